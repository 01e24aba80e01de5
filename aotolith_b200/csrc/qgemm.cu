// Packed 4-bit GEMM for several activation rows (prefill): y[M,N] = x[M,K] . W[N,K]^T.
//
// The weight is read from HBM once per 128 activation rows and is never materialised: every
// warp turns its 16-row x 128-column block of packed words into bf16 A fragments in registers -
// code (exact) times scale, rounded once to bf16, which is bit for bit the weight the reference
// materialises before its dense product - and multiplies it against the activation tile staged
// in shared memory (mma.sync m16n8k16, fp32 accumulate). The product is computed transposed
// (rows of W are the M dimension of the mma, activation rows its N dimension), so the fragment
// layout of the GEMV kernel is reused unchanged.
//
// CTA = WN x WM warps: WN row tiles of 16 weight rows, WM slices of the 128-row activation
// tile. The activation tile of one 128-column block (128 x 128 bf16) is staged with the same
// in-chunk permutation the fragments use and double buffered; the next block's packed words are
// requested before the current block is multiplied.
#include <cuda_fp16.h>

#include "qgemv_core.cuh"

namespace aoto {

constexpr int GEMM_M_TILE = 128;               // activation rows per CTA
constexpr int GEMM_ROW_BYTES = 256 + 64;       // one staged row: 16 chunks of 16 B + padding
constexpr int GEMM_STAGE_BYTES = GEMM_M_TILE * GEMM_ROW_BYTES;

struct GemmParams {
  const bf16* x;
  const uint32_t* w;
  const bf16* s;
  const bf16* addend;
  const bf16* gate;
  bf16* out;
  int M, N, K;
  int addend_kind, epilogue;
  float alpha, beta;
};

// exact (136 + code) pairs -> bf16(code * scale) pairs
__device__ __forceinline__ uint32_t scaled_pair(uint32_t biased, __nv_bfloat162 scale2) {
  __nv_bfloat162 v = *reinterpret_cast<__nv_bfloat162*>(&biased);
  const __nv_bfloat162 offset = __float2bfloat162_rn(136.f);
  v = __hmul2(__hsub2(v, offset), scale2);
  return *reinterpret_cast<uint32_t*>(&v);
}

template <int WN, int WM>
__global__ void __launch_bounds__(WN * WM * 32)
qgemm_mma_kernel(const GemmParams p) {
  constexpr int THREADS = WN * WM * 32;
  constexpr int M_PER_WARP = GEMM_M_TILE / WM;   // activation rows a warp covers
  constexpr int NT = M_PER_WARP / 8;             // mma n-tiles per warp
  extern __shared__ uint4 smem[];
  unsigned char* stage[2] = {reinterpret_cast<unsigned char*>(smem),
                             reinterpret_cast<unsigned char*>(smem) + GEMM_STAGE_BYTES};

  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int g = lane >> 2, t = lane & 3;
  const int wn = warp % WN, wm = warp / WN;
  const int K = p.K, N = p.N, M = p.M;
  const int nblocks = K >> 7;
  const int row_u4 = K >> 5, row_sc = K >> 6;
  const int tile = blockIdx.x * WN + wn;
  const int m_base = blockIdx.y * GEMM_M_TILE;
  const int rlo = min(tile * 16 + g, N - 1), rhi = min(tile * 16 + g + 8, N - 1);
  const uint4* wq = reinterpret_cast<const uint4*>(p.w);

  auto load_weights = [&](int kb, WeightItem* it) {
    it->lo = ldg_nc_u4(wq + (size_t)rlo * row_u4 + kb * 4 + t);
    it->hi = ldg_nc_u4(wq + (size_t)rhi * row_u4 + kb * 4 + t);
    it->slo = __ldg(reinterpret_cast<const uint32_t*>(p.s + (size_t)rlo * row_sc + kb * 2));
    it->shi = __ldg(reinterpret_cast<const uint32_t*>(p.s + (size_t)rhi * row_sc + kb * 2));
  };
  // Block kb of the activation tile travels global -> registers (before the block's mma) ->
  // shared memory (after them): chunk q = 4*t' + j of a row goes to slot 4*j + t', with its
  // eight values in fragment order [0,4,1,5,2,6,3,7].
  constexpr int CHUNKS = GEMM_M_TILE * 16 / THREADS;
  uint4 held[CHUNKS];
  auto fetch_x = [&](int kb) {
#pragma unroll
    for (int u = 0; u < CHUNKS; ++u) {
      const int c = tid + u * THREADS;
      const int m = m_base + (c >> 4);
      held[u] = make_uint4(0u, 0u, 0u, 0u);
      if (m < M) held[u] = __ldg(reinterpret_cast<const uint4*>(p.x + (size_t)m * K + kb * 128 + (c & 15) * 8));
    }
  };
  auto store_x = [&](unsigned char* dst) {
#pragma unroll
    for (int u = 0; u < CHUNKS; ++u) {
      const int c = tid + u * THREADS;
      const int r = c >> 4, q = c & 15;
      const uint4 v = held[u];
      uint4 o;
      o.x = __byte_perm(v.x, v.z, 0x5410);  // (x0, x4)
      o.y = __byte_perm(v.x, v.z, 0x7632);  // (x1, x5)
      o.z = __byte_perm(v.y, v.w, 0x5410);  // (x2, x6)
      o.w = __byte_perm(v.y, v.w, 0x7632);  // (x3, x7)
      const int slot = (q & 3) * 4 + (q >> 2);
      *reinterpret_cast<uint4*>(dst + (size_t)r * GEMM_ROW_BYTES + slot * 16) = o;
    }
  };

  float acc[NT][4];
#pragma unroll
  for (int i = 0; i < NT; ++i) acc[i][0] = acc[i][1] = acc[i][2] = acc[i][3] = 0.f;

  WeightItem current, next;
  load_weights(0, &current);
  next = current;
  fetch_x(0);
  store_x(stage[0]);
  __syncthreads();

  for (int kb = 0; kb < nblocks; ++kb) {
    const unsigned char* xs = stage[kb & 1];
    const bool more = kb + 1 < nblocks;
    if (more) {
      load_weights(kb + 1, &next);
      fetch_x(kb + 1);
    }
    // A fragments of this block: bf16(code * scale), the scale of the group the codes are in
    const __nv_bfloat162 s_lo_a = __bfloat162bfloat162(__ushort_as_bfloat16((unsigned short)(current.slo & 0xffffu)));
    const __nv_bfloat162 s_lo_b = __bfloat162bfloat162(__ushort_as_bfloat16((unsigned short)(current.slo >> 16)));
    const __nv_bfloat162 s_hi_a = __bfloat162bfloat162(__ushort_as_bfloat16((unsigned short)(current.shi & 0xffffu)));
    const __nv_bfloat162 s_hi_b = __bfloat162bfloat162(__ushort_as_bfloat16((unsigned short)(current.shi >> 16)));
    // lanes t = 0,1 hold codes of the block's first group, t = 2,3 of its second
    const __nv_bfloat162 s_lo = (t < 2) ? s_lo_a : s_lo_b;
    const __nv_bfloat162 s_hi = (t < 2) ? s_hi_a : s_hi_b;
    const uint32_t wl[4] = {current.lo.x, current.lo.y, current.lo.z, current.lo.w};
    const uint32_t wh[4] = {current.hi.x, current.hi.y, current.hi.z, current.hi.w};
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const uint32_t a0 = scaled_pair(AOTO_NIB(wl[j], 0), s_lo), a1 = scaled_pair(AOTO_NIB(wh[j], 0), s_hi);
      const uint32_t a2 = scaled_pair(AOTO_NIB(wl[j], 4), s_lo), a3 = scaled_pair(AOTO_NIB(wh[j], 4), s_hi);
      const uint32_t a4 = scaled_pair(AOTO_NIB(wl[j], 8), s_lo), a5 = scaled_pair(AOTO_NIB(wh[j], 8), s_hi);
      const uint32_t a6 = scaled_pair(AOTO_NIB(wl[j], 12), s_lo), a7 = scaled_pair(AOTO_NIB(wh[j], 12), s_hi);
#pragma unroll
      for (int i = 0; i < NT; ++i) {
        const int r = wm * M_PER_WARP + i * 8 + g;
        const uint4 b = *reinterpret_cast<const uint4*>(xs + (size_t)r * GEMM_ROW_BYTES + (j * 4 + t) * 16);
        mma_16816(acc[i], a0, a1, a2, a3, b.x, b.y);
        mma_16816(acc[i], a4, a5, a6, a7, b.z, b.w);
      }
    }
    // the other buffer was last read in the previous iteration, which ended with a barrier
    if (more) store_x(stage[(kb + 1) & 1]);
    current = next;
    __syncthreads();
  }

  // epilogue: acc[i] = {(row g, m 2t), (row g, m 2t+1), (row g+8, m 2t), (row g+8, m 2t+1)}
#pragma unroll
  for (int i = 0; i < NT; ++i) {
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const int n = tile * 16 + g + (e >> 1) * 8;
      const int m = m_base + wm * M_PER_WARP + i * 8 + 2 * t + (e & 1);
      if (n >= N || m >= M) continue;
      float y = p.alpha * acc[i][e];
      if (p.addend_kind == AOTO_ADDEND_VECTOR) y = fmaf(p.beta, __bfloat162float(p.addend[n]), y);
      else if (p.addend_kind == AOTO_ADDEND_FULL) y = fmaf(p.beta, __bfloat162float(p.addend[(size_t)m * N + n]), y);
      if (p.epilogue == AOTO_EPILOGUE_SILU_MUL) {
        const float gate = __bfloat162float(p.gate[(size_t)m * N + n]);
        y = y * (gate / (1.f + expf(-gate)));
      }
      p.out[(size_t)m * N + n] = __float2bfloat16_rn(y);
    }
  }
}

template <int WN, int WM>
static int launch_gemm(const GemmParams& p, cudaStream_t stream) {
  auto kernel = qgemm_mma_kernel<WN, WM>;
  const size_t smem = 2 * (size_t)GEMM_STAGE_BYTES;
  static PerDeviceOnce raised;
  if (raise_dynamic_smem(kernel, smem, raised) != AOTO_OK) return AOTO_ERR_LAUNCH;
  const int tiles = (p.N + 15) / 16;
  dim3 grid((tiles + WN - 1) / WN, (p.M + GEMM_M_TILE - 1) / GEMM_M_TILE), block(WN * WM * 32);
  return launch_kernel(kernel, grid, block, smem, stream, false, p);
}

bool qgemm_applies(const aoto_qmatmul_args& a) {
  return a.M > 1 && a.group_size == 64 && (a.K % 128) == 0 && a.norm_weight == nullptr &&
         a.epilogue != AOTO_EPILOGUE_SILU_MUL_PAIRED;
}

int qgemm_launch(const aoto_qmatmul_args& a, cudaStream_t stream) {
  GemmParams p;
  p.x = (const bf16*)a.x;
  p.w = (const uint32_t*)a.packed;
  p.s = (const bf16*)a.scales;
  p.addend = (const bf16*)a.addend;
  p.gate = (const bf16*)a.gate;
  p.out = (bf16*)a.out;
  p.M = a.M; p.N = a.N; p.K = a.K;
  p.addend_kind = a.addend_kind; p.epilogue = a.epilogue;
  p.alpha = a.alpha; p.beta = a.beta;
  const int tiles = (a.N + 15) / 16;
  const int m_tiles = (a.M + GEMM_M_TILE - 1) / GEMM_M_TILE;
  // narrow matrices: fewer weight rows per CTA so that more SMs take part
  if ((tiles / 4) * m_tiles < 74) return launch_gemm<2, 4>(p, stream);
  return launch_gemm<4, 2>(p, stream);
}

}  // namespace aoto
