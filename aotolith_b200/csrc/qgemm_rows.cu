// Packed 4-bit products for a FEW activation rows (2..16): a decode step over several tokens,
// the short buckets of a prompt pass.
//
// The large-tile kernels spend such a product on latency: a 128-row activation tile is staged and
// multiplied block after block of K behind a CTA-wide barrier, eleven microseconds for seven
// blocks however few rows are real. Here the product is shaped like the one-row GEMV instead. The
// whole activation [rows, K] is staged in shared memory once (in the fragment order of the GEMM
// kernel); a CTA owns a tile of sixteen weight rows and its eight warps SHARE the 128-column blocks
// of K, each with the packed words of its next blocks already requested; every warp turns its block
// into bf16(code * scale) A fragments - the weight the reference materialises, bit for bit - and
// multiplies them against eight (or sixteen) activation rows at once: the activation rows are the
// columns of the mma. The warps' partial C tiles meet in shared memory; 128 (256) threads add them
// in a fixed order and run the epilogue. A persistent grid walks the tiles.
#include "qgemv_core.cuh"

namespace aoto {

constexpr int QR_WARPS = 8;
constexpr int QR_AHEAD = 2;  // 128-column blocks of a warp in flight

struct RowsParams {
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
__device__ __forceinline__ uint32_t rows_scaled_pair(uint32_t biased, __nv_bfloat162 scale2) {
  __nv_bfloat162 v = *reinterpret_cast<__nv_bfloat162*>(&biased);
  v = __hmul2(__hsub2(v, __float2bfloat162_rn(136.f)), scale2);
  return *reinterpret_cast<uint32_t*>(&v);
}

// One staged row: K bf16 and 64 bytes, so that neighbouring rows start 16 banks apart.
__host__ __device__ inline size_t rows_row_bytes(int K) { return (size_t)K * 2 + 64; }

template <int NT>  // mma n-tiles: 8 * NT staged activation rows
__global__ void __launch_bounds__(QR_WARPS * 32)
qgemm_rows_kernel(const RowsParams p) {
  extern __shared__ uint4 smem[];
  constexpr int ROWS = 8 * NT;
  const int K = p.K, N = p.N, M = p.M;
  const int nblocks = K >> 7, row_u4 = K >> 5, row_sc = K >> 6, chunks = K >> 3;
  const size_t row_bytes = rows_row_bytes(K);
  unsigned char* xs = reinterpret_cast<unsigned char*>(smem);
  float* part = reinterpret_cast<float*>(xs + (size_t)ROWS * row_bytes);  // [warp][NT*4][32]
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int g = lane >> 2, t = lane & 3;
  const int tiles = (N + 15) >> 4;

  pdl_wait_for_producers();
  pdl_release_dependents();
  // Stage the activation: chunk q = 4*t' + j of a 128-column block goes to slot 4*j + t' with its
  // eight values in fragment order [0,4,1,5,2,6,3,7]; rows beyond M are zero.
  for (int c = tid; c < ROWS * chunks; c += QR_WARPS * 32) {
    const int r = c / chunks, cc = c - r * chunks;
    const int kb = cc >> 4, q = cc & 15;
    uint4 v = make_uint4(0u, 0u, 0u, 0u);
    if (r < M) v = *reinterpret_cast<const uint4*>(p.x + (size_t)r * K + (size_t)cc * 8);
    uint4 o;
    o.x = __byte_perm(v.x, v.z, 0x5410);  // (x0, x4)
    o.y = __byte_perm(v.x, v.z, 0x7632);  // (x1, x5)
    o.z = __byte_perm(v.y, v.w, 0x5410);  // (x2, x6)
    o.w = __byte_perm(v.y, v.w, 0x7632);  // (x3, x7)
    const int slot = (q & 3) * 4 + (q >> 2);
    *reinterpret_cast<uint4*>(xs + (size_t)r * row_bytes + (size_t)kb * 256 + slot * 16) = o;
  }
  __syncthreads();

  const uint4* wq = reinterpret_cast<const uint4*>(p.w);
  for (int tile = blockIdx.x; tile < tiles; tile += gridDim.x) {
    const int rlo = min(tile * 16 + g, N - 1), rhi = min(tile * 16 + g + 8, N - 1);
    float acc[NT][4];
#pragma unroll
    for (int i = 0; i < NT; ++i) acc[i][0] = acc[i][1] = acc[i][2] = acc[i][3] = 0.f;

    for (int kb0 = warp; kb0 < nblocks; kb0 += QR_WARPS * QR_AHEAD) {
      WeightItem item[QR_AHEAD];
#pragma unroll
      for (int a = 0; a < QR_AHEAD; ++a) {
        const int kb = kb0 + a * QR_WARPS;
        if (kb < nblocks) {
          item[a].lo = ldg_nc_u4(wq + (size_t)rlo * row_u4 + kb * 4 + t);
          item[a].hi = ldg_nc_u4(wq + (size_t)rhi * row_u4 + kb * 4 + t);
          item[a].slo = __ldg(reinterpret_cast<const uint32_t*>(p.s + (size_t)rlo * row_sc + kb * 2));
          item[a].shi = __ldg(reinterpret_cast<const uint32_t*>(p.s + (size_t)rhi * row_sc + kb * 2));
        }
      }
#pragma unroll
      for (int a = 0; a < QR_AHEAD; ++a) {
        const int kb = kb0 + a * QR_WARPS;
        if (kb >= nblocks) break;
        const WeightItem& it = item[a];
        // lanes t = 0,1 hold codes of the block's first group, t = 2,3 of its second
        const unsigned short raw_lo = (unsigned short)(t < 2 ? (it.slo & 0xffffu) : (it.slo >> 16));
        const unsigned short raw_hi = (unsigned short)(t < 2 ? (it.shi & 0xffffu) : (it.shi >> 16));
        const __nv_bfloat162 s_lo = __bfloat162bfloat162(__ushort_as_bfloat16(raw_lo));
        const __nv_bfloat162 s_hi = __bfloat162bfloat162(__ushort_as_bfloat16(raw_hi));
        const uint32_t wl[4] = {it.lo.x, it.lo.y, it.lo.z, it.lo.w};
        const uint32_t wh[4] = {it.hi.x, it.hi.y, it.hi.z, it.hi.w};
        const unsigned char* xb = xs + (size_t)kb * 256 + t * 16;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const uint32_t a0 = rows_scaled_pair(AOTO_NIB(wl[j], 0), s_lo), a1 = rows_scaled_pair(AOTO_NIB(wh[j], 0), s_hi);
          const uint32_t a2 = rows_scaled_pair(AOTO_NIB(wl[j], 4), s_lo), a3 = rows_scaled_pair(AOTO_NIB(wh[j], 4), s_hi);
          const uint32_t a4 = rows_scaled_pair(AOTO_NIB(wl[j], 8), s_lo), a5 = rows_scaled_pair(AOTO_NIB(wh[j], 8), s_hi);
          const uint32_t a6 = rows_scaled_pair(AOTO_NIB(wl[j], 12), s_lo), a7 = rows_scaled_pair(AOTO_NIB(wh[j], 12), s_hi);
#pragma unroll
          for (int i = 0; i < NT; ++i) {
            const uint4 b = *reinterpret_cast<const uint4*>(xb + (size_t)(i * 8 + g) * row_bytes + j * 64);
            mma_16816(acc[i], a0, a1, a2, a3, b.x, b.y);
            mma_16816(acc[i], a4, a5, a6, a7, b.z, b.w);
          }
        }
      }
    }

    // the warps' partial tiles meet in shared memory
#pragma unroll
    for (int i = 0; i < NT; ++i)
#pragma unroll
      for (int e = 0; e < 4; ++e) part[((size_t)warp * NT * 4 + i * 4 + e) * 32 + lane] = acc[i][e];
    __syncthreads();
    for (int u = tid; u < NT * 4 * 32; u += QR_WARPS * 32) {
      // element u = (i, e, lane) of a C tile: row g (+8 for e >= 2) of W, activation i*8 + 2t + (e & 1)
      const int ie = u >> 5, ln = u & 31;
      const int i = ie >> 2, e = ie & 3;
      const int n = tile * 16 + (ln >> 2) + (e >> 1) * 8;
      const int m = i * 8 + 2 * (ln & 3) + (e & 1);
      float total = 0.f;
#pragma unroll
      for (int w = 0; w < QR_WARPS; ++w) total += part[(size_t)w * NT * 4 * 32 + u];
      if (n < N && m < M) {
        float y = p.alpha * total;
        if (p.addend_kind == AOTO_ADDEND_VECTOR) y = fmaf(p.beta, __bfloat162float(p.addend[n]), y);
        else if (p.addend_kind == AOTO_ADDEND_FULL) y = fmaf(p.beta, __bfloat162float(p.addend[(size_t)m * N + n]), y);
        if (p.epilogue == AOTO_EPILOGUE_SILU_MUL) {
          const float gate = __bfloat162float(p.gate[(size_t)m * N + n]);
          y = y * (gate / (1.f + expf(-gate)));
        }
        p.out[(size_t)m * N + n] = __float2bfloat16_rn(y);
      }
    }
    __syncthreads();  // the next tile overwrites the partial tiles
  }
}

static size_t rows_smem_bytes(int nt, int K) {
  return (size_t)8 * nt * rows_row_bytes(K) + (size_t)QR_WARPS * nt * 4 * 32 * 4;
}

// Two to sixteen activation rows whose staged copy fits shared memory beside the partial tiles.
bool qgemm_rows_applies(const aoto_qmatmul_args& a) {
  if (a.M < 2 || a.M > 16 || a.group_size != 64 || (a.K % 128) != 0 || a.N < 16) return false;
  if (a.norm_weight != nullptr || a.epilogue == AOTO_EPILOGUE_SILU_MUL_PAIRED) return false;
  if (a.flags & (AOTO_FLAG_WEIGHT_BITS_8 | AOTO_FLAG_WEIGHT_DENSE)) return false;
  return rows_smem_bytes(a.M <= 8 ? 1 : 2, a.K) <= 200 * 1024;
}

template <int NT>
static int launch_rows(const RowsParams& p, cudaStream_t stream) {
  auto kernel = qgemm_rows_kernel<NT>;
  const size_t smem = rows_smem_bytes(NT, p.K);
  static PerDeviceOnce raised;
  if (raise_dynamic_smem(kernel, 200 * 1024, raised) != AOTO_OK) return AOTO_ERR_LAUNCH;
  int resident = 0;
  if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&resident, kernel, QR_WARPS * 32, smem) != cudaSuccess || resident < 1) {
    (void)cudaGetLastError();
    resident = 1;
  }
  const int tiles = (p.N + 15) / 16;
  const int most = 148 * resident;
  return launch_kernel(kernel, dim3(tiles < most ? tiles : most), dim3(QR_WARPS * 32), smem, stream, false, p);
}

int qgemm_rows_launch(const aoto_qmatmul_args& a, cudaStream_t stream) {
  if (!qgemm_rows_applies(a)) return AOTO_ERR_UNSUPPORTED;
  RowsParams p;
  p.x = (const bf16*)a.x;
  p.w = (const uint32_t*)a.packed;
  p.s = (const bf16*)a.scales;
  p.addend = (const bf16*)a.addend;
  p.gate = (const bf16*)a.gate;
  p.out = (bf16*)a.out;
  p.M = a.M; p.N = a.N; p.K = a.K;
  p.addend_kind = a.addend_kind; p.epilogue = a.epilogue;
  p.alpha = a.alpha; p.beta = a.beta;
  return a.M <= 8 ? launch_rows<1>(p, stream) : launch_rows<2>(p, stream);
}

}  // namespace aoto
