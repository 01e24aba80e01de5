// Packed 8-bit projections: y[M,N] = x[M,K] . W[N,K]^T with W as signed 8-bit codes, four to a
// 32-bit word (code k of a word at bit 8k, two's complement), one scale per group along K.
//
// First kernel of the eight-bit path: a warp per weight row (a few CTAs per SM, each warp walking
// rows a grid stride apart), the lanes stride over units of eight codes (two words, one 8-byte
// load), MR activation rows of the CTA staged in shared memory so that a decoded weight is used
// MR times. Every weight is rounded to bf16 as
// code * scale before it is multiplied - the value the dequantise-then-multiply form of the
// reference materialises - and products accumulate in fp32. The single-row form (MR = 1) takes
// the fused RMS-norm prologue and the paired gate/up epilogue like the four-bit GEMV.
#include "qgemv_core.cuh"

namespace aoto {

constexpr int I8_WARPS = 8;

__device__ __forceinline__ void i8_decode8(const uint2 words, const float scale, float (&w)[8]) {
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int lo = ((int)(words.x << (24 - 8 * i))) >> 24;
    const int hi = ((int)(words.y << (24 - 8 * i))) >> 24;
    w[i] = round_bf16((float)lo * scale);
    w[4 + i] = round_bf16((float)hi * scale);
  }
}

template <int MR>
__global__ void __launch_bounds__(I8_WARPS * 32)
qmatmul_i8_kernel(const GemvParams p, const int M) {
  extern __shared__ uint4 smem[];
  const int K = p.K, N = p.N, chunks = K >> 3;
  uint4* xs = smem;                                            // MR rows of K bf16
  float* red = reinterpret_cast<float*>(xs + (size_t)MR * chunks);
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int m0 = blockIdx.y * MR;
  pdl_wait_for_producers();
  pdl_release_dependents();
  if (MR == 1) {
    stage_activation<false>(p, p.x + (size_t)m0 * K, xs, nullptr, red);
  } else {
    const uint4* xv = reinterpret_cast<const uint4*>(p.x);
    for (int c = tid; c < MR * chunks; c += blockDim.x) {
      const int r = c / chunks, j = c - r * chunks;
      xs[c] = (m0 + r < M) ? xv[(size_t)(m0 + r) * chunks + j] : make_uint4(0u, 0u, 0u, 0u);
    }
    __syncthreads();
  }

  const int row_sc = K / p.group;
  const bool paired = p.epilogue == AOTO_EPILOGUE_SILU_MUL_PAIRED;
  // The grid is a few CTAs per SM, not one per eight rows: a warp walks rows n, n + stride, ...
  // so that staging the activation is paid once per CTA and not once per 8 x K bytes of weight.
  for (int n = blockIdx.x * I8_WARPS + warp; n < N; n += gridDim.x * I8_WARPS) {
  const uint2* w0 = reinterpret_cast<const uint2*>(p.w0) + (size_t)n * chunks;
  const uint2* w1 = reinterpret_cast<const uint2*>(p.w1) + (size_t)n * chunks;
  float acc[MR], acc2[MR];
#pragma unroll
  for (int r = 0; r < MR; ++r) acc[r] = acc2[r] = 0.f;
  // With a single activation row several units of a lane are requested before the first is used
  // (a row is short, K bytes); with staged rows the registers go to the accumulators instead.
  constexpr int AHEAD = MR == 1 ? 4 : 1;
  const bf16* sc0 = p.s0 + (size_t)n * row_sc;
  const bf16* sc1 = paired ? p.s1 + (size_t)n * row_sc : sc0;
  for (int j0 = lane; j0 < chunks; j0 += 32 * AHEAD) {
    uint2 q0[AHEAD], q1[AHEAD];
    float scale0[AHEAD], scale1[AHEAD];
#pragma unroll
    for (int a = 0; a < AHEAD; ++a) {
      const int j = j0 + 32 * a;
      q0[a] = q1[a] = make_uint2(0u, 0u);
      scale0[a] = scale1[a] = 0.f;
      if (j < chunks) {
        const int gidx = (j * 8) / p.group;
        q0[a] = __ldg(w0 + j);
        scale0[a] = ldg_nc_bf16(sc0 + gidx);
        if (paired) {
          q1[a] = __ldg(w1 + j);
          scale1[a] = ldg_nc_bf16(sc1 + gidx);
        }
      }
    }
#pragma unroll
    for (int a = 0; a < AHEAD; ++a) {
      const int j = j0 + 32 * a;
      if (j >= chunks) break;
      float w[8], v[8];
      i8_decode8(q0[a], scale0[a], w);
      if (paired) i8_decode8(q1[a], scale1[a], v);
#pragma unroll
      for (int r = 0; r < MR; ++r) {
        float xf[8];
        unpack8(xs[(size_t)r * chunks + j], xf);
#pragma unroll
        for (int i = 0; i < 8; ++i) acc[r] = fmaf(w[i], xf[i], acc[r]);
        if (paired) {
#pragma unroll
          for (int i = 0; i < 8; ++i) acc2[r] = fmaf(v[i], xf[i], acc2[r]);
        }
      }
    }
  }
#pragma unroll
  for (int r = 0; r < MR; ++r) {
    const float total = warp_sum(acc[r]);
    const float total2 = paired ? warp_sum(acc2[r]) : 0.f;
    const int m = m0 + r;
    if (lane == 0 && m < M) p.out[(size_t)m * N + n] = __float2bfloat16_rn(finish_output(p, m, n, total, total2));
  }
  }  // rows of this warp
}

// W[n, 4j+i] = bf16(code) * bf16(scale[n, (4j+i)/group]) rounded once to bf16; a thread per unit
// of eight codes.
__global__ void __launch_bounds__(256)
dequantize_i8_kernel(const uint2* __restrict__ packed, const bf16* __restrict__ scales, uint4* __restrict__ out,
                     const int64_t units, const int chunks, const int group) {
  const int64_t u = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (u >= units) return;
  const int64_t n = u / chunks;
  const int j = (int)(u - n * chunks);
  const int row_sc = chunks * 8 / group;
  float w[8];
  i8_decode8(__ldg(packed + u), __bfloat162float(scales[n * row_sc + (j * 8) / group]), w);
  uint4 o;
  o.x = pack_bf16x2(w[0], w[1]);
  o.y = pack_bf16x2(w[2], w[3]);
  o.z = pack_bf16x2(w[4], w[5]);
  o.w = pack_bf16x2(w[6], w[7]);
  out[u] = o;
}

// Shapes the eight-bit kernel takes: units of eight codes along K and per group, K small enough
// for MR staged rows; norm and the paired form only with a single activation row.
bool qmatmul_i8_supported(const aoto_qmatmul_args& a) {
  if (a.M <= 0 || a.N <= 0 || a.K <= 0 || a.group_size <= 0) return false;
  if ((a.K % 8) != 0 || (a.group_size % 8) != 0 || (a.K % a.group_size) != 0 || a.K > 32768) return false;
  if (a.M > 1 && (a.norm_weight != nullptr || a.epilogue == AOTO_EPILOGUE_SILU_MUL_PAIRED)) return false;
  return true;
}

template <int MR>
static int launch_i8(const GemvParams& p, int M, cudaStream_t stream, bool pdl) {
  const size_t smem = (size_t)MR * p.K * 2 + 32 * 4;
  auto kernel = qmatmul_i8_kernel<MR>;
  if (smem > 48 * 1024) {
    static PerDeviceOnce raised;
    if (raise_dynamic_smem(kernel, 160 * 1024, raised) != AOTO_OK) return AOTO_ERR_LAUNCH;
    if (smem > 160 * 1024) return AOTO_ERR_UNSUPPORTED;
  }
  const int row_groups = (M + MR - 1) / MR;
  const int wanted = (p.N + I8_WARPS - 1) / I8_WARPS;
  const int per_group = 148 * 6 / (row_groups < 6 ? row_groups : 6);  // about six CTAs per SM in all
  dim3 grid(wanted < per_group ? wanted : per_group, row_groups), block(I8_WARPS * 32);
  return launch_kernel(kernel, grid, block, smem, stream, pdl, p, M);
}

int qmatmul_i8_launch(const aoto_qmatmul_args& a, cudaStream_t stream) {
  if (!qmatmul_i8_supported(a)) return AOTO_ERR_UNSUPPORTED;
  if (!aligned_to(a.packed, 8) || (a.packed2 && !aligned_to(a.packed2, 8))) return AOTO_ERR_ARGUMENT;
  GemvParams p;
  p.x = (const bf16*)a.x;
  p.w0 = (const uint32_t*)a.packed;
  p.s0 = (const bf16*)a.scales;
  p.w1 = (const uint32_t*)a.packed2;
  p.s1 = (const bf16*)a.scales2;
  p.addend = (const bf16*)a.addend;
  p.gate = (const bf16*)a.gate;
  p.norm_w = (const bf16*)a.norm_weight;
  p.out = (bf16*)a.out;
  p.N = a.N; p.K = a.K; p.group = a.group_size;
  p.addend_kind = a.addend_kind; p.epilogue = a.epilogue;
  p.alpha = a.alpha; p.beta = a.beta; p.eps = a.rms_norm_eps;
  const bool pdl = (a.flags & AOTO_FLAG_PDL) != 0;
  if (a.M == 1) return launch_i8<1>(p, a.M, stream, pdl);
  // more staged rows reuse a decoded weight more often; 8 rows of K <= 8192 fit 128 KB
  if (a.M >= 8 && a.K <= 8192) return launch_i8<8>(p, a.M, stream, pdl);
  if (a.M >= 4 && a.K <= 16384) return launch_i8<4>(p, a.M, stream, pdl);
  return launch_i8<2>(p, a.M, stream, pdl);
}

const char* qmatmul_i8_variant(const aoto_qmatmul_args& a) { return a.M == 1 ? "qgemv_i8" : "qgemm_i8_rows"; }

int dequantize_i8_launch(const aoto_dequantize_args& a, cudaStream_t stream) {
  if ((a.K % 8) != 0 || (a.group_size % 8) != 0 || (a.K % a.group_size) != 0) return AOTO_ERR_UNSUPPORTED;
  const int chunks = a.K / 8;
  const int64_t units = (int64_t)a.N * chunks;
  const int64_t blocks = (units + 255) / 256;
  if (blocks > 0x7fffffff) return AOTO_ERR_UNSUPPORTED;
  return launch_kernel(dequantize_i8_kernel, dim3((unsigned)blocks), dim3(256), 0, stream, false,
                       (const uint2*)a.packed, (const bf16*)a.scales, (uint4*)a.out, units, chunks, a.group_size);
}

}  // namespace aoto
