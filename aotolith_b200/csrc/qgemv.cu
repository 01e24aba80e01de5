// Packed 4-bit GEMV (single activation row per grid.y slice) for sm_100a.
//
// Two kernels:
//
//  * qgemv_mma_kernel  - group 64, K % 128 == 0. The weight stream is the only
//    HBM traffic that matters, so the kernel is built around it: every lane
//    issues 128-bit loads of packed words, nibbles are turned into bf16 values
//    in registers with one logic op per code pair, and the multiply-accumulate
//    runs on the tensor pipe (mma.sync m16n8k16, fp32 accumulate) so the ALU
//    only pays for the decode. One warp owns a 16-row x 128-column block of W
//    at a time; the warps of a CTA split K and reduce through shared memory in
//    a fixed order, so results are deterministic.
//
//  * qgemv_generic_kernel - any group size that is a multiple of 8 and any K
//    that is a multiple of it; one warp per output row, scalar decode. It is
//    the shape-complete variant small test models and odd shapes use.
//
// Both apply the optional RMS-norm prologue to the activation row while
// staging it in shared memory (fp32 statistics, x_hat rounded to bf16), and
// the epilogues of the packed matmul/addmm operation.
#include "qgemv_core.cuh"

namespace aoto {

// Block = 16 rows x 128 columns of W (two groups of 64). Lane (g = lane/4,
// t = lane%4) holds codes [32t, 32t+32) of rows g and g+8. The eight mma of a
// block all accumulate into one C tile; B column parity separates the two
// groups (even columns see only x of the first group, odd of the second), so
// C[row][0] and C[row][1] are the two per-group code sums of that row.
template <int RT, int UK, bool PAIRED>
__global__ void __launch_bounds__(256)
qgemv_mma_kernel(const GemvParams p) {
  constexpr int MATS = PAIRED ? 2 : 1;
  extern __shared__ uint4 smem[];
  const int K = p.K, N = p.N;
  const int nblocks = K >> 7, groups = K >> 6, chunks = K >> 3;
  const int W = blockDim.x >> 5;
  uint4* xs = smem;
  uint4* zero16 = xs + chunks;  // directly after the 16-byte chunks, so it is 16-byte aligned
  float* xsum = reinterpret_cast<float*>(zero16 + 1);
  float* csum = xsum + groups;
  float* part = csum + chunks;
  float* red = part + MATS * RT * W * 16;

  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int g = lane >> 2, t = lane & 3;
  const int m = blockIdx.y;
  if (tid == 0) *zero16 = make_uint4(0u, 0u, 0u, 0u);
  const int tile0 = blockIdx.x * RT;
  const int per_rt = (nblocks + W - 1) / W;
  const int row_u4 = K >> 5;   // uint4 per packed row
  const int row_sc = K >> 6;   // scales per row

  int rlo[RT], rhi[RT];
#pragma unroll
  for (int rt = 0; rt < RT; ++rt) {
    rlo[rt] = min((tile0 + rt) * 16 + g, N - 1);
    rhi[rt] = min((tile0 + rt) * 16 + g + 8, N - 1);
  }

  WeightItem item[MATS][RT][UK];
  auto load_batch = [&](int step) {
#pragma unroll
    for (int u = 0; u < UK; ++u) {
      const int kb = warp + (step + u) * W;
      if (kb < nblocks) {
#pragma unroll
        for (int mat = 0; mat < MATS; ++mat) {
          const uint4* wq = reinterpret_cast<const uint4*>(mat == 0 ? p.w0 : p.w1);
          const bf16* sc = mat == 0 ? p.s0 : p.s1;
#pragma unroll
          for (int rt = 0; rt < RT; ++rt) {
            WeightItem& it = item[mat][rt][u];
            it.lo = ldg_nc_u4(wq + (size_t)rlo[rt] * row_u4 + kb * 4 + t);
            it.hi = ldg_nc_u4(wq + (size_t)rhi[rt] * row_u4 + kb * 4 + t);
            it.slo = __ldg(reinterpret_cast<const uint32_t*>(sc + (size_t)rlo[rt] * row_sc + kb * 2));
            it.shi = __ldg(reinterpret_cast<const uint32_t*>(sc + (size_t)rhi[rt] * row_sc + kb * 2));
          }
        }
      }
    }
  };

  // Weights do not depend on the producer of x: start streaming them before
  // waiting for it.
  load_batch(0);
  pdl_wait_for_producers();
  pdl_release_dependents();

  stage_activation<true>(p, p.x + (size_t)m * K, xs, csum, red);
  for (int gidx = tid; gidx < groups; gidx += blockDim.x) {
    float s = 0.f;
#pragma unroll
    for (int c = 0; c < 8; ++c) s += csum[gidx * 8 + c];
    xsum[gidx] = 136.f * s;
  }
  __syncthreads();

  float acc[MATS][RT][2];
#pragma unroll
  for (int mat = 0; mat < MATS; ++mat)
#pragma unroll
    for (int rt = 0; rt < RT; ++rt) acc[mat][rt][0] = acc[mat][rt][1] = 0.f;

  // even B columns carry the first group of the block, odd ones the second
  const BSource bs = b_source(xs, zero16, lane);

  for (int step = 0; step < per_rt; step += UK) {
    if (step > 0) load_batch(step);
#pragma unroll
    for (int u = 0; u < UK; ++u) {
      const int kb = warp + (step + u) * W;
      if (kb < nblocks) {
#pragma unroll
        for (int mat = 0; mat < MATS; ++mat) {
#pragma unroll
          for (int rt = 0; rt < RT; ++rt) {
            float lo, hi;
            mma_block(item[mat][rt][u], bs, kb, xsum, lo, hi);
            acc[mat][rt][0] += lo;
            acc[mat][rt][1] += hi;
          }
        }
      }
    }
  }

  if (t == 0) {
#pragma unroll
    for (int mat = 0; mat < MATS; ++mat)
#pragma unroll
      for (int rt = 0; rt < RT; ++rt) {
        float* dst = part + ((mat * RT + rt) * W + warp) * 16;
        dst[g] = acc[mat][rt][0];
        dst[g + 8] = acc[mat][rt][1];
      }
  }
  __syncthreads();
  if (tid < RT * 16) {
    const int rt = tid >> 4, r = tid & 15;
    const int n = (tile0 + rt) * 16 + r;
    if (n < N) {
      float total = 0.f, total2 = 0.f;
      for (int w = 0; w < W; ++w) total += part[((0 * RT + rt) * W + w) * 16 + r];
      if (PAIRED)
        for (int w = 0; w < W; ++w) total2 += part[((1 * RT + rt) * W + w) * 16 + r];
      p.out[(size_t)m * N + n] = __float2bfloat16_rn(finish_output(p, m, n, total, total2));
    }
  }
}

// One warp per output row; lanes stride over the packed words.
__global__ void __launch_bounds__(256)
qgemv_generic_kernel(const GemvParams p) {
  extern __shared__ uint4 smem[];
  const int K = p.K, N = p.N, chunks = K >> 3;
  uint4* xs = smem;
  float* red = reinterpret_cast<float*>(xs + chunks);
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int W = blockDim.x >> 5;
  const int m = blockIdx.y;
  pdl_wait_for_producers();
  pdl_release_dependents();
  stage_activation<false>(p, p.x + (size_t)m * K, xs, nullptr, red);

  const int n = blockIdx.x * W + warp;
  if (n >= N) return;
  const int words = K >> 3;
  const int row_sc = K / p.group;
  const bool paired = p.epilogue == AOTO_EPILOGUE_SILU_MUL_PAIRED;
  float acc = 0.f, acc2 = 0.f;
  for (int j = lane; j < words; j += 32) {
    float xf[8];
    unpack8(xs[j], xf);
    const int gidx = (j * 8) / p.group;
    {
      const uint32_t word = __ldg(p.w0 + (size_t)n * words + j);
      const float scale = __bfloat162float(p.s0[(size_t)n * row_sc + gidx]);
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        const int code = ((int)(word << (28 - 4 * i))) >> 28;
        acc = fmaf((float)code, xf[i] * scale, acc);
      }
    }
    if (paired) {
      const uint32_t word = __ldg(p.w1 + (size_t)n * words + j);
      const float scale = __bfloat162float(p.s1[(size_t)n * row_sc + gidx]);
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        const int code = ((int)(word << (28 - 4 * i))) >> 28;
        acc2 = fmaf((float)code, xf[i] * scale, acc2);
      }
    }
  }
  acc = warp_sum(acc);
  acc2 = warp_sum(acc2);
  if (lane == 0) p.out[(size_t)m * N + n] = __float2bfloat16_rn(finish_output(p, m, n, acc, acc2));
}

// ---------------------------------------------------------------------------
// host side
// ---------------------------------------------------------------------------

struct GemvPlan {
  bool fast;
  int W, RT, UK;
  const char* name;
};

static GemvPlan plan_gemv(const aoto_qmatmul_args& a) {
  GemvPlan plan = {false, 8, 1, 1, "qgemv_generic"};
  const bool paired = a.epilogue == AOTO_EPILOGUE_SILU_MUL_PAIRED;
  if (a.group_size != 64 || (a.K % 128) != 0 || a.K > 32768) return plan;
  plan.fast = true;
  const int nblocks = a.K / 128;
  int W = 8;
  if (nblocks % 8 != 0) {
    if (nblocks % 7 == 0) W = 7;
    else if (nblocks % 6 == 0) W = 6;
    else if (nblocks % 5 == 0) W = 5;
  }
  if (nblocks < W) W = nblocks;
  plan.W = W;
  const int per_rt = (nblocks + W - 1) / W;
  const int tiles = (a.N + 15) / 16;
  const bool big = tiles >= 148 * 16;
  if (!paired) {
    if (per_rt == 1) { plan.RT = big ? 4 : 1; plan.UK = 1; }
    else if (per_rt >= 4) { plan.RT = 1; plan.UK = 4; }
    else if (big) { plan.RT = 2; plan.UK = 2; }
    else { plan.RT = 1; plan.UK = 2; }
  } else {
    if (per_rt == 1) { plan.RT = big ? 2 : 1; plan.UK = 1; }
    else { plan.RT = 1; plan.UK = 2; }
  }
  plan.name = paired ? "qgemv_mma_paired" : "qgemv_mma";
  return plan;
}

template <int RT, int UK, bool PAIRED>
static int launch_mma(const GemvParams& p, const GemvPlan& plan, int M, cudaStream_t stream, bool pdl) {
  constexpr int MATS = PAIRED ? 2 : 1;
  const size_t smem = (size_t)p.K * 2 + (size_t)(p.K / 64) * 4 + (size_t)(p.K / 8) * 4 +
                      (size_t)MATS * RT * plan.W * 16 * 4 + 32 * 4 + 16;
  auto kernel = qgemv_mma_kernel<RT, UK, PAIRED>;
  if (smem > 48 * 1024) {
    static PerDeviceOnce raised;
    if (raise_dynamic_smem(kernel, 100 * 1024, raised) != AOTO_OK) return AOTO_ERR_LAUNCH;
  }
  const int tiles = (p.N + 15) / 16;
  dim3 grid((tiles + RT - 1) / RT, M), block(plan.W * 32);
  return launch_kernel(kernel, grid, block, smem, stream, pdl, p);
}

static int check_args(const aoto_qmatmul_args& a, bool pointers) {
  const bool dense = (a.flags & AOTO_FLAG_WEIGHT_DENSE) != 0;  // bf16 weights: no scales, no groups
  if (a.M <= 0 || a.N <= 0 || a.K <= 0) return AOTO_ERR_ARGUMENT;
  if (!dense && (a.group_size <= 0 || a.group_size % 8 != 0 || a.K % a.group_size != 0)) return AOTO_ERR_ARGUMENT;
  if (dense && (a.flags & AOTO_FLAG_WEIGHT_BITS_8)) return AOTO_ERR_ARGUMENT;
  if (a.addend_kind < AOTO_ADDEND_NONE || a.addend_kind > AOTO_ADDEND_FULL) return AOTO_ERR_ARGUMENT;
  if (a.epilogue < AOTO_EPILOGUE_NONE || a.epilogue > AOTO_EPILOGUE_SILU_MUL_PAIRED) return AOTO_ERR_ARGUMENT;
  if (!pointers) return AOTO_OK;
  if (!a.x || !a.packed || (!dense && !a.scales) || !a.out) return AOTO_ERR_ARGUMENT;
  if (a.addend_kind != AOTO_ADDEND_NONE && !a.addend) return AOTO_ERR_ARGUMENT;
  if (a.epilogue == AOTO_EPILOGUE_SILU_MUL && !a.gate) return AOTO_ERR_ARGUMENT;
  if (a.epilogue == AOTO_EPILOGUE_SILU_MUL_PAIRED && (!a.packed2 || (!dense && !a.scales2))) return AOTO_ERR_ARGUMENT;
  if (!aligned_to(a.x, 16) || !aligned_to(a.packed, 16) || (!dense && !aligned_to(a.scales, 4))) return AOTO_ERR_ARGUMENT;
  if (a.norm_weight && !aligned_to(a.norm_weight, 16)) return AOTO_ERR_ARGUMENT;
  if (a.packed2 && (!aligned_to(a.packed2, 16) || (!dense && !aligned_to(a.scales2, 4)))) return AOTO_ERR_ARGUMENT;
  return AOTO_OK;
}

int qgemv_launch(const aoto_qmatmul_args& a, cudaStream_t stream) {
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
  const GemvPlan plan = plan_gemv(a);
  if (!plan.fast) {
    if (a.K > 49152) return AOTO_ERR_UNSUPPORTED;
    const size_t smem = (size_t)a.K * 2 + 32 * 4;
    if (smem > 48 * 1024) {
      static PerDeviceOnce raised;
      if (raise_dynamic_smem(qgemv_generic_kernel, 100 * 1024, raised) != AOTO_OK) return AOTO_ERR_LAUNCH;
    }
    dim3 grid((a.N + 7) / 8, a.M), block(256);
    return launch_kernel(qgemv_generic_kernel, grid, block, smem, stream, pdl, p);
  }
  const bool paired = a.epilogue == AOTO_EPILOGUE_SILU_MUL_PAIRED;
#define AOTO_CASE(rt, uk, pr) \
  if (plan.RT == rt && plan.UK == uk && paired == pr) return launch_mma<rt, uk, pr>(p, plan, a.M, stream, pdl);
  AOTO_CASE(1, 1, false)
  AOTO_CASE(1, 2, false)
  AOTO_CASE(1, 4, false)
  AOTO_CASE(2, 2, false)
  AOTO_CASE(4, 1, false)
  AOTO_CASE(1, 1, true)
  AOTO_CASE(1, 2, true)
  AOTO_CASE(2, 1, true)
#undef AOTO_CASE
  return AOTO_ERR_UNSUPPORTED;
}

int qgemv_check(const aoto_qmatmul_args& a, bool pointers) { return check_args(a, pointers); }
const char* qgemv_variant(const aoto_qmatmul_args& a) { return plan_gemv(a).name; }

}  // namespace aoto
