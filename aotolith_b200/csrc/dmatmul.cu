// Dense bf16 projections: y[M,N] = x[M,K] . W[N,K]^T with W as it is stored by the model.
//
// First kernel of the dense (unquantised) decoders: a warp per weight row (a few CTAs per SM, each
// warp walking rows a grid stride apart), lanes stride over 16-byte units of eight weights, MR
// activation rows of the CTA staged in shared memory so that a loaded weight is used MR times;
// products accumulate in fp32 and are rounded once. The single-row form takes the paired gate/up
// epilogue; bias, residual and the y * silu(gate) epilogue work with any number of rows. A decode
// step streams 2 bytes per weight, four times the packed form: the kernel is bound by HBM for one
// row and by its re-reads of the weight (M / MR passes) for a prompt.
#include "qgemv_core.cuh"

namespace aoto {

constexpr int DM_WARPS = 8;

template <int MR>
__global__ void __launch_bounds__(DM_WARPS * 32)
dmatmul_kernel(const GemvParams p, const int M) {
  extern __shared__ uint4 smem[];
  const int K = p.K, N = p.N, chunks = K >> 3;
  uint4* xs = smem;  // MR rows of K bf16
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int m0 = blockIdx.y * MR;
  pdl_wait_for_producers();
  pdl_release_dependents();
  {
    const uint4* xv = reinterpret_cast<const uint4*>(p.x);
    for (int c = tid; c < MR * chunks; c += blockDim.x) {
      const int r = c / chunks, j = c - r * chunks;
      xs[c] = (m0 + r < M) ? xv[(size_t)(m0 + r) * chunks + j] : make_uint4(0u, 0u, 0u, 0u);
    }
    __syncthreads();
  }
  const bool paired = p.epilogue == AOTO_EPILOGUE_SILU_MUL_PAIRED;
  for (int n = blockIdx.x * DM_WARPS + warp; n < N; n += gridDim.x * DM_WARPS) {
    const uint4* w0 = reinterpret_cast<const uint4*>(p.w0) + (size_t)n * chunks;
    const uint4* w1 = reinterpret_cast<const uint4*>(p.w1) + (size_t)n * chunks;
    float acc[MR], acc2[MR];
#pragma unroll
    for (int r = 0; r < MR; ++r) acc[r] = acc2[r] = 0.f;
    // with a single activation row several units of a lane are requested before the first is used
    constexpr int AHEAD = MR == 1 ? 4 : 2;
    for (int j0 = lane; j0 < chunks; j0 += 32 * AHEAD) {
      uint4 q0[AHEAD], q1[AHEAD];
#pragma unroll
      for (int a = 0; a < AHEAD; ++a) {
        const int j = j0 + 32 * a;
        q0[a] = q1[a] = make_uint4(0u, 0u, 0u, 0u);
        if (j < chunks) {
          q0[a] = ldg_nc_u4(w0 + j);
          if (paired) q1[a] = ldg_nc_u4(w1 + j);
        }
      }
#pragma unroll
      for (int a = 0; a < AHEAD; ++a) {
        const int j = j0 + 32 * a;
        if (j >= chunks) break;
        float w[8], v[8];
        unpack8(q0[a], w);
        if (paired) unpack8(q1[a], v);
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
  }
}

// Shapes the dense kernel takes: rows of whole 16-byte units, short enough for MR staged rows;
// no norm prologue (dense graphs keep the norm as an operation of its own), the paired form
// only with a single activation row, operands on 16-byte boundaries.
bool dmatmul_supported(const aoto_qmatmul_args& a) {
  if (a.M <= 0 || a.N <= 0 || a.K <= 0) return false;
  if ((a.K % 8) != 0 || a.K > 32768) return false;
  if (a.norm_weight != nullptr) return false;
  if (a.M > 1 && a.epilogue == AOTO_EPILOGUE_SILU_MUL_PAIRED) return false;
  // activation and weight rows are read as 16-byte units
  if (((uintptr_t)a.x | (uintptr_t)a.packed | (uintptr_t)a.packed2) & 15) return false;
  return true;
}

template <int MR>
static int launch_dense(const GemvParams& p, int M, cudaStream_t stream, bool pdl) {
  const size_t smem = (size_t)MR * p.K * 2;
  auto kernel = dmatmul_kernel<MR>;
  if (smem > 48 * 1024) {
    static PerDeviceOnce raised;
    if (raise_dynamic_smem(kernel, 160 * 1024, raised) != AOTO_OK) return AOTO_ERR_LAUNCH;
    if (smem > 160 * 1024) return AOTO_ERR_UNSUPPORTED;
  }
  const int row_groups = (M + MR - 1) / MR;
  const int wanted = (p.N + DM_WARPS - 1) / DM_WARPS;
  const int per_group = 148 * 6 / (row_groups < 6 ? row_groups : 6);  // about six CTAs per SM in all
  dim3 grid(wanted < per_group ? wanted : per_group, row_groups), block(DM_WARPS * 32);
  return launch_kernel(kernel, grid, block, smem, stream, pdl, p, M);
}

int dmatmul_launch(const aoto_qmatmul_args& a, cudaStream_t stream) {
  if (!dmatmul_supported(a)) return AOTO_ERR_UNSUPPORTED;
  GemvParams p;
  p.x = (const bf16*)a.x;
  p.w0 = (const uint32_t*)a.packed;
  p.s0 = nullptr;
  p.w1 = (const uint32_t*)a.packed2;
  p.s1 = nullptr;
  p.addend = (const bf16*)a.addend;
  p.gate = (const bf16*)a.gate;
  p.norm_w = nullptr;
  p.out = (bf16*)a.out;
  p.N = a.N; p.K = a.K; p.group = a.K;
  p.addend_kind = a.addend_kind; p.epilogue = a.epilogue;
  p.alpha = a.alpha; p.beta = a.beta; p.eps = 0.f;
  const bool pdl = (a.flags & AOTO_FLAG_PDL) != 0;
  if (a.M == 1) return launch_dense<1>(p, a.M, stream, pdl);
  if (a.M >= 8 && a.K <= 8192) return launch_dense<8>(p, a.M, stream, pdl);
  if (a.M >= 4 && a.K <= 16384) return launch_dense<4>(p, a.M, stream, pdl);
  return launch_dense<2>(p, a.M, stream, pdl);
}

const char* dmatmul_variant(const aoto_qmatmul_args& a) { return a.M == 1 ? "dgemv" : "dgemm_rows"; }

}  // namespace aoto
