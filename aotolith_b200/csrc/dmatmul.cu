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

// ---------------------------------------------------------------------------
// One activation row on the tensor pipe
// ---------------------------------------------------------------------------
//
// The warp-per-row kernel above spends a lane sixteen conversions and eight multiply-adds on every
// 16-byte unit and issues in 61 % of all cycles at half the DRAM rate. Here the multiply-add goes
// to `mma.sync m16n8k16`: a warp owns a tile of sixteen weight rows; lane (g, t) loads 16 bytes of
// row g and of row g+8 - eight consecutive weights, four lanes cover 32 - and uses them as they
// come as the A fragments of two instructions. The fragment slots of a lane then hold weights
// 8t..8t+3 (first instruction) and 8t+4..8t+7 (second) of the 32-weight step instead of the
// architectural 2t, 2t+1, 2t+8, 2t+9; a dot product does not care, as long as column 0 of B holds
// the activations in the same order, which is the lane's own 16-byte unit of x. The other seven
// columns of B are zero. Per step and lane: two 16-byte loads, one shared-memory load, two mma.
// SPLIT = false: a warp walks whole rows (vocabulary-sized N). SPLIT = true: a CTA owns one tile
// and its warps share the steps of K (layer-sized N, where tiles are fewer than warps).
constexpr int DV_WARPS = 8;
constexpr int DV_AHEAD = 4;  // 32-weight steps of a lane in flight

template <bool PAIRED, bool SPLIT>
__global__ void __launch_bounds__(DV_WARPS * 32)
dgemv_mma_kernel(const GemvParams p) {
  extern __shared__ uint4 smem[];
  const int K = p.K, N = p.N, steps = K >> 5, units = K >> 3;
  uint4* xs = smem;            // the activation row; one zero unit behind it
  uint4* zero = xs + units;
  float* part = reinterpret_cast<float*>(zero + 1);  // SPLIT: [matrix][warp][16] partial sums
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int g = lane >> 2, t = lane & 3;
  const int tiles = (N + 15) >> 4;
  pdl_wait_for_producers();
  pdl_release_dependents();
  {
    const uint4* xv = reinterpret_cast<const uint4*>(p.x);
    for (int c = tid; c < units; c += blockDim.x) xs[c] = xv[c];
    if (tid == 0) *zero = make_uint4(0u, 0u, 0u, 0u);
    __syncthreads();
  }
  // column 0 of B belongs to the lanes with g == 0; the others multiply by zero
  const uint4* bsrc = g == 0 ? xs + t : zero;
  const int bstride = g == 0 ? 4 : 0;
  const int first_tile = SPLIT ? blockIdx.x : blockIdx.x * DV_WARPS + warp;
  const int tile_stride = SPLIT ? gridDim.x : gridDim.x * DV_WARPS;
  const int first_step = SPLIT ? warp : 0;
  const int step_stride = SPLIT ? DV_WARPS : 1;
  for (int tile = first_tile; tile < tiles; tile += tile_stride) {
    const int row_lo = min(tile * 16 + g, N - 1), row_hi = min(tile * 16 + g + 8, N - 1);
    const uint4* a_lo = reinterpret_cast<const uint4*>(p.w0) + (size_t)row_lo * units + t;
    const uint4* a_hi = reinterpret_cast<const uint4*>(p.w0) + (size_t)row_hi * units + t;
    const uint4* b_lo = reinterpret_cast<const uint4*>(p.w1) + (size_t)row_lo * units + t;
    const uint4* b_hi = reinterpret_cast<const uint4*>(p.w1) + (size_t)row_hi * units + t;
    float c0[4] = {0.f, 0.f, 0.f, 0.f}, c1[4] = {0.f, 0.f, 0.f, 0.f};
    for (int s0 = first_step; s0 < steps; s0 += step_stride * DV_AHEAD) {
      uint4 lo[DV_AHEAD], hi[DV_AHEAD], lo2[DV_AHEAD], hi2[DV_AHEAD];
#pragma unroll
      for (int a = 0; a < DV_AHEAD; ++a) {
        const int s = s0 + a * step_stride;
        if (s < steps) {
          lo[a] = ldg_nc_u4(a_lo + s * 4);
          hi[a] = ldg_nc_u4(a_hi + s * 4);
          if (PAIRED) {
            lo2[a] = ldg_nc_u4(b_lo + s * 4);
            hi2[a] = ldg_nc_u4(b_hi + s * 4);
          }
        }
      }
#pragma unroll
      for (int a = 0; a < DV_AHEAD; ++a) {
        const int s = s0 + a * step_stride;
        if (s >= steps) break;
        const uint4 xq = bsrc[s * bstride];
        mma_16816(c0, lo[a].x, hi[a].x, lo[a].y, hi[a].y, xq.x, xq.y);
        mma_16816(c0, lo[a].z, hi[a].z, lo[a].w, hi[a].w, xq.z, xq.w);
        if (PAIRED) {
          mma_16816(c1, lo2[a].x, hi2[a].x, lo2[a].y, hi2[a].y, xq.x, xq.y);
          mma_16816(c1, lo2[a].z, hi2[a].z, lo2[a].w, hi2[a].w, xq.z, xq.w);
        }
      }
    }
    // column 0 of the C tile: lanes with t == 0 hold row g in c[0] and row g+8 in c[2]
    if (!SPLIT) {
      if (t == 0) {
        const int n_lo = tile * 16 + g, n_hi = n_lo + 8;
        if (n_lo < N) p.out[n_lo] = __float2bfloat16_rn(finish_output(p, 0, n_lo, c0[0], c1[0]));
        if (n_hi < N) p.out[n_hi] = __float2bfloat16_rn(finish_output(p, 0, n_hi, c0[2], c1[2]));
      }
    } else {
      if (t == 0) {
        part[warp * 16 + g] = c0[0];
        part[warp * 16 + g + 8] = c0[2];
        if (PAIRED) {
          part[(DV_WARPS + warp) * 16 + g] = c1[0];
          part[(DV_WARPS + warp) * 16 + g + 8] = c1[2];
        }
      }
      __syncthreads();
      if (tid < 16) {
        const int n = tile * 16 + tid;
        if (n < N) {
          float total = 0.f, total2 = 0.f;
#pragma unroll
          for (int w = 0; w < DV_WARPS; ++w) total += part[w * 16 + tid];
          if (PAIRED) {
#pragma unroll
            for (int w = 0; w < DV_WARPS; ++w) total2 += part[(DV_WARPS + w) * 16 + tid];
          }
          p.out[n] = __float2bfloat16_rn(finish_output(p, 0, n, total, total2));
        }
      }
      __syncthreads();  // the next tile overwrites the partial sums
    }
  }
}

static bool dgemv_mma_applies(const aoto_qmatmul_args& a) {
  if (a.M != 1 || (a.K % 32) != 0 || a.N < 16) return false;
  // the gate/up pair over long rows measured faster a warp per row (4096 x 14336 twice: 41.1 us
  // against 43.9 us here, where two matrices' fragments leave two CTAs per SM)
  if (a.epilogue == AOTO_EPILOGUE_SILU_MUL_PAIRED && a.K >= 2048) return false;
  return true;
}

template <bool PAIRED, bool SPLIT>
static int launch_dgemv_mma(const GemvParams& p, cudaStream_t stream, bool pdl) {
  auto kernel = dgemv_mma_kernel<PAIRED, SPLIT>;
  const size_t smem = (size_t)p.K * 2 + 16 + (SPLIT ? (size_t)2 * DV_WARPS * 16 * 4 : 0);
  if (smem > 48 * 1024) {
    static PerDeviceOnce raised;
    if (raise_dynamic_smem(kernel, 96 * 1024, raised) != AOTO_OK) return AOTO_ERR_LAUNCH;
  }
  const int tiles = (p.N + 15) / 16;
  // a persistent grid of the CTAs that are resident together (no second, partial wave)
  int resident = 0;
  if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&resident, kernel, DV_WARPS * 32, smem) != cudaSuccess || resident < 1) {
    (void)cudaGetLastError();
    resident = 1;
  }
  const int wanted = SPLIT ? tiles : (tiles + DV_WARPS - 1) / DV_WARPS;
  const int most = 148 * resident;
  return launch_kernel(kernel, dim3(wanted < most ? wanted : most), dim3(DV_WARPS * 32), smem, stream, pdl, p);
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
  if (dgemv_mma_applies(a)) {
    const bool paired = a.epilogue == AOTO_EPILOGUE_SILU_MUL_PAIRED;
    const bool split = (a.N + 15) / 16 < 148 * DV_WARPS;  // fewer tiles than warps: share K inside a CTA
    if (paired) return split ? launch_dgemv_mma<true, true>(p, stream, pdl) : launch_dgemv_mma<true, false>(p, stream, pdl);
    return split ? launch_dgemv_mma<false, true>(p, stream, pdl) : launch_dgemv_mma<false, false>(p, stream, pdl);
  }
  if (a.M == 1) return launch_dense<1>(p, a.M, stream, pdl);
  if (a.M >= 8 && a.K <= 8192) return launch_dense<8>(p, a.M, stream, pdl);
  if (a.M >= 4 && a.K <= 16384) return launch_dense<4>(p, a.M, stream, pdl);
  return launch_dense<2>(p, a.M, stream, pdl);
}

const char* dmatmul_variant(const aoto_qmatmul_args& a) {
  if (dgemv_mma_applies(a)) return "dgemv_mma";
  return a.M == 1 ? "dgemv" : "dgemm_rows";
}

}  // namespace aoto
