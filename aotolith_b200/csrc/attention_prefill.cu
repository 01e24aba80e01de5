// Prefill attention, tiled: one CTA per (64 query rows, query head), four warps of 16 rows.
//
// K and V of the head's kv head stream through shared memory in tiles of 64 keys (cp.async,
// two stages); S = Q.K^T and O += P.V run on the tensor pipe (mma.sync m16n8k16, fp32
// accumulate) with the running row maximum and sum of the online softmax in registers. The
// probabilities go back into the second product as bf16 A fragments straight from the S
// accumulators; V fragments are read with a transposing ldmatrix. Scores are scaled in fp32,
// the additive mask (0 / -inf, any pattern: causal, left padding) is applied per element, rows
// with no admitted key produce zeros.
#include "attention.cuh"

namespace aoto {

constexpr int PF_BQ = 64, PF_BK = 64, PF_THREADS = 128;

__device__ __forceinline__ void pf_cp16(void* smem_dst, const void* gmem_src) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"((uint32_t)__cvta_generic_to_shared(smem_dst)), "l"(gmem_src) : "memory");
}

__device__ __forceinline__ void pf_mma(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

// Two 8x8 b16 matrices, transposed: rows are keys in shared memory, the fragment wants
// (k = key, n = dim) pairs along k.
__device__ __forceinline__ void pf_ldmatrix_x2_trans(uint32_t& r0, uint32_t& r1, const void* smem_row) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x2.trans.shared.b16 {%0, %1}, [%2];"
               : "=r"(r0), "=r"(r1) : "r"((uint32_t)__cvta_generic_to_shared(smem_row)));
}

template <int D>
__global__ void __launch_bounds__(PF_THREADS)
attention_prefill_mma_kernel(const AttnParams p) {
  constexpr int PITCH = D * 2 + 16;      // bytes of a staged row; the pad spreads rows over the banks
  constexpr int KSTEPS = D / 16;         // k steps of Q.K^T
  constexpr int DTILES = D / 8;          // n tiles of P.V
  constexpr int CHUNKS = D / 8;          // 16-byte chunks of a row
  extern __shared__ uint4 pf_smem[];
  unsigned char* qs = reinterpret_cast<unsigned char*>(pf_smem);
  unsigned char* ks = qs + PF_BQ * PITCH;
  unsigned char* vs = ks + 2 * PF_BK * PITCH;

  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int g = lane >> 2, t = lane & 3;
  const int head = blockIdx.y, q0 = blockIdx.x * PF_BQ;
  const int kvh = head / (p.QH / p.KVH);
  const int Lq = p.Lq, Lk = p.Lk;
  const bf16* qbase = p.q + (size_t)head * Lq * D;
  const bf16* kbase = p.k + (size_t)kvh * Lk * D;
  const bf16* vbase = p.v + (size_t)kvh * Lk * D;
  const int last_key = p.causal ? min(Lk, q0 + PF_BQ) : Lk;
  const int tiles = (last_key + PF_BK - 1) / PF_BK;

  auto load_rows = [&](unsigned char* dst, const bf16* src, int first, int limit) {
    for (int c = tid; c < PF_BK * CHUNKS; c += PF_THREADS) {
      const int r = c / CHUNKS, j = c - r * CHUNKS;
      unsigned char* to = dst + (size_t)r * PITCH + j * 16;
      if (first + r < limit) pf_cp16(to, src + (size_t)(first + r) * D + j * 8);
      else *reinterpret_cast<uint4*>(to) = make_uint4(0u, 0u, 0u, 0u);
    }
  };
  load_rows(qs, qbase, q0, Lq);
  load_rows(ks, kbase, 0, Lk);
  load_rows(vs, vbase, 0, Lk);
  asm volatile("cp.async.commit_group;" ::: "memory");

  float o[DTILES][4];
#pragma unroll
  for (int i = 0; i < DTILES; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f;
  float row_max[2] = {-INFINITY, -INFINITY}, row_sum[2] = {0.f, 0.f};
  uint32_t qa[KSTEPS][4];
  const int row_lo = q0 + warp * 16 + g, row_hi = row_lo + 8;

  for (int j = 0; j < tiles; ++j) {
    const int stage = j & 1;
    if (j + 1 < tiles) {
      load_rows(ks + (size_t)(stage ^ 1) * PF_BK * PITCH, kbase, (j + 1) * PF_BK, Lk);
      load_rows(vs + (size_t)(stage ^ 1) * PF_BK * PITCH, vbase, (j + 1) * PF_BK, Lk);
      asm volatile("cp.async.commit_group;" ::: "memory");
      asm volatile("cp.async.wait_group 1;" ::: "memory");
    } else {
      asm volatile("cp.async.wait_group 0;" ::: "memory");
    }
    __syncthreads();
    if (j == 0) {
      const unsigned char* qlo = qs + (size_t)(warp * 16 + g) * PITCH;
      const unsigned char* qhi = qlo + 8 * PITCH;
#pragma unroll
      for (int kk = 0; kk < KSTEPS; ++kk) {
        qa[kk][0] = *reinterpret_cast<const uint32_t*>(qlo + (kk * 16 + 2 * t) * 2);
        qa[kk][1] = *reinterpret_cast<const uint32_t*>(qhi + (kk * 16 + 2 * t) * 2);
        qa[kk][2] = *reinterpret_cast<const uint32_t*>(qlo + (kk * 16 + 8 + 2 * t) * 2);
        qa[kk][3] = *reinterpret_cast<const uint32_t*>(qhi + (kk * 16 + 8 + 2 * t) * 2);
      }
    }
    const unsigned char* kt = ks + (size_t)stage * PF_BK * PITCH;
    const unsigned char* vt = vs + (size_t)stage * PF_BK * PITCH;

    // S = Q.K^T for 16 rows x 64 keys
    float s[8][4];
#pragma unroll
    for (int n = 0; n < 8; ++n) s[n][0] = s[n][1] = s[n][2] = s[n][3] = 0.f;
#pragma unroll
    for (int kk = 0; kk < KSTEPS; ++kk) {
#pragma unroll
      for (int n = 0; n < 8; ++n) {
        const unsigned char* krow = kt + (size_t)(n * 8 + g) * PITCH + (kk * 16 + 2 * t) * 2;
        pf_mma(s[n], qa[kk], *reinterpret_cast<const uint32_t*>(krow), *reinterpret_cast<const uint32_t*>(krow + 16));
      }
    }

    // scale, mask, running maximum
    float tile_max[2] = {-INFINITY, -INFINITY};
#pragma unroll
    for (int n = 0; n < 8; ++n) {
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const int row = (e & 2) ? row_hi : row_lo;
        const int key = j * PF_BK + n * 8 + 2 * t + (e & 1);
        float value = -INFINITY;
        if (row < Lq && key < Lk && !(p.causal && key > row)) {
          const float add = p.mask ? __bfloat162float(p.mask[(size_t)row * Lk + key]) : 0.f;
          value = s[n][e] * p.scale + add;
        }
        s[n][e] = value;
        tile_max[e >> 1] = fmaxf(tile_max[e >> 1], value);
      }
    }
    float correction[2];
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      float m = tile_max[h];
      m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, 1));
      m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, 2));
      const float m_new = fmaxf(row_max[h], m);
      correction[h] = (row_max[h] == -INFINITY) ? 0.f : expf(row_max[h] - m_new);
      row_max[h] = m_new;
      row_sum[h] *= correction[h];
    }
    // probabilities (bf16 A fragments of the second product) and the row sums of this tile
    uint32_t pa[4][4];
#pragma unroll
    for (int n = 0; n < 8; ++n) {
      float e4[4];
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const float m = row_max[e >> 1];
        e4[e] = (s[n][e] == -INFINITY) ? 0.f : expf(s[n][e] - m);
        row_sum[e >> 1] += e4[e];
      }
      pa[n >> 1][(n & 1) * 2 + 0] = pack_bf16x2(e4[0], e4[1]);  // row g, keys 2t, 2t+1 of this n tile
      pa[n >> 1][(n & 1) * 2 + 1] = pack_bf16x2(e4[2], e4[3]);  // row g + 8
    }
#pragma unroll
    for (int i = 0; i < DTILES; ++i) {
      o[i][0] *= correction[0]; o[i][1] *= correction[0];
      o[i][2] *= correction[1]; o[i][3] *= correction[1];
    }
    // O += P.V
#pragma unroll
    for (int kk = 0; kk < 4; ++kk) {
      const unsigned char* vrow = vt + (size_t)(kk * 16 + (lane & 15)) * PITCH;
#pragma unroll
      for (int i = 0; i < DTILES; ++i) {
        uint32_t b0, b1;
        pf_ldmatrix_x2_trans(b0, b1, vrow + i * 16);
        pf_mma(o[i], pa[kk], b0, b1);
      }
    }
    __syncthreads();  // the other stage is refilled at the top of the next iteration
  }

#pragma unroll
  for (int h = 0; h < 2; ++h) {
    row_sum[h] += __shfl_xor_sync(0xffffffffu, row_sum[h], 1);
    row_sum[h] += __shfl_xor_sync(0xffffffffu, row_sum[h], 2);
  }
  const float inv_lo = row_sum[0] > 0.f ? 1.f / row_sum[0] : 0.f;
  const float inv_hi = row_sum[1] > 0.f ? 1.f / row_sum[1] : 0.f;
  bf16* out = p.out + (size_t)head * Lq * D;
#pragma unroll
  for (int i = 0; i < DTILES; ++i) {
    if (row_lo < Lq)
      *reinterpret_cast<uint32_t*>(out + (size_t)row_lo * D + i * 8 + 2 * t) = pack_bf16x2(o[i][0] * inv_lo, o[i][1] * inv_lo);
    if (row_hi < Lq)
      *reinterpret_cast<uint32_t*>(out + (size_t)row_hi * D + i * 8 + 2 * t) = pack_bf16x2(o[i][2] * inv_hi, o[i][3] * inv_hi);
  }
}

bool attention_prefill_mma_applies(const AttnParams& p) {
  const uintptr_t bits = reinterpret_cast<uintptr_t>(p.q) | reinterpret_cast<uintptr_t>(p.k) |
                         reinterpret_cast<uintptr_t>(p.v) | reinterpret_cast<uintptr_t>(p.out);
  return (p.D == 64 || p.D == 128) && p.Lq >= 16 && (bits & 15) == 0;
}

template <int D>
static int launch_prefill(const AttnParams& p, cudaStream_t stream) {
  constexpr size_t smem = (size_t)(PF_BQ + 4 * PF_BK) * (D * 2 + 16);
  static bool raised = false;
  if (!raised) {
    if (cudaFuncSetAttribute(attention_prefill_mma_kernel<D>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess) {
      (void)cudaGetLastError();
      return AOTO_ERR_LAUNCH;
    }
    raised = true;
  }
  dim3 grid((p.Lq + PF_BQ - 1) / PF_BQ, p.QH);
  return launch_kernel(attention_prefill_mma_kernel<D>, grid, dim3(PF_THREADS), smem, stream, false, p);
}

int attention_prefill_mma_launch(const AttnParams& p, cudaStream_t stream) {
  return p.D == 64 ? launch_prefill<64>(p, stream) : launch_prefill<128>(p, stream);
}

}  // namespace aoto
