// Prefill attention, tiled: one CTA per (64 query rows, query head), four warps of 16 rows.
//
// K and V of the head's kv head stream through shared memory in tiles of 64 keys (cp.async,
// two stages, one barrier per tile); S = Q.K^T and O += P.V run on the tensor pipe (mma.sync
// m16n8k16, fp32 accumulate, B fragments by ldmatrix.x4) with the running row maximum and sum of
// the online softmax in registers. Scores are kept in the base-2 domain (the scale carries
// log2 e, exponentials are ex2.approx). The probabilities go back into the second product as bf16
// A fragments straight from the S accumulators; V fragments are read with a transposing ldmatrix.
// The additive mask (0 / -inf, any pattern: causal, left padding, banded) is applied per element;
// rows with no admitted key produce zeros.
//
// With a workspace, attention_mask_classes_kernel first sorts the 64 x 64 tiles of the mask into
// "no key admitted", "adds zero everywhere" and "mixed": the first kind is neither loaded nor
// multiplied, the second reads no mask. Without one every tile is visited, same result. The query
// tiles of a head are launched last-first, because under a causal mask the late ones are the long ones.
#include <type_traits>

#include "attention.cuh"

namespace aoto {

constexpr int PF_BQ = 64, PF_BK = 64, PF_THREADS = 128;
constexpr int PF_MAX_KEY_TILES = 1024;  // key tiles a CTA keeps classes for (65 536 keys)
constexpr unsigned char PF_TILE_NONE = 0, PF_TILE_MIXED = 1, PF_TILE_ZERO = 2;
constexpr int PF_CLASS_WARPS = 8;
constexpr int PF_MASK_NONE = 0, PF_MASK_PAIRS = 1, PF_MASK_SINGLE = 2;
constexpr int PF_CLASS_MIN_KEYS = 256;  // shorter windows have too few tiles to pay for the extra launch

__device__ __forceinline__ void pf_cp16(void* smem_dst, const void* gmem_src) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"((uint32_t)__cvta_generic_to_shared(smem_dst)), "l"(gmem_src) : "memory");
}

__device__ __forceinline__ void pf_mma(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

// Four 8x8 b16 matrices, transposed: rows are keys in shared memory, the fragment wants
// (k = key, n = dim) pairs along k.
__device__ __forceinline__ void pf_ldmatrix_x4_trans(uint32_t (&r)[4], const void* smem_row) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0, %1, %2, %3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"((uint32_t)__cvta_generic_to_shared(smem_row)));
}

// One warp per (64 query rows, 64 keys) tile of the additive mask: 512 16-byte chunks, sixteen per
// lane and all in flight at once. The class goes to classes[q_tile * key_tiles + key_tile].
__global__ void __launch_bounds__(PF_CLASS_WARPS * 32)
attention_mask_classes_kernel(const bf16* __restrict__ mask, unsigned char* __restrict__ classes,
                              int Lq, int Lk, int q_tiles, int key_tiles) {
  const int lane = threadIdx.x & 31;
  const int tile = blockIdx.x * PF_CLASS_WARPS + (threadIdx.x >> 5);
  if (tile >= q_tiles * key_tiles) return;
  const int qt = tile / key_tiles, kt = tile - qt * key_tiles;
  const int q0 = qt * PF_BQ, k0 = kt * PF_BK;
  uint4 m[16];
  bool inside[16];
#pragma unroll
  for (int u = 0; u < 16; ++u) {
    const int c = lane + 32 * u;
    const int row = q0 + (c >> 3), key = k0 + (c & 7) * 8;   // Lk is a multiple of 8: a chunk is inside or outside
    inside[u] = row < Lq && key < Lk;
    m[u] = make_uint4(0u, 0u, 0u, 0u);
    if (inside[u]) m[u] = *reinterpret_cast<const uint4*>(mask + (size_t)row * Lk + key);
  }
  bool any_admitted = false, all_zero = true;
#pragma unroll
  for (int u = 0; u < 16; ++u) {
    if (inside[u]) {
      // -inf in bf16 is 0xFF80: a word of two excluded keys is 0xFF80FF80; two zeros are 0
      any_admitted |= m[u].x != 0xFF80FF80u || m[u].y != 0xFF80FF80u || m[u].z != 0xFF80FF80u || m[u].w != 0xFF80FF80u;
      all_zero &= (m[u].x | m[u].y | m[u].z | m[u].w) == 0u;
    }
  }
  any_admitted = __any_sync(0xffffffffu, any_admitted);
  all_zero = __all_sync(0xffffffffu, all_zero);
  if (lane == 0) classes[tile] = !any_admitted ? PF_TILE_NONE : (all_zero ? PF_TILE_ZERO : PF_TILE_MIXED);
}

// Four 8x8 b16 matrices as they lie in shared memory (rows are keys, the fragment wants the pair
// of dims 2t, 2t+1 of key g).
__device__ __forceinline__ void pf_ldmatrix_x4(uint32_t (&r)[4], const void* smem_row) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0, %1, %2, %3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"((uint32_t)__cvta_generic_to_shared(smem_row)));
}

// 2^x on the special-function unit; -inf gives 0.
__device__ __forceinline__ float pf_exp2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
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
  // The late query tiles of a causal prompt visit the most key tiles: they are launched first, so
  // that the short ones fill in behind them.
  const int q_tile = gridDim.x - 1 - blockIdx.x;
  const int head = blockIdx.y, q0 = q_tile * PF_BQ;
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
  // Classes of the key tiles for this tile of query rows, written by attention_mask_classes_kernel
  // when the caller gave a workspace: 0 = no key admitted (the tile is neither loaded nor
  // multiplied), 2 = the mask adds zero everywhere (no mask loads), 1 = mixed. With a causal
  // prompt mask that halves the work and confines the mask loads to the diagonal tiles; with left
  // padding it drops the padded keys.
  __shared__ unsigned char tile_class[PF_MAX_KEY_TILES];
  const bool classed = p.tile_classes != nullptr;
  const bool mask_pairs = (Lk & 1) == 0 && (reinterpret_cast<uintptr_t>(p.mask) & 3) == 0;
  if (classed) {
    const unsigned char* mine = p.tile_classes + (size_t)q_tile * p.key_tiles;
    for (int i = tid; i < tiles; i += PF_THREADS) tile_class[i] = mine[i];
    __syncthreads();
  }
  auto tile_admitted = [&](int j) { return !classed || tile_class[j] != PF_TILE_NONE; };
  // the admitted tiles in order: `next_tile(j)` is the first admitted tile at or after j
  auto next_tile = [&](int j) {
    while (j < tiles && !tile_admitted(j)) ++j;
    return j;
  };
  const int first = next_tile(0);

  load_rows(qs, qbase, q0, Lq);
  if (first < tiles) {
    load_rows(ks, kbase, first * PF_BK, Lk);
    load_rows(vs, vbase, first * PF_BK, Lk);
  }
  asm volatile("cp.async.commit_group;" ::: "memory");

  float o[DTILES][4];
#pragma unroll
  for (int i = 0; i < DTILES; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f;
  // scores are kept in the base-2 domain: exp(x) = 2^(x * log2 e), one multiply folded into the scale
  constexpr float LOG2E = 1.4426950408889634f;
  const float scale_log2 = p.scale * LOG2E;
  float row_max[2] = {-INFINITY, -INFINITY}, row_sum[2] = {0.f, 0.f};
  uint32_t qa[KSTEPS][4];
  const int row_lo = q0 + warp * 16 + g, row_hi = row_lo + 8;

  int stage = 0;
  bool have_q = false;
  for (int j = first; j < tiles; stage ^= 1) {
    const int following = next_tile(j + 1);
    asm volatile("cp.async.wait_group 0;" ::: "memory");  // tile j (and, the first time, Q)
    __syncthreads();
    // Every warp is past the products of the previous tile, so its stage is free: the next tile is
    // requested now and lands while this one is multiplied. One barrier per tile.
    if (following < tiles) {
      load_rows(ks + (size_t)(stage ^ 1) * PF_BK * PITCH, kbase, following * PF_BK, Lk);
      load_rows(vs + (size_t)(stage ^ 1) * PF_BK * PITCH, vbase, following * PF_BK, Lk);
      asm volatile("cp.async.commit_group;" ::: "memory");
    }
    if (!have_q) {
      have_q = true;
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
    for (int kk = 0; kk < KSTEPS; kk += 2) {
      // one ldmatrix.x4 per 8 keys fetches the B fragments of two k steps: lanes 8m..8m+7 address
      // the rows of matrix m = (k step, low or high eight dims)
      uint32_t b[8][4];
#pragma unroll
      for (int n = 0; n < 8; ++n)
        pf_ldmatrix_x4(b[n], kt + (size_t)(n * 8 + (lane & 7)) * PITCH + (kk * 16 + (lane >> 3) * 8) * 2);
#pragma unroll
      for (int n = 0; n < 8; ++n) pf_mma(s[n], qa[kk], b[n][0], b[n][1]);
#pragma unroll
      for (int n = 0; n < 8; ++n) pf_mma(s[n], qa[kk + 1], b[n][2], b[n][3]);
    }

    // Scale, mask, running maximum. Three forms of the mask term, chosen per tile and the same for
    // the whole warp: none (no mask, or a tile where it adds zero everywhere), pairs of neighbouring
    // keys in one 32-bit load (even window, 4-byte aligned mask), single elements.
    float tile_max[2] = {-INFINITY, -INFINITY};
    auto scores = [&](auto mode_tag, auto edge_tag) {
      constexpr int MODE = decltype(mode_tag)::value;
      constexpr bool EDGE = decltype(edge_tag)::value;  // false: every (row, key) of the warp's tile is in range and admitted by the causal rule
      const int key_base = j * PF_BK + 2 * t;
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        const int row = h ? row_hi : row_lo;
        const bf16* mask_row = MODE != PF_MASK_NONE ? p.mask + (size_t)row * Lk + key_base : nullptr;
#pragma unroll
        for (int n = 0; n < 8; ++n) {
          const int key = key_base + n * 8;
          float add0 = 0.f, add1 = 0.f;
          if (MODE == PF_MASK_PAIRS) {
            if (!EDGE || (row < Lq && key < Lk)) {  // the window is even: key + 1 is inside as well
              const uint32_t pair = *reinterpret_cast<const uint32_t*>(mask_row + n * 8);
              add0 = __uint_as_float(pair << 16);
              add1 = __uint_as_float(pair & 0xFFFF0000u);
            }
          } else if (MODE == PF_MASK_SINGLE) {
            if (!EDGE || (row < Lq && key < Lk)) add0 = __bfloat162float(mask_row[n * 8]);
            if (!EDGE || (row < Lq && key + 1 < Lk)) add1 = __bfloat162float(mask_row[n * 8 + 1]);
          }
          const bool in0 = !EDGE || (row < Lq && key < Lk && !(p.causal && key > row));
          const bool in1 = !EDGE || (row < Lq && key + 1 < Lk && !(p.causal && key + 1 > row));
          const float v0 = in0 ? s[n][2 * h] * scale_log2 + add0 * LOG2E : -INFINITY;
          const float v1 = in1 ? s[n][2 * h + 1] * scale_log2 + add1 * LOG2E : -INFINITY;
          s[n][2 * h] = v0;
          s[n][2 * h + 1] = v1;
          tile_max[h] = fmaxf(tile_max[h], fmaxf(v0, v1));
        }
      }
    };
    const bool edge = q0 + PF_BQ > Lq || (j + 1) * PF_BK > Lk || (p.causal && (j + 1) * PF_BK - 1 > q0 + warp * 16);
    const int mode = (p.mask == nullptr || (classed && tile_class[j] == PF_TILE_ZERO)) ? PF_MASK_NONE
                     : (mask_pairs ? PF_MASK_PAIRS : PF_MASK_SINGLE);
    using Edge = std::true_type;
    using Inner = std::false_type;
    if (mode == PF_MASK_NONE) {
      if (edge) scores(std::integral_constant<int, PF_MASK_NONE>(), Edge()); else scores(std::integral_constant<int, PF_MASK_NONE>(), Inner());
    } else if (mode == PF_MASK_PAIRS) {
      if (edge) scores(std::integral_constant<int, PF_MASK_PAIRS>(), Edge()); else scores(std::integral_constant<int, PF_MASK_PAIRS>(), Inner());
    } else {
      if (edge) scores(std::integral_constant<int, PF_MASK_SINGLE>(), Edge()); else scores(std::integral_constant<int, PF_MASK_SINGLE>(), Inner());
    }
    float correction[2];
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      float m = tile_max[h];
      m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, 1));
      m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, 2));
      const float m_new = fmaxf(row_max[h], m);
      correction[h] = (row_max[h] == -INFINITY) ? 0.f : pf_exp2(row_max[h] - m_new);
      row_max[h] = m_new;
      row_sum[h] *= correction[h];
    }
    // probabilities (bf16 A fragments of the second product) and the row sums of this tile
    // a row with no admitted key so far has maximum -inf: subtract 0 instead, every term is 2^(-inf)
    const float max_or_zero[2] = {row_max[0] == -INFINITY ? 0.f : row_max[0], row_max[1] == -INFINITY ? 0.f : row_max[1]};
    uint32_t pa[4][4];
#pragma unroll
    for (int n = 0; n < 8; ++n) {
      float e4[4];
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        e4[e] = pf_exp2(s[n][e] - max_or_zero[e >> 1]);  // 2^(-inf) = 0 for an excluded key
        row_sum[e >> 1] += e4[e];
      }
      pa[n >> 1][(n & 1) * 2 + 0] = pack_bf16x2(e4[0], e4[1]);  // row g, keys 2t, 2t+1 of this n tile
      pa[n >> 1][(n & 1) * 2 + 1] = pack_bf16x2(e4[2], e4[3]);  // row g + 8
    }
    // after the first tiles the running maximum seldom moves: the accumulator is rescaled only
    // when some row of the warp needs it
    if (__any_sync(0xffffffffu, correction[0] != 1.f || correction[1] != 1.f)) {
#pragma unroll
      for (int i = 0; i < DTILES; ++i) {
        o[i][0] *= correction[0]; o[i][1] *= correction[0];
        o[i][2] *= correction[1]; o[i][3] *= correction[1];
      }
    }
    // O += P.V
#pragma unroll
    for (int kk = 0; kk < 4; ++kk) {
      const unsigned char* vrow = vt + (size_t)(kk * 16 + (lane & 15)) * PITCH;
#pragma unroll
      for (int i = 0; i < DTILES; i += 2) {
        // lanes 0-15 address the 16 keys at dims 8i.., lanes 16-31 the same keys at dims 8(i+1)..
        uint32_t b[4];
        pf_ldmatrix_x4_trans(b, vrow + (i + (lane >> 4)) * 16);
        pf_mma(o[i], pa[kk], b[0], b[1]);
        pf_mma(o[i + 1], pa[kk], b[2], b[3]);
      }
    }
    j = following;
  }
  asm volatile("cp.async.wait_group 0;" ::: "memory");  // a query tile with no admitted key tile never waited for Q

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

// Workspace the tile classes want (behind the counter header every workspace starts with), or 0
// when the mask is absent, short or not addressable in 16-byte chunks.
int64_t attention_prefill_scratch_bytes(const AttnParams& p) {
  if (!attention_prefill_mma_applies(p) || p.mask == nullptr || p.Lk < PF_CLASS_MIN_KEYS || (p.Lk & 7) != 0 ||
      (reinterpret_cast<uintptr_t>(p.mask) & 15) != 0)
    return 0;
  const int64_t q_tiles = (p.Lq + PF_BQ - 1) / PF_BQ, key_tiles = (p.Lk + PF_BK - 1) / PF_BK;
  if (key_tiles > PF_MAX_KEY_TILES) return 0;
  return SCRATCH_HEADER_BYTES + ((q_tiles * key_tiles + 15) & ~(int64_t)15);
}

template <int D>
static int launch_prefill(const AttnParams& p, cudaStream_t stream) {
  constexpr size_t smem = (size_t)(PF_BQ + 4 * PF_BK) * (D * 2 + 16);
  static PerDeviceOnce raised;
  if (raise_dynamic_smem(attention_prefill_mma_kernel<D>, smem, raised) != AOTO_OK) return AOTO_ERR_LAUNCH;
  dim3 grid((p.Lq + PF_BQ - 1) / PF_BQ, p.QH);
  return launch_kernel(attention_prefill_mma_kernel<D>, grid, dim3(PF_THREADS), smem, stream, false, p);
}

int attention_prefill_mma_launch(const AttnParams& given, int64_t scratch_bytes, cudaStream_t stream) {
  AttnParams p = given;
  p.tile_classes = nullptr;
  p.key_tiles = 0;
  // The workspace is optional: without it every tile is visited and the mask is read element by element.
  const int64_t need = attention_prefill_scratch_bytes(p);
  if (need > 0 && p.scratch != nullptr && scratch_bytes >= need) {
    const int q_tiles = (p.Lq + PF_BQ - 1) / PF_BQ;
    p.key_tiles = (p.Lk + PF_BK - 1) / PF_BK;
    unsigned char* classes = reinterpret_cast<unsigned char*>(p.scratch) + SCRATCH_HEADER_BYTES;
    p.tile_classes = classes;
    const int warps = q_tiles * p.key_tiles;
    const int status = launch_kernel(attention_mask_classes_kernel, dim3((warps + PF_CLASS_WARPS - 1) / PF_CLASS_WARPS),
                                     dim3(PF_CLASS_WARPS * 32), 0, stream, false, p.mask, classes, p.Lq, p.Lk, q_tiles, p.key_tiles);
    if (status != AOTO_OK) return status;
  }
  return p.D == 64 ? launch_prefill<64>(p, stream) : launch_prefill<128>(p, stream);
}

}  // namespace aoto
