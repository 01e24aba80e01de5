// One decode step as one persistent cooperative kernel.
//
// Every CTA of the grid (one per SM) walks the same stage program. A stage is a
// packed projection (GEMV), one layer's cache update + attention, or the greedy
// pick; consecutive stages are separated by a grid-wide barrier built from one
// 64-bit arrival counter (release add, acquire poll, bounded). The barrier is
// split into arrive and wait, and a GEMV stage requests its first batch of
// weights between the two: weights do not depend on activations, so the HBM
// stream keeps flowing while the grid synchronises.
//
// Activations written by one stage and read by the next go through L2
// (ld.global.cg / cp.async.cg): L1 is not coherent across SMs and activation
// buffers are reused from layer to layer.
#include <cooperative_groups.h>

#include "qgemv_core.cuh"

namespace aoto {

constexpr int STEP_THREADS = 512;
constexpr int STEP_WARPS = STEP_THREADS / 32;
constexpr int STEP_MAX_K = 16384;          // activation row staged in shared memory
constexpr int STEP_MAX_ITEMS = 256;        // (tile, block) items of one round
constexpr int STEP_BATCH = 4;              // items a warp holds in registers at once
constexpr long long STEP_SPIN_LIMIT = 1ll << 22;
constexpr int PICK_COUNTER_BASE = 0;       // payload offset (floats) of the per-CTA maxima

struct StepControl {
  unsigned long long* arrive;  // sync_words[0]
  unsigned long long* epoch;   // sync_words[1]
  int* status;
  float* scratch;
};

struct GridSync {
  unsigned long long* arrive;
  unsigned long long base;
  unsigned int ctas;
  int* status;
};

__device__ __forceinline__ unsigned long long ld_acquire_u64(const unsigned long long* ptr) {
  unsigned long long v;
  asm volatile("ld.acquire.gpu.global.u64 %0, [%1];" : "=l"(v) : "l"(ptr) : "memory");
  return v;
}

// Every thread's writes of the finished stage become visible, then the CTA is counted.
__device__ __forceinline__ void grid_arrive(const GridSync& gs) {
  __threadfence();
  __syncthreads();
  if (threadIdx.x == 0) {
    asm volatile("red.release.gpu.global.add.u64 [%0], %1;" ::"l"(gs.arrive), "l"(1ull) : "memory");
  }
}

// Wait until every CTA has arrived `index + 1` times since the launch began.
// Returns false (and records 1 + index) when the bounded wait runs out.
__device__ __forceinline__ bool grid_wait(const GridSync& gs, int index, int* flag_smem) {
  if (threadIdx.x == 0) {
    const unsigned long long target = gs.base + (unsigned long long)(index + 1) * gs.ctas;
    long long spins = 0;
    int ok = 1;
    while (ld_acquire_u64(gs.arrive) < target) {
      if (++spins > STEP_SPIN_LIMIT) { ok = 0; break; }
    }
    if (!ok) atomicCAS(gs.status, 0, index + 1);
    *flag_smem = ok;
  }
  __syncthreads();
  return *flag_smem != 0;
}

__device__ __forceinline__ uint4 ldcg_u4(const void* ptr) {
  uint4 v;
  asm volatile("ld.global.cg.v4.u32 {%0,%1,%2,%3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(ptr));
  return v;
}

__device__ __forceinline__ void cp_async_16_cg(void* smem_dst, const void* gmem_src) {
  const uint32_t dst = (uint32_t)__cvta_generic_to_shared(smem_dst);
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(gmem_src) : "memory");
}

struct StepSmem {
  uint4* xs;        // STEP_MAX_K / 8 permuted activation chunks
  float* xsum;      // STEP_MAX_K / 64
  float* csum;      // STEP_MAX_K / 8
  float* part;      // STEP_MAX_ITEMS * 16
  float* red;       // 64
  int* flag;        // 4
  unsigned char* tile;  // attention tiles and scores
};

// ---------------------------------------------------------------------------
// GEMV stage
// ---------------------------------------------------------------------------

struct RoundPlan {
  int tiles, nblocks, mats, my_tiles, tiles_per_round, per_tile;
};

__device__ __forceinline__ RoundPlan plan_rounds(const aoto_step_stage& st) {
  RoundPlan r;
  r.tiles = (st.N + 15) >> 4;
  r.nblocks = st.K >> 7;
  r.mats = st.epilogue == AOTO_EPILOGUE_SILU_MUL_PAIRED ? 2 : 1;
  r.per_tile = r.nblocks * r.mats;
  const int c = blockIdx.x, G = gridDim.x;
  r.my_tiles = r.tiles > c ? (r.tiles - c + G - 1) / G : 0;
  int tpr = 64 / r.per_tile;
  if (tpr < 1) tpr = 1;
  if (tpr > 8) tpr = 8;
  r.tiles_per_round = tpr;
  return r;
}

// item q of a round -> global tile, matrix, k block; false past the end
__device__ __forceinline__ bool item_of(const RoundPlan& r, int round, int q, int* tile, int* mat, int* kb) {
  const int tl = q / r.per_tile;
  const int local = round * r.tiles_per_round + tl;
  if (tl >= r.tiles_per_round || local >= r.my_tiles) return false;
  const int rem = q - tl * r.per_tile;
  *mat = rem / r.nblocks;
  *kb = rem - *mat * r.nblocks;
  *tile = blockIdx.x + local * gridDim.x;
  return true;
}

__device__ __forceinline__ void load_item(const aoto_step_stage& st, int tile, int mat, int kb,
                                          int g, int t, WeightItem* it) {
  const int K = st.K;
  const int row_u4 = K >> 5, row_sc = K >> 6;
  const int rlo = min(tile * 16 + g, st.N - 1), rhi = min(tile * 16 + g + 8, st.N - 1);
  const uint4* wq = reinterpret_cast<const uint4*>(mat == 0 ? st.packed : st.packed2);
  const bf16* sc = reinterpret_cast<const bf16*>(mat == 0 ? st.scales : st.scales2);
  it->lo = ldg_nc_u4(wq + (size_t)rlo * row_u4 + kb * 4 + t);
  it->hi = ldg_nc_u4(wq + (size_t)rhi * row_u4 + kb * 4 + t);
  it->slo = __ldg(reinterpret_cast<const uint32_t*>(sc + (size_t)rlo * row_sc + kb * 2));
  it->shi = __ldg(reinterpret_cast<const uint32_t*>(sc + (size_t)rhi * row_sc + kb * 2));
}

__device__ void stage_gemv(const aoto_step_stage& st, const StepSmem& sm, const GridSync& gs,
                           int wait_index, const StepControl& ctl, bool* alive) {
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int g = lane >> 2, t = lane & 3;
  const int K = st.K, N = st.N;
  const RoundPlan rp = plan_rounds(st);
  const int rounds = (rp.my_tiles + rp.tiles_per_round - 1) / rp.tiles_per_round;

  // first batch of the first round: requested before the barrier is waited for
  WeightItem items[STEP_BATCH];
  int it_tile[STEP_BATCH], it_mat[STEP_BATCH], it_kb[STEP_BATCH], it_q[STEP_BATCH];
  bool it_ok[STEP_BATCH];
  auto load_batch = [&](int round, int first) {
#pragma unroll
    for (int b = 0; b < STEP_BATCH; ++b) {
      const int q = warp + (first + b) * STEP_WARPS;
      it_q[b] = q;
      it_ok[b] = q < STEP_MAX_ITEMS && item_of(rp, round, q, &it_tile[b], &it_mat[b], &it_kb[b]);
      if (it_ok[b]) load_item(st, it_tile[b], it_mat[b], it_kb[b], g, t, &items[b]);
    }
  };
  if (rounds > 0) load_batch(0, 0);

  if (wait_index >= 0 && !grid_wait(gs, wait_index, sm.flag)) { *alive = false; return; }

  // ---- stage the activation row (one round trip: x, norm weight together) ----
  const int chunks = K >> 3;
  const bf16* x = reinterpret_cast<const bf16*>(st.x);
  if (st.x_index != nullptr) {
    long long row = *reinterpret_cast<const volatile long long*>(st.x_index);
    if (row < 0) row = 0;
    if (row >= st.x_rows) row = st.x_rows - 1;
    x += (size_t)row * K;
  }
  const uint4* wv = reinterpret_cast<const uint4*>(st.norm_weight);
  constexpr int MAXC = STEP_MAX_K / 8 / STEP_THREADS;  // chunks a thread may own
  uint4 xr[MAXC], wr[MAXC];
  float ss = 0.f;
#pragma unroll
  for (int i = 0; i < MAXC; ++i) {
    const int c = tid + i * STEP_THREADS;
    if (c < chunks) {
      xr[i] = ldcg_u4(x + (size_t)c * 8);
      if (wv != nullptr) wr[i] = __ldg(wv + c);
    }
  }
  if ((st.flags & AOTO_STAGE_FLAG_STEP_INPUTS) && blockIdx.x == gridDim.x - 1) {
    const int valid = *reinterpret_cast<const volatile int*>(st.counters);
    if (tid == 0) st.position_out[0] = (long long)(valid - 1);
    for (int i = tid; i < st.capacity; i += STEP_THREADS) st.mask_out[i] = i >= st.capacity - valid ? 1 : 0;
  }
#pragma unroll
  for (int i = 0; i < MAXC; ++i) {
    const int c = tid + i * STEP_THREADS;
    if (c < chunks) {
      if (st.x_copy != nullptr && blockIdx.x == 0) reinterpret_cast<uint4*>(st.x_copy)[c] = xr[i];
      float f[8];
      unpack8(xr[i], f);
#pragma unroll
      for (int j = 0; j < 8; ++j) ss = fmaf(f[j], f[j], ss);
    }
  }
  float inv = 1.f;
  if (wv != nullptr) inv = rsqrtf(block_sum(ss, sm.red) / (float)K + st.rms_norm_eps);
#pragma unroll
  for (int i = 0; i < MAXC; ++i) {
    const int c = tid + i * STEP_THREADS;
    if (c < chunks) {
      float f[8];
      unpack8(xr[i], f);
      if (wv != nullptr) {
        float w[8];
        unpack8(wr[i], w);
#pragma unroll
        for (int j = 0; j < 8; ++j) f[j] = round_bf16((f[j] * inv) * w[j]);
      }
      uint4 o;
      o.x = pack_bf16x2(f[0], f[4]); o.y = pack_bf16x2(f[1], f[5]);
      o.z = pack_bf16x2(f[2], f[6]); o.w = pack_bf16x2(f[3], f[7]);
      sm.csum[c] = ((f[0] + f[1]) + (f[2] + f[3])) + ((f[4] + f[5]) + (f[6] + f[7]));
      sm.xs[c] = o;
    }
  }
  __syncthreads();
  for (int gi = tid; gi < (K >> 6); gi += STEP_THREADS) {
    float s = 0.f;
#pragma unroll
    for (int c = 0; c < 8; ++c) s += sm.csum[gi * 8 + c];
    sm.xsum[gi] = 136.f * s;
  }
  __syncthreads();

  // ---- rounds ----
  GemvParams ep;
  ep.addend = reinterpret_cast<const bf16*>(st.addend);
  ep.gate = nullptr;
  ep.N = N; ep.K = K; ep.addend_kind = st.addend_kind; ep.epilogue = st.epilogue;
  ep.alpha = st.alpha; ep.beta = st.beta; ep.eps = st.rms_norm_eps;
  bf16* out = reinterpret_cast<bf16*>(st.out);
  const bool keep = ((g & 1) == (t >> 1));
  float best_v = -INFINITY;
  int best_i = 0x7fffffff;

  for (int round = 0; round < rounds; ++round) {
    const int items_in_round = min(rp.tiles_per_round, rp.my_tiles - round * rp.tiles_per_round) * rp.per_tile;
    const int per_warp = (items_in_round + STEP_WARPS - 1) / STEP_WARPS;
    for (int first = 0; first < per_warp; first += STEP_BATCH) {
      if (round > 0 || first > 0) load_batch(round, first);
#pragma unroll
      for (int b = 0; b < STEP_BATCH; ++b) {
        if (!it_ok[b]) continue;
        const int kb = it_kb[b];
        uint4 bf[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          bf[j] = sm.xs[kb * 16 + t * 4 + j];
          if (!keep) bf[j] = make_uint4(0u, 0u, 0u, 0u);
        }
        const float2 off = *reinterpret_cast<const float2*>(sm.xsum + kb * 2);
        const WeightItem& it = items[b];
        const uint32_t wl[4] = {it.lo.x, it.lo.y, it.lo.z, it.lo.w};
        const uint32_t wh[4] = {it.hi.x, it.hi.y, it.hi.z, it.hi.w};
        float c[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          mma_16816(c, AOTO_NIB(wl[j], 0), AOTO_NIB(wh[j], 0), AOTO_NIB(wl[j], 4), AOTO_NIB(wh[j], 4),
                    bf[j].x, bf[j].y);
          mma_16816(c, AOTO_NIB(wl[j], 8), AOTO_NIB(wh[j], 8), AOTO_NIB(wl[j], 12), AOTO_NIB(wh[j], 12),
                    bf[j].z, bf[j].w);
        }
        if (t == 0) {
          float* dst = sm.part + it_q[b] * 16;
          dst[g] = bf16x2_lo(it.slo) * (c[0] - off.x) + bf16x2_hi(it.slo) * (c[1] - off.y);
          dst[g + 8] = bf16x2_lo(it.shi) * (c[2] - off.x) + bf16x2_hi(it.shi) * (c[3] - off.y);
        }
      }
    }
    __syncthreads();
    const int tiles_here = items_in_round / rp.per_tile;
    if (tid < tiles_here * 16) {
      const int tl = tid >> 4, r = tid & 15;
      const int tile = blockIdx.x + (round * rp.tiles_per_round + tl) * gridDim.x;
      const int n = tile * 16 + r;
      if (n < N) {
        const float* p0 = sm.part + (tl * rp.per_tile) * 16 + r;
        float total = 0.f, total2 = 0.f;
        for (int kb = 0; kb < rp.nblocks; ++kb) total += p0[kb * 16];
        if (rp.mats == 2)
          for (int kb = 0; kb < rp.nblocks; ++kb) total2 += p0[(rp.nblocks + kb) * 16];
        const bf16 y = __float2bfloat16_rn(finish_output(ep, 0, n, total, total2));
        out[n] = y;
        if (st.flags & AOTO_STAGE_FLAG_ARGMAX) {
          float v = __bfloat162float(y);
          if (v != v) v = INFINITY;
          if (v > best_v || (v == best_v && n < best_i)) { best_v = v; best_i = n; }
        }
      }
    }
    __syncthreads();
  }

  if (st.flags & AOTO_STAGE_FLAG_ARGMAX) {
    // the CTA's best (value, first index) goes to scratch for the pick stage
    float* sv = sm.red;
    int* si = reinterpret_cast<int*>(sm.red + 32);
#pragma unroll
    for (int offset = 16; offset > 0; offset >>= 1) {
      const float ov = __shfl_xor_sync(0xffffffffu, best_v, offset);
      const int oi = __shfl_xor_sync(0xffffffffu, best_i, offset);
      if (ov > best_v || (ov == best_v && oi < best_i)) { best_v = ov; best_i = oi; }
    }
    if (lane == 0) { sv[warp] = best_v; si[warp] = best_i; }
    __syncthreads();
    if (tid == 0) {
      for (int w = 1; w < STEP_WARPS; ++w)
        if (sv[w] > best_v || (sv[w] == best_v && si[w] < best_i)) { best_v = sv[w]; best_i = si[w]; }
      float* payload = ctl.scratch + SCRATCH_HEADER_BYTES / 4 + PICK_COUNTER_BASE;
      payload[2 * blockIdx.x] = best_v;
      reinterpret_cast<int*>(payload)[2 * blockIdx.x + 1] = best_i;
    }
  }
}

// ---------------------------------------------------------------------------
// attention stage: rotate q and k, write the shifted window, attend
// ---------------------------------------------------------------------------

__device__ __forceinline__ int attention_tile_keys(int head_dim) { return head_dim <= 64 ? 256 : 128; }

__device__ __forceinline__ float rotate_from(const bf16* head, const bf16* cos_row, const bf16* sin_row,
                                             int d, int D) {
  const int half = D >> 1;
  const float v = ldcg_bf16(head + d);
  const float partner = d < half ? -ldcg_bf16(head + d + half) : ldcg_bf16(head + d - half);
  return round_bf16(round_bf16(v * __bfloat162float(cos_row[d])) +
                    round_bf16(partner * __bfloat162float(sin_row[d])));
}

__device__ void stage_attention(const aoto_step_stage& st, const StepSmem& sm, const StepControl& ctl) {
  const int D = st.head_dim, C = st.capacity, KVH = st.kv_heads, QH = st.query_heads;
  const int G = QH / KVH;
  const int TK = attention_tile_keys(D);
  const int splits = (C + TK - 1) / TK;
  if ((int)blockIdx.x >= KVH * splits) return;
  const int kvh = blockIdx.x / splits, split = blockIdx.x - kvh * splits;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int row_bytes = D * 2 + 16;
  unsigned char* kt = sm.tile;
  unsigned char* vt = kt + (size_t)TK * row_bytes;
  float* qs = reinterpret_cast<float*>(vt + (size_t)TK * row_bytes);
  float* sc = qs + G * D;
  float* stat = sc + G * TK;
  float* madd = stat + G * 2;

  const int k0 = split * TK;
  const int nkeys = min(TK, C - k0);
  const int chunks = D >> 3;
  const bf16* kin = reinterpret_cast<const bf16*>(st.cache_in) + (size_t)kvh * C * D;
  const bf16* vin = reinterpret_cast<const bf16*>(st.cache_in) + ((size_t)KVH + kvh) * C * D;
  bf16* kout = reinterpret_cast<bf16*>(st.cache_out) + (size_t)kvh * C * D;
  bf16* vout = reinterpret_cast<bf16*>(st.cache_out) + ((size_t)KVH + kvh) * C * D;
  const bf16* row = reinterpret_cast<const bf16*>(st.row);

  // window slot j of the new cache is slot j + 1 of the old one; the last slot is the new pair
  for (int c = tid; c < nkeys * chunks; c += STEP_THREADS) {
    const int r = c / chunks, j = c - r * chunks;
    const int slot = k0 + r;
    if (slot < C - 1) {
      cp_async_16_cg(kt + (size_t)r * row_bytes + j * 16, kin + (size_t)(slot + 1) * D + j * 8);
      cp_async_16_cg(vt + (size_t)r * row_bytes + j * 16, vin + (size_t)(slot + 1) * D + j * 8);
    }
  }
  long long pos = *reinterpret_cast<const volatile long long*>(st.position);
  if (pos < 0) pos = 0;
  if (pos >= st.table_rows) pos = st.table_rows - 1;
  const bf16* cos_row = reinterpret_cast<const bf16*>(st.cos_table) + (size_t)pos * D;
  const bf16* sin_row = reinterpret_cast<const bf16*>(st.sin_table) + (size_t)pos * D;
  for (int i = tid; i < G * D; i += STEP_THREADS) {
    const int h = i / D, d = i - h * D;
    qs[i] = rotate_from(row + st.query_start + (size_t)(kvh * G + h) * D, cos_row, sin_row, d, D) * st.scale;
  }
  if (k0 + nkeys == C) {  // this CTA owns the last slot: rotated key and value of the step
    const int r = C - 1 - k0;
    for (int d = tid; d < D; d += STEP_THREADS) {
      const float kv = rotate_from(row + st.key_start + (size_t)kvh * D, cos_row, sin_row, d, D);
      reinterpret_cast<bf16*>(kt + (size_t)r * row_bytes)[d] = __float2bfloat16_rn(kv);
      unsigned short raw;
      asm volatile("ld.global.cg.u16 %0, [%1];" : "=h"(raw) : "l"(row + st.value_start + (size_t)kvh * D + d));
      reinterpret_cast<unsigned short*>(vt + (size_t)r * row_bytes)[d] = raw;
    }
  }
  for (int i = tid; i < TK; i += STEP_THREADS)
    madd[i] = (i < nkeys && st.mask[k0 + i]) ? 0.f : -INFINITY;
  asm volatile("cp.async.commit_group;\ncp.async.wait_group 0;" ::: "memory");
  __syncthreads();

  // the shifted window goes out to the next cache while it is scored
  for (int c = tid; c < nkeys * chunks; c += STEP_THREADS) {
    const int r = c / chunks, j = c - r * chunks;
    const size_t dst = (size_t)(k0 + r) * D + j * 8;
    *reinterpret_cast<uint4*>(kout + dst) = *reinterpret_cast<const uint4*>(kt + (size_t)r * row_bytes + j * 16);
    *reinterpret_cast<uint4*>(vout + dst) = *reinterpret_cast<const uint4*>(vt + (size_t)r * row_bytes + j * 16);
  }

  for (int item = tid; item < G * TK; item += STEP_THREADS) {
    const int h = item / TK, key = item - h * TK;
    float s = -INFINITY;
    const float m_add = madd[key];
    if (m_add != -INFINITY) {
      const uint4* krow = reinterpret_cast<const uint4*>(kt + (size_t)key * row_bytes);
      const float* qh = qs + h * D;
      float dot = 0.f;
      for (int j = 0; j < chunks; ++j) {
        const uint4 kk = krow[j];
        const float* q8 = qh + j * 8;
        dot = fmaf(bf16x2_lo(kk.x), q8[0], dot); dot = fmaf(bf16x2_hi(kk.x), q8[1], dot);
        dot = fmaf(bf16x2_lo(kk.y), q8[2], dot); dot = fmaf(bf16x2_hi(kk.y), q8[3], dot);
        dot = fmaf(bf16x2_lo(kk.z), q8[4], dot); dot = fmaf(bf16x2_hi(kk.z), q8[5], dot);
        dot = fmaf(bf16x2_lo(kk.w), q8[6], dot); dot = fmaf(bf16x2_hi(kk.w), q8[7], dot);
      }
      s = dot;
    }
    sc[item] = s;
  }
  __syncthreads();
  for (int h = warp; h < G; h += STEP_WARPS) {
    float m = -INFINITY;
    for (int key = lane; key < TK; key += 32) m = fmaxf(m, sc[h * TK + key]);
    m = warp_max(m);
    const float m_safe = (m == -INFINITY) ? 0.f : m;
    float l = 0.f;
    for (int key = lane; key < TK; key += 32) {
      const float s = sc[h * TK + key];
      const float e = (s == -INFINITY) ? 0.f : expf(s - m_safe);
      sc[h * TK + key] = e;
      l += e;
    }
    l = warp_sum(l);
    if (lane == 0) { stat[2 * h] = m; stat[2 * h + 1] = l; }
  }
  __syncthreads();
  const int pairs = D >> 1;
  bf16* out = reinterpret_cast<bf16*>(st.attn_out);
  float* partials = ctl.scratch + SCRATCH_HEADER_BYTES / 4 + 2 * gridDim.x;  // after the pick payload
  for (int item = tid; item < G * pairs; item += STEP_THREADS) {
    const int h = item / pairs, dp = item - h * pairs;
    float a0 = 0.f, a1 = 0.f;
    const float* w = sc + h * TK;
    for (int key = 0; key < nkeys; ++key) {
      const float wk = w[key];
      if (wk != 0.f) {
        const uint32_t vv = *reinterpret_cast<const uint32_t*>(vt + (size_t)key * row_bytes + dp * 4);
        a0 = fmaf(wk, bf16x2_lo(vv), a0);
        a1 = fmaf(wk, bf16x2_hi(vv), a1);
      }
    }
    const int head = kvh * G + h;
    if (splits == 1) {
      const float l = stat[2 * h + 1];
      const float inv = l > 0.f ? 1.f / l : 0.f;
      *reinterpret_cast<uint32_t*>(out + (size_t)head * D + dp * 2) = pack_bf16x2(a0 * inv, a1 * inv);
    } else {
      float* dst = partials + ((size_t)head * splits + split) * (D + 2);
      dst[2 + dp * 2] = a0;
      dst[3 + dp * 2] = a1;
      if (dp == 0) { dst[0] = stat[2 * h]; dst[1] = stat[2 * h + 1]; }
    }
  }
  if (splits == 1) return;

  int* counters = reinterpret_cast<int*>(ctl.scratch);
  __threadfence();
  __syncthreads();
  if (tid == 0) {
    const int arrived = atomicAdd(counters + kvh, 1);
    const int last = arrived == splits - 1;
    if (last) counters[kvh] = 0;
    *sm.flag = last;
  }
  __syncthreads();
  if (!*sm.flag) return;
  __threadfence();
  for (int item = tid; item < G * D; item += STEP_THREADS) {
    const int h = item / D, d = item - h * D;
    const int head = kvh * G + h;
    const float* base = partials + (size_t)head * splits * (D + 2);
    float m = -INFINITY;
    for (int s2 = 0; s2 < splits; ++s2) m = fmaxf(m, __ldcg(base + (size_t)s2 * (D + 2)));
    float acc = 0.f, l = 0.f;
    if (m != -INFINITY) {
      for (int s2 = 0; s2 < splits; ++s2) {
        const float* part = base + (size_t)s2 * (D + 2);
        const float pm = __ldcg(part);
        const float w = (pm == -INFINITY) ? 0.f : expf(pm - m);
        acc = fmaf(w, __ldcg(part + 2 + d), acc);
        l = fmaf(w, __ldcg(part + 1), l);
      }
    }
    out[(size_t)head * D + d] = __float2bfloat16_rn(l > 0.f ? acc / l : 0.f);
  }
}

// ---------------------------------------------------------------------------
// pick stage: CTA 0 reduces the per-CTA maxima the LM-head stage left
// ---------------------------------------------------------------------------
__device__ void stage_pick(const aoto_step_stage& st, const StepControl& ctl) {
  if (blockIdx.x != 0 || threadIdx.x >= 32) return;
  const float* payload = ctl.scratch + SCRATCH_HEADER_BYTES / 4 + PICK_COUNTER_BASE;
  float bv = -INFINITY;
  int bi = 0x7fffffff;
  for (int c = threadIdx.x; c < (int)gridDim.x; c += 32) {
    const float v = __ldcg(payload + 2 * c);
    const int i = __ldcg(reinterpret_cast<const int*>(payload) + 2 * c + 1);
    if (v > bv || (v == bv && i < bi)) { bv = v; bi = i; }
  }
#pragma unroll
  for (int offset = 16; offset > 0; offset >>= 1) {
    const float ov = __shfl_xor_sync(0xffffffffu, bv, offset);
    const int oi = __shfl_xor_sync(0xffffffffu, bi, offset);
    if (ov > bv || (ov == bv && oi < bi)) { bv = ov; bi = oi; }
  }
  if (threadIdx.x == 0) {
    st.token[0] = (long long)bi;
    if (st.counters != nullptr) {
      const int step = st.counters[1];
      if (st.generated != nullptr && step < st.generated_capacity) st.generated[step] = (long long)bi;
      st.counters[0] += 1;
      st.counters[1] = step + 1;
    }
  }
}

__global__ void __launch_bounds__(STEP_THREADS, 1)
decode_step_kernel(const aoto_step_stage* __restrict__ stages, int stage_count, StepControl ctl) {
  extern __shared__ uint4 smem_raw[];
  __shared__ aoto_step_stage stage;
  StepSmem sm;
  sm.xs = smem_raw;
  sm.xsum = reinterpret_cast<float*>(sm.xs + STEP_MAX_K / 8);
  sm.csum = sm.xsum + STEP_MAX_K / 64;
  sm.part = sm.csum + STEP_MAX_K / 8;
  sm.red = sm.part + STEP_MAX_ITEMS * 16;
  sm.flag = reinterpret_cast<int*>(sm.red + 64);
  sm.tile = reinterpret_cast<unsigned char*>(sm.flag + 4);

  __shared__ unsigned long long epoch_smem;
  if (threadIdx.x == 0) epoch_smem = ld_acquire_u64(ctl.epoch);
  __syncthreads();
  GridSync gs;
  gs.arrive = ctl.arrive;
  gs.ctas = gridDim.x;
  gs.status = ctl.status;
  gs.base = epoch_smem * (unsigned long long)stage_count * gridDim.x;

  bool alive = true;
  for (int s = 0; s < stage_count && alive; ++s) {
    __syncthreads();
    // every thread copies a slice of the descriptor
    {
      const int words = sizeof(aoto_step_stage) / 4;
      const uint32_t* src = reinterpret_cast<const uint32_t*>(stages + s);
      uint32_t* dst = reinterpret_cast<uint32_t*>(&stage);
      for (int i = threadIdx.x; i < words; i += STEP_THREADS) dst[i] = __ldg(src + i);
    }
    __syncthreads();
    if (stage.kind == AOTO_STAGE_GEMV) {
      stage_gemv(stage, sm, gs, s - 1, ctl, &alive);
    } else {
      if (s > 0 && !grid_wait(gs, s - 1, sm.flag)) { alive = false; break; }
      if (stage.kind == AOTO_STAGE_ATTENTION) stage_attention(stage, sm, ctl);
      else if (stage.kind == AOTO_STAGE_PICK) stage_pick(stage, ctl);
    }
    if (alive) grid_arrive(gs);
  }
  // the last CTA-independent duty: open the next launch's epoch once everyone is done
  if (alive && blockIdx.x == 0) {
    if (grid_wait(gs, stage_count - 1, sm.flag) && threadIdx.x == 0) {
      asm volatile("st.release.gpu.global.u64 [%0], %1;" ::"l"(ctl.epoch), "l"(epoch_smem + 1) : "memory");
    }
  }
}

static size_t step_smem_bytes(int max_head_dim, int max_group) {
  size_t fixed = (size_t)STEP_MAX_K / 8 * 16 + (size_t)STEP_MAX_K / 64 * 4 + (size_t)STEP_MAX_K / 8 * 4 +
                 (size_t)STEP_MAX_ITEMS * 16 * 4 + 64 * 4 + 16;
  const int D = max_head_dim > 0 ? max_head_dim : 64;
  const int G = max_group > 0 ? max_group : 1;
  const int TK = D <= 64 ? 256 : 128;
  const size_t attention = (size_t)2 * TK * (D * 2 + 16) + ((size_t)G * D + (size_t)G * TK + (size_t)G * 2 + TK) * 4;
  return fixed + attention;
}

static int check_stage(const aoto_step_stage& st) {
  if (st.kind == AOTO_STAGE_GEMV) {
    if (st.N <= 0 || st.K <= 0 || st.K > STEP_MAX_K || (st.K & 127) || st.group_size != 64) return 0;
    if (st.epilogue == AOTO_EPILOGUE_SILU_MUL) return 0;
    const int per_tile = (st.K >> 7) * (st.epilogue == AOTO_EPILOGUE_SILU_MUL_PAIRED ? 2 : 1);
    if (per_tile > STEP_MAX_ITEMS) return 0;
    return 1;
  }
  if (st.kind == AOTO_STAGE_ATTENTION) {
    if (st.head_dim <= 0 || (st.head_dim & 7) || st.head_dim > 128) return 0;
    if (st.kv_heads <= 0 || st.query_heads % st.kv_heads) return 0;
    if (st.query_heads / st.kv_heads > 16 || st.kv_heads > SCRATCH_MAX_COUNTERS) return 0;
    if (st.capacity <= 0) return 0;
    return 1;
  }
  return st.kind == AOTO_STAGE_PICK;
}

}  // namespace aoto

using namespace aoto;

extern "C" int aoto_sm100_decode_step_stage_size(void) { return (int)sizeof(aoto_step_stage); }

extern "C" int aoto_sm100_decode_step_supported(const aoto_step_stage* stages, int32_t count) {
  if (!stages || count <= 0) return 0;
  for (int i = 0; i < count; ++i)
    if (!check_stage(stages[i])) return 0;
  return 1;
}

extern "C" int64_t aoto_sm100_decode_step_scratch_bytes(const aoto_step_stage* stages, int32_t count) {
  if (!stages || count <= 0) return 0;
  int64_t need = SCRATCH_HEADER_BYTES + 2 * 1024 * 4;  // pick payload for up to 1024 CTAs
  for (int i = 0; i < count; ++i) {
    const aoto_step_stage& st = stages[i];
    if (st.kind != AOTO_STAGE_ATTENTION) continue;
    const int TK = st.head_dim <= 64 ? 256 : 128;
    const int splits = (st.capacity + TK - 1) / TK;
    const int64_t bytes = SCRATCH_HEADER_BYTES + 2 * 1024 * 4 +
                          (int64_t)st.query_heads * splits * (st.head_dim + 2) * 4;
    if (bytes > need) need = bytes;
  }
  return need;
}

extern "C" int aoto_sm100_decode_step(const aoto_decode_step_args* a, void* stream_) {
  if (!a || !a->stages || a->stage_count <= 0 || !a->sync_words || !a->status || !a->scratch)
    return AOTO_ERR_ARGUMENT;
  int device = 0, sms = 0, coop = 0;
  if (cudaGetDevice(&device) != cudaSuccess) return AOTO_ERR_LAUNCH;
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device);
  cudaDeviceGetAttribute(&coop, cudaDevAttrCooperativeLaunch, device);
  if (!coop) return AOTO_ERR_UNSUPPORTED;
  size_t smem = step_smem_bytes(128, 16);
  if (step_smem_bytes(64, 16) > smem) smem = step_smem_bytes(64, 16);
  static bool raised = false;
  if (!raised) {
    if (cudaFuncSetAttribute(decode_step_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess) {
      (void)cudaGetLastError();
      return AOTO_ERR_LAUNCH;
    }
    raised = true;
  }
  int per_sm = 0;
  if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, decode_step_kernel, STEP_THREADS, smem) != cudaSuccess ||
      per_sm < 1) {
    (void)cudaGetLastError();
    return AOTO_ERR_UNSUPPORTED;
  }
  int ctas = a->ctas > 0 ? a->ctas : sms;
  if (ctas > sms * per_sm) ctas = sms * per_sm;  // every CTA must be resident: they wait on one another
  if (ctas > 1024) ctas = 1024;
  StepControl ctl;
  ctl.arrive = reinterpret_cast<unsigned long long*>(a->sync_words);
  ctl.epoch = ctl.arrive + 1;
  ctl.status = a->status;
  ctl.scratch = reinterpret_cast<float*>(a->scratch);
  cudaLaunchConfig_t config = {};
  config.gridDim = dim3(ctas);
  config.blockDim = dim3(STEP_THREADS);
  config.dynamicSmemBytes = smem;
  config.stream = (cudaStream_t)stream_;
  cudaLaunchAttribute attribute[1];
  attribute[0].id = cudaLaunchAttributeCooperative;
  attribute[0].val.cooperative = 1;
  config.attrs = attribute;
  config.numAttrs = 1;
  const aoto_step_stage* stages = a->stages;
  int count = a->stage_count;
  if (cudaLaunchKernelEx(&config, decode_step_kernel, stages, count, ctl) != cudaSuccess) {
    (void)cudaGetLastError();
    return AOTO_ERR_LAUNCH;
  }
  return AOTO_OK;
}
