// One decode step as one persistent cooperative kernel, without barriers.
//
// Every CTA of the grid (one per SM) walks the same stage program. A stage is a
// packed projection (GEMV), one layer's cache update + attention, or the greedy
// pick. Intermediate vectors are exchanged as 8-byte "stamped" words - two bf16
// values and the launch's 32-bit epoch - written with single 8-byte stores. A
// consumer polls exactly the words it needs until they carry the epoch, so a
// stage starts on a CTA one L2 round trip after its inputs were produced, with
// no grid-wide synchronisation, fence or arrival counter on the critical path.
// A projection requests its first batch of weights BEFORE it polls its input
// row: weights do not depend on activations, so the HBM stream never waits for
// the dependency chain.
//
// Polls are bounded (POLL_LIMIT rounds); a CTA whose poll runs out records the
// stage in `status` and leaves, and its consumers run out in turn.
#include "qgemv_core.cuh"

namespace aoto {

constexpr int STEP_THREADS = 256;
constexpr int STEP_WARPS = STEP_THREADS / 32;
constexpr int STEP_MAX_K = 16384;      // activation row staged in shared memory
constexpr int STEP_MAX_ITEMS = 336;    // partial sums kept in shared memory (6 chunks of 56 blocks)
constexpr int POLL_SLICES = 3;         // 32-byte chunks of the input row a thread polls at once
constexpr int POLL_LIMIT = 1 << 20;    // rounds of a bounded poll (each is >= one L2 round trip)
constexpr int ATT_TILE = 64;           // keys per attention item
constexpr int MAX_GROUP = 16;          // query heads per kv head
constexpr int ITEM_BYTES = 16 * 64 + 16 * 4;    // one 16-row x 128-column block: codes, then 16 scale pairs
constexpr int ITEM_SLOTS = 14;                 // blocks a warp keeps in shared memory: two banks of seven
constexpr int BANK_SLOTS = ITEM_SLOTS / 2;
constexpr int CHUNK_ITEMS = BANK_SLOTS * STEP_WARPS;  // blocks of one chunk of a CTA's list
constexpr int PART_ITEMS = 6 * CHUNK_ITEMS;    // ring of partial sums: a tile spans at most three chunks and a
                                               // warp runs at most two chunks ahead of the last barrier
constexpr int RING_SLOT_BYTES = 7680;  // one 16-row weight tile with its scales (K <= 896)
constexpr int RING_DEPTH = STEP_WARPS <= 8 ? 2 : 1;  // ring slots a warp owns
constexpr int RING_SLOTS = RING_DEPTH * STEP_WARPS;

struct StepControl {
  uint32_t epoch;
  int* status;
  float* scratch;
  unsigned long long* trace;
};

__device__ __forceinline__ unsigned long long global_timer_ns() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}
__device__ __forceinline__ void trace_mark(const StepControl& ctl, int stage, int which) {
  if (ctl.trace != nullptr && blockIdx.x == 0 && threadIdx.x == 0) ctl.trace[stage * 8 + which] = global_timer_ns();
}

// ---- stamped words ---------------------------------------------------------
__device__ __forceinline__ void st_stamped(void* ptr, uint32_t data, uint32_t stamp) {
  asm volatile("st.volatile.global.v2.u32 [%0], {%1, %2};" ::"l"(ptr), "r"(data), "r"(stamp) : "memory");
}
__device__ __forceinline__ uint2 ld_stamped(const void* ptr) {
  uint2 v;
  asm volatile("ld.volatile.global.v2.u32 {%0, %1}, [%2];" : "=r"(v.x), "=r"(v.y) : "l"(ptr) : "memory");
  return v;
}
// two consecutive stamped words (16-byte aligned)
__device__ __forceinline__ uint4 ld_stamped_pair(const void* ptr) {
  uint4 v;
  asm volatile("ld.volatile.global.v4.u32 {%0, %1, %2, %3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(ptr) : "memory");
  return v;
}

__device__ __forceinline__ void cp_async_16_cg(void* smem_dst, const void* gmem_src) {
  const uint32_t dst = (uint32_t)__cvta_generic_to_shared(smem_dst);
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(gmem_src) : "memory");
}

// ---- bulk copies into shared memory, completion counted by an mbarrier ----
__device__ __forceinline__ uint32_t smem_address(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void mbar_init(unsigned long long* bar, int count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_address(bar)), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(unsigned long long* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_address(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(unsigned long long* bar, uint32_t parity) {
  uint32_t done;
  asm volatile(
      "{\n.reg .pred p;\nmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\nselp.u32 %0, 1, 0, p;\n}\n"
      : "=r"(done) : "r"(smem_address(bar)), "r"(parity) : "memory");
  return done != 0;
}
// global -> this CTA's shared memory; both addresses 16-byte aligned, bytes a multiple of 16
__device__ __forceinline__ void bulk_load(void* smem_dst, const void* gmem_src, uint32_t bytes, unsigned long long* bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
               ::"r"(smem_address(smem_dst)), "l"(gmem_src), "r"(bytes), "r"(smem_address(bar)) : "memory");
}
__device__ __forceinline__ void fence_async_proxy() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }

// Shared-memory accesses by 32-bit shared address. The kernel's shared-memory pointers travel
// through a struct, where the compiler no longer knows their address space and falls back to
// generic loads with 64-bit address arithmetic; the block loop states the space itself.
__device__ __forceinline__ uint4 lds128(uint32_t address) {
  uint4 v;
  asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(address));
  return v;
}
__device__ __forceinline__ uint32_t lds32(uint32_t address) {
  uint32_t v;
  asm volatile("ld.shared.u32 %0, [%1];" : "=r"(v) : "r"(address));
  return v;
}
__device__ __forceinline__ float2 lds64f(uint32_t address) {
  float2 v;
  asm volatile("ld.shared.v2.f32 {%0,%1}, [%2];" : "=f"(v.x), "=f"(v.y) : "r"(address));
  return v;
}
__device__ __forceinline__ void sts32f(uint32_t address, float value) {
  asm volatile("st.shared.f32 [%0], %1;" ::"r"(address), "f"(value) : "memory");
}

// One 16 x 128 block with every operand addressed in shared memory: `b_address` is where this
// lane's B fragments of the block start (the staged row, or a zero page for the lanes whose
// column belongs to the other group), `offset_address` the block's pair of 136*sum(x) values.
__device__ __forceinline__ void mma_block_shared(const WeightItem& it, uint32_t b_address, uint32_t offset_address,
                                                 float& lo, float& hi) {
  const float2 off = lds64f(offset_address);
  float c[4] = {-off.x, -off.y, -off.x, -off.y};
  const uint32_t wl[4] = {it.lo.x, it.lo.y, it.lo.z, it.lo.w};
  const uint32_t wh[4] = {it.hi.x, it.hi.y, it.hi.z, it.hi.w};
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    const uint4 b = lds128(b_address + j * 16);
    mma_16816(c, AOTO_NIB(wl[j], 0), AOTO_NIB(wh[j], 0), AOTO_NIB(wl[j], 4), AOTO_NIB(wh[j], 4), b.x, b.y);
    mma_16816(c, AOTO_NIB(wl[j], 8), AOTO_NIB(wh[j], 8), AOTO_NIB(wl[j], 12), AOTO_NIB(wh[j], 12), b.z, b.w);
  }
  lo = fmaf(bf16x2_lo(it.slo), c[0], bf16x2_hi(it.slo) * c[1]);
  hi = fmaf(bf16x2_lo(it.shi), c[2], bf16x2_hi(it.shi) * c[3]);
}

__device__ __forceinline__ void cp_async_4(void* smem_dst, const void* gmem_src) {
  const uint32_t dst = (uint32_t)__cvta_generic_to_shared(smem_dst);
  asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(dst), "l"(gmem_src) : "memory");
}

struct StepSmem {
  uint4* xs;            // STEP_MAX_K / 8 permuted activation chunks
  uint4* nw;            // STEP_MAX_K / 8 chunks of the norm weight
  float* xsum;          // STEP_MAX_K / 64
  float* part;          // STEP_MAX_ITEMS * 16
  float* red;           // 64
  int* flag;            // 4 ints, then a 64-byte zero page
  unsigned long long* bars;  // RING_SLOTS mbarriers
  uint32_t* ring_uses;       // completed phases of every ring slot
  unsigned char* tile;  // attention tiles, scores, row values; or the weight ring of a GEMV stage
};

// A CTA gave up: remember where, once.
__device__ __forceinline__ void give_up(const StepControl& ctl, int stage) {
  if (threadIdx.x == 0) atomicCAS(ctl.status, 0, stage + 1);
}

// ---------------------------------------------------------------------------
// GEMV stage
// ---------------------------------------------------------------------------
struct RoundPlan {
  int tiles, nblocks, mats, my_tiles, per_tile;
  float inv_per_tile, inv_nblocks;  // exact for the small quotients taken here (< 2^10)
};

__device__ __forceinline__ int small_div(int a, float inv_b) { return __float2int_rd(((float)a + 0.5f) * inv_b); }

// Quotients here are small (< 2^10) and the operands below 2^20, where the reciprocal form is
// exact; it replaces integer divisions that cost ~30 instructions each at the head of a stage.
__device__ __forceinline__ RoundPlan plan_rounds(const aoto_step_stage& st) {
  RoundPlan r;
  r.tiles = (st.N + 15) >> 4;
  r.nblocks = st.K >> 7;
  r.mats = st.epilogue == AOTO_EPILOGUE_SILU_MUL_PAIRED ? 2 : 1;
  r.per_tile = r.nblocks * r.mats;
  const int c = blockIdx.x, G = gridDim.x;
  r.inv_per_tile = __frcp_rn((float)r.per_tile);
  r.inv_nblocks = __frcp_rn((float)r.nblocks);
  r.my_tiles = r.tiles > c ? small_div(r.tiles - c + G - 1, __frcp_rn((float)G)) : 0;
  return r;
}

// Returns false when a poll ran out (the caller leaves the kernel).
__device__ bool stage_gemv(const aoto_step_stage& shared_stage, const StepSmem& sm, const StepControl& ctl, int stage_index) {
  // The descriptor lives in shared memory; a private copy keeps its fields in registers, so that
  // they are not read again after every barrier and volatile access.
  const aoto_step_stage st = shared_stage;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int g = lane >> 2, t = lane & 3;
  const int K = st.K, N = st.N;
  const uint32_t epoch = ctl.epoch;
  const RoundPlan rp = plan_rounds(st);
  trace_mark(ctl, stage_index, 0);

  // ---- weights first: they do not depend on the input row ----
  // Chunk mode: the CTA's blocks - (tile, matrix, k block), tile-major - form one list that is cut
  // into chunks of 56; block i of a chunk belongs to warp i % 8 and travels global -> shared
  // memory with cp.async into one of the warp's two banks of seven slots. Two chunks are in
  // flight before anything waits; a bank is refilled by its warp as soon as the warp has
  // multiplied it (no CTA-wide synchronisation for the ring), none of it occupies registers.
  unsigned char* my_slots = sm.tile + (size_t)warp * ITEM_SLOTS * ITEM_BYTES;
  const int total_items = rp.my_tiles * rp.per_tile;
  const int chunks_total = (total_items + CHUNK_ITEMS - 1) / CHUNK_ITEMS;
  auto locate = [&](int idx, int* tile, int* mat, int* kb) {
    const int lt = small_div(idx, rp.inv_per_tile);
    const int j = idx - lt * rp.per_tile;
    *mat = small_div(j, rp.inv_nblocks);
    *kb = j - *mat * rp.nblocks;
    *tile = blockIdx.x + lt * gridDim.x;
  };
  auto request_chunk = [&](int chunk) {
    if (chunk < chunks_total) {
      const int r = lane >> 1, half = lane & 1;
      unsigned char* bank = my_slots + (size_t)(chunk & 1) * BANK_SLOTS * ITEM_BYTES;
      for (int i = 0; i < BANK_SLOTS; ++i) {
        const int idx = chunk * CHUNK_ITEMS + warp + i * STEP_WARPS;
        if (idx >= total_items) break;
        int tile, mat, kb;
        locate(idx, &tile, &mat, &kb);
        unsigned char* slot = bank + (size_t)i * ITEM_BYTES;
        const unsigned char* wbytes = reinterpret_cast<const unsigned char*>(mat == 0 ? st.packed : st.packed2);
        const unsigned char* sbytes = reinterpret_cast<const unsigned char*>(mat == 0 ? st.scales : st.scales2);
        const int n = min(tile * 16 + r, N - 1);
        const unsigned char* src = wbytes + (size_t)n * (K >> 1) + (size_t)kb * 64 + half * 32;
        cp_async_16_cg(slot + r * 64 + half * 32, src);
        cp_async_16_cg(slot + r * 64 + half * 32 + 16, src + 16);
        if (lane < 16) {
          const int ns = min(tile * 16 + lane, N - 1);
          cp_async_4(slot + 1024 + lane * 4, sbytes + (size_t)ns * (K >> 5) + (size_t)kb * 4);
        }
      }
    }
    asm volatile("cp.async.commit_group;" ::: "memory");  // an empty group keeps the count uniform
  };
  // A stage with many small tiles per CTA (K <= 896 and no second matrix: the LM head of the 0.5B
  // shape) runs in "ring mode": every warp owns whole tiles and streams them through a ring in
  // shared memory. A tile's 16 packed rows are one contiguous run of global memory, and so are
  // its scales, so two bulk copies fetch a tile; every warp owns two ring slots and keeps both
  // in flight, accumulates in registers and stores its rows itself, with no CTA-wide
  // synchronisation between tiles.
  const bool ring_mode = rp.my_tiles >= STEP_WARPS && st.addend_mode <= AOTO_STAGE_ADDEND_PLAIN &&
                         rp.mats == 1 && (N & 15) == 0 && 17 * K <= 2 * RING_SLOT_BYTES &&
                         ((reinterpret_cast<uintptr_t>(st.packed) | reinterpret_cast<uintptr_t>(st.scales)) & 15) == 0;
  unsigned char* my_ring = sm.tile + (size_t)warp * RING_DEPTH * RING_SLOT_BYTES;
  unsigned long long* my_bars = sm.bars + warp * RING_DEPTH;
  uint32_t ring_uses[RING_DEPTH];
  bool ring_pending[RING_DEPTH];
#pragma unroll
  for (int d = 0; d < RING_DEPTH; ++d) { ring_uses[d] = 0u; ring_pending[d] = false; }
  auto ring_issue = [&](int local_tile, int slot) {
    ring_pending[slot] = true;
    if (lane == 0) {
      const int tile = blockIdx.x + local_tile * gridDim.x;
      const uint32_t weight_bytes = 16u * (uint32_t)(K >> 1), scale_bytes = 16u * (uint32_t)(K >> 5);
      unsigned char* dst = my_ring + (size_t)slot * RING_SLOT_BYTES;
      fence_async_proxy();  // earlier reads and writes of this slot come before the copy
      mbar_expect_tx(my_bars + slot, weight_bytes + scale_bytes);
      bulk_load(dst, reinterpret_cast<const unsigned char*>(st.packed) + (size_t)tile * weight_bytes, weight_bytes, my_bars + slot);
      bulk_load(dst + weight_bytes, reinterpret_cast<const unsigned char*>(st.scales) + (size_t)tile * scale_bytes, scale_bytes, my_bars + slot);
    }
  };
  // Bounded wait for a slot's copies; false if they never landed.
  auto ring_wait = [&](int slot) {
    const uint32_t parity = ring_uses[slot] & 1u;
    int spins = 0;
    while (!mbar_try_wait(my_bars + slot, parity))
      if (++spins > POLL_LIMIT) return false;
    ring_uses[slot] += 1u;
    ring_pending[slot] = false;
    return true;
  };
  // Leave nothing in flight into this CTA's shared memory (used on the way out after a failure).
  auto ring_drain = [&]() {
    asm volatile("cp.async.wait_group 0;" ::: "memory");
    bool ok = true;
#pragma unroll
    for (int slot = 0; slot < RING_DEPTH; ++slot)
      if (ring_pending[slot]) ok = ring_wait(slot) && ok;
    if (lane == 0) {
#pragma unroll
      for (int d = 0; d < RING_DEPTH; ++d) sm.ring_uses[warp * RING_DEPTH + d] = ring_uses[d];
    }
    return ok;
  };
  if (ring_mode) {
#pragma unroll
    for (int d = 0; d < RING_DEPTH; ++d) {
      ring_uses[d] = sm.ring_uses[warp * RING_DEPTH + d];
      if (warp + d * STEP_WARPS < rp.my_tiles) ring_issue(warp + d * STEP_WARPS, d);
    }
  } else {
    request_chunk(0);
    request_chunk(1);
  }

  long long gather_row = 0;
  if (st.x_index != nullptr) {
    gather_row = *reinterpret_cast<const volatile long long*>(st.x_index);
    if (gather_row < 0) gather_row = 0;
    if (gather_row >= st.x_rows) gather_row = st.x_rows - 1;
  }

  // ---- the addend of the first round does not depend on the input row either ----
  float addend0 = 0.f;
  uint2 addend0_word = make_uint2(0u, 0u);
  {
    const int tl0 = tid >> 4, r0 = tid & 15;
    const int tiles0 = min(STEP_THREADS / 16, rp.my_tiles);
    const int n0 = (blockIdx.x + tl0 * gridDim.x) * 16 + r0;
    if (tl0 < tiles0 && n0 < N) {
      if (st.addend_mode == AOTO_STAGE_ADDEND_PLAIN) {
        addend0 = ldg_nc_bf16(reinterpret_cast<const bf16*>(st.addend) + n0);
      } else if (st.addend_mode == AOTO_STAGE_ADDEND_GATHER) {
        addend0 = ldg_nc_bf16(reinterpret_cast<const bf16*>(st.addend) + (size_t)gather_row * N + n0);
      } else if (st.addend_mode == AOTO_STAGE_ADDEND_STAMPED) {
        addend0_word = ld_stamped(reinterpret_cast<const unsigned char*>(st.addend) + (size_t)(n0 >> 1) * 8);
      }
    }
  }

  // ---- input row: gather it, or poll its stamped words; raw chunks go to shared memory ----
  const int chunks = K >> 3;
  const uint4* wv = reinterpret_cast<const uint4*>(st.norm_weight);
  if (wv != nullptr) {
    for (int c = tid; c < chunks; c += STEP_THREADS) cp_async_16_cg(sm.nw + c, wv + c);
    asm volatile("cp.async.commit_group;" ::: "memory");
  }
  float ss = 0.f;
  auto keep_chunk = [&](int c, const uint4 v) {
    sm.xs[c] = v;
    if (wv != nullptr) {
      float f[8];
      unpack8(v, f);
#pragma unroll
      for (int j = 0; j < 8; ++j) ss = fmaf(f[j], f[j], ss);
    }
  };
  if (st.flags & AOTO_STAGE_FLAG_X_GATHER) {
    const uint4* xrow = reinterpret_cast<const uint4*>(reinterpret_cast<const bf16*>(st.x) + (size_t)gather_row * K);
    for (int c = tid; c < chunks; c += STEP_THREADS) keep_chunk(c, ldg_nc_u4(xrow + c));
  } else {
    const unsigned char* xw = reinterpret_cast<const unsigned char*>(st.x);
    int polls = 0;
    for (int base = 0; base < chunks; base += POLL_SLICES * STEP_THREADS) {
      bool done[POLL_SLICES];
#pragma unroll
      for (int i = 0; i < POLL_SLICES; ++i) done[i] = (base + tid + i * STEP_THREADS) >= chunks;
      while (true) {
        bool ready = true;
        uint4 a[POLL_SLICES], b[POLL_SLICES];
#pragma unroll
        for (int i = 0; i < POLL_SLICES; ++i) {
          if (done[i]) continue;
          const int c = base + tid + i * STEP_THREADS;
          a[i] = ld_stamped_pair(xw + (size_t)c * 32);
          b[i] = ld_stamped_pair(xw + (size_t)c * 32 + 16);
        }
#pragma unroll
        for (int i = 0; i < POLL_SLICES; ++i) {
          if (done[i]) continue;
          if (a[i].y == epoch && a[i].w == epoch && b[i].y == epoch && b[i].w == epoch) {
            keep_chunk(base + tid + i * STEP_THREADS, make_uint4(a[i].x, a[i].z, b[i].x, b[i].z));
            done[i] = true;
          } else {
            ready = false;
          }
        }
        if (__syncthreads_and(ready)) break;
        if (++polls > POLL_LIMIT) { ring_drain(); give_up(ctl, stage_index); return false; }
      }
    }
  }
  trace_mark(ctl, stage_index, 1);

  // Norm statistic: one shared-memory hop (per-warp partial sums, then every thread adds them
  // in warp order). Stages alternate between the two halves of `red`, so no barrier is needed
  // to protect it from the previous stage's readers.
  float inv = 1.f;
  if (wv != nullptr) {
    ss = warp_sum(ss);
    float* slot = sm.red + (stage_index & 1) * 32;
    if (lane == 0) slot[warp] = ss;
    asm volatile("cp.async.wait_group 0;" ::: "memory");
    __syncthreads();
    float total = 0.f;
#pragma unroll
    for (int w = 0; w < STEP_WARPS; ++w) total += slot[w];
    inv = rsqrtf(total / (float)K + st.rms_norm_eps);
  }
  // Normalise, store in fragment order (in place: a thread rewrites the chunks it wrote), and
  // sum each group of 64 (eight consecutive chunks, i.e. eight consecutive lanes) with three
  // shuffles.
  for (int base = 0; base < chunks; base += STEP_THREADS) {
    const int c = base + tid;
    float chunk_sum = 0.f;
    if (c < chunks) {
      float f[8];
      unpack8(sm.xs[c], f);
      if (wv != nullptr) {
        float w[8];
        unpack8(sm.nw[c], w);
#pragma unroll
        for (int j = 0; j < 8; ++j) f[j] = round_bf16((f[j] * inv) * w[j]);
      }
      uint4 o;
      o.x = pack_bf16x2(f[0], f[4]); o.y = pack_bf16x2(f[1], f[5]);
      o.z = pack_bf16x2(f[2], f[6]); o.w = pack_bf16x2(f[3], f[7]);
      chunk_sum = ((f[0] + f[1]) + (f[2] + f[3])) + ((f[4] + f[5]) + (f[6] + f[7]));
      sm.xs[c] = o;
    }
    chunk_sum += __shfl_xor_sync(0xffffffffu, chunk_sum, 1);
    chunk_sum += __shfl_xor_sync(0xffffffffu, chunk_sum, 2);
    chunk_sum += __shfl_xor_sync(0xffffffffu, chunk_sum, 4);
    if (c < chunks && (lane & 7) == 0) sm.xsum[c >> 3] = 136.f * chunk_sum;
  }
  __syncthreads();
  trace_mark(ctl, stage_index, 2);

  // ---- chunks: multiply a bank, refill it, reduce the tiles that are complete ----
  bf16* out_plain = reinterpret_cast<bf16*>(st.out);
  unsigned char* out_words = reinterpret_cast<unsigned char*>(st.out);
  const BSource bs = b_source(sm.xs, reinterpret_cast<const uint4*>(sm.flag) + 1, lane);
  // the same choice for the chunk loop, as shared addresses: lanes of the other group's column read
  // a 64-byte zero page for every block, the others 64 bytes of the staged row per block
  const bool keeps_x = ((g & 1) == (t >> 1));
  const uint32_t b_address = keeps_x ? smem_address(sm.xs) + (uint32_t)t * 64 : smem_address(reinterpret_cast<const uint4*>(sm.flag) + 1);
  const uint32_t b_step = keeps_x ? 256u : 0u;
  const uint32_t xsum_address = smem_address(sm.xsum);
  const uint32_t part_address = smem_address(sm.part) + (uint32_t)g * 4;
  const uint32_t lane_item_offset = (uint32_t)(g * 64 + t * 16);   // codes of row g; row g + 8 is 512 bytes on
  const uint32_t lane_scale_offset = 1024u + (uint32_t)g * 4 - lane_item_offset;  // relative to the slot address above
  float best_v = -INFINITY;
  int best_i = 0x7fffffff;
  int polls = 0;

  // Epilogue and store of one warp-owned tile: lane (g, t = 0) holds rows g and g + 8.
  auto finish_tile = [&](int tile, float gate_lo, float gate_hi, float up_lo, float up_hi) {
    uint32_t bits[2];
#pragma unroll
    for (int half = 0; half < 2; ++half) {
      const int n = tile * 16 + g + half * 8;
      float y = st.alpha * (half ? gate_hi : gate_lo);
      if (st.addend_mode == AOTO_STAGE_ADDEND_PLAIN && n < N)
        y = fmaf(st.beta, __bfloat162float(reinterpret_cast<const bf16*>(st.addend)[n]), y);
      if (st.epilogue == AOTO_EPILOGUE_SILU_MUL_PAIRED) {
        const float gate = round_bf16(y);
        y = (st.alpha * (half ? up_hi : up_lo)) * (gate / (1.f + expf(-gate)));
      }
      bits[half] = float_to_bf16_bits(y);
    }
    const uint32_t next_lo = __shfl_down_sync(0xffffffffu, bits[0], 4);
    const uint32_t next_hi = __shfl_down_sync(0xffffffffu, bits[1], 4);
    if (t == 0) {
#pragma unroll
      for (int half = 0; half < 2; ++half) {
        const int n = tile * 16 + g + half * 8;
        if (n >= N) continue;
        if (st.flags & AOTO_STAGE_FLAG_OUT_PLAIN) {
          out_plain[n] = __ushort_as_bfloat16((unsigned short)bits[half]);
        } else if ((g & 1) == 0) {
          st_stamped(out_words + (size_t)(n >> 1) * 8, bits[half] | ((half ? next_hi : next_lo) << 16), epoch);
        }
        if (st.flags & AOTO_STAGE_FLAG_ARGMAX) {
          float v = __uint_as_float(bits[half] << 16);
          if (v != v) v = INFINITY;
          if (v > best_v || (v == best_v && n < best_i)) { best_v = v; best_i = n; }
        }
      }
    }
  };

  if (ring_mode) {
    const int row_u4 = K >> 5;    // 16-byte words of a packed row
    const int scale_row = K >> 5;  // bytes of a row of scales
    bool ring_ok = true;
    bool marked = false;
    int use = 0;
    for (int local_tile = warp; local_tile < rp.my_tiles; local_tile += STEP_WARPS, ++use) {
      const int slot = use % RING_DEPTH;
      if (!ring_wait(slot)) { ring_ok = false; break; }
      // shared addresses of this lane's codes (rows g and g + 8) and scale pairs in the slot
      const uint32_t base = smem_address(my_ring) + (uint32_t)slot * RING_SLOT_BYTES;
      uint32_t codes = base + (uint32_t)(g * row_u4 + t) * 16;
      uint32_t pairs = base + 16u * (uint32_t)(K >> 1) + (uint32_t)(g * scale_row);
      const uint32_t codes_hi = 8u * (uint32_t)row_u4 * 16, pairs_hi = 8u * (uint32_t)scale_row;
      uint32_t b_at = b_address, x_at = xsum_address;
      float a_lo = 0.f, a_hi = 0.f;
#pragma unroll 2
      for (int kb = 0; kb < rp.nblocks; ++kb) {
        WeightItem it;
        it.lo = lds128(codes);
        it.hi = lds128(codes + codes_hi);
        it.slo = lds32(pairs);
        it.shi = lds32(pairs + pairs_hi);
        float lo, hi;
        mma_block_shared(it, b_at, x_at, lo, hi);
        a_lo += lo;
        a_hi += hi;
        codes += 64; pairs += 4; b_at += b_step; x_at += 8;
      }
      if (!marked) { trace_mark(ctl, stage_index, 3); marked = true; }
      __syncwarp();  // every lane is done with the slot before it is refilled
      if (local_tile + RING_DEPTH * STEP_WARPS < rp.my_tiles) ring_issue(local_tile + RING_DEPTH * STEP_WARPS, slot);
      finish_tile(blockIdx.x + local_tile * gridDim.x, a_lo, a_hi, 0.f, 0.f);
    }
    if (!ring_ok) ring_drain();
    if (lane == 0) {
#pragma unroll
      for (int d = 0; d < RING_DEPTH; ++d) sm.ring_uses[warp * RING_DEPTH + d] = ring_uses[d];
    }
    if (__syncthreads_or(!ring_ok)) { give_up(ctl, stage_index); return false; }
  }

  int finished = 0;  // local tiles whose epilogue has run
  for (int chunk = 0; chunk < (ring_mode ? 0 : chunks_total); ++chunk) {
    asm volatile("cp.async.wait_group 1;" ::: "memory");  // everything but the newest group has landed
    __syncwarp();
    {
      // this warp's blocks of the chunk are idx0, idx0 + 8, ...: position in the tile and in the
      // ring of partial sums advance by eight per block, no division inside the loop
      const int idx0 = chunk * CHUNK_ITEMS + warp;
      const int count = idx0 < total_items ? min(BANK_SLOTS, (total_items - idx0 + STEP_WARPS - 1) / STEP_WARPS) : 0;
      int j = idx0 - small_div(idx0, rp.inv_per_tile) * rp.per_tile;  // block within its tile
      int pos = idx0 % PART_ITEMS;
      uint32_t slot = smem_address(my_slots) + (uint32_t)((chunk & 1) * BANK_SLOTS * ITEM_BYTES) + lane_item_offset;
      for (int i = 0; i < count; ++i) {
        const int kb = j >= rp.nblocks ? j - rp.nblocks : j;
        WeightItem it;
        it.lo = lds128(slot);
        it.hi = lds128(slot + 512);
        it.slo = lds32(slot + lane_scale_offset);
        it.shi = lds32(slot + lane_scale_offset + 32);
        float lo, hi;
        mma_block_shared(it, b_address + (uint32_t)kb * b_step, xsum_address + (uint32_t)kb * 8, lo, hi);
        if (t == 0) {
          sts32f(part_address + (uint32_t)pos * 64, lo);
          sts32f(part_address + (uint32_t)pos * 64 + 32, hi);
        }
        slot += ITEM_BYTES;
        j += STEP_WARPS;
        while (j >= rp.per_tile) j -= rp.per_tile;
        pos += STEP_WARPS;
        if (pos >= PART_ITEMS) pos -= PART_ITEMS;
      }
    }
    __syncwarp();                // every lane has read the bank
    request_chunk(chunk + 2);    // refill it
    if (chunk == 0) trace_mark(ctl, stage_index, 3);
    // tiles whose last block lies in this chunk are complete after the barrier
    const int done_items = min(total_items, (chunk + 1) * CHUNK_ITEMS);
    const int complete = small_div(done_items, rp.inv_per_tile);
    if (complete == finished) continue;  // uniform: a long tile is still being summed
    __syncthreads();
    if (chunk == 0) trace_mark(ctl, stage_index, 4);
    for (int first = finished; first < complete; first += STEP_THREADS / 16) {
      // reduce over k blocks in a fixed order, epilogue, store
      const int tl = first + (tid >> 4), r = tid & 15;
      const int tile = blockIdx.x + tl * gridDim.x;
      const int n = tile * 16 + r;
      const bool valid = tl < complete && n < N;
      const bool prefetched = tl == (tid >> 4);  // the addend requested before the input was polled
      float y = 0.f;
      if (valid) {
        int base = (tl * rp.per_tile) % PART_ITEMS;
        const uint32_t row_address = smem_address(sm.part) + (uint32_t)r * 4;
        // fixed order: four interleaved partial sums over the k blocks (in registers), then their sum
        auto next = [&]() {
          const float v = __uint_as_float(lds32(row_address + (uint32_t)base * 64));
          if (++base == PART_ITEMS) base = 0;
          return v;
        };
        auto sum_blocks = [&]() {
          float s0 = 0.f, s1 = 0.f, s2 = 0.f, s3 = 0.f;
          int kb = 0;
          for (; kb + 4 <= rp.nblocks; kb += 4) {
            s0 += next(); s1 += next(); s2 += next(); s3 += next();
          }
          for (; kb < rp.nblocks; ++kb) s0 += next();
          return (s0 + s1) + (s2 + s3);
        };
        const float total = sum_blocks();
        const float total2 = rp.mats == 2 ? sum_blocks() : 0.f;
        y = st.alpha * total;
        if (st.addend_mode == AOTO_STAGE_ADDEND_PLAIN) {
          const float a = prefetched ? addend0 : __bfloat162float(reinterpret_cast<const bf16*>(st.addend)[n]);
          y = fmaf(st.beta, a, y);
        } else if (st.addend_mode == AOTO_STAGE_ADDEND_GATHER) {
          const float a = prefetched
                              ? addend0
                              : __bfloat162float(reinterpret_cast<const bf16*>(st.addend)[(size_t)gather_row * N + n]);
          y = fmaf(st.beta, a, y);
        } else if (st.addend_mode == AOTO_STAGE_ADDEND_STAMPED) {
          const unsigned char* words = reinterpret_cast<const unsigned char*>(st.addend) + (size_t)(n >> 1) * 8;
          uint2 w = prefetched ? addend0_word : ld_stamped(words);
          while (w.y != epoch && ++polls <= POLL_LIMIT) w = ld_stamped(words);
          y = fmaf(st.beta, (n & 1) ? bf16x2_hi(w.x) : bf16x2_lo(w.x), y);
        }
        if (st.epilogue == AOTO_EPILOGUE_SILU_MUL_PAIRED) {
          const float gate = round_bf16(y);
          y = (st.alpha * total2) * (gate / (1.f + expf(-gate)));
        }
      }
      const uint32_t bits = float_to_bf16_bits(y);
      const uint32_t neighbour = __shfl_down_sync(0xffffffffu, bits, 1);
      if (valid) {
        if (st.flags & AOTO_STAGE_FLAG_OUT_PLAIN) {
          out_plain[n] = __ushort_as_bfloat16((unsigned short)bits);
        } else if ((r & 1) == 0) {
          st_stamped(out_words + (size_t)(n >> 1) * 8, bits | (neighbour << 16), epoch);
        }
        if (st.flags & AOTO_STAGE_FLAG_ARGMAX) {
          float v = __uint_as_float(bits << 16);
          if (v != v) v = INFINITY;
          if (v > best_v || (v == best_v && n < best_i)) { best_v = v; best_i = n; }
        }
      }
    }
    finished = complete;
    if (chunk == 0) trace_mark(ctl, stage_index, 5);
  }
  asm volatile("cp.async.wait_group 0;" ::: "memory");
  if (__syncthreads_or(polls > POLL_LIMIT)) { give_up(ctl, stage_index); return false; }
  trace_mark(ctl, stage_index, 6);

  if (st.flags & AOTO_STAGE_FLAG_ARGMAX) {
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
      unsigned char* payload = reinterpret_cast<unsigned char*>(ctl.scratch) + SCRATCH_HEADER_BYTES;
      st_stamped(payload + (size_t)blockIdx.x * 16, __float_as_uint(best_v), epoch);
      st_stamped(payload + (size_t)blockIdx.x * 16 + 8, (uint32_t)best_i, epoch);
    }
  }
  trace_mark(ctl, stage_index, 7);
  return true;
}

// ---------------------------------------------------------------------------
// attention stage: rotate q and k, write the shifted window, attend
// ---------------------------------------------------------------------------
__device__ __forceinline__ float rotate_smem(const float* head, const bf16* cos_row, const bf16* sin_row, int d, int D) {
  const int half = D >> 1;
  const float v = head[d];
  const float partner = d < half ? -head[d + half] : head[d - half];
  return round_bf16(round_bf16(v * __bfloat162float(cos_row[d])) +
                    round_bf16(partner * __bfloat162float(sin_row[d])));
}

// Bytes of the tile region the whole-window form of the attention stage needs.
__host__ __device__ inline size_t window_attention_bytes(int capacity, int head_dim) {
  const size_t tiles = (size_t)2 * capacity * (head_dim * 2 + 16);
  const size_t floats = (size_t)3 * head_dim + head_dim + 2 * (size_t)capacity + (size_t)STEP_WARPS * 2 * head_dim + 64;
  return tiles + floats * 4 + 64;
}
constexpr size_t STEP_TILE_REGION_BYTES = (size_t)RING_SLOTS * RING_SLOT_BYTES;

// Attention stage, whole-window form: one CTA per QUERY head holds the whole window of its kv
// head in shared memory, so a head is finished where it started - no split, no merge through
// scratch, no second exchange. The CTAs of a group read the same window (from L2) and share the
// write of the shifted window into the next cache. Used when the window fits the tile region.
__device__ bool stage_attention_window(const aoto_step_stage& st, const StepSmem& sm, const StepControl& ctl, int stage_index) {
  const int D = st.head_dim, C = st.capacity, KVH = st.kv_heads, QH = st.query_heads;
  const int G = QH / KVH;
  trace_mark(ctl, stage_index, 0);
  if ((int)blockIdx.x >= QH) {
    trace_mark(ctl, stage_index, 1);
    trace_mark(ctl, stage_index, 6);
    trace_mark(ctl, stage_index, 7);
    return true;
  }
  const uint32_t epoch = ctl.epoch;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int head = blockIdx.x, kvh = head / G, member = head - kvh * G;
  const int row_bytes = D * 2 + 16, chunks = D >> 3, pairs = D >> 1;
  unsigned char* kt = sm.tile;
  unsigned char* vt = kt + (size_t)C * row_bytes;
  float* rowv = reinterpret_cast<float*>(vt + (size_t)C * row_bytes);  // raw q head, k, v of the step: 3*D
  float* qs = rowv + 3 * D;                                            // rotated, scaled query: D
  float* sc = qs + D;                                                  // scores / probabilities: C
  float* madd = sc + C;                                                // additive mask: C
  float* pv = madd + C;                                                // partial P.V: slices * D
  float* red = pv + STEP_WARPS * 2 * D;                                // 64

  int valid_length = 0;
  long long pos;
  if (st.flags & AOTO_STAGE_FLAG_WINDOW) {
    valid_length = *reinterpret_cast<const volatile int*>(st.counters);
    pos = valid_length - 1;
  } else {
    pos = *reinterpret_cast<const volatile long long*>(st.position);
  }
  if (pos < 0) pos = 0;
  if (pos >= st.table_rows) pos = st.table_rows - 1;
  const bf16* cos_row = reinterpret_cast<const bf16*>(st.cos_table) + (size_t)pos * D;
  const bf16* sin_row = reinterpret_cast<const bf16*>(st.sin_table) + (size_t)pos * D;
  const bf16* kin = reinterpret_cast<const bf16*>(st.cache_in) + (size_t)kvh * C * D;
  const bf16* vin = reinterpret_cast<const bf16*>(st.cache_in) + ((size_t)KVH + kvh) * C * D;
  bf16* kout = reinterpret_cast<bf16*>(st.cache_out) + (size_t)kvh * C * D;
  bf16* vout = reinterpret_cast<bf16*>(st.cache_out) + ((size_t)KVH + kvh) * C * D;

  // slot j of the new window is slot j + 1 of the old one; the last slot is this step's pair
  for (int c = tid; c < (C - 1) * chunks; c += STEP_THREADS) {
    const int r = c / chunks, j = c - r * chunks;
    cp_async_16_cg(kt + (size_t)r * row_bytes + j * 16, kin + (size_t)(r + 1) * D + j * 8);
    cp_async_16_cg(vt + (size_t)r * row_bytes + j * 16, vin + (size_t)(r + 1) * D + j * 8);
  }
  asm volatile("cp.async.commit_group;" ::: "memory");
  for (int i = tid; i < C; i += STEP_THREADS) {
    const bool attend = (st.flags & AOTO_STAGE_FLAG_WINDOW) ? (i >= C - valid_length) : (st.mask[i] != 0);
    madd[i] = attend ? 0.f : -INFINITY;
  }

  // this head's query and its kv head's key and value of the step: poll the stamped projection row
  {
    const unsigned char* row_words = reinterpret_cast<const unsigned char*>(st.row);
    const int total_words = 3 * pairs;
    int polls = 0;
    bool pending = tid < total_words;
    while (true) {
      bool ready = true;
      if (pending) {
        int element;
        if (tid < pairs) element = st.query_start + head * D + 2 * tid;
        else if (tid < 2 * pairs) element = st.key_start + kvh * D + 2 * (tid - pairs);
        else element = st.value_start + kvh * D + 2 * (tid - 2 * pairs);
        const uint2 v = ld_stamped(row_words + (size_t)(element >> 1) * 8);
        if (v.y == epoch) {
          rowv[2 * tid] = bf16x2_lo(v.x);
          rowv[2 * tid + 1] = bf16x2_hi(v.x);
          pending = false;
        } else {
          ready = false;
        }
      }
      if (__syncthreads_and(ready)) break;
      if (++polls > POLL_LIMIT) {
        asm volatile("cp.async.wait_group 0;" ::: "memory");
        give_up(ctl, stage_index);
        return false;
      }
    }
  }
  trace_mark(ctl, stage_index, 1);

  for (int d = tid; d < D; d += STEP_THREADS) {
    qs[d] = rotate_smem(rowv, cos_row, sin_row, d, D) * st.scale;
    reinterpret_cast<bf16*>(kt + (size_t)(C - 1) * row_bytes)[d] =
        __float2bfloat16_rn(rotate_smem(rowv + D, cos_row, sin_row, d, D));
    reinterpret_cast<bf16*>(vt + (size_t)(C - 1) * row_bytes)[d] = __float2bfloat16_rn(rowv[2 * D + d]);
  }
  asm volatile("cp.async.wait_group 0;" ::: "memory");
  __syncthreads();

  // the members of a group share the write of the shifted window into the next cache
  {
    const int share = (C + G - 1) / G;
    const int first = member * share, last = min(C, first + share);
    for (int c = tid; c < (last - first) * chunks; c += STEP_THREADS) {
      const int r = first + c / chunks, j = c % chunks;
      const size_t dst = (size_t)r * D + j * 8;
      *reinterpret_cast<uint4*>(kout + dst) = *reinterpret_cast<const uint4*>(kt + (size_t)r * row_bytes + j * 16);
      *reinterpret_cast<uint4*>(vout + dst) = *reinterpret_cast<const uint4*>(vt + (size_t)r * row_bytes + j * 16);
    }
  }

  // scores: thread <-> key
  float local_max = -INFINITY;
  for (int key = tid; key < C; key += STEP_THREADS) {
    float s = -INFINITY;
    if (madd[key] != -INFINITY) {
      const uint4* krow = reinterpret_cast<const uint4*>(kt + (size_t)key * row_bytes);
      const float4* q4 = reinterpret_cast<const float4*>(qs);
      float d0 = 0.f, d1 = 0.f, d2 = 0.f, d3 = 0.f;
      for (int j = 0; j < chunks; ++j) {
        const uint4 kk = krow[j];
        const float4 qa = q4[2 * j], qb = q4[2 * j + 1];
        d0 = fmaf(bf16x2_lo(kk.x), qa.x, d0); d1 = fmaf(bf16x2_hi(kk.x), qa.y, d1);
        d2 = fmaf(bf16x2_lo(kk.y), qa.z, d2); d3 = fmaf(bf16x2_hi(kk.y), qa.w, d3);
        d0 = fmaf(bf16x2_lo(kk.z), qb.x, d0); d1 = fmaf(bf16x2_hi(kk.z), qb.y, d1);
        d2 = fmaf(bf16x2_lo(kk.w), qb.z, d2); d3 = fmaf(bf16x2_hi(kk.w), qb.w, d3);
      }
      s = (d0 + d1) + (d2 + d3);
    }
    sc[key] = s;
    local_max = fmaxf(local_max, s);
  }
  local_max = warp_max(local_max);
  if (lane == 0) red[warp] = local_max;
  __syncthreads();
  float m = red[0];
#pragma unroll
  for (int w = 1; w < STEP_WARPS; ++w) m = fmaxf(m, red[w]);
  const float m_safe = (m == -INFINITY) ? 0.f : m;
  float local_sum = 0.f;
  for (int key = tid; key < C; key += STEP_THREADS) {
    const float s = sc[key];
    const float e = (s == -INFINITY) ? 0.f : expf(s - m_safe);
    sc[key] = e;
    local_sum += e;
  }
  local_sum = warp_sum(local_sum);
  if (lane == 0) red[32 + warp] = local_sum;
  __syncthreads();
  float l = 0.f;
#pragma unroll
  for (int w = 0; w < STEP_WARPS; ++w) l += red[32 + w];

  // P.V: thread <-> (key slice, dim pair); the slices are summed in a fixed order afterwards
  const int slices = STEP_THREADS / pairs;
  const int per_slice = (C + slices - 1) / slices;
  {
    const int slice = tid / pairs, dp = tid - slice * pairs;
    float a0 = 0.f, a1 = 0.f;
    if (slice < slices) {
      const int k_begin = slice * per_slice, k_end = min(C, k_begin + per_slice);
      for (int key = k_begin; key < k_end; ++key) {
        const float w = sc[key];
        if (w != 0.f) {
          const uint32_t v = *reinterpret_cast<const uint32_t*>(vt + (size_t)key * row_bytes + dp * 4);
          a0 = fmaf(w, bf16x2_lo(v), a0);
          a1 = fmaf(w, bf16x2_hi(v), a1);
        }
      }
      pv[(slice * pairs + dp) * 2] = a0;
      pv[(slice * pairs + dp) * 2 + 1] = a1;
    }
  }
  __syncthreads();
  if (tid < pairs) {
    float a0 = 0.f, a1 = 0.f;
    for (int slice = 0; slice < slices; ++slice) {
      a0 += pv[(slice * pairs + tid) * 2];
      a1 += pv[(slice * pairs + tid) * 2 + 1];
    }
    const float inv = l > 0.f ? 1.f / l : 0.f;
    unsigned char* out_words = reinterpret_cast<unsigned char*>(st.attn_out);
    st_stamped(out_words + ((size_t)head * pairs + tid) * 8, pack_bf16x2(a0 * inv, a1 * inv), epoch);
  }
  __syncthreads();
  trace_mark(ctl, stage_index, 6);
  trace_mark(ctl, stage_index, 7);
  return true;
}

__device__ bool stage_attention(const aoto_step_stage& shared_stage, const StepSmem& sm, const StepControl& ctl, int stage_index) {
  const aoto_step_stage st = shared_stage;
  const int D = st.head_dim, C = st.capacity, KVH = st.kv_heads, QH = st.query_heads;
  if (window_attention_bytes(C, D) <= STEP_TILE_REGION_BYTES && QH <= (int)gridDim.x &&
      STEP_THREADS >= 3 * (D >> 1) && STEP_THREADS % (D >> 1) == 0)
    return stage_attention_window(st, sm, ctl, stage_index);
  const int G = QH / KVH;
  const int TK = ATT_TILE;
  const int splits = (C + TK - 1) / TK;
  const int total_items = KVH * splits;
  trace_mark(ctl, stage_index, 0);
  if ((int)blockIdx.x >= total_items) {
    trace_mark(ctl, stage_index, 1);
    trace_mark(ctl, stage_index, 6);
    trace_mark(ctl, stage_index, 7);
    return true;
  }
  const uint32_t epoch = ctl.epoch;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int row_bytes = D * 2 + 16;
  unsigned char* kt = sm.tile;
  unsigned char* vt = kt + (size_t)TK * (128 * 2 + 16);
  float* rowv = reinterpret_cast<float*>(vt + (size_t)TK * (128 * 2 + 16));  // (G+2)*D raw q heads, k, v
  float* qs = rowv + (MAX_GROUP + 2) * 128;                                  // G*D rotated, scaled
  float* sc = qs + MAX_GROUP * 128;                                          // G*TK
  float* stat = sc + MAX_GROUP * TK;                                         // G*2
  float* madd = stat + MAX_GROUP * 2;                                        // TK
  float* pv = madd + TK;                                                     // 2*G*D halves of P.V

  int valid_length = 0;
  long long pos;
  if (st.flags & AOTO_STAGE_FLAG_WINDOW) {
    valid_length = *reinterpret_cast<const volatile int*>(st.counters);
    pos = valid_length - 1;
  } else {
    pos = *reinterpret_cast<const volatile long long*>(st.position);
  }
  if (pos < 0) pos = 0;
  if (pos >= st.table_rows) pos = st.table_rows - 1;
  const bf16* cos_row = reinterpret_cast<const bf16*>(st.cos_table) + (size_t)pos * D;
  const bf16* sin_row = reinterpret_cast<const bf16*>(st.sin_table) + (size_t)pos * D;
  const unsigned char* row_words = reinterpret_cast<const unsigned char*>(st.row);
  unsigned char* out_words = reinterpret_cast<unsigned char*>(st.attn_out);
  float* partials = reinterpret_cast<float*>(reinterpret_cast<unsigned char*>(ctl.scratch) + SCRATCH_HEADER_BYTES + 16 * 1024);
  int* counters = reinterpret_cast<int*>(ctl.scratch);
  bool first_item = true;

  for (int item = blockIdx.x; item < total_items; item += gridDim.x) {
    const int kvh = item / splits, split = item - kvh * splits;
    const int k0 = split * TK;
    const int nkeys = min(TK, C - k0);
    const int chunks = D >> 3;
    const bf16* kin = reinterpret_cast<const bf16*>(st.cache_in) + (size_t)kvh * C * D;
    const bf16* vin = reinterpret_cast<const bf16*>(st.cache_in) + ((size_t)KVH + kvh) * C * D;
    bf16* kout = reinterpret_cast<bf16*>(st.cache_out) + (size_t)kvh * C * D;
    bf16* vout = reinterpret_cast<bf16*>(st.cache_out) + ((size_t)KVH + kvh) * C * D;

    // window slot j of the new cache is slot j + 1 of the old one; the last slot is the new pair
    for (int c = tid; c < TK * chunks; c += STEP_THREADS) {
      const int r = c / chunks, j = c - r * chunks;
      const int slot = k0 + r;
      if (r < nkeys && slot < C - 1) {
        cp_async_16_cg(kt + (size_t)r * row_bytes + j * 16, kin + (size_t)(slot + 1) * D + j * 8);
        cp_async_16_cg(vt + (size_t)r * row_bytes + j * 16, vin + (size_t)(slot + 1) * D + j * 8);
      } else if (r >= nkeys) {
        *reinterpret_cast<uint4*>(kt + (size_t)r * row_bytes + j * 16) = make_uint4(0u, 0u, 0u, 0u);
        *reinterpret_cast<uint4*>(vt + (size_t)r * row_bytes + j * 16) = make_uint4(0u, 0u, 0u, 0u);
      }
    }
    asm volatile("cp.async.commit_group;" ::: "memory");
    for (int i = tid; i < TK; i += STEP_THREADS) {
      bool attend = false;
      if (i < nkeys) {
        attend = (st.flags & AOTO_STAGE_FLAG_WINDOW) ? (k0 + i >= C - valid_length) : (st.mask[k0 + i] != 0);
      }
      madd[i] = attend ? 0.f : -INFINITY;
    }

    // the step's q heads of this group, k and v: poll the stamped projection row
    {
      const int words_q = (G * D) >> 1, words_kv = D >> 1;
      const int total_words = words_q + 2 * words_kv;
      int polls = 0;
      int w = tid;
      bool pending = w < total_words;
      while (true) {
        bool ready = true;
        if (pending) {
          int element;  // first element of the word in the projection row
          if (w < words_q) element = st.query_start + kvh * G * D + 2 * w;
          else if (w < words_q + words_kv) element = st.key_start + kvh * D + 2 * (w - words_q);
          else element = st.value_start + kvh * D + 2 * (w - words_q - words_kv);
          const uint2 v = ld_stamped(row_words + (size_t)(element >> 1) * 8);
          if (v.y == epoch) {
            rowv[2 * w] = bf16x2_lo(v.x);
            rowv[2 * w + 1] = bf16x2_hi(v.x);
            w += STEP_THREADS;
            pending = w < total_words;
            ready = !pending;
          } else {
            ready = false;
          }
        }
        if (__syncthreads_and(ready)) break;
        if (++polls > POLL_LIMIT) { give_up(ctl, stage_index); return false; }
      }
    }
    if (first_item) trace_mark(ctl, stage_index, 1);

    for (int i = tid; i < G * D; i += STEP_THREADS) {
      const int h = i / D, d = i - h * D;
      qs[i] = rotate_smem(rowv + h * D, cos_row, sin_row, d, D) * st.scale;
    }
    asm volatile("cp.async.wait_group 0;" ::: "memory");
    if (k0 + nkeys == C) {  // this item owns the last slot: rotated key and value of the step
      const int r = C - 1 - k0;
      for (int d = tid; d < D; d += STEP_THREADS) {
        reinterpret_cast<bf16*>(kt + (size_t)r * row_bytes)[d] =
            __float2bfloat16_rn(rotate_smem(rowv + G * D, cos_row, sin_row, d, D));
        reinterpret_cast<bf16*>(vt + (size_t)r * row_bytes)[d] = __float2bfloat16_rn(rowv[(G + 1) * D + d]);
      }
    }
    __syncthreads();

    // the shifted window goes out to the next cache
    for (int c = tid; c < nkeys * chunks; c += STEP_THREADS) {
      const int r = c / chunks, j = c - r * chunks;
      const size_t dst = (size_t)(k0 + r) * D + j * 8;
      *reinterpret_cast<uint4*>(kout + dst) = *reinterpret_cast<const uint4*>(kt + (size_t)r * row_bytes + j * 16);
      *reinterpret_cast<uint4*>(vout + dst) = *reinterpret_cast<const uint4*>(vt + (size_t)r * row_bytes + j * 16);
    }

    // scores: thread <-> (head, key); four partial sums for instruction-level parallelism
    for (int it = tid; it < G * TK; it += STEP_THREADS) {
      const int h = it / TK, key = it - h * TK;
      float s = -INFINITY;
      if (madd[key] != -INFINITY) {
        const uint4* krow = reinterpret_cast<const uint4*>(kt + (size_t)key * row_bytes);
        const float4* qh = reinterpret_cast<const float4*>(qs + h * D);
        float d0 = 0.f, d1 = 0.f, d2 = 0.f, d3 = 0.f;
        for (int j = 0; j < chunks; ++j) {
          const uint4 kk = krow[j];
          const float4 qa = qh[2 * j], qb = qh[2 * j + 1];
          d0 = fmaf(bf16x2_lo(kk.x), qa.x, d0); d1 = fmaf(bf16x2_hi(kk.x), qa.y, d1);
          d2 = fmaf(bf16x2_lo(kk.y), qa.z, d2); d3 = fmaf(bf16x2_hi(kk.y), qa.w, d3);
          d0 = fmaf(bf16x2_lo(kk.z), qb.x, d0); d1 = fmaf(bf16x2_hi(kk.z), qb.y, d1);
          d2 = fmaf(bf16x2_lo(kk.w), qb.z, d2); d3 = fmaf(bf16x2_hi(kk.w), qb.w, d3);
        }
        s = (d0 + d1) + (d2 + d3);
      }
      sc[it] = s;
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
    // P.V: thread <-> (key half, head, dim pair); unrolled, no branches
    const int pairs = D >> 1;
    const int per_half = G * pairs;
    for (int it = tid; it < 2 * per_half; it += STEP_THREADS) {
      const int half = it / per_half, rest = it - half * per_half;
      const int h = rest / pairs, dp = rest - h * pairs;
      const float* w = sc + h * TK + half * (TK / 2);
      const unsigned char* vbase = vt + (size_t)(half * (TK / 2)) * row_bytes + dp * 4;
      float a0 = 0.f, a1 = 0.f, b0 = 0.f, b1 = 0.f;
#pragma unroll 4
      for (int key = 0; key < TK / 2; key += 2) {
        const float w0 = w[key], w1 = w[key + 1];
        const uint32_t v0 = *reinterpret_cast<const uint32_t*>(vbase + (size_t)key * row_bytes);
        const uint32_t v1 = *reinterpret_cast<const uint32_t*>(vbase + (size_t)(key + 1) * row_bytes);
        a0 = fmaf(w0, w0 != 0.f ? bf16x2_lo(v0) : 0.f, a0);
        a1 = fmaf(w0, w0 != 0.f ? bf16x2_hi(v0) : 0.f, a1);
        b0 = fmaf(w1, w1 != 0.f ? bf16x2_lo(v1) : 0.f, b0);
        b1 = fmaf(w1, w1 != 0.f ? bf16x2_hi(v1) : 0.f, b1);
      }
      pv[(half * per_half + rest) * 2] = a0 + b0;
      pv[(half * per_half + rest) * 2 + 1] = a1 + b1;
    }
    __syncthreads();
    for (int rest = tid; rest < per_half; rest += STEP_THREADS) {
      const int h = rest / pairs, dp = rest - h * pairs;
      const float a0 = pv[rest * 2] + pv[(per_half + rest) * 2];
      const float a1 = pv[rest * 2 + 1] + pv[(per_half + rest) * 2 + 1];
      const int head = kvh * G + h;
      if (splits == 1) {
        const float l = stat[2 * h + 1];
        const float inv = l > 0.f ? 1.f / l : 0.f;
        st_stamped(out_words + ((size_t)head * pairs + dp) * 8, pack_bf16x2(a0 * inv, a1 * inv), epoch);
      } else {
        float* dst = partials + ((size_t)head * splits + split) * (D + 2);
        dst[2 + dp * 2] = a0;
        dst[3 + dp * 2] = a1;
        if (dp == 0) { dst[0] = stat[2 * h]; dst[1] = stat[2 * h + 1]; }
      }
    }
    if (splits > 1) {
      __threadfence();
      __syncthreads();
      if (tid == 0) {
        const int arrived = atomicAdd(counters + kvh, 1);
        const int last = arrived == splits - 1;
        if (last) counters[kvh] = 0;
        *sm.flag = last;
      }
      __syncthreads();
      if (*sm.flag) {
        __threadfence();
        for (int rest = tid; rest < per_half; rest += STEP_THREADS) {
          const int h = rest / pairs, dp = rest - h * pairs;
          const int head = kvh * G + h;
          const float* base = partials + (size_t)head * splits * (D + 2);
          float m = -INFINITY;
          for (int s2 = 0; s2 < splits; ++s2) m = fmaxf(m, __ldcg(base + (size_t)s2 * (D + 2)));
          float acc0 = 0.f, acc1 = 0.f, l = 0.f;
          if (m != -INFINITY) {
            for (int s2 = 0; s2 < splits; ++s2) {
              const float* part = base + (size_t)s2 * (D + 2);
              const float pm = __ldcg(part);
              const float wgt = (pm == -INFINITY) ? 0.f : expf(pm - m);
              acc0 = fmaf(wgt, __ldcg(part + 2 + dp * 2), acc0);
              acc1 = fmaf(wgt, __ldcg(part + 3 + dp * 2), acc1);
              l = fmaf(wgt, __ldcg(part + 1), l);
            }
          }
          const float inv = l > 0.f ? 1.f / l : 0.f;
          st_stamped(out_words + ((size_t)head * pairs + dp) * 8, pack_bf16x2(acc0 * inv, acc1 * inv), epoch);
        }
      }
    }
    __syncthreads();
    first_item = false;
  }
  trace_mark(ctl, stage_index, 6);
  trace_mark(ctl, stage_index, 7);
  return true;
}

// ---------------------------------------------------------------------------
// pick stage: CTA 0 polls the per-CTA maxima the LM-head stage left
// ---------------------------------------------------------------------------
__device__ bool stage_pick(const aoto_step_stage& st, const StepControl& ctl, int stage_index) {
  trace_mark(ctl, stage_index, 0);
  if (blockIdx.x != 0) return true;
  const unsigned char* payload = reinterpret_cast<const unsigned char*>(ctl.scratch) + SCRATCH_HEADER_BYTES;
  if (threadIdx.x < 32) {
    float bv = -INFINITY;
    int bi = 0x7fffffff;
    int polls = 0;
    bool failed = false;
    for (int c = threadIdx.x; c < (int)gridDim.x && !failed; c += 32) {
      uint2 a = ld_stamped(payload + (size_t)c * 16), b = ld_stamped(payload + (size_t)c * 16 + 8);
      while (a.y != ctl.epoch || b.y != ctl.epoch) {
        if (++polls > POLL_LIMIT) { failed = true; break; }
        a = ld_stamped(payload + (size_t)c * 16);
        b = ld_stamped(payload + (size_t)c * 16 + 8);
      }
      const float v = __uint_as_float(a.x);
      const int i = (int)b.x;
      if (v > bv || (v == bv && i < bi)) { bv = v; bi = i; }
    }
    failed = __any_sync(0xffffffffu, failed);
#pragma unroll
    for (int offset = 16; offset > 0; offset >>= 1) {
      const float ov = __shfl_xor_sync(0xffffffffu, bv, offset);
      const int oi = __shfl_xor_sync(0xffffffffu, bi, offset);
      if (ov > bv || (ov == bv && oi < bi)) { bv = ov; bi = oi; }
    }
    trace_mark(ctl, stage_index, 1);
    if (threadIdx.x == 0 && !failed) {
      st.token[0] = (long long)bi;
      if (st.counters != nullptr) {
        const int step = st.counters[1];
        if (st.generated != nullptr && step < st.generated_capacity) st.generated[step] = (long long)bi;
        st.counters[0] += 1;
        st.counters[1] = step + 1;
      }
    }
    if (threadIdx.x == 0 && failed) atomicCAS(ctl.status, 0, stage_index + 1);
  }
  trace_mark(ctl, stage_index, 6);
  trace_mark(ctl, stage_index, 7);
  return true;
}

__global__ void __launch_bounds__(STEP_THREADS, 1)
decode_step_kernel(const aoto_step_stage* __restrict__ stages, int stage_count, StepControl ctl) {
  extern __shared__ uint4 smem_raw[];
  __shared__ aoto_step_stage stage_buffer[2];
  StepSmem sm;
  sm.xs = smem_raw;
  sm.nw = sm.xs + STEP_MAX_K / 8;
  sm.xsum = reinterpret_cast<float*>(sm.nw + STEP_MAX_K / 8);
  sm.part = sm.xsum + STEP_MAX_K / 64;
  sm.red = sm.part + STEP_MAX_ITEMS * 16;
  sm.flag = reinterpret_cast<int*>(sm.red + 64);
  sm.bars = reinterpret_cast<unsigned long long*>(sm.flag + 20);
  sm.ring_uses = reinterpret_cast<uint32_t*>(sm.bars + RING_SLOTS);
  sm.tile = reinterpret_cast<unsigned char*>(sm.ring_uses + RING_SLOTS);
  if (threadIdx.x == 0) {
    for (int i = 1; i <= 4; ++i) *(reinterpret_cast<uint4*>(sm.flag) + i) = make_uint4(0u, 0u, 0u, 0u);
    for (int i = 0; i < RING_SLOTS; ++i) { mbar_init(sm.bars + i, 1); sm.ring_uses[i] = 0u; }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }

  // Stage descriptors are double buffered: the next one is requested while the current
  // stage runs, so a stage never starts with a round trip for its own description.
  constexpr int WORDS = sizeof(aoto_step_stage) / 4;
  if (threadIdx.x < WORDS)
    reinterpret_cast<uint32_t*>(&stage_buffer[0])[threadIdx.x] = ldg_nc_u32(reinterpret_cast<const uint32_t*>(stages) + threadIdx.x);
  __syncthreads();
  for (int s = 0; s < stage_count; ++s) {
    uint32_t next_word = 0;
    if (threadIdx.x < WORDS && s + 1 < stage_count)
      next_word = ldg_nc_u32(reinterpret_cast<const uint32_t*>(stages + s + 1) + threadIdx.x);
    const aoto_step_stage& stage = stage_buffer[s & 1];
    bool alive = true;
    if (stage.kind == AOTO_STAGE_GEMV) alive = stage_gemv(stage, sm, ctl, s);
    else if (stage.kind == AOTO_STAGE_ATTENTION) alive = stage_attention(stage, sm, ctl, s);
    else if (stage.kind == AOTO_STAGE_PICK) alive = stage_pick(stage, ctl, s);
    if (!alive) return;
    if (threadIdx.x < WORDS) reinterpret_cast<uint32_t*>(&stage_buffer[(s + 1) & 1])[threadIdx.x] = next_word;
    __syncthreads();
  }
}

static size_t step_smem_bytes() {
  const size_t fixed = (size_t)STEP_MAX_K / 8 * 16 * 2 + (size_t)STEP_MAX_K / 64 * 4 +
                       (size_t)STEP_MAX_ITEMS * 16 * 4 + 64 * 4 + 80 + (size_t)RING_SLOTS * (8 + 4);
  const size_t attention = (size_t)2 * ATT_TILE * (128 * 2 + 16) +
                           ((size_t)(MAX_GROUP + 2) * 128 + (size_t)MAX_GROUP * 128 + (size_t)MAX_GROUP * ATT_TILE +
                            (size_t)MAX_GROUP * 2 + ATT_TILE + (size_t)2 * MAX_GROUP * 128) * 4;
  const size_t ring = (size_t)RING_SLOTS * RING_SLOT_BYTES;
  return fixed + (attention > ring ? attention : ring);
}

static int check_stage(const aoto_step_stage& st) {
  if (st.kind == AOTO_STAGE_GEMV) {
    if (st.N <= 0 || (st.N & 1) || st.K <= 0 || st.K > STEP_MAX_K || (st.K & 127) || st.group_size != 64) return 0;
    if (st.epilogue == AOTO_EPILOGUE_SILU_MUL) return 0;
    if (st.addend_mode < AOTO_STAGE_ADDEND_NONE || st.addend_mode > AOTO_STAGE_ADDEND_GATHER) return 0;
    if (st.addend_mode == AOTO_STAGE_ADDEND_GATHER && st.x_index == nullptr) return 0;
    if ((st.flags & AOTO_STAGE_FLAG_X_GATHER) && (st.x_index == nullptr || st.x_rows <= 0)) return 0;
    const int per_tile = (st.K >> 7) * (st.epilogue == AOTO_EPILOGUE_SILU_MUL_PAIRED ? 2 : 1);
    if (per_tile > ITEM_SLOTS * STEP_WARPS) return 0;  // a tile's blocks must fit one round of slots
    return 1;
  }
  if (st.kind == AOTO_STAGE_ATTENTION) {
    if (st.head_dim <= 0 || (st.head_dim & 7) || st.head_dim > 128) return 0;
    if (st.kv_heads <= 0 || st.query_heads % st.kv_heads) return 0;
    if (st.query_heads / st.kv_heads > MAX_GROUP || st.kv_heads > SCRATCH_MAX_COUNTERS) return 0;
    if (st.capacity <= 0) return 0;
    if ((st.query_start | st.key_start | st.value_start) & 1) return 0;
    return 1;
  }
  return st.kind == AOTO_STAGE_PICK;
}

}  // namespace aoto

using namespace aoto;

extern "C" int aoto_sm100_decode_step_stage_size(void) { return (int)sizeof(aoto_step_stage); }

extern "C" int64_t aoto_sm100_stamped_bytes(int64_t count) { return (count + 1) / 2 * 8; }

extern "C" int aoto_sm100_decode_step_supported(const aoto_step_stage* stages, int32_t count) {
  if (!stages || count <= 0) return 0;
  for (int i = 0; i < count; ++i)
    if (!check_stage(stages[i])) return 0;
  return 1;
}

extern "C" int64_t aoto_sm100_decode_step_scratch_bytes(const aoto_step_stage* stages, int32_t count) {
  if (!stages || count <= 0) return 0;
  // header | per-CTA maxima (16 KiB: up to 1024 CTAs x 16 B) | attention partials
  int64_t need = SCRATCH_HEADER_BYTES + 16 * 1024;
  for (int i = 0; i < count; ++i) {
    const aoto_step_stage& st = stages[i];
    if (st.kind != AOTO_STAGE_ATTENTION) continue;
    const int splits = (st.capacity + ATT_TILE - 1) / ATT_TILE;
    const int64_t bytes = SCRATCH_HEADER_BYTES + 16 * 1024 +
                          (int64_t)st.query_heads * splits * (st.head_dim + 2) * 4;
    if (bytes > need) need = bytes;
  }
  return need;
}

extern "C" int aoto_sm100_decode_step(const aoto_decode_step_args* a, void* stream_) {
  if (!a || !a->stages || a->stage_count <= 0 || !a->status || !a->scratch || a->epoch == 0)
    return AOTO_ERR_ARGUMENT;
  int device = 0, sms = 0, coop = 0;
  if (cudaGetDevice(&device) != cudaSuccess) return AOTO_ERR_LAUNCH;
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device);
  cudaDeviceGetAttribute(&coop, cudaDevAttrCooperativeLaunch, device);
  if (!coop) return AOTO_ERR_UNSUPPORTED;
  const size_t smem = step_smem_bytes();
  static PerDeviceOnce raised;
  if (raise_dynamic_smem(decode_step_kernel, smem, raised) != AOTO_OK) return AOTO_ERR_LAUNCH;
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
  ctl.epoch = a->epoch;
  ctl.status = a->status;
  ctl.scratch = reinterpret_cast<float*>(a->scratch);
  ctl.trace = reinterpret_cast<unsigned long long*>(a->trace);
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
