// One decode step as one persistent kernel whose weights run ahead of the dependency chain.
//
// The grid is one CTA of sixteen warps per SM. The host lays the packed weights out ONCE as
// one byte stream per (CTA, warp): the 16 x 128 blocks the warp will multiply, stage after
// stage, already in tensor-core fragment order, cut into pieces of at most three blocks with a
// 16-byte header each. A warp keeps `ring_depth` pieces in flight into its own ring in shared
// memory with bulk copies (cp.async.bulk + mbarrier, no multicast) and refills a slot the
// moment it has multiplied it, across stage boundaries. When the input row of a stage arrives,
// its weights have been resident for several stages.
//
// Stages exchange their vectors as 8-byte stamped words {two bf16, launch epoch} through L2;
// a consumer polls the words it needs until they carry the epoch. No grid-wide barrier exists.
// Every wait - on a stamped word or on an mbarrier - is bounded: a CTA whose wait runs out
// records the stage in `status`, waits (bounded) for its own copies in flight and returns.
#include "qgemv_core.cuh"

namespace aoto {

constexpr int SS_WARPS = AOTO_STREAM_WARPS;
constexpr int SS_THREADS = SS_WARPS * 32;
constexpr int SS_BLOCK_BYTES = AOTO_STREAM_BLOCK_BYTES;
constexpr int SS_SLOT_BYTES = AOTO_STREAM_SLOT_BYTES;
constexpr int SS_MAX_K = 16384;
constexpr int SS_POLL_LIMIT = 1 << 20;  // rounds of a bounded poll (each is at least one L2 round trip)
constexpr int SS_PART_SLOTS = AOTO_STREAM_PART_SLOTS + SS_WARPS;  // shared tiles, then one private slot per warp
constexpr int SS_PART_BYTES = 128;      // [matrix][row] floats of one share
constexpr int SS_MAX_WINDOW_KEYS = 16;  // keys per warp whose rows travel into shared memory a layer ahead; a
                                        // longer window is read from L2 in passes of sixteen keys per warp

// ---------------------------------------------------------------------------
// shared-memory layout, computed identically on both sides
// ---------------------------------------------------------------------------
struct SSLayout {
  uint32_t ring, bars, kvbars, stages, table, work, xs, xsum, part, red, rotary, kv, total;
  int keys_per_warp;  // rows of a warp's key / value buffers (short window)
  int long_window;    // the window does not fit the buffers: only the step's own key and value rows are kept
  int slices_max;     // long window: most slices a kv head's window is cut into (stride of the partial results)
};

__host__ __device__ inline uint32_t ss_align(uint32_t v, uint32_t a) { return (v + a - 1) / a * a; }

__host__ __device__ inline int ss_slices_max(int ctas, int kv_heads, int capacity) {
  const int by_grid = ctas / (kv_heads > 0 ? kv_heads : 1), by_keys = (capacity + 15) / 16;
  const int slices = by_grid < by_keys ? by_grid : by_keys;
  return slices > 1 ? slices : 1;
}

__host__ __device__ inline SSLayout ss_layout(int stage_count, int max_k, int depth, int capacity, int head_dim,
                                              bool has_attention, bool force_long = false, int group = 1,
                                              int slices_max = 1) {
  SSLayout L;
  uint32_t off = 0;
  L.ring = off; off += (uint32_t)SS_WARPS * depth * SS_SLOT_BYTES;
  L.bars = off; off += (uint32_t)SS_WARPS * AOTO_STREAM_MAX_RING * 8;
  L.kvbars = off; off += (uint32_t)SS_WARPS * 8;
  L.stages = off; off += (uint32_t)stage_count * (uint32_t)sizeof(aoto_stream_stage);
  L.table = off; off += ss_align((uint32_t)stage_count * 4, 16);
  // work region: the staged row, its group sums and the partial sums of a GEMV stage; an
  // attention stage uses the same bytes for its row values, query and per-warp results
  L.work = off;
  L.xs = off;
  const uint32_t xs_bytes = (uint32_t)max_k * 2;
  L.xsum = L.xs + xs_bytes;
  const uint32_t xsum_bytes = ss_align((uint32_t)(max_k / 128) * 8, 16);
  L.part = L.xsum + xsum_bytes;
  uint32_t work_bytes = xs_bytes + xsum_bytes + (uint32_t)SS_PART_SLOTS * SS_PART_BYTES;
  const int keys_per_warp = has_attention ? (capacity + SS_WARPS - 1) / SS_WARPS : 0;
  const bool long_window = has_attention && (force_long || keys_per_warp > SS_MAX_WINDOW_KEYS);
  uint32_t attention_bytes =
      has_attention ? (uint32_t)(4 * head_dim + SS_WARPS * (head_dim + 2) + SS_WARPS * 16 + 4 * 16) * 4 : 0;
  if (long_window) {
    // raw q (group heads), k, v; rotated q; per (warp, head) results or the staged slices of one head;
    // per (warp, head) key weights; per-warp factors; per-slice factors
    const int rows = SS_WARPS * group > slices_max ? SS_WARPS * group : slices_max;
    const int weight_heads = group > 4 ? group : 4;  // a warp scores four heads at a time
    attention_bytes = (uint32_t)((2 * group + 2) * head_dim + rows * (head_dim + 2) + SS_WARPS * weight_heads * 16 +
                                 SS_WARPS * 16 + 4 * slices_max) * 4;
  }
  if (attention_bytes > work_bytes) work_bytes = attention_bytes;
  off += ss_align(work_bytes, 16);
  L.red = off; off += 64 * 4;
  L.rotary = off; off += has_attention ? (uint32_t)head_dim * 4 : 0;  // cos row, sin row of the step's position
  L.keys_per_warp = keys_per_warp;
  L.long_window = long_window;
  L.slices_max = long_window ? slices_max : 0;
  L.kv = off;
  if (L.long_window) off += ss_align((uint32_t)2 * head_dim * 2, 16);
  else off += has_attention ? (uint32_t)SS_WARPS * 2 * L.keys_per_warp * head_dim * 2 : 0;
  L.total = off;
  return L;
}

// ---------------------------------------------------------------------------
// small device helpers
// ---------------------------------------------------------------------------
__device__ __forceinline__ uint32_t ss_smem(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void ss_st_stamped(void* ptr, uint32_t data, uint32_t stamp) {
  const unsigned long long word = (unsigned long long)data | ((unsigned long long)stamp << 32);
  asm volatile("st.relaxed.gpu.global.u64 [%0], %1;" ::"l"(ptr), "l"(word) : "memory");
}
// the same word for a reader on another GPU
__device__ __forceinline__ void ss_st_stamped_sys(void* ptr, uint32_t data, uint32_t stamp) {
  const unsigned long long word = (unsigned long long)data | ((unsigned long long)stamp << 32);
  asm volatile("st.relaxed.sys.global.u64 [%0], %1;" ::"l"(ptr), "l"(word) : "memory");
}
__device__ __forceinline__ uint4 ss_ld_stamped_pair_sys(const void* ptr) {
  uint4 v;
  asm volatile("ld.relaxed.sys.global.v4.u32 {%0, %1, %2, %3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(ptr) : "memory");
  return v;
}
__device__ __forceinline__ uint2 ss_ld_stamped_sys(const void* ptr) {
  unsigned long long word;
  asm volatile("ld.relaxed.sys.global.u64 %0, [%1];" : "=l"(word) : "l"(ptr) : "memory");
  return make_uint2((uint32_t)word, (uint32_t)(word >> 32));
}
__device__ __forceinline__ uint2 ss_ld_stamped(const void* ptr) {
  unsigned long long word;
  asm volatile("ld.relaxed.gpu.global.u64 %0, [%1];" : "=l"(word) : "l"(ptr) : "memory");
  return make_uint2((uint32_t)word, (uint32_t)(word >> 32));
}
// two consecutive stamped words; each carries its own stamp, so the pair needs no atomicity
__device__ __forceinline__ uint4 ss_ld_stamped_pair(const void* ptr) {
  uint4 v;
  asm volatile("ld.relaxed.gpu.global.v4.u32 {%0, %1, %2, %3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(ptr) : "memory");
  return v;
}
__device__ __forceinline__ int ss_ld_status(const int* status) {
  int v;
  asm volatile("ld.relaxed.gpu.global.s32 %0, [%1];" : "=r"(v) : "l"(status) : "memory");
  return v;
}

__device__ __forceinline__ void ss_mbar_init(uint32_t bar, int count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void ss_mbar_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool ss_mbar_try_wait(uint32_t bar, uint32_t parity) {
  uint32_t done;
  asm volatile(
      "{\n.reg .pred p;\nmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\nselp.u32 %0, 1, 0, p;\n}\n"
      : "=r"(done) : "r"(bar), "r"(parity) : "memory");
  return done != 0;
}
// Bounded wait for a phase of an mbarrier; false if it never completed.
__device__ __forceinline__ bool ss_mbar_wait(uint32_t bar, uint32_t parity) {
  for (int spins = 0; spins < SS_POLL_LIMIT / 8; ++spins)  // a try_wait may itself block for a while
    if (ss_mbar_try_wait(bar, parity)) return true;
  return false;
}
// global -> this CTA's shared memory; both addresses 16-byte aligned, bytes a multiple of 16
__device__ __forceinline__ void ss_bulk_load(uint32_t smem_dst, const void* gmem_src, uint32_t bytes, uint32_t bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
               ::"r"(smem_dst), "l"(gmem_src), "r"(bytes), "r"(bar) : "memory");
}
__device__ __forceinline__ void ss_fence_async_proxy() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }

// Shared-memory accesses by 32-bit shared address. They are ordinary (not volatile) loads: the
// compiler may schedule them freely between the barriers and fences that carry "memory".
__device__ __forceinline__ uint4 ss_lds128(uint32_t address) {
  uint4 v;
  asm("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(address) : "memory");
  return v;
}
__device__ __forceinline__ uint32_t ss_lds32(uint32_t address) {
  uint32_t v;
  asm("ld.shared.u32 %0, [%1];" : "=r"(v) : "r"(address) : "memory");
  return v;
}
__device__ __forceinline__ float ss_ldsf(uint32_t address) { return __uint_as_float(ss_lds32(address)); }
__device__ __forceinline__ float2 ss_lds64f(uint32_t address) {
  float2 v;
  asm("ld.shared.v2.f32 {%0,%1}, [%2];" : "=f"(v.x), "=f"(v.y) : "r"(address) : "memory");
  return v;
}
__device__ __forceinline__ float4 ss_lds128f(uint32_t address) {
  float4 v;
  asm("ld.shared.v4.f32 {%0,%1,%2,%3}, [%4];" : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "r"(address) : "memory");
  return v;
}
__device__ __forceinline__ void ss_sts32(uint32_t address, uint32_t value) {
  asm volatile("st.shared.u32 [%0], %1;" ::"r"(address), "r"(value) : "memory");
}
__device__ __forceinline__ void ss_stsf(uint32_t address, float value) { ss_sts32(address, __float_as_uint(value)); }

__device__ __forceinline__ void ss_mma(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0,
                                       uint32_t b1) {
  asm("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// The SM's own cycle counter: reading it costs a few cycles, so the marks do not stretch what
// they measure (the global nanosecond timer takes hundreds of cycles per read).
// Maximum of a float over the warp with one integer reduction: IEEE floats order like
// sign-magnitude integers, so flipping the magnitude bits of negatives gives a monotonic key.
__device__ __forceinline__ float ss_warp_max(float v) {
  int key = __float_as_int(v);
  key ^= (key >> 31) & 0x7fffffff;
  key = __reduce_max_sync(0xffffffffu, key);
  key ^= (key >> 31) & 0x7fffffff;
  return __int_as_float(key);
}

// ---------------------------------------------------------------------------
// kernel state
// ---------------------------------------------------------------------------
// The SM's instruction cache holds 32 KB (measured on this part: a loop body of 2048
// instructions issues at 1.0 cycles per instruction, one of 2560 at 2.7, and every jump into
// code that is not resident costs an L2 round trip). A step walks the same code ~120 times,
// so the whole kernel is kept inside the cache: one code path per stage kind, loops instead of
// unrolled copies, approximate intrinsics where the result is rounded to bf16 anyway.
struct SSParams {
  aoto_stream_step_args a;
  SSLayout L;
};

// A warp's view of its stream. Uniform over the lanes of the warp.
struct WarpStream {
  unsigned long long issue_offset;  // byte offset in the stream of the next piece to request
  uint32_t ring;                    // shared address of the warp's first slot
  uint32_t bars;                    // shared address of the warp's first mbarrier
  uint32_t next_stage;              // stage of the next piece to multiply
  uint32_t slot, parity;            // where that piece is (or will be)
  uint32_t issue_slot;              // slot the next request goes to
  int in_flight;                    // pieces requested and not yet multiplied
};

// Every CTA's per-stage timeline on the one clock all SMs share (slow to read: the traced
// instantiation of the kernel is for diagnosis, never for timing).
__device__ __noinline__ void ss_trace(const SSParams& p, int stage, int which) {
  if (threadIdx.x != 0) return;
  unsigned long long t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  p.a.trace[((size_t)blockIdx.x * p.a.stage_count + stage) * 8 + which] = t;
}

__device__ __noinline__ void ss_give_up(const SSParams& p, int stage) {
  if (threadIdx.x == 0) atomicCAS(p.a.status, 0, stage + 1);
}

// Request one piece of `bytes` into the warp's next slot (lane 0 only issues). The slot was
// only READ through the generic proxy and __syncwarp ordered those reads before this point: a
// write by the async proxy needs no proxy fence after reads.
__device__ __forceinline__ void ss_request(const SSParams& p, WarpStream& ws, uint32_t bytes, int lane) {
  if (lane == 0) {
    const uint32_t bar = ws.bars + ws.issue_slot * 8;
    ss_mbar_expect_tx(bar, bytes);
    ss_bulk_load(ws.ring + ws.issue_slot * SS_SLOT_BYTES,
                 reinterpret_cast<const unsigned char*>(p.a.stream) + ws.issue_offset, bytes, bar);
  }
  ws.issue_offset += bytes;
  ws.issue_slot = ws.issue_slot + 1 == (uint32_t)p.a.ring_depth ? 0u : ws.issue_slot + 1;
  ws.in_flight += 1;
}

// ---------------------------------------------------------------------------
// one 16 x 128 block from shared memory
// ---------------------------------------------------------------------------
// `block` is the shared address of the block, `xb` of this lane's B fragments of the block's
// columns (the staged row in fragment order: 256 bytes a block), `sums` of the block's pair of
// 136*sum(x) values. The two scale groups of a block are independent accumulator chains of
// four mma each, issued alternately. Returns the contributions to rows g (lo) and g + 8 (hi),
// identical on the four lanes of a quad.
#define SS_NIB(word, shift) ((((word) >> (shift)) & 0x000F000Fu) ^ 0x43084308u)

__device__ __forceinline__ void ss_block(uint32_t block, uint32_t xb, uint32_t sums, int lane, float& lo, float& hi) {
  const uint4 l = ss_lds128(block + (uint32_t)lane * 16);
  const uint4 h = ss_lds128(block + 512 + (uint32_t)lane * 16);
  const uint32_t slo = ss_lds32(block + 1024 + (uint32_t)(lane >> 2) * 4);
  const uint32_t shi = ss_lds32(block + 1056 + (uint32_t)(lane >> 2) * 4);
  const float2 off = ss_lds64f(sums);
  float ca[4] = {-off.x, -off.x, -off.x, -off.x};
  float cb[4] = {-off.y, -off.y, -off.y, -off.y};
  const uint4 b0 = ss_lds128(xb), b2 = ss_lds128(xb + 128);
  ss_mma(ca, SS_NIB(l.x, 0), SS_NIB(h.x, 0), SS_NIB(l.x, 4), SS_NIB(h.x, 4), b0.x, b0.y);
  ss_mma(cb, SS_NIB(l.z, 0), SS_NIB(h.z, 0), SS_NIB(l.z, 4), SS_NIB(h.z, 4), b2.x, b2.y);
  ss_mma(ca, SS_NIB(l.x, 8), SS_NIB(h.x, 8), SS_NIB(l.x, 12), SS_NIB(h.x, 12), b0.z, b0.w);
  ss_mma(cb, SS_NIB(l.z, 8), SS_NIB(h.z, 8), SS_NIB(l.z, 12), SS_NIB(h.z, 12), b2.z, b2.w);
  const uint4 b1 = ss_lds128(xb + 64), b3 = ss_lds128(xb + 192);
  ss_mma(ca, SS_NIB(l.y, 0), SS_NIB(h.y, 0), SS_NIB(l.y, 4), SS_NIB(h.y, 4), b1.x, b1.y);
  ss_mma(cb, SS_NIB(l.w, 0), SS_NIB(h.w, 0), SS_NIB(l.w, 4), SS_NIB(h.w, 4), b3.x, b3.y);
  ss_mma(ca, SS_NIB(l.y, 8), SS_NIB(h.y, 8), SS_NIB(l.y, 12), SS_NIB(h.y, 12), b1.z, b1.w);
  ss_mma(cb, SS_NIB(l.w, 8), SS_NIB(h.w, 8), SS_NIB(l.w, 12), SS_NIB(h.w, 12), b3.z, b3.w);
  lo = fmaf(bf16x2_lo(slo), ca[0], bf16x2_hi(slo) * cb[0]);
  hi = fmaf(bf16x2_lo(shi), ca[2], bf16x2_hi(shi) * cb[2]);
}

// ---------------------------------------------------------------------------
// GEMV stage
// ---------------------------------------------------------------------------
struct Best {
  float value;
  int index;
};

// Where chunk c (columns 8c..8c+7) of the staged row lives: k step (c & 15) >> 1 of block
// c >> 4, slots 0-7 or 8-15 of that step. Lane t of a quad wants, per pair of steps q, the 16
// bytes {b0(2q), b1(2q), b0(2q+1), b1(2q+1)} where b0 = slots (2t, 2t+1), b1 = (2t+8, 2t+9):
// the chunk's four pairs go to this address and the three 16-byte steps after it.
__device__ __forceinline__ uint32_t ss_chunk_address(uint32_t xs, int c) {
  return xs + (uint32_t)(c >> 4) * 256 + (uint32_t)((c & 15) >> 2) * 64 + (uint32_t)(c & 3) * 4;
}

// The CTA's largest logit (first index on ties) for the pick stage: once per step, out of line.
__device__ __noinline__ void ss_publish_best(const SSParams& p, float bv, int bi, unsigned char* smem) {
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  float* sv = reinterpret_cast<float*>(smem + p.L.red);
  int* si = reinterpret_cast<int*>(sv + 32);
#pragma unroll 1
  for (int offset = 16; offset > 0; offset >>= 1) {
    const float ov = __shfl_xor_sync(0xffffffffu, bv, offset);
    const int oi = __shfl_xor_sync(0xffffffffu, bi, offset);
    if (ov > bv || (ov == bv && oi < bi)) { bv = ov; bi = oi; }
  }
  __syncthreads();  // the finishers' maxima are in; `red` is free of the norm statistic
  if (lane == 0) { sv[warp] = bv; si[warp] = bi; }
  __syncthreads();
  if (tid == 0) {
#pragma unroll 1
    for (int w = 1; w < SS_WARPS; ++w)
      if (sv[w] > bv || (sv[w] == bv && si[w] < bi)) { bv = sv[w]; bi = si[w]; }
    unsigned char* payload = reinterpret_cast<unsigned char*>(p.a.scratch);
    ss_st_stamped(payload + (size_t)blockIdx.x * 16, __float_as_uint(bv), p.a.epoch);
    ss_st_stamped(payload + (size_t)blockIdx.x * 16 + 8, (uint32_t)bi, p.a.epoch);
  }
}

// Element n of a stamped addend, polled until it carries the epoch (`rows` > 1: the sum of the rows
// of an exchanged vector, N values a row). False when the poll ran out.
__device__ __noinline__ bool ss_stamped_addend(const void* addend, int n, int N, int rows, uint32_t epoch, float& value) {
  float total = 0.f;
  for (int r = 0; r < rows; ++r) {
    const unsigned char* at = reinterpret_cast<const unsigned char*>(addend) + (size_t)r * ((size_t)N * 4) + (size_t)(n >> 1) * 8;
    uint2 w = rows > 1 ? ss_ld_stamped_sys(at) : ss_ld_stamped(at);
    for (int polls = 0; w.y != epoch; ++polls) {
      if (polls > SS_POLL_LIMIT) return false;
      w = rows > 1 ? ss_ld_stamped_sys(at) : ss_ld_stamped(at);
    }
    total += (n & 1) ? bf16x2_hi(w.x) : bf16x2_lo(w.x);
  }
  value = rows > 1 ? round_bf16(total) : total;
  return true;
}

// Returns false when a wait ran out (every thread of the CTA gets the same answer).
//
// Only the work that must be done by every warp is done by every warp: the row is fetched,
// normalised and staged by the warps that own chunks of it (four for K = 896), a tile shared
// between warps is finished by the one warp whose duty it is, and a warp with nothing to do in
// a phase waits at the barrier and leaves the issue slots to the others.
template <bool TRACE, bool SHARDED>
__device__ __forceinline__ bool ss_gemv(const SSParams& p, const aoto_stream_stage& st, int stage_index, uint32_t entry,
                                        WarpStream& ws, Best& best, unsigned char* smem) {
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int K = st.K, N = st.N;
  const uint32_t epoch = p.a.epoch;
  const uint32_t stage_flags = st.flags, addend_mode = st.addend_mode;
  const int tile0 = (int)(entry & 0xFFFFu);
  const bool shares_tiles = (entry >> 31) != 0;
  const uint32_t xs = ss_smem(smem + p.L.xs), xsum = ss_smem(smem + p.L.xsum), part = ss_smem(smem + p.L.part);
  const uint32_t stat = ss_smem(smem + p.L.red) + (uint32_t)(stage_index & 1) * 128;  // stages alternate halves
  if (TRACE) ss_trace(p, stage_index, 0);

  long long gather_row = 0;
  if ((stage_flags & AOTO_STAGE_FLAG_X_GATHER) || addend_mode == AOTO_STAGE_ADDEND_GATHER) {
    gather_row = *reinterpret_cast<const volatile long long*>(p.a.x_index);
    gather_row = max(0ll, min(gather_row, (long long)p.a.x_rows - 1));
  }
  // which shared tile this warp finishes after the multiply, and that tile's addend: both loads
  // are off the critical path here (the row is still being fetched) and on it later
  uint32_t duty = 0;
  if (shares_tiles) duty = ldg_nc_u32(p.a.duties + ((size_t)stage_index * gridDim.x + blockIdx.x) * SS_WARPS + warp);

  // ---- the input row ----
  // Pass 1 (the warps that own chunks of the row): fetch the chunk, park it in its place in the
  // staged row, add up its squares. Pass 2, after the warps' sums have met: normalise the chunk
  // in place (if the stage has a norm) and publish the group sums the multiply subtracts.
  const int chunks = K >> 3;
  const uint4* wv = reinterpret_cast<const uint4*>(st.norm_weight);
  const bool has_norm = wv != nullptr;
  const bool stager = warp * 32 < chunks;
  const int per_thread = (chunks + SS_THREADS - 1) / SS_THREADS;
  bool failed = false;
  if (stager) {
    const unsigned char* words = reinterpret_cast<const unsigned char*>(st.x);
    const bool gathers = (stage_flags & AOTO_STAGE_FLAG_X_GATHER) != 0;
    if (gathers) words += (size_t)gather_row * K * 2;
    float squares = 0.f;
    int rounds = 0;
#pragma unroll 1
    for (int i = 0; i < per_thread; ++i) {
      const int c = min(tid + i * SS_THREADS, chunks - 1);  // lanes past the row repeat its last chunk
      uint4 raw;
      if (gathers) {
        raw = ldg_nc_u4(reinterpret_cast<const uint4*>(words) + c);
      } else {
        if (SHARDED && (stage_flags & AOTO_STAGE_FLAG_X_SUM)) {
          // an exchanged vector: the chunk is the sum of every rank's row, added in rank order in fp32
          // and rounded once (what an all-reduce of bf16 rows gives)
          while (true) {
            float v0 = 0.f, v1 = 0.f, v2 = 0.f, v3 = 0.f, v4 = 0.f, v5 = 0.f, v6 = 0.f, v7 = 0.f;
            bool here = true;
#pragma unroll 1
            for (int r = 0; r < p.a.world; ++r) {
              const unsigned char* row = words + (size_t)r * ((size_t)K * 4) + (size_t)c * 32;
              const uint4 a = ss_ld_stamped_pair_sys(row), b = ss_ld_stamped_pair_sys(row + 16);
              here = here && a.y == epoch && a.w == epoch && b.y == epoch && b.w == epoch;
              v0 += bf16x2_lo(a.x); v1 += bf16x2_hi(a.x); v2 += bf16x2_lo(a.z); v3 += bf16x2_hi(a.z);
              v4 += bf16x2_lo(b.x); v5 += bf16x2_hi(b.x); v6 += bf16x2_lo(b.z); v7 += bf16x2_hi(b.z);
            }
            raw = make_uint4(pack_bf16x2(v0, v1), pack_bf16x2(v2, v3), pack_bf16x2(v4, v5), pack_bf16x2(v6, v7));
            if (__all_sync(0xffffffffu, here)) break;
            if (++rounds > SS_POLL_LIMIT || ((rounds & 255) == 0 && ss_ld_status(p.a.status) != 0)) { failed = true; break; }
          }
        } else {
          while (true) {
            const uint4 a = ss_ld_stamped_pair(words + (size_t)c * 32), b = ss_ld_stamped_pair(words + (size_t)c * 32 + 16);
            raw = make_uint4(a.x, a.z, b.x, b.z);
            if (__all_sync(0xffffffffu, a.y == epoch && a.w == epoch && b.y == epoch && b.w == epoch)) break;
            // a CTA that gave up elsewhere ends every other wait early
            if (++rounds > SS_POLL_LIMIT || ((rounds & 255) == 0 && ss_ld_status(p.a.status) != 0)) { failed = true; break; }
          }
        }
      }
      const uint32_t at = ss_chunk_address(xs, c);
      ss_sts32(at, raw.x); ss_sts32(at + 16, raw.y); ss_sts32(at + 32, raw.z); ss_sts32(at + 48, raw.w);
      if (tid + i * SS_THREADS < chunks) {
        squares = fmaf(bf16x2_lo(raw.x), bf16x2_lo(raw.x), squares); squares = fmaf(bf16x2_hi(raw.x), bf16x2_hi(raw.x), squares);
        squares = fmaf(bf16x2_lo(raw.y), bf16x2_lo(raw.y), squares); squares = fmaf(bf16x2_hi(raw.y), bf16x2_hi(raw.y), squares);
        squares = fmaf(bf16x2_lo(raw.z), bf16x2_lo(raw.z), squares); squares = fmaf(bf16x2_hi(raw.z), bf16x2_hi(raw.z), squares);
        squares = fmaf(bf16x2_lo(raw.w), bf16x2_lo(raw.w), squares); squares = fmaf(bf16x2_hi(raw.w), bf16x2_hi(raw.w), squares);
      }
    }
    squares = warp_sum(squares);
    if (lane == 0) ss_stsf(stat + (uint32_t)warp * 4, squares);
  } else if (lane == 0) {
    ss_stsf(stat + (uint32_t)warp * 4, 0.f);
  }
  float duty_addend = 0.f;
  bool alive = true;
  if (duty != 0 && lane < 16 && addend_mode != AOTO_STAGE_ADDEND_NONE) {
    const int n = min((tile0 + (int)(duty & 0x7FFFu)) * 16 + lane, N - 1);
    if (addend_mode == AOTO_STAGE_ADDEND_STAMPED) {
      // an intermediate that was produced stages ago: its poll is a formality
      alive = ss_stamped_addend(st.addend, n, N, (SHARDED && (stage_flags & AOTO_STAGE_FLAG_ADDEND_SUM)) ? p.a.world : 1, epoch,
                                duty_addend);
    } else {
      const size_t row = addend_mode == AOTO_STAGE_ADDEND_GATHER ? (size_t)gather_row * N : 0;
      duty_addend = ldg_nc_bf16(reinterpret_cast<const bf16*>(st.addend) + row + n);
    }
  }
  if (__syncthreads_or(failed)) {  // the warps' sums of squares meet
    ss_give_up(p, stage_index);
    return false;
  }
  if (TRACE) ss_trace(p, stage_index, 1);
  if (stager) {
    float inv = 1.f;
    if (has_norm) {
      // the sixteen sums in a fixed order (a tree: the result does not depend on timing)
      const float4 a = ss_lds128f(stat), b = ss_lds128f(stat + 16), c4 = ss_lds128f(stat + 32), d = ss_lds128f(stat + 48);
      const float total = (((a.x + a.y) + (a.z + a.w)) + ((b.x + b.y) + (b.z + b.w))) +
                          (((c4.x + c4.y) + (c4.z + c4.w)) + ((d.x + d.y) + (d.z + d.w)));
      inv = rsqrtf(__fdividef(total, (float)K) + st.rms_norm_eps);
    }
#pragma unroll 1
    for (int i = 0; i < per_thread; ++i) {
      const int c = tid + i * SS_THREADS;
      const bool mine = c < chunks;
      const uint32_t at = ss_chunk_address(xs, min(c, chunks - 1));
      uint4 o = make_uint4(ss_lds32(at), ss_lds32(at + 16), ss_lds32(at + 32), ss_lds32(at + 48));
      if (has_norm) {
        const uint4 w = ldg_nc_u4(wv + min(c, chunks - 1));
        o.x = pack_bf16x2((bf16x2_lo(o.x) * inv) * bf16x2_lo(w.x), (bf16x2_hi(o.x) * inv) * bf16x2_hi(w.x));
        o.y = pack_bf16x2((bf16x2_lo(o.y) * inv) * bf16x2_lo(w.y), (bf16x2_hi(o.y) * inv) * bf16x2_hi(w.y));
        o.z = pack_bf16x2((bf16x2_lo(o.z) * inv) * bf16x2_lo(w.z), (bf16x2_hi(o.z) * inv) * bf16x2_hi(w.z));
        o.w = pack_bf16x2((bf16x2_lo(o.w) * inv) * bf16x2_lo(w.w), (bf16x2_hi(o.w) * inv) * bf16x2_hi(w.w));
        if (mine) { ss_sts32(at, o.x); ss_sts32(at + 16, o.y); ss_sts32(at + 32, o.z); ss_sts32(at + 48, o.w); }
      }
      // the rounded values are what is multiplied and what is summed; a group of 64 columns is
      // eight consecutive chunks, i.e. eight consecutive lanes
      float chunk_sum = ((bf16x2_lo(o.x) + bf16x2_hi(o.x)) + (bf16x2_lo(o.y) + bf16x2_hi(o.y))) +
                        ((bf16x2_lo(o.z) + bf16x2_hi(o.z)) + (bf16x2_lo(o.w) + bf16x2_hi(o.w)));
      if (!mine) chunk_sum = 0.f;
      chunk_sum += __shfl_xor_sync(0xffffffffu, chunk_sum, 1);
      chunk_sum += __shfl_xor_sync(0xffffffffu, chunk_sum, 2);
      chunk_sum += __shfl_xor_sync(0xffffffffu, chunk_sum, 4);
      if (mine && (lane & 7) == 0) ss_stsf(xsum + (uint32_t)(c >> 3) * 4, 136.f * chunk_sum);
    }
  }
  __syncthreads();
  if (TRACE) ss_trace(p, stage_index, 3);

  // ---- the multiply, then (one site for both) the finishing of a tile ----
  const bool paired = st.epilogue == AOTO_EPILOGUE_SILU_MUL_PAIRED;
  const uint32_t xb = xs + (uint32_t)(lane & 3) * 16;
  float acc0 = 0.f, acc1 = 0.f, acc2 = 0.f, acc3 = 0.f;  // [matrix][rows g, g + 8]
  bool met = false, first_piece = true;
#pragma unroll 1
  while (true) {
    int finish_tile = -1, finish_parts = 0;
    uint32_t finish_first = 0;
    float finish_addend = 0.f;
    if (ws.next_stage == (uint32_t)stage_index) {
      if (!ss_mbar_wait(ws.bars + ws.slot * 8, ws.parity)) { alive = false; break; }
      const uint32_t slot = ws.ring + ws.slot * SS_SLOT_BYTES;
      // header: {next_stage | nblocks << 16 | flags << 24} {byte offset of the columns in the staged row}
      //         {byte offset of the partial slot | tile << 16} {bytes of the piece ring_depth ahead}
      const uint4 h = ss_lds128(slot);
      const int nblocks = (int)((h.x >> 16) & 0xFFu);
      const uint32_t flags = h.x >> 24;
      float lo_sum = 0.f, hi_sum = 0.f;
#pragma unroll 1
      for (int b = 0; b < nblocks; ++b) {
        float lo, hi;
        ss_block(slot + 16 + (uint32_t)b * SS_BLOCK_BYTES, xb + h.y + (uint32_t)b * 256, xsum + (h.y >> 5) + (uint32_t)b * 8,
                 lane, lo, hi);
        lo_sum += lo;
        hi_sum += hi;
      }
      if (flags & AOTO_PIECE_MAT1) { acc2 += lo_sum; acc3 += hi_sum; } else { acc0 += lo_sum; acc1 += hi_sum; }
      __syncwarp();  // every lane is done with the slot before it is refilled
      ws.next_stage = h.x & 0xFFFFu;
      ws.slot += 1;
      if (ws.slot == (uint32_t)p.a.ring_depth) { ws.slot = 0; ws.parity ^= 1u; }
      ws.in_flight -= 1;
      if (h.w != 0) ss_request(p, ws, h.w, lane);
      if (TRACE && first_piece) { ss_trace(p, stage_index, 4); first_piece = false; }
      if (flags & AOTO_PIECE_SEG_END) {
        // the share's sums go to its partial slot (a whole tile has a slot of the warp's own)
        const uint32_t at = part + (h.z & 0xFFFFu) + (uint32_t)(lane >> 2) * 4;
        if ((lane & 3) == 0) {
          ss_stsf(at, acc0);
          ss_stsf(at + 32, acc1);
          ss_stsf(at + 64, acc2);
          ss_stsf(at + 96, acc3);
        }
        acc0 = acc1 = acc2 = acc3 = 0.f;
        if (flags & AOTO_PIECE_WHOLE) {
          finish_tile = tile0 + (int)(h.z >> 16);
          finish_first = part + (h.z & 0xFFFFu);
          finish_parts = 1;
          if (lane < 16 && addend_mode != AOTO_STAGE_ADDEND_NONE) {
            // whole tiles carry a residual only in large models, where the load hides behind other warps
            const int n = min(finish_tile * 16 + lane, N - 1);
            if (addend_mode == AOTO_STAGE_ADDEND_STAMPED) {
              if (!ss_stamped_addend(st.addend, n, N, (SHARDED && (stage_flags & AOTO_STAGE_FLAG_ADDEND_SUM)) ? p.a.world : 1,
                                     epoch, finish_addend))
                alive = false;
            } else {
              const size_t row = addend_mode == AOTO_STAGE_ADDEND_GATHER ? (size_t)gather_row * N : 0;
              finish_addend = ldg_nc_bf16(reinterpret_cast<const bf16*>(st.addend) + row + n);
            }
          }
        }
      }
    } else if (!met) {
      // tiles shared between warps: meet, then the warp whose duty it is sums the shares
      if (TRACE) ss_trace(p, stage_index, 5);
      met = true;
      if (shares_tiles) {
        if (__syncthreads_or(!alive)) break;
        if (TRACE) ss_trace(p, stage_index, 6);
        if (duty != 0) {
          finish_tile = tile0 + (int)(duty & 0x7FFFu);
          finish_first = part + ((duty >> 16) & 0xFFu) * SS_PART_BYTES;
          finish_parts = (int)(duty >> 24);
          finish_addend = duty_addend;
        }
      }
    } else {
      break;
    }
    if (finish_tile >= 0) {
      // lanes 0-15 hold rows 0-15 of the tile (lanes 16-31 the same rows of the second matrix):
      // sum the shares in a fixed order, alpha, addend, paired SiLU, round, store, track the maximum
      __syncwarp();
      const int n = finish_tile * 16 + (lane & 15);
      float total = 0.f;
      {
        const uint32_t at = finish_first + (uint32_t)lane * 4;  // [matrix][row] floats of a share
#pragma unroll 1
        for (int i = 0; i < finish_parts; ++i) total += ss_ldsf(at + (uint32_t)i * SS_PART_BYTES);
      }
      const float second = __shfl_down_sync(0xffffffffu, total, 16);
      float y = st.alpha * total;
      if (addend_mode != AOTO_STAGE_ADDEND_NONE) y = fmaf(st.beta, finish_addend, y);
      if (paired) {
        const float gate = round_bf16(y);
        y = (st.alpha * second) * __fdividef(gate, 1.f + __expf(-gate));
      }
      const uint32_t bits = float_to_bf16_bits(y);
      const uint32_t neighbour = __shfl_down_sync(0xffffffffu, bits, 1);
      if (lane < 16 && n < N) {
        if (stage_flags & AOTO_STAGE_FLAG_OUT_PLAIN) {
          reinterpret_cast<bf16*>(st.out)[n] = __ushort_as_bfloat16((unsigned short)bits);
          float v = __uint_as_float(bits << 16);
          if (v != v) v = INFINITY;
          if (v > best.value || (v == best.value && n < best.index)) { best.value = v; best.index = n; }
        } else if ((lane & 1) == 0) {
          unsigned char* at = reinterpret_cast<unsigned char*>(st.out) + (size_t)(n >> 1) * 8;
          if (SHARDED && (stage_flags & AOTO_STAGE_FLAG_TO_PEERS)) {
            // this rank's row of the exchanged vector, on every rank: plain 8-byte stores over NVLink,
            // data and stamp in one word
            at += (size_t)p.a.rank * ((size_t)N * 4);
#pragma unroll 1
            for (int q = 0; q < p.a.world; ++q) ss_st_stamped_sys(at + p.a.peer_delta[q], bits | (neighbour << 16), epoch);
          } else {
            ss_st_stamped(at, bits | (neighbour << 16), epoch);
          }
        }
      }
      __syncwarp();  // a warp's own slot is read before its next whole tile overwrites it
    }
  }
  // a stage without shared tiles still meets once (the staged row stays until every warp has
  // used it); so does a warp that left the loop because a wait ran out
  if (!shares_tiles || !alive) alive = !__syncthreads_or(!alive);
  if (!alive) {
    ss_give_up(p, stage_index);
    return false;
  }
  if (stage_flags & AOTO_STAGE_FLAG_ARGMAX) ss_publish_best(p, best.value, best.index, smem);
  if (TRACE) ss_trace(p, stage_index, 7);
  return true;
}

// ---------------------------------------------------------------------------
// attention stage, window in shared memory: one CTA per query head over the whole window
// ---------------------------------------------------------------------------
// What a warp of a head CTA needs to know about its share of the window. The same for every
// layer of a launch (the window length is a property of the step), so it is worked out once.
struct WindowShare {
  int head, kvh, member;    // this CTA's query head (-1: none), its kv head, the head's rank in the group
  int k0, nkeys, old_keys;  // keys [k0, k0 + nkeys) of the new window; the first old_keys come from the cache
  int first_valid;          // slots below it are outside the window (window mode)
  uint32_t kbuf, vbuf, bar; // shared addresses of the warp's key rows, value rows and mbarrier
  uint32_t new_key, new_value;  // where this step's rotated key / value rows go (the owner warp's buffers)
};

__device__ __noinline__ WindowShare ss_window_share(const SSParams& p, int warp, int valid_length, unsigned char* smem) {
  WindowShare w;
  const int C = p.a.capacity, D = p.a.head_dim, QH = p.a.query_heads;
  w.head = (int)blockIdx.x < QH && p.a.first_attention >= 0 ? (int)blockIdx.x : -1;
  const int G = QH / max(p.a.kv_heads, 1);
  w.kvh = max(w.head, 0) / max(G, 1);
  w.member = max(w.head, 0) - w.kvh * G;
  w.first_valid = p.a.window ? max(0, C - valid_length) : 0;
  const int per = max(1, (C - w.first_valid + SS_WARPS - 1) / SS_WARPS);
  w.k0 = min(C, w.first_valid + warp * per);
  w.nkeys = min(C, w.k0 + per) - w.k0;
  w.old_keys = max(0, min(w.k0 + w.nkeys, C - 1) - w.k0);  // slot C - 1 is this step's key
  const uint32_t rows = (uint32_t)p.L.keys_per_warp * D * 2;
  const uint32_t kv = ss_smem(smem + p.L.kv);
  w.kbuf = kv + (uint32_t)warp * 2 * rows;
  w.vbuf = w.kbuf + rows;
  w.bar = ss_smem(smem + p.L.kvbars) + (uint32_t)warp * 8;
  const int owner = (C - 1 - w.first_valid) / per;
  const int owner_k0 = w.first_valid + owner * per;
  w.new_key = kv + (uint32_t)owner * 2 * rows + (uint32_t)(C - 1 - owner_k0) * D * 2;
  w.new_value = w.new_key + rows;
  if (p.L.long_window) {  // no buffers: the step's own rows only
    w.kbuf = w.vbuf = 0;
    w.new_key = kv;
    w.new_value = kv + (uint32_t)D * 2;
  }
  return w;
}

// Request this warp's share of a layer's window: new slot j is old slot j + 1.
__device__ __forceinline__ void ss_request_window(const SSParams& p, const aoto_stream_stage& st, const WindowShare& w,
                                                  int lane) {
  if (w.head < 0 || w.old_keys <= 0 || lane != 0 || p.L.long_window) return;
  const int D = p.a.head_dim, C = p.a.capacity;
  const bf16* kin = reinterpret_cast<const bf16*>(st.addend) + ((size_t)w.kvh * C + w.k0 + 1) * D;
  const bf16* vin = kin + (size_t)p.a.kv_heads * C * D;
  const uint32_t bytes = (uint32_t)w.old_keys * D * 2;
  ss_fence_async_proxy();  // this step's key row was written into the buffers through the generic proxy
  ss_mbar_expect_tx(w.bar, 2 * bytes);
  ss_bulk_load(w.kbuf, kin, bytes, w.bar);
  ss_bulk_load(w.vbuf, vin, bytes, w.bar);
}

// Slot j of the next cache is slot j + 1 of this one, for every key and value plane of the
// layer: a plain copy that touches nothing the step computes with. `me` of `movers` CTAs.
__device__ __noinline__ void ss_move_window(const void* cache_in, void* cache_out, int planes, int capacity, int chunks,
                                            int me, int movers) {
  const uint4* src = reinterpret_cast<const uint4*>(cache_in);
  uint4* dst = reinterpret_cast<uint4*>(cache_out);
  const int per_plane = (capacity - 1) * chunks;
  const int total = planes * per_plane;  // one flat range: every mover takes an equal share of all planes
#pragma unroll 2
  for (int i = me * SS_THREADS + (int)threadIdx.x; i < total; i += movers * SS_THREADS) {
    const int plane = i / per_plane;
    const size_t at = (size_t)plane * capacity * chunks + (size_t)(i - plane * per_plane);
    dst[at] = ldg_nc_u4(src + at + chunks);
  }
}

// ---------------------------------------------------------------------------
// attention stage, long window: a kv head's window spread over many CTAs
// ---------------------------------------------------------------------------
// One SM cannot take a long window in from L2 fast enough (a head's 1 280 keys of 128 dims are
// 655 KB; ~5 us per 128 KB were measured), so the window of every kv head is cut into `slices`
// runs of keys and CTA (kv head, slice) scores ALL query heads of the group against its run - the
// key and value rows are read once for the group. Each warp takes a share of the run, in passes of
// sixteen keys (two lanes per key, alternate 16-byte chunks of the row, every load of a pass
// issued before anything is computed), up to four heads at a time in registers with an online
// softmax. The CTA's per-head partial result (max, sum, weighted values) goes out as fp32 stamped
// words; CTA h < query_heads then polls head h's partials of all slices, merges them and publishes
// the head's output as the short form does. The step's own key/value (slot C - 1) stay in shared
// memory; the unit that owns the last slot writes them into the next cache. Afterwards every CTA
// moves an equal share of the cache window.
//
// Every attention stage has a region of partial results of its own: the stamp of a word is the
// launch's, so a merge could not tell this layer's word from one the previous layer left.
template <bool TRACE>
__device__ __noinline__ bool ss_attention_spread(const SSParams& p, const aoto_stream_stage& st, int stage_index,
                                                 int valid_length, unsigned char* smem) {
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int D = p.a.head_dim, C = p.a.capacity, KVH = p.a.kv_heads, QH = p.a.query_heads;
  const int G = QH / KVH, pairs = D >> 1;
  const int cta = (int)blockIdx.x, ctas = (int)gridDim.x;
  const uint32_t epoch = p.a.epoch;
  if (TRACE) ss_trace(p, stage_index, 0);

  // geometry of the step's window (the same on every CTA)
  const int first_valid = p.a.window ? max(0, C - valid_length) : 0;
  const int window = C - first_valid;
  const int slices = max(1, min(min(ctas / KVH, (window + 15) >> 4), p.L.slices_max));
  const int run = (window + slices - 1) / slices;          // keys of a slice
  const int last_slice = (C - 1 - first_valid) / run;      // the slice that holds this step's key
  const bool unit = cta < KVH * slices;
  const int kvh = unit ? cta / slices : 0, slice = unit ? cta - kvh * slices : 0;
  const int s0 = min(C, first_valid + slice * run), s1 = min(C, s0 + run);
  const int per = max(1, (s1 - s0 + SS_WARPS - 1) / SS_WARPS);
  const int k0 = min(s1, s0 + warp * per), nkeys = unit ? min(s1, k0 + per) - k0 : 0;
  const bool merges = cta < QH;
  const size_t head_stride = (size_t)p.L.slices_max * (D + 2) * 8;  // bytes of one head's partials
  // a region per attention stage: the stamp is the launch's, so words a previous layer of the
  // same launch left would pass for this layer's
  unsigned char* partials = reinterpret_cast<unsigned char*>(p.a.scratch) + (size_t)ctas * 16 +
                            (size_t)st.ordinal * QH * head_stride;

  const uint32_t rowv = ss_smem(smem + p.L.work);                       // raw q (G heads), k, v: (G + 2) * D floats
  const uint32_t qs = rowv + (uint32_t)(G + 2) * D * 4;                 // rotated, scaled queries: G * D floats
  const uint32_t merge = qs + (uint32_t)G * D * 4;                      // [warp][head]: m, l, D sums / staged slices
  const int merge_rows = max(SS_WARPS * G, p.L.slices_max);
  const uint32_t weights = merge + (uint32_t)merge_rows * (D + 2) * 4;  // [warp][head in group of four][16]
  const int weight_heads = max(G, 4);
  const uint32_t factors = weights + (uint32_t)SS_WARPS * weight_heads * 64;  // [warp][16]
  const uint32_t slice_factors = factors + (uint32_t)SS_WARPS * 64;     // [4 warps][slices_max]
  const uint32_t rotary = ss_smem(smem + p.L.rotary);
  const uint32_t new_key = ss_smem(smem + p.L.kv), new_value = new_key + (uint32_t)D * 2;
  const int dims = D >> 5;
  bool failed = false;

  if (unit) {
    if (nkeys > 0) {  // this warp's rows are asked for now: the projection the stage waits for gives them time
      const int old = min(k0 + nkeys, C - 1) - k0;
      const unsigned char* kin = reinterpret_cast<const unsigned char*>(st.addend) + ((size_t)kvh * C + k0 + 1) * D * 2;
      const unsigned char* vin = kin + (size_t)KVH * C * D * 2;
      for (int o = lane * 128; o < old * D * 2; o += 32 * 128) {
        asm volatile("prefetch.global.L2 [%0];" ::"l"(kin + o));
        asm volatile("prefetch.global.L2 [%0];" ::"l"(vin + o));
      }
    }
    __syncthreads();  // the previous stage's last readers of the work region are done
    // the group's queries and the kv head's key and value of the step
    const int words = (G + 2) * pairs;
    if (tid < ((words + 31) & ~31)) {
      const bool mine = tid < words;
      int element = p.a.query_start + kvh * G * D + 2 * tid;
      if (tid >= (G + 1) * pairs) element = p.a.value_start + kvh * D + 2 * (tid - (G + 1) * pairs);
      else if (tid >= G * pairs) element = p.a.key_start + kvh * D + 2 * (tid - G * pairs);
      const unsigned char* at = reinterpret_cast<const unsigned char*>(st.x) + (size_t)(element >> 1) * 8;
#pragma unroll 1
      for (int rounds = 1;; ++rounds) {
        const uint2 v = mine ? ss_ld_stamped(at) : make_uint2(0u, epoch);
        if (v.y == epoch && mine) {
          ss_stsf(rowv + (uint32_t)tid * 8, bf16x2_lo(v.x));
          ss_stsf(rowv + (uint32_t)tid * 8 + 4, bf16x2_hi(v.x));
        }
        if (__all_sync(0xffffffffu, v.y == epoch)) break;
        if (rounds > SS_POLL_LIMIT || ((rounds & 255) == 0 && ss_ld_status(p.a.status) != 0)) { failed = true; break; }
      }
    }
  }
  if (__syncthreads_or(failed)) {
    ss_give_up(p, stage_index);
    return false;
  }
  if (TRACE) ss_trace(p, stage_index, 1);

  if (unit) {
    // rotate the group's queries (bf16 rounding points of the unfused form) and the key
    const int hd = D >> 1;
#pragma unroll 1
    for (int i = tid; i < (G + 1) * D; i += SS_THREADS) {
      const int d = i % D;
      const uint32_t cs = ss_lds32(rotary + (uint32_t)(d & ~1) * 2), sn = ss_lds32(rotary + (uint32_t)(D + (d & ~1)) * 2);
      const float c = (d & 1) ? bf16x2_hi(cs) : bf16x2_lo(cs), sine = (d & 1) ? bf16x2_hi(sn) : bf16x2_lo(sn);
      const int other = d < hd ? i + hd : i - hd;
      const float sign = d < hd ? -1.f : 1.f;
      const float r = round_bf16(round_bf16(ss_ldsf(rowv + (uint32_t)i * 4) * c) +
                                 round_bf16(sign * ss_ldsf(rowv + (uint32_t)other * 4) * sine));
      if (i < G * D) {
        ss_stsf(qs + (uint32_t)i * 4, r * p.a.scale);
      } else {
        const uint32_t key_bits = float_to_bf16_bits(r);
        const uint32_t value_bits = float_to_bf16_bits(ss_ldsf(rowv + (uint32_t)(i + D) * 4));
        asm volatile("st.shared.u16 [%0], %1;" ::"r"(new_key + (uint32_t)d * 2), "h"((unsigned short)key_bits) : "memory");
        asm volatile("st.shared.u16 [%0], %1;" ::"r"(new_value + (uint32_t)d * 2), "h"((unsigned short)value_bits) : "memory");
        if (slice == last_slice) {
          bf16* kout = reinterpret_cast<bf16*>(const_cast<void*>(st.norm_weight)) + ((size_t)kvh * C + (C - 1)) * D;
          kout[d] = __ushort_as_bfloat16((unsigned short)key_bits);
          kout[(size_t)KVH * C * D + d] = __ushort_as_bfloat16((unsigned short)value_bits);
        }
      }
    }
    __syncthreads();
    if (TRACE) ss_trace(p, stage_index, 2);

    // Every warp attends its keys, four heads of the group at a time, eight keys a pass: lane
    // 4 * key + head scores one (key, head) pair over the whole row (the four lanes of a key read the
    // same addresses), the eight lanes of a head share its running maximum and sum, and for the
    // weighted values every lane owns D / 32 dimensions of all four heads. The loops are kept
    // rolled: this code runs once per layer and warp, and what it costs is fetching it.
    const bf16* kplane = reinterpret_cast<const bf16*>(st.addend) + (size_t)kvh * C * D;  // new slot j = old slot j + 1
    const bf16* vplane = kplane + (size_t)KVH * C * D;
    const unsigned char* own_key = smem + p.L.kv;                      // the step's own rows (slot C - 1)
    const unsigned char* own_value = own_key + (size_t)D * 2;
    const uint32_t my_weights = weights + (uint32_t)warp * weight_heads * 64;  // [head of the group of four][8 keys]
    const int hl = lane & 3, kl = lane >> 2;
#pragma unroll 1
    for (int g0 = 0; g0 < G; g0 += 4) {
      const bool has_head = g0 + hl < G;
      float m = -INFINITY, l = 0.f;   // of head g0 + hl (the same on its eight lanes)
      float a[4][4];                  // [head of the group][dimension of this lane]
#pragma unroll
      for (int h = 0; h < 4; ++h) a[h][0] = a[h][1] = a[h][2] = a[h][3] = 0.f;
#pragma unroll 1
      for (int c0 = 0; c0 < nkeys; c0 += 8) {
        const int key = c0 + kl, slot = k0 + key;
        bool attend = false;
        if (key < nkeys && has_head) attend = p.a.window ? slot >= first_valid : p.a.mask[slot] != 0;
        float sc = -INFINITY;
        if (attend) {
          const uint4* krow = slot == C - 1 ? reinterpret_cast<const uint4*>(own_key)
                                            : reinterpret_cast<const uint4*>(kplane + (size_t)(slot + 1) * D);
          const uint32_t qrow = qs + (uint32_t)((g0 + hl) * D) * 4;
          float d0 = 0.f, d1 = 0.f, d2 = 0.f, d3 = 0.f;
#pragma unroll 8
          for (int c = 0; c < (D >> 3); ++c) {
            const uint4 kk = krow[c];
            const float4 qa = ss_lds128f(qrow + (uint32_t)c * 32), qb = ss_lds128f(qrow + (uint32_t)c * 32 + 16);
            d0 = fmaf(bf16x2_lo(kk.x), qa.x, d0); d1 = fmaf(bf16x2_hi(kk.x), qa.y, d1);
            d2 = fmaf(bf16x2_lo(kk.y), qa.z, d2); d3 = fmaf(bf16x2_hi(kk.y), qa.w, d3);
            d0 = fmaf(bf16x2_lo(kk.z), qb.x, d0); d1 = fmaf(bf16x2_hi(kk.z), qb.y, d1);
            d2 = fmaf(bf16x2_lo(kk.w), qb.z, d2); d3 = fmaf(bf16x2_hi(kk.w), qb.w, d3);
          }
          sc = (d0 + d1) + (d2 + d3);
        }
        // maximum and sum over the eight keys of the head (lanes that differ in bits 2-4)
        float mc = sc;
        mc = fmaxf(mc, __shfl_xor_sync(0xffffffffu, mc, 4));
        mc = fmaxf(mc, __shfl_xor_sync(0xffffffffu, mc, 8));
        mc = fmaxf(mc, __shfl_xor_sync(0xffffffffu, mc, 16));
        const float m_new = fmaxf(m, mc);
        const float keep = m == -INFINITY ? 0.f : __expf(m - m_new);
        const float e = sc == -INFINITY ? 0.f : __expf(sc - m_new);
        float es = e;
        es += __shfl_xor_sync(0xffffffffu, es, 4);
        es += __shfl_xor_sync(0xffffffffu, es, 8);
        es += __shfl_xor_sync(0xffffffffu, es, 16);
        l = fmaf(l, keep, es);
        m = m_new;
        ss_stsf(my_weights + (uint32_t)hl * 64 + (uint32_t)kl * 4, e);
        __syncwarp();
#pragma unroll
        for (int h = 0; h < 4; ++h) {
          const float kh = __shfl_sync(0xffffffffu, keep, h);  // lane h holds head g0 + h
          a[h][0] *= kh; a[h][1] *= kh; a[h][2] *= kh; a[h][3] *= kh;
        }
        const int count = min(8, nkeys - c0);
#pragma unroll 4
        for (int j = 0; j < count; ++j) {
          const int vslot = k0 + c0 + j;
          const unsigned char* vrow = vslot == C - 1 ? own_value
                                                     : reinterpret_cast<const unsigned char*>(vplane + (size_t)(vslot + 1) * D);
          uint2 v = make_uint2(0u, 0u);
          if (dims == 4) v = *reinterpret_cast<const uint2*>(vrow + (size_t)lane * 8);
          else v.x = *reinterpret_cast<const uint32_t*>(vrow + (size_t)lane * 4);
          const float v0 = bf16x2_lo(v.x), v1 = bf16x2_hi(v.x), v2 = bf16x2_lo(v.y), v3 = bf16x2_hi(v.y);
#pragma unroll
          for (int h = 0; h < 4; ++h) {
            const float wt = ss_ldsf(my_weights + (uint32_t)h * 64 + (uint32_t)j * 4);
            a[h][0] = fmaf(wt, v0, a[h][0]); a[h][1] = fmaf(wt, v1, a[h][1]);
            a[h][2] = fmaf(wt, v2, a[h][2]); a[h][3] = fmaf(wt, v3, a[h][3]);
          }
        }
        __syncwarp();  // the weights are read: the next pass may overwrite them
      }
#pragma unroll
      for (int h = 0; h < 4; ++h) {
        if (g0 + h < G) {
          const uint32_t mine = merge + (uint32_t)((warp * G + g0 + h) * (D + 2)) * 4;
          const float mh = __shfl_sync(0xffffffffu, m, h), lh = __shfl_sync(0xffffffffu, l, h);
          if (lane == 0) { ss_stsf(mine, mh); ss_stsf(mine + 4, lh); }
          ss_stsf(mine + 8 + (uint32_t)lane * dims * 4, a[h][0]);
          ss_stsf(mine + 12 + (uint32_t)lane * dims * 4, a[h][1]);
          if (dims == 4) { ss_stsf(mine + 16 + (uint32_t)lane * dims * 4, a[h][2]); ss_stsf(mine + 20 + (uint32_t)lane * dims * 4, a[h][3]); }
        }
      }
    }
    if (TRACE) ss_trace(p, stage_index, 3);
    __syncthreads();
    if (TRACE) ss_trace(p, stage_index, 4);

    // the CTA's result per head: the sixteen warps merged in a fixed order, published as fp32 words
    // (a warp's thirty-two elements belong to one head, so the sixteen factors are computed once per warp)
#pragma unroll 1
    for (int i = tid; i < G * D; i += SS_THREADS) {
      const int g = i / D, d = i - g * D;
      const uint32_t row = merge + (uint32_t)(((lane & (SS_WARPS - 1)) * G + g) * (D + 2)) * 4;
      const float wm = lane < SS_WARPS ? ss_ldsf(row) : -INFINITY;
      const float wl = lane < SS_WARPS ? ss_ldsf(row + 4) : 0.f;
      const float mx = ss_warp_max(wm);
      const float factor = wm == -INFINITY ? 0.f : __expf(wm - mx);
      const uint32_t mine = factors + (uint32_t)warp * 64;
      __syncwarp();
      if (lane < SS_WARPS) ss_stsf(mine + (uint32_t)lane * 4, factor);
      const float den = warp_sum(factor * wl);
      __syncwarp();
      float n0 = 0.f, n1 = 0.f;
#pragma unroll 2
      for (int w2 = 0; w2 < SS_WARPS; w2 += 2) {
        n0 = fmaf(ss_ldsf(mine + (uint32_t)w2 * 4), ss_ldsf(merge + (uint32_t)((w2 * G + g) * (D + 2) + 2 + d) * 4), n0);
        n1 = fmaf(ss_ldsf(mine + (uint32_t)w2 * 4 + 4), ss_ldsf(merge + (uint32_t)(((w2 + 1) * G + g) * (D + 2) + 2 + d) * 4), n1);
      }
      unsigned char* out = partials + (size_t)(kvh * G + g) * head_stride + (size_t)slice * (D + 2) * 8;
      ss_st_stamped(out + (size_t)(2 + d) * 8, __float_as_uint(n0 + n1), epoch);
      if (d == 0) {
        ss_st_stamped(out, __float_as_uint(mx), epoch);
        ss_st_stamped(out + 8, __float_as_uint(den), epoch);
      }
    }
  }
  if (TRACE) ss_trace(p, stage_index, 5);

  if (merges) {
    // head `cta`: its partial results of all slices, merged, and published as the head's output
    __syncthreads();  // the merge rows are read: the area now stages the slices
    const unsigned char* from = partials + (size_t)cta * head_stride;
    const int words = slices * (D + 2);
    int rounds = 0;
#pragma unroll 1
    for (int i = tid; i < words; i += SS_THREADS) {
      uint2 v = ss_ld_stamped(from + (size_t)i * 8);
      while (v.y != epoch) {
        if (++rounds > SS_POLL_LIMIT || ((rounds & 255) == 0 && ss_ld_status(p.a.status) != 0)) { failed = true; break; }
        v = ss_ld_stamped(from + (size_t)i * 8);
      }
      ss_sts32(merge + (uint32_t)i * 4, v.x);
    }
    if (__syncthreads_or(failed)) {
      ss_give_up(p, stage_index);
      return false;
    }
    if (tid < D) {
      const uint32_t mine = slice_factors + (uint32_t)warp * (uint32_t)p.L.slices_max * 4;
      float mx = -INFINITY;
      for (int s2 = lane; s2 < slices; s2 += 32) mx = fmaxf(mx, ss_ldsf(merge + (uint32_t)(s2 * (D + 2)) * 4));
      mx = ss_warp_max(mx);
      float den = 0.f;
      for (int s2 = lane; s2 < slices; s2 += 32) {
        const float sm = ss_ldsf(merge + (uint32_t)(s2 * (D + 2)) * 4);
        const float factor = sm == -INFINITY ? 0.f : __expf(sm - mx);
        ss_stsf(mine + (uint32_t)s2 * 4, factor);
        den = fmaf(factor, ss_ldsf(merge + (uint32_t)(s2 * (D + 2) + 1) * 4), den);
      }
      den = warp_sum(den);
      __syncwarp();
      float num = 0.f;
#pragma unroll 2
      for (int s2 = 0; s2 < slices; ++s2)
        num = fmaf(ss_ldsf(mine + (uint32_t)s2 * 4), ss_ldsf(merge + (uint32_t)(s2 * (D + 2) + 2 + tid) * 4), num);
      const float result = den > 0.f ? __fdividef(num, den) : 0.f;
      const uint32_t bits = float_to_bf16_bits(result);
      const uint32_t neighbour = __shfl_down_sync(0xffffffffu, bits, 1);
      if ((tid & 1) == 0)
        ss_st_stamped(reinterpret_cast<unsigned char*>(st.out) + ((size_t)cta * pairs + (tid >> 1)) * 8,
                      bits | (neighbour << 16), epoch);
    }
  }
  if (TRACE) ss_trace(p, stage_index, 6);

  // the cache window: every CTA moves an equal share
  ss_move_window(st.addend, const_cast<void*>(st.norm_weight), 2 * KVH, C, D >> 3, cta, ctas);
  __syncthreads();  // the work region is free for the next stage
  if (TRACE) ss_trace(p, stage_index, 7);
  return true;
}

template <bool TRACE>
__device__ __forceinline__ bool ss_attention(const SSParams& p, const aoto_stream_stage& st, int stage_index,
                                             const WindowShare& w, uint32_t& kv_parity, bool& kv_pending,
                                             unsigned char* smem) {
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int D = p.a.head_dim, C = p.a.capacity, KVH = p.a.kv_heads, QH = p.a.query_heads;
  const uint32_t epoch = p.a.epoch;
  if (TRACE) ss_trace(p, stage_index, 0);

  // the CTAs without a head move the window (every CTA does when each one has a head)
  const int helpers = (int)gridDim.x - QH;
  if (w.head < 0) {
    ss_move_window(st.addend, const_cast<void*>(st.norm_weight), 2 * KVH, C, D >> 3, (int)blockIdx.x - QH, helpers);
    if (TRACE) ss_trace(p, stage_index, 7);
    return true;
  }

  const int pairs = D >> 1;
  __syncthreads();  // the previous stage's last readers of the work region are done
  const uint32_t rowv = ss_smem(smem + p.L.work);  // raw q head, k, v of the step: 3 * D floats
  const uint32_t qs = rowv + (uint32_t)3 * D * 4;  // rotated, scaled query: D floats
  const uint32_t merge = qs + (uint32_t)D * 4;     // per warp: m, l, then D sums
  const uint32_t weights = merge + (uint32_t)SS_WARPS * (D + 2) * 4 + (uint32_t)warp * 64;  // this warp's key weights
  const uint32_t rotary = ss_smem(smem + p.L.rotary);  // cos row, sin row (bf16)

  // this head's query and its kv head's key and value of the step: the warps that own words of
  // the stamped projection row poll them, the others go straight to the barrier
  bool failed = false;
  if (tid < ((3 * pairs + 31) & ~31)) {
    const bool mine = tid < 3 * pairs;
    int element = p.a.query_start + w.head * D + 2 * tid;
    if (tid >= 2 * pairs) element = p.a.value_start + w.kvh * D + 2 * (tid - 2 * pairs);
    else if (tid >= pairs) element = p.a.key_start + w.kvh * D + 2 * (tid - pairs);
    const unsigned char* at = reinterpret_cast<const unsigned char*>(st.x) + (size_t)(element >> 1) * 8;
#pragma unroll 1
    for (int rounds = 1;; ++rounds) {
      const uint2 v = mine ? ss_ld_stamped(at) : make_uint2(0u, epoch);
      if (v.y == epoch && mine) {
        ss_stsf(rowv + (uint32_t)tid * 8, bf16x2_lo(v.x));
        ss_stsf(rowv + (uint32_t)tid * 8 + 4, bf16x2_hi(v.x));
      }
      if (__all_sync(0xffffffffu, v.y == epoch)) break;
      if (rounds > SS_POLL_LIMIT || ((rounds & 255) == 0 && ss_ld_status(p.a.status) != 0)) { failed = true; break; }
    }
  }
  if (__syncthreads_or(failed)) {
    ss_give_up(p, stage_index);
    return false;
  }
  if (TRACE) ss_trace(p, stage_index, 1);

  // rotate; this step's key and value join the window of the warp that owns the last slot
  if (tid < D) {
    const int half = D >> 1;
    const uint32_t cs = ss_lds32(rotary + (uint32_t)(tid & ~1) * 2), sn = ss_lds32(rotary + (uint32_t)(D + (tid & ~1)) * 2);
    const float c = (tid & 1) ? bf16x2_hi(cs) : bf16x2_lo(cs), sine = (tid & 1) ? bf16x2_hi(sn) : bf16x2_lo(sn);
    const int other = tid < half ? tid + half : tid - half;
    const float sign = tid < half ? -1.f : 1.f;
    const float q = round_bf16(round_bf16(ss_ldsf(rowv + (uint32_t)tid * 4) * c) +
                               round_bf16(sign * ss_ldsf(rowv + (uint32_t)other * 4) * sine));
    const float k = round_bf16(round_bf16(ss_ldsf(rowv + (uint32_t)(D + tid) * 4) * c) +
                               round_bf16(sign * ss_ldsf(rowv + (uint32_t)(D + other) * 4) * sine));
    ss_stsf(qs + (uint32_t)tid * 4, q * p.a.scale);
    const uint32_t key_bits = float_to_bf16_bits(k), value_bits = float_to_bf16_bits(ss_ldsf(rowv + (uint32_t)(2 * D + tid) * 4));
    asm volatile("st.shared.u16 [%0], %1;" ::"r"(w.new_key + (uint32_t)tid * 2), "h"((unsigned short)key_bits) : "memory");
    asm volatile("st.shared.u16 [%0], %1;" ::"r"(w.new_value + (uint32_t)tid * 2), "h"((unsigned short)value_bits) : "memory");
    if (w.member == 0) {
      bf16* kout = reinterpret_cast<bf16*>(const_cast<void*>(st.norm_weight)) + ((size_t)w.kvh * C + (C - 1)) * D;
      kout[tid] = __ushort_as_bfloat16((unsigned short)key_bits);
      kout[(size_t)KVH * C * D + tid] = __ushort_as_bfloat16((unsigned short)value_bits);
    }
  }
  __syncthreads();
  if (TRACE) ss_trace(p, stage_index, 2);

  // every warp attends its keys: two lanes per key for the scores, the lanes split the head
  // dimension for the weighted sum of values
  bool alive = true;
  if (kv_pending && w.old_keys > 0) alive = ss_mbar_wait(w.bar, kv_parity);
  if (TRACE) ss_trace(p, stage_index, 3);
  {
    const int key = lane >> 1, half = lane & 1;
    const int half_chunks = D >> 4;  // 16-byte chunks of half a row
    float s = -INFINITY;
    bool attend = false;
    if (alive && key < w.nkeys) attend = p.a.window ? w.k0 + key >= w.first_valid : p.a.mask[w.k0 + key] != 0;
    if (attend) {
      const uint32_t krow = w.kbuf + (uint32_t)key * D * 2 + (uint32_t)half * D;
      const uint32_t qrow = qs + (uint32_t)half * (D >> 1) * 4;
      float d0 = 0.f, d1 = 0.f, d2 = 0.f, d3 = 0.f;
#pragma unroll 1
      for (int i = 0; i < half_chunks; ++i) {
        const int ci = (i + key) & (half_chunks - 1);  // rows are 2*D bytes apart: rotate the chunk order by key
        const uint4 kk = ss_lds128(krow + (uint32_t)ci * 16);
        const float4 qa = ss_lds128f(qrow + (uint32_t)ci * 32), qb = ss_lds128f(qrow + (uint32_t)ci * 32 + 16);
        d0 = fmaf(bf16x2_lo(kk.x), qa.x, d0); d1 = fmaf(bf16x2_hi(kk.x), qa.y, d1);
        d2 = fmaf(bf16x2_lo(kk.y), qa.z, d2); d3 = fmaf(bf16x2_hi(kk.y), qa.w, d3);
        d0 = fmaf(bf16x2_lo(kk.z), qb.x, d0); d1 = fmaf(bf16x2_hi(kk.z), qb.y, d1);
        d2 = fmaf(bf16x2_lo(kk.w), qb.z, d2); d3 = fmaf(bf16x2_hi(kk.w), qb.w, d3);
      }
      s = (d0 + d1) + (d2 + d3);
    }
    const float other = __shfl_xor_sync(0xffffffffu, s, 1);
    s = attend ? s + other : -INFINITY;
    const float m = ss_warp_max(s);
    const float e = s == -INFINITY ? 0.f : __expf(s - m);
    // the warp's weights go through shared memory: the weighted sum below reads them as
    // broadcasts and needs no shuffle per key
    if (half == 0) ss_stsf(weights + (uint32_t)key * 4, e);
    __syncwarp();
    // weighted values: lane holds D / 32 consecutive dimensions; every lane also sums the weights
    const int dims = D >> 5;  // 2 or 4
    float a0 = 0.f, a1 = 0.f, a2 = 0.f, a3 = 0.f, l = 0.f;
    const uint32_t vrow = w.vbuf + (uint32_t)lane * dims * 2;
#pragma unroll 2
    for (int j = 0; j < w.nkeys; ++j) {
      const float wt = ss_ldsf(weights + (uint32_t)j * 4);
      const uint32_t v0 = ss_lds32(vrow + (uint32_t)j * D * 2);
      a0 = fmaf(wt, bf16x2_lo(v0), a0);
      a1 = fmaf(wt, bf16x2_hi(v0), a1);
      if (dims == 4) {
        const uint32_t v1 = ss_lds32(vrow + (uint32_t)j * D * 2 + 4);
        a2 = fmaf(wt, bf16x2_lo(v1), a2);
        a3 = fmaf(wt, bf16x2_hi(v1), a3);
      }
      l += wt;
    }
    const uint32_t mine = merge + (uint32_t)warp * (D + 2) * 4;
    if (lane == 0) { ss_stsf(mine, m); ss_stsf(mine + 4, l); }
    ss_stsf(mine + 8 + (uint32_t)lane * dims * 4, a0);
    ss_stsf(mine + 12 + (uint32_t)lane * dims * 4, a1);
    if (dims == 4) { ss_stsf(mine + 16 + (uint32_t)lane * dims * 4, a2); ss_stsf(mine + 20 + (uint32_t)lane * dims * 4, a3); }
  }
  if (TRACE) ss_trace(p, stage_index, 4);
  if (__syncthreads_or(!alive)) {
    ss_give_up(p, stage_index);
    return false;
  }
  if (TRACE) ss_trace(p, stage_index, 5);
  if (kv_pending) { kv_parity ^= 1u; kv_pending = false; }

  // merge the warps' results in a fixed order; the sixteen rescaling factors are computed once
  // per merging warp (one lane each) instead of once per output dimension
  if (tid < D) {
    const uint32_t factors = merge + (uint32_t)SS_WARPS * (D + 2) * 4 + SS_WARPS * 64 + (uint32_t)warp * 64;
    const uint32_t row = merge + (uint32_t)(lane & (SS_WARPS - 1)) * (D + 2) * 4;
    const float wm = lane < SS_WARPS ? ss_ldsf(row) : -INFINITY;
    const float wl = lane < SS_WARPS ? ss_ldsf(row + 4) : 0.f;
    const float m = ss_warp_max(wm);
    const float factor = wm == -INFINITY ? 0.f : __expf(wm - m);
    if (lane < SS_WARPS) ss_stsf(factors + (uint32_t)lane * 4, factor);
    const float den = warp_sum(factor * wl);
    __syncwarp();
    float n0 = 0.f, n1 = 0.f;
#pragma unroll 2
    for (int i = 0; i < SS_WARPS; i += 2) {
      n0 = fmaf(ss_ldsf(factors + (uint32_t)i * 4), ss_ldsf(merge + (uint32_t)(i * (D + 2) + 2 + tid) * 4), n0);
      n1 = fmaf(ss_ldsf(factors + (uint32_t)i * 4 + 4), ss_ldsf(merge + (uint32_t)((i + 1) * (D + 2) + 2 + tid) * 4), n1);
    }
    const float out = den > 0.f ? __fdividef(n0 + n1, den) : 0.f;
    const uint32_t bits = float_to_bf16_bits(out);
    const uint32_t neighbour = __shfl_down_sync(0xffffffffu, bits, 1);
    if ((tid & 1) == 0)
      ss_st_stamped(reinterpret_cast<unsigned char*>(st.out) + ((size_t)w.head * pairs + (tid >> 1)) * 8,
                    bits | (neighbour << 16), epoch);
  }
  if (TRACE) ss_trace(p, stage_index, 6);

  // the next layer's window starts travelling: every warp is done with its buffers
  if (st.next_attention >= 0) {
    const aoto_stream_stage* all = reinterpret_cast<const aoto_stream_stage*>(smem + p.L.stages);
    ss_request_window(p, all[st.next_attention], w, lane);
    kv_pending = true;
  }
  if (helpers <= 0) ss_move_window(st.addend, const_cast<void*>(st.norm_weight), 2 * KVH, C, D >> 3, w.head, QH);
  __syncthreads();  // the work region is free for the next stage
  if (TRACE) ss_trace(p, stage_index, 7);
  return true;
}

// ---------------------------------------------------------------------------
// pick stage: CTA 0 polls the per-CTA maxima the ARGMAX stage left
// ---------------------------------------------------------------------------
template <bool SHARDED>
__device__ __noinline__ void ss_pick(const SSParams& p, int stage_index) {
  if (blockIdx.x != 0 || threadIdx.x >= 32) return;
  const unsigned char* payload = reinterpret_cast<const unsigned char*>(p.a.scratch);
  float bv = -INFINITY;
  int bi = 0x7fffffff;
  int polls = 0;
  bool failed = false;
#pragma unroll 1
  for (int c = threadIdx.x; c < (int)gridDim.x && !failed; c += 32) {
    uint2 a = ss_ld_stamped(payload + (size_t)c * 16), b = ss_ld_stamped(payload + (size_t)c * 16 + 8);
    while (a.y != p.a.epoch || b.y != p.a.epoch) {
      if (++polls > SS_POLL_LIMIT) { failed = true; break; }
      a = ss_ld_stamped(payload + (size_t)c * 16);
      b = ss_ld_stamped(payload + (size_t)c * 16 + 8);
    }
    const float v = __uint_as_float(a.x);
    const int i = (int)b.x;
    if (v > bv || (v == bv && i < bi)) { bv = v; bi = i; }
  }
  failed = __any_sync(0xffffffffu, failed);
#pragma unroll 1
  for (int offset = 16; offset > 0; offset >>= 1) {
    const float ov = __shfl_xor_sync(0xffffffffu, bv, offset);
    const int oi = __shfl_xor_sync(0xffffffffu, bi, offset);
    if (ov > bv || (ov == bv && oi < bi)) { bv = ov; bi = oi; }
  }
  if (SHARDED && p.a.world > 1 && !failed) {
    // every rank holds a slice of the vocabulary: the ranks' best (logit, index in the whole
    // vocabulary) meet in every rank's exchange slots; the largest wins, the lowest index on ties
    bi += p.a.vocab_offset;
    unsigned char* slots = reinterpret_cast<unsigned char*>(p.a.pick_exchange);
    if (threadIdx.x == 0) {
#pragma unroll 1
      for (int q = 0; q < p.a.world; ++q) {
        unsigned char* at = slots + (size_t)p.a.rank * 16 + p.a.peer_delta[q];
        ss_st_stamped_sys(at, __float_as_uint(bv), p.a.epoch);
        ss_st_stamped_sys(at + 8, (uint32_t)bi, p.a.epoch);
      }
    }
    bv = -INFINITY;
    bi = 0x7fffffff;
    if ((int)threadIdx.x < p.a.world) {
      const unsigned char* at = slots + (size_t)threadIdx.x * 16;
      uint2 a = ss_ld_stamped_sys(at), b = ss_ld_stamped_sys(at + 8);
      for (int waits = 0; a.y != p.a.epoch || b.y != p.a.epoch; ++waits) {
        if (waits > SS_POLL_LIMIT || ((waits & 255) == 255 && ss_ld_status(p.a.status) != 0)) { failed = true; break; }
        a = ss_ld_stamped_sys(at);
        b = ss_ld_stamped_sys(at + 8);
      }
      bv = __uint_as_float(a.x);
      bi = (int)b.x;
    }
    failed = __any_sync(0xffffffffu, failed);
#pragma unroll 1
    for (int offset = 16; offset > 0; offset >>= 1) {
      const float ov = __shfl_xor_sync(0xffffffffu, bv, offset);
      const int oi = __shfl_xor_sync(0xffffffffu, bi, offset);
      if (ov > bv || (ov == bv && oi < bi)) { bv = ov; bi = oi; }
    }
  }
  if (threadIdx.x == 0 && !failed) {
    p.a.token[0] = (long long)bi;
    if (p.a.counters != nullptr) {
      const int step = p.a.counters[1];
      if (p.a.generated != nullptr && step < p.a.generated_capacity) p.a.generated[step] = (long long)bi;
      p.a.counters[0] += 1;
      p.a.counters[1] = step + 1;
    }
  }
  if (threadIdx.x == 0 && failed) atomicCAS(p.a.status, 0, stage_index + 1);
}

// Everything a CTA sets up once per launch: descriptors and its column of the table into shared
// memory, barriers, the rotary rows of the step's position, and every warp's first requests.
__device__ __noinline__ void ss_start(const SSParams& p, unsigned char* smem, WarpStream& ws, int valid_length,
                                      long long position) {
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int depth = p.a.ring_depth;
  {
    const uint4* src = reinterpret_cast<const uint4*>(p.a.stages);
    uint4* dst = reinterpret_cast<uint4*>(smem + p.L.stages);
    const int words = p.a.stage_count * (int)(sizeof(aoto_stream_stage) / 16);
    for (int i = tid; i < words; i += SS_THREADS) dst[i] = ldg_nc_u4(src + i);
    uint32_t* table = reinterpret_cast<uint32_t*>(smem + p.L.table);
    for (int s = tid; s < p.a.stage_count; s += SS_THREADS)
      table[s] = ldg_nc_u32(p.a.cta_table + (size_t)s * gridDim.x + blockIdx.x);
  }
  if (tid == 0) {
    for (int i = 0; i < SS_WARPS * AOTO_STREAM_MAX_RING; ++i) ss_mbar_init(ss_smem(smem + p.L.bars) + i * 8, 1);
    for (int i = 0; i < SS_WARPS; ++i) ss_mbar_init(ss_smem(smem + p.L.kvbars) + i * 8, 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (p.a.first_attention >= 0 && ((int)blockIdx.x < p.a.query_heads || p.L.long_window) && tid < 2 * p.a.head_dim) {
    // the rotary rows of the step's position: fetched once, off every layer's critical path
    long long pos = max(0ll, min(position, (long long)p.a.table_rows - 1));
    const int D = p.a.head_dim;
    const bf16* table = reinterpret_cast<const bf16*>(tid < D ? p.a.cos_table : p.a.sin_table);
    reinterpret_cast<bf16*>(smem + p.L.rotary)[tid] = table[(size_t)pos * D + (tid < D ? tid : tid - D)];
  }
  __syncthreads();
  // every warp starts its stream: `depth` pieces in flight before anything is awaited
  const uint4 start = ldg_nc_u4(reinterpret_cast<const uint4*>(p.a.starts) + (size_t)blockIdx.x * SS_WARPS + warp);
  ws.issue_offset = (unsigned long long)start.x * 16ull;
  ws.ring = ss_smem(smem + p.L.ring) + (uint32_t)warp * depth * SS_SLOT_BYTES;
  ws.bars = ss_smem(smem + p.L.bars) + (uint32_t)warp * AOTO_STREAM_MAX_RING * 8;
  ws.next_stage = start.z >> 16;
  ws.slot = 0; ws.parity = 0; ws.issue_slot = 0; ws.in_flight = 0;
  const uint32_t sizes[3] = {(start.y & 0xFFFFu) * 16u, (start.y >> 16) * 16u, (start.z & 0xFFFFu) * 16u};
#pragma unroll
  for (int i = 0; i < AOTO_STREAM_MAX_RING; ++i)
    if (i < depth && sizes[i] != 0) ss_request(p, ws, sizes[i], lane);
}

template <bool TRACE, bool LONG, bool SHARDED>
__global__ void __launch_bounds__(SS_THREADS, 1) stream_step_kernel(const __grid_constant__ SSParams p) {
  extern __shared__ uint4 ss_raw[];
  unsigned char* smem = reinterpret_cast<unsigned char*>(ss_raw);
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;

  // the step's position and window
  int valid_length = 0;
  long long position = 0;
  if (p.a.window) {
    valid_length = *reinterpret_cast<const volatile int*>(p.a.counters);
    position = valid_length - 1;
  } else if (p.a.position != nullptr) {
    position = *reinterpret_cast<const volatile long long*>(p.a.position);
  }
  WarpStream ws;
  ss_start(p, smem, ws, valid_length, position);
  uint32_t kv_parity = 0;
  bool kv_pending = false;
  const aoto_stream_stage* stages = reinterpret_cast<const aoto_stream_stage*>(smem + p.L.stages);
  const WindowShare share = ss_window_share(p, warp, valid_length, smem);
  if (!LONG && p.a.first_attention >= 0) {
    ss_request_window(p, stages[p.a.first_attention], share, lane);
    kv_pending = true;
  }

  Best best;
  best.value = -INFINITY;
  best.index = 0x7fffffff;
  const uint32_t* table = reinterpret_cast<const uint32_t*>(smem + p.L.table);
  bool alive = true;
#pragma unroll 1
  for (int s = 0; s < p.a.stage_count && alive; ++s) {
    const aoto_stream_stage& st = stages[s];
    if (st.kind == AOTO_STAGE_GEMV) {
      const uint32_t entry = table[s];
      if (((entry >> 16) & 0x7FFFu) != 0) {
        alive = ss_gemv<TRACE, SHARDED>(p, st, s, entry, ws, best, smem);
      } else if ((st.flags & AOTO_STAGE_FLAG_ARGMAX) && tid == 0) {
        // a CTA without rows of the last projection still answers the pick stage's poll
        unsigned char* payload = reinterpret_cast<unsigned char*>(p.a.scratch);
        ss_st_stamped(payload + (size_t)blockIdx.x * 16, __float_as_uint(-INFINITY), p.a.epoch);
        ss_st_stamped(payload + (size_t)blockIdx.x * 16 + 8, 0x7fffffffu, p.a.epoch);
      }
    } else if (st.kind == AOTO_STAGE_ATTENTION) {
      if constexpr (LONG) alive = ss_attention_spread<TRACE>(p, st, s, valid_length, smem);
      else alive = ss_attention<TRACE>(p, st, s, share, kv_parity, kv_pending, smem);
    } else if (st.kind == AOTO_STAGE_PICK) {
      ss_pick<SHARDED>(p, s);
    }
  }
  if (!alive) {
    // a wait ran out: nothing may still be travelling into this CTA's shared memory when it leaves
    while (ws.in_flight > 0) {
      ss_mbar_wait(ws.bars + ws.slot * 8, ws.parity);
      ws.slot += 1;
      if (ws.slot == (uint32_t)p.a.ring_depth) { ws.slot = 0; ws.parity ^= 1u; }
      ws.in_flight -= 1;
    }
    if (kv_pending && share.head >= 0 && share.old_keys > 0) ss_mbar_wait(share.bar, kv_parity);
  }
}

static int ss_check(const aoto_stream_step_args& a, SSLayout* layout) {
  if (a.stage_count <= 0 || a.stage_count >= (int)AOTO_STREAM_NO_STAGE || a.ctas <= 0 || a.ctas > 1024) return 0;
  if (a.ring_depth < 2 || a.ring_depth > AOTO_STREAM_MAX_RING) return 0;
  if (a.max_k <= 0 || a.max_k > SS_MAX_K || (a.max_k & 127)) return 0;
  if (a.world < 0 || a.world > 8 || (a.world > 1 && (a.rank < 0 || a.rank >= a.world))) return 0;
  const bool has_attention = a.first_attention >= 0;
  if (has_attention) {
    if (a.head_dim != 64 && a.head_dim != 128) return 0;
    if (a.kv_heads <= 0 || a.query_heads <= 0 || a.query_heads % a.kv_heads) return 0;
    if (a.query_heads > a.ctas || a.capacity < 2) return 0;
    if (a.capacity > (1 << 20)) return 0;
    if (3 * (a.head_dim >> 1) > SS_THREADS) return 0;
    if ((a.query_start | a.key_start | a.value_start) & 1) return 0;
    if (a.table_rows <= 0 || a.attention_stages <= 0) return 0;
  }
  const int group = has_attention ? a.query_heads / a.kv_heads : 1;
  const int slices_max = has_attention ? ss_slices_max(a.ctas, a.kv_heads, a.capacity) : 1;
  *layout = ss_layout(a.stage_count, a.max_k, a.ring_depth, a.capacity, a.head_dim, has_attention, false, group, slices_max);
  if (has_attention && !layout->long_window) {
    // wide heads and long rows together can leave no room for the per-warp key / value buffers:
    // the window is then read from L2 as a long one is
    int device = 0, limit = 227 * 1024;
    if (cudaGetDevice(&device) != cudaSuccess ||
        cudaDeviceGetAttribute(&limit, cudaDevAttrMaxSharedMemoryPerBlockOptin, device) != cudaSuccess) {
      (void)cudaGetLastError();
      limit = 227 * 1024;
    }
    if ((int64_t)layout->total > (int64_t)limit)
      *layout = ss_layout(a.stage_count, a.max_k, a.ring_depth, a.capacity, a.head_dim, has_attention, true, group,
                          slices_max);
  }
  // the spread form polls the group's queries, key and value with one thread per stamped word
  if (layout->long_window && (group + 2) * (a.head_dim >> 1) > SS_THREADS) return 0;
  return 1;
}

// Scratch the kernel needs: the per-CTA maxima of the pick stage, then (long window) every head's
// partial attention results of all slices.
static int64_t ss_scratch_bytes(const aoto_stream_step_args& a, const SSLayout& L) {
  int64_t need = (int64_t)a.ctas * 16;
  if (L.long_window) need += (int64_t)a.attention_stages * a.query_heads * L.slices_max * (a.head_dim + 2) * 8;
  return need;
}

}  // namespace aoto

using namespace aoto;

extern "C" int aoto_sm100_stream_stage_size(void) { return (int)sizeof(aoto_stream_stage); }
extern "C" int aoto_sm100_stream_args_size(void) { return (int)sizeof(aoto_stream_step_args); }

extern "C" int64_t aoto_sm100_stream_step_scratch_bytes(int32_t ctas) { return ctas > 0 ? (int64_t)ctas * 16 : 0; }

extern "C" int64_t aoto_sm100_stream_step_smem_bytes(const aoto_stream_step_args* a) {
  SSLayout L;
  if (!a || !ss_check(*a, &L)) return -1;
  return (int64_t)L.total;
}

extern "C" int64_t aoto_sm100_stream_step_scratch_bytes_for(const aoto_stream_step_args* a) {
  SSLayout L;
  if (!a || !ss_check(*a, &L)) return -1;
  return ss_scratch_bytes(*a, L);
}

extern "C" int aoto_sm100_stream_step(const aoto_stream_step_args* a, void* stream_) {
  if (!a || !a->stages || !a->cta_table || !a->duties || !a->starts || !a->stream || !a->status || !a->scratch ||
      a->epoch == 0)
    return AOTO_ERR_ARGUMENT;
  if (!aligned_to(a->stream, 16) || !aligned_to(a->stages, 16) || !aligned_to(a->starts, 16)) return AOTO_ERR_ARGUMENT;
  if (a->scratch_bytes < aoto_sm100_stream_step_scratch_bytes(a->ctas)) return AOTO_ERR_ARGUMENT;
  SSParams params;
  params.a = *a;
  if (params.a.world <= 1) {  // one GPU: nothing is exchanged
    params.a.world = 1;
    params.a.rank = 0;
  } else if (!a->pick_exchange) {
    return AOTO_ERR_ARGUMENT;
  }
  if (!ss_check(*a, &params.L)) return AOTO_ERR_UNSUPPORTED;
  if (a->scratch_bytes < ss_scratch_bytes(*a, params.L)) return AOTO_ERR_ARGUMENT;
  int device = 0, sms = 0, coop = 0, smem_limit = 0;
  if (cudaGetDevice(&device) != cudaSuccess) {
    (void)cudaGetLastError();
    return AOTO_ERR_LAUNCH;
  }
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device);
  cudaDeviceGetAttribute(&coop, cudaDevAttrCooperativeLaunch, device);
  cudaDeviceGetAttribute(&smem_limit, cudaDevAttrMaxSharedMemoryPerBlockOptin, device);
  if (!coop || (int64_t)params.L.total > (int64_t)smem_limit) return AOTO_ERR_UNSUPPORTED;
  // two instantiations: the marks of the per-stage timeline cost issue slots, so the kernel that
  // serves requests carries none
  // and two more for the window form, so that neither carries the other's code
  const bool traced = a->trace != nullptr, lengthy = params.L.long_window != 0, sharded = params.a.world > 1;
  // the exchange between GPUs is a third switch: a single GPU's kernel carries none of its code
  using Kernel = void (*)(const SSParams);
  static const Kernel kernels[8] = {
      stream_step_kernel<false, false, false>, stream_step_kernel<false, false, true>,
      stream_step_kernel<false, true, false>,  stream_step_kernel<false, true, true>,
      stream_step_kernel<true, false, false>,  stream_step_kernel<true, false, true>,
      stream_step_kernel<true, true, false>,   stream_step_kernel<true, true, true>,
  };
  const int which = (traced ? 4 : 0) + (lengthy ? 2 : 0) + (sharded ? 1 : 0);
  Kernel kernel = kernels[which];
  static PerDeviceOnce raised[8];
  if (raise_dynamic_smem(kernel, (size_t)smem_limit, raised[which]) != AOTO_OK) return AOTO_ERR_LAUNCH;
  int per_sm = 0;
  if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, kernel, SS_THREADS, params.L.total) != cudaSuccess ||
      per_sm < 1) {
    (void)cudaGetLastError();
    return AOTO_ERR_UNSUPPORTED;
  }
  if (a->ctas > sms * per_sm) return AOTO_ERR_UNSUPPORTED;  // every CTA must be resident: they wait on one another
  cudaLaunchConfig_t config = {};
  config.gridDim = dim3(a->ctas);
  config.blockDim = dim3(SS_THREADS);
  config.dynamicSmemBytes = params.L.total;
  config.stream = (cudaStream_t)stream_;
  cudaLaunchAttribute attribute[1];
  attribute[0].id = cudaLaunchAttributeCooperative;
  attribute[0].val.cooperative = 1;
  config.attrs = attribute;
  config.numAttrs = 1;
  if (cudaLaunchKernelEx(&config, kernel, params) != cudaSuccess) {
    (void)cudaGetLastError();
    return AOTO_ERR_LAUNCH;
  }
  return AOTO_OK;
}
