// Grouped-query attention over the static bf16 KV cache.
//
//  * decode (q_len == 1): FlashDecoding-style. grid = (kv heads, key splits);
//    each CTA stages its K/V tiles with async copies, scores them for every
//    query head of the group, keeps fp32 softmax statistics and a partial
//    weighted sum of V. With one split the CTA writes the output rows itself;
//    with several it writes (max, sum, acc[D]) to scratch and the last CTA of
//    the kv head to arrive merges them in split order.
//  * prefill (q_len > 1): one warp per (head, query row), keys in tiles of 32
//    with an online softmax.
//
// Softmax follows the "safe" rule of the reference: a row whose keys are all
// masked produces zeros, never NaN.
#include "attention.cuh"

namespace aoto {

constexpr int DECODE_THREADS = 128;

__device__ __forceinline__ void cp_async_16(void* smem_dst, const void* gmem_src) {
  const uint32_t dst = (uint32_t)__cvta_generic_to_shared(smem_dst);
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(gmem_src) : "memory");
}
__device__ __forceinline__ void cp_async_wait_all() {
  asm volatile("cp.async.commit_group;\ncp.async.wait_group 0;" ::: "memory");
}

// Decode: one CTA per (kv head, key split). The CTA pulls its K and V tiles
// into shared memory with 16-byte async copies issued all at once (a decode
// step is latency bound: what matters is that every load of the CTA is in
// flight together), scores them against ALL query heads of the group (the
// tiles are read from HBM once per group, not once per query head), and keeps
// fp32 softmax statistics. With several splits the partial (max, sum, acc[D])
// of every query head goes to scratch and the last CTA of the kv head to
// finish merges them in split order; the arrival counter it used is left at
// zero for the next launch.
//
// Rows of the shared tiles are padded by 16 bytes so that a warp reading one
// key per lane touches every bank once.
__global__ void __launch_bounds__(DECODE_THREADS)
attention_decode_kernel(const AttnParams p) {
  extern __shared__ uint4 smem4[];
  const int D = p.D, G = p.QH / p.KVH, TK = p.keys_per_split;
  const int row_bytes = D * 2 + 16;
  unsigned char* kt = reinterpret_cast<unsigned char*>(smem4);
  unsigned char* vt = kt + (size_t)TK * row_bytes;
  float* qs = reinterpret_cast<float*>(vt + (size_t)TK * row_bytes);  // G*D, scaled
  float* sc = qs + G * D;                                             // G*TK scores -> weights
  float* stat = sc + G * TK;                                          // G*2 (max, sum)
  float* madd = stat + G * 2;                                         // TK additive mask
  __shared__ int is_last;

  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int kvh = blockIdx.x, split = blockIdx.y;
  const int k0 = split * TK;
  const int nkeys = min(TK, p.Lk - k0);
  pdl_wait_for_producers();
  pdl_release_dependents();

  // all loads of the tile first
  const int chunks = D >> 3;  // 16-byte chunks per row
  const bf16* kbase = p.k + ((size_t)kvh * p.Lk + k0) * D;
  const bf16* vbase = p.v + ((size_t)kvh * p.Lk + k0) * D;
  for (int c = tid; c < nkeys * chunks; c += DECODE_THREADS) {
    const int r = c / chunks, j = c - r * chunks;
    cp_async_16(kt + (size_t)r * row_bytes + j * 16, kbase + (size_t)r * D + j * 8);
    cp_async_16(vt + (size_t)r * row_bytes + j * 16, vbase + (size_t)r * D + j * 8);
  }
  for (int i = tid; i < G * D; i += DECODE_THREADS)
    qs[i] = __bfloat162float(p.q[(size_t)kvh * G * D + i]) * p.scale;
  for (int i = tid; i < TK; i += DECODE_THREADS)
    madd[i] = (i < nkeys) ? (p.mask ? __bfloat162float(p.mask[k0 + i]) : 0.f) : -INFINITY;
  cp_async_wait_all();
  __syncthreads();

  // scores: thread <-> (key, head) pairs
  for (int item = tid; item < G * TK; item += DECODE_THREADS) {
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
      s = dot + m_add;
    }
    sc[item] = s;
  }
  __syncthreads();
  // per-head max and sum: one warp per head (round robin)
  for (int h = warp; h < G; h += DECODE_THREADS / 32) {
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
  // P.V: thread <-> (head, dim pair)
  const int pairs = D >> 1;
  for (int item = tid; item < G * pairs; item += DECODE_THREADS) {
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
    if (p.splits == 1) {
      const float l = stat[2 * h + 1];
      const float inv = l > 0.f ? 1.f / l : 0.f;
      *reinterpret_cast<uint32_t*>(p.out + (size_t)head * D + dp * 2) = pack_bf16x2(a0 * inv, a1 * inv);
    } else {
      float* dst = p.scratch + SCRATCH_HEADER_BYTES / 4 + ((size_t)head * p.splits + split) * (D + 2);
      dst[2 + dp * 2] = a0;
      dst[3 + dp * 2] = a1;
      if (dp == 0) { dst[0] = stat[2 * h]; dst[1] = stat[2 * h + 1]; }
    }
  }
  if (p.splits == 1) return;

  // last CTA of this kv head merges the splits
  int* counters = reinterpret_cast<int*>(p.scratch);
  __threadfence();
  __syncthreads();
  if (tid == 0) {
    const int arrived = atomicAdd(counters + kvh, 1);
    is_last = (arrived == p.splits - 1);
    if (is_last) counters[kvh] = 0;  // ready for the next launch
  }
  __syncthreads();
  if (!is_last) return;
  __threadfence();
  // The partial results of the kv head's query heads lie next to each other in scratch. They are
  // staged in this CTA's shared memory (free now) with coalesced loads that are all in flight
  // together - as many heads at a time as fit - and merged from there: read one by one from L2,
  // the 3 * splits dependent-latency loads of every output element were most of a long window's
  // kernel time.
  const int per_head = p.splits * (D + 2);
  const int region = (2 * TK * row_bytes) / 4 + G * D + G * TK + G * 2 + TK;  // floats of the dynamic region
  const float* group = p.scratch + SCRATCH_HEADER_BYTES / 4 + (size_t)kvh * G * per_head;
  float* staged = reinterpret_cast<float*>(smem4);
  const int heads_per_round = min(G, region / per_head);
  if (heads_per_round >= 1) {
    for (int h0 = 0; h0 < G; h0 += heads_per_round) {
      const int heads = min(heads_per_round, G - h0);
      const float* from = group + (size_t)h0 * per_head;
      __syncthreads();  // the previous round's readers are done with the staging area
#pragma unroll 8
      for (int i = tid; i < heads * per_head; i += DECODE_THREADS) staged[i] = __ldcg(from + i);
      __syncthreads();
      for (int item = tid; item < heads * D; item += DECODE_THREADS) {
        const int h = item / D, d = item - h * D;
        const float* base = staged + h * per_head;
        float m = -INFINITY;
        for (int s2 = 0; s2 < p.splits; ++s2) m = fmaxf(m, base[s2 * (D + 2)]);
        float acc = 0.f, l = 0.f;
        if (m != -INFINITY) {
          for (int s2 = 0; s2 < p.splits; ++s2) {
            const float* part = base + s2 * (D + 2);
            const float pm = part[0];
            const float w = (pm == -INFINITY) ? 0.f : expf(pm - m);
            acc = fmaf(w, part[2 + d], acc);
            l = fmaf(w, part[1], l);
          }
        }
        p.out[(size_t)(kvh * G + h0 + h) * D + d] = __float2bfloat16_rn(l > 0.f ? acc / l : 0.f);
      }
    }
    return;
  }
  // more splits than one head's partials fit in shared memory: merge straight from L2
  for (int item = tid; item < G * D; item += DECODE_THREADS) {
    const int h = item / D, d = item - h * D;
    const int head = kvh * G + h;
    const float* base = p.scratch + SCRATCH_HEADER_BYTES / 4 + (size_t)head * p.splits * (D + 2);
    float m = -INFINITY;
    for (int s2 = 0; s2 < p.splits; ++s2) m = fmaxf(m, __ldcg(base + (size_t)s2 * (D + 2)));
    float acc = 0.f, l = 0.f;
    if (m != -INFINITY) {
      for (int s2 = 0; s2 < p.splits; ++s2) {
        const float* part = base + (size_t)s2 * (D + 2);
        const float pm = __ldcg(part);
        const float w = (pm == -INFINITY) ? 0.f : expf(pm - m);
        acc = fmaf(w, __ldcg(part + 2 + d), acc);
        l = fmaf(w, __ldcg(part + 1), l);
      }
    }
    p.out[(size_t)head * D + d] = __float2bfloat16_rn(l > 0.f ? acc / l : 0.f);
  }
}

// Prefill: warp per (head, query row). Lanes hold one key each while scoring a
// tile of 32 keys, then cover D while accumulating P.V.
constexpr int PREFILL_WARPS = 4;
constexpr int MAX_D_PER_LANE = 8;  // D <= 256

__global__ void __launch_bounds__(PREFILL_WARPS * 32)
attention_prefill_kernel(const AttnParams p) {
  extern __shared__ float sm[];
  const int D = p.D;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int64_t rowid = (int64_t)blockIdx.x * PREFILL_WARPS + warp;
  float* qs = sm + warp * D;
  if (rowid >= (int64_t)p.QH * p.Lq) return;
  const int head = (int)(rowid / p.Lq), qi = (int)(rowid % p.Lq);
  const int kvh = head / (p.QH / p.KVH);
  const bf16* qrow = p.q + ((size_t)head * p.Lq + qi) * D;
  for (int d = lane; d < D; d += 32) qs[d] = __bfloat162float(qrow[d]) * p.scale;
  __syncwarp();
  const bf16* kbase = p.k + (size_t)kvh * p.Lk * D;
  const bf16* vbase = p.v + (size_t)kvh * p.Lk * D;
  const bf16* mrow = p.mask ? p.mask + (size_t)qi * p.Lk : nullptr;

  float m = -INFINITY, l = 0.f;
  float acc[MAX_D_PER_LANE];
#pragma unroll
  for (int i = 0; i < MAX_D_PER_LANE; ++i) acc[i] = 0.f;
  const int last_key = p.causal ? min(p.Lk, qi + 1) : p.Lk;

  for (int t0 = 0; t0 < last_key; t0 += 32) {
    const int key = t0 + lane;
    float s = -INFINITY;
    if (key < last_key) {
      const float madd = mrow ? __bfloat162float(mrow[key]) : 0.f;
      if (madd != -INFINITY) {
        const uint32_t* krow = reinterpret_cast<const uint32_t*>(kbase + (size_t)key * D);
        float dot = 0.f;
        for (int d2 = 0; d2 < (D >> 1); ++d2) {
          const uint32_t kk = krow[d2];
          dot = fmaf(bf16x2_lo(kk), qs[2 * d2], dot);
          dot = fmaf(bf16x2_hi(kk), qs[2 * d2 + 1], dot);
        }
        s = dot + madd;
      }
    }
    const float tile_max = warp_max(s);
    if (tile_max == -INFINITY) continue;  // whole tile masked (warp-uniform)
    const float m_new = fmaxf(m, tile_max);
    const float correction = (m == -INFINITY) ? 0.f : expf(m - m_new);
    const float e = (s == -INFINITY) ? 0.f : expf(s - m_new);
    l = l * correction + warp_sum(e);
#pragma unroll
    for (int i = 0; i < MAX_D_PER_LANE; ++i) acc[i] *= correction;
    const int tile = min(32, last_key - t0);
    for (int j = 0; j < tile; ++j) {
      const float w = __shfl_sync(0xffffffffu, e, j);
      if (w != 0.f) {
        const bf16* vrow = vbase + (size_t)(t0 + j) * D;
#pragma unroll
        for (int i = 0; i < MAX_D_PER_LANE; ++i) {
          const int d = lane + 32 * i;
          if (d < D) acc[i] = fmaf(w, __bfloat162float(vrow[d]), acc[i]);
        }
      }
    }
    m = m_new;
  }
  const float inv = l > 0.f ? 1.f / l : 0.f;
  bf16* orow = p.out + ((size_t)head * p.Lq + qi) * D;
#pragma unroll
  for (int i = 0; i < MAX_D_PER_LANE; ++i) {
    const int d = lane + 32 * i;
    if (d < D) orow[d] = __float2bfloat16_rn(acc[i] * inv);
  }
}

// Keys per CTA and number of splits for the decode kernel. Short contexts are
// latency bound: small tiles so that a handful of CTAs per kv head share the
// window. Long contexts are bandwidth bound: enough CTAs to cover the machine,
// tiles capped by shared memory.
static void decode_tiling(const aoto_attention_args& a, int* keys_per_split, int* splits) {
  int tile = a.head_dim <= 128 ? 64 : 32;
  if (a.kv_len <= 32) tile = 32;
  *keys_per_split = tile;
  *splits = (a.kv_len + tile - 1) / tile;
}

}  // namespace aoto

using namespace aoto;

extern "C" int64_t aoto_sm100_attention_scratch_bytes(const aoto_attention_args* a) {
  if (!a || a->q_len <= 0 || a->kv_len <= 0 || a->head_dim <= 0) return 0;
  if (a->q_len > 1) {
    // the tiled prefill kernel classifies the tiles of a long mask into an optional workspace
    AttnParams p = {};
    p.q = (const bf16*)a->q; p.k = (const bf16*)a->k; p.v = (const bf16*)a->v;
    p.mask = (const bf16*)a->mask; p.out = (bf16*)a->out;
    p.Lq = a->q_len; p.Lk = a->kv_len; p.D = a->head_dim;
    return attention_prefill_scratch_bytes(p);
  }
  int tile, splits;
  decode_tiling(*a, &tile, &splits);
  if (splits == 1) return 0;
  return SCRATCH_HEADER_BYTES + (int64_t)a->query_heads * splits * (a->head_dim + 2) * 4;
}

extern "C" int aoto_sm100_attention(const aoto_attention_args* a, void* stream_) {
  cudaStream_t stream = (cudaStream_t)stream_;
  if (!a || !a->q || !a->k || !a->v || !a->out) return AOTO_ERR_ARGUMENT;
  if (a->query_heads <= 0 || a->kv_heads <= 0 || a->q_len <= 0 || a->kv_len <= 0 || a->head_dim <= 0)
    return AOTO_ERR_ARGUMENT;
  if (a->query_heads % a->kv_heads != 0) return AOTO_ERR_ARGUMENT;
  if ((a->head_dim & 1) || a->head_dim > 256) return AOTO_ERR_UNSUPPORTED;
  if (!aligned_to(a->k, 4) || !aligned_to(a->v, 4)) return AOTO_ERR_ARGUMENT;
  AttnParams p = {};
  p.q = (const bf16*)a->q; p.k = (const bf16*)a->k; p.v = (const bf16*)a->v;
  p.mask = (const bf16*)a->mask; p.out = (bf16*)a->out; p.scratch = (float*)a->scratch;
  p.QH = a->query_heads; p.KVH = a->kv_heads; p.Lq = a->q_len; p.Lk = a->kv_len; p.D = a->head_dim;
  p.causal = a->causal; p.scale = a->scale;
  // One query under the top-left aligned causal rule sees key 0 only; the split-KV decode kernel
  // attends the whole window, so that case goes to the prefill kernels, which apply the rule.
  const bool causal_single = a->causal && a->kv_len > 1;
  if (a->q_len == 1 && !causal_single) {
    if ((a->head_dim & 7) || !aligned_to(a->k, 16) || !aligned_to(a->v, 16)) return AOTO_ERR_UNSUPPORTED;
    decode_tiling(*a, &p.keys_per_split, &p.splits);
    if (p.splits > 1) {
      if (a->kv_heads > SCRATCH_MAX_COUNTERS) return AOTO_ERR_UNSUPPORTED;
      const int64_t need = aoto_sm100_attention_scratch_bytes(a);
      if (!a->scratch || a->scratch_bytes < need || !aligned_to(a->scratch, 4)) return AOTO_ERR_ARGUMENT;
    }
    const int G = a->query_heads / a->kv_heads;
    const size_t smem = (size_t)2 * p.keys_per_split * (a->head_dim * 2 + 16) +
                        ((size_t)G * a->head_dim + (size_t)G * p.keys_per_split + (size_t)G * 2 +
                         p.keys_per_split) * 4;
    if (smem > 48 * 1024) {
      static PerDeviceOnce raised;
      if (raise_dynamic_smem(attention_decode_kernel, 160 * 1024, raised) != AOTO_OK) return AOTO_ERR_LAUNCH;
      if (smem > 160 * 1024) return AOTO_ERR_UNSUPPORTED;
    }
    return launch_kernel(attention_decode_kernel, dim3(a->kv_heads, p.splits), dim3(DECODE_THREADS),
                         smem, stream, false, p);
  }
  p.splits = 1;
  p.keys_per_split = 0;
  if (attention_prefill_mma_applies(p)) return attention_prefill_mma_launch(p, a->scratch ? a->scratch_bytes : 0, stream);
  const int64_t rows = (int64_t)a->query_heads * a->q_len;
  const size_t smem = (size_t)PREFILL_WARPS * a->head_dim * 4;
  return launch_kernel(attention_prefill_kernel, dim3((unsigned)((rows + PREFILL_WARPS - 1) / PREFILL_WARPS)),
                       dim3(PREFILL_WARPS * 32), smem, stream, false, p);
}


// ---------------------------------------------------------------------------
// Decode attention for callers that must not allocate
// ---------------------------------------------------------------------------
//
// Some hosts of this library are not allowed to allocate device memory once they are running: a
// serving process whose memory was carved up at start-up and which treats any later cudaMalloc
// as a bug, an integrator that links the library into a runtime with its own sealed pool and no
// way to hand a workspace through, a latency-critical loop where the allocator (which may
// synchronise the whole device) is banned outright. The split-KV decode kernel needs a scratch
// buffer for its per-split partial results, and every other route to it goes through a buffer
// the caller allocates. This entry point gives such callers the same kernel with the scratch in
// a fixed array that is part of the library image.
//
// The array is AOTO_STATIC_SCRATCH_BYTES long and every GPU that loads the library holds one
// copy of it until the process exits. `static_scratch` below is the HOST-side handle of that
// array, not a device address; the device address is looked up once per device with
// cudaGetSymbolAddress (with that device current) and cached.
static __device__ __align__(256) unsigned char static_scratch[AOTO_STATIC_SCRATCH_BYTES];

namespace {
void* static_scratch_address[MAX_DEVICES] = {};

// Device address of the static scratch array on the current device, or nullptr.
void* static_scratch_on_current_device() {
  int device = -1;
  if (cudaGetDevice(&device) != cudaSuccess || device < 0 || device >= MAX_DEVICES) {
    (void)cudaGetLastError();
    return nullptr;
  }
  if (static_scratch_address[device] == nullptr) {
    void* address = nullptr;
    if (cudaGetSymbolAddress(&address, static_scratch) != cudaSuccess || address == nullptr) {
      (void)cudaGetLastError();
      return nullptr;
    }
    static_scratch_address[device] = address;  // racing first calls store the same value
  }
  return static_scratch_address[device];
}
}  // namespace

extern "C" int64_t aoto_sm100_attention_static_scratch_limit(void) { return AOTO_STATIC_SCRATCH_BYTES; }

extern "C" int aoto_sm100_attention_decode_static(const aoto_attention_args* a, void* stream_) {
  if (!a) return AOTO_ERR_ARGUMENT;
  if (a->q_len != 1) return AOTO_ERR_UNSUPPORTED;  // the prefill kernel runs without a workspace: call aoto_sm100_attention
  const int64_t need = aoto_sm100_attention_scratch_bytes(a);
  if (need > AOTO_STATIC_SCRATCH_BYTES) return AOTO_ERR_TOO_LARGE;
  void* scratch = static_scratch_on_current_device();
  if (scratch == nullptr) return AOTO_ERR_LAUNCH;
  cudaStream_t stream = (cudaStream_t)stream_;
  if (need > 0) {
    // The arrival counters at the head of the array must be zero when the kernel starts. The
    // kernel leaves them at zero, but the array is shared by every call and keeps whatever the
    // last one left behind (an aborted launch included), so they are cleared on the stream.
    if (cudaMemsetAsync(scratch, 0, SCRATCH_HEADER_BYTES, stream) != cudaSuccess) {
      (void)cudaGetLastError();
      return AOTO_ERR_LAUNCH;
    }
  }
  aoto_attention_args with_scratch = *a;
  with_scratch.scratch = scratch;
  with_scratch.scratch_bytes = AOTO_STATIC_SCRATCH_BYTES;
  return aoto_sm100_attention(&with_scratch, stream_);
}
