// Grouped-query attention over the static bf16 KV cache.
//
//  * decode (q_len == 1): FlashDecoding-style. grid = (query heads, key splits);
//    each CTA scores its key range, keeps fp32 softmax statistics and a partial
//    weighted sum of V. With one split the CTA writes the output row itself;
//    with several it writes (max, sum, acc[D]) to scratch and a small combine
//    kernel merges them in split order.
//  * prefill (q_len > 1): one warp per (head, query row), keys in tiles of 32
//    with an online softmax.
//
// Softmax follows the "safe" rule of the reference: a row whose keys are all
// masked produces zeros, never NaN.
#include "common.cuh"

namespace aoto {

struct AttnParams {
  const bf16* q;
  const bf16* k;
  const bf16* v;
  const bf16* mask;
  bf16* out;
  float* scratch;
  int QH, KVH, Lq, Lk, D;
  int causal, splits, keys_per_split;
  float scale;
};

constexpr int DECODE_THREADS = 128;

__global__ void __launch_bounds__(DECODE_THREADS)
attention_decode_kernel(const AttnParams p) {
  extern __shared__ float sm[];
  const int D = p.D;
  float* qs = sm;                       // D
  float* sc = qs + D;                   // keys_per_split
  float* red = sc + p.keys_per_split;   // 32
  float* pv = red + 32;                 // parts * D
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int head = blockIdx.x, split = blockIdx.y;
  const int kvh = head / (p.QH / p.KVH);
  const int k0 = split * p.keys_per_split;
  const int k1 = min(p.Lk, k0 + p.keys_per_split);
  const int nkeys = k1 - k0;
  pdl_wait_for_producers();
  pdl_release_dependents();

  for (int d = tid; d < D; d += DECODE_THREADS)
    qs[d] = __bfloat162float(p.q[(size_t)head * D + d]) * p.scale;
  __syncthreads();

  const bf16* kbase = p.k + (size_t)kvh * p.Lk * D;
  const bf16* vbase = p.v + (size_t)kvh * p.Lk * D;

  // scores: one warp per key, lanes over D (pairs)
  float local_max = -INFINITY;
  for (int i = warp; i < nkeys; i += DECODE_THREADS / 32) {
    const int key = k0 + i;
    float madd = 0.f;
    if (p.mask != nullptr) madd = __bfloat162float(p.mask[key]);
    float s = -INFINITY;
    if (madd != -INFINITY) {  // warp-uniform: skip masked keys without reading them
      const uint32_t* krow = reinterpret_cast<const uint32_t*>(kbase + (size_t)key * D);
      float dot = 0.f;
      for (int d2 = lane; d2 < (D >> 1); d2 += 32) {
        const uint32_t kk = krow[d2];
        dot = fmaf(bf16x2_lo(kk), qs[2 * d2], dot);
        dot = fmaf(bf16x2_hi(kk), qs[2 * d2 + 1], dot);
      }
      s = warp_sum(dot) + madd;
    }
    if (lane == 0) sc[i] = s;
    local_max = fmaxf(local_max, s);
  }
  // block max
  __syncthreads();
  if (lane == 0) red[warp] = local_max;
  __syncthreads();
  float m = -INFINITY;
  for (int w = 0; w < DECODE_THREADS / 32; ++w) m = fmaxf(m, red[w]);
  const float m_safe = (m == -INFINITY) ? 0.f : m;

  float lsum = 0.f;
  for (int i = tid; i < nkeys; i += DECODE_THREADS) {
    const float s = sc[i];
    const float e = (s == -INFINITY) ? 0.f : expf(s - m_safe);
    sc[i] = e;
    lsum += e;
  }
  const float l = block_sum(lsum, red);  // also orders the sc[] writes

  // P.V: threads_per_row lanes cover D in pairs; the remaining factor splits keys
  const int tpr = D >> 1;
  const int parts = DECODE_THREADS / tpr;  // >= 1 because D <= 256
  const int part = tid / tpr, dpair = tid % tpr;
  float a0 = 0.f, a1 = 0.f;
  if (part < parts) {
    for (int i = part; i < nkeys; i += parts) {
      const float w = sc[i];
      if (w != 0.f) {
        const uint32_t vv = reinterpret_cast<const uint32_t*>(vbase + (size_t)(k0 + i) * D)[dpair];
        a0 = fmaf(w, bf16x2_lo(vv), a0);
        a1 = fmaf(w, bf16x2_hi(vv), a1);
      }
    }
    pv[part * D + 2 * dpair] = a0;
    pv[part * D + 2 * dpair + 1] = a1;
  }
  __syncthreads();
  for (int d = tid; d < D; d += DECODE_THREADS) {
    float acc = 0.f;
    for (int q = 0; q < parts; ++q) acc += pv[q * D + d];
    if (p.splits == 1) {
      const float inv = l > 0.f ? 1.f / l : 0.f;
      p.out[(size_t)head * D + d] = __float2bfloat16_rn(acc * inv);
    } else {
      float* dst = p.scratch + ((size_t)head * p.splits + split) * (D + 2);
      dst[2 + d] = acc;
      if (d == 0) { dst[0] = m; dst[1] = l; }
    }
  }
}

__global__ void __launch_bounds__(128)
attention_combine_kernel(const AttnParams p) {
  const int head = blockIdx.x, D = p.D;
  const float* base = p.scratch + (size_t)head * p.splits * (D + 2);
  float m = -INFINITY;
  for (int s = 0; s < p.splits; ++s) m = fmaxf(m, base[(size_t)s * (D + 2)]);
  for (int d = threadIdx.x; d < D; d += blockDim.x) {
    float acc = 0.f, l = 0.f;
    if (m != -INFINITY) {
      for (int s = 0; s < p.splits; ++s) {
        const float* part = base + (size_t)s * (D + 2);
        const float w = (part[0] == -INFINITY) ? 0.f : expf(part[0] - m);
        acc = fmaf(w, part[2 + d], acc);
        l = fmaf(w, part[1], l);
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

static int decode_splits(const aoto_attention_args& a) {
  // one split per 512 keys keeps every CTA's score buffer small and gives the
  // long-context case enough CTAs to cover the machine
  if (a.kv_len <= 1024) return 1;
  return (a.kv_len + 511) / 512;
}

}  // namespace aoto

using namespace aoto;

extern "C" int64_t aoto_sm100_attention_scratch_bytes(const aoto_attention_args* a) {
  if (!a || a->q_len != 1) return 0;
  const int splits = decode_splits(*a);
  if (splits == 1) return 0;
  return (int64_t)a->query_heads * splits * (a->head_dim + 2) * 4;
}

extern "C" int aoto_sm100_attention(const aoto_attention_args* a, void* stream_) {
  cudaStream_t stream = (cudaStream_t)stream_;
  if (!a || !a->q || !a->k || !a->v || !a->out) return AOTO_ERR_ARGUMENT;
  if (a->query_heads <= 0 || a->kv_heads <= 0 || a->q_len <= 0 || a->kv_len <= 0 || a->head_dim <= 0)
    return AOTO_ERR_ARGUMENT;
  if (a->query_heads % a->kv_heads != 0) return AOTO_ERR_ARGUMENT;
  if ((a->head_dim & 1) || a->head_dim > 256) return AOTO_ERR_UNSUPPORTED;
  if (!aligned_to(a->k, 4) || !aligned_to(a->v, 4)) return AOTO_ERR_ARGUMENT;
  AttnParams p;
  p.q = (const bf16*)a->q; p.k = (const bf16*)a->k; p.v = (const bf16*)a->v;
  p.mask = (const bf16*)a->mask; p.out = (bf16*)a->out; p.scratch = (float*)a->scratch;
  p.QH = a->query_heads; p.KVH = a->kv_heads; p.Lq = a->q_len; p.Lk = a->kv_len; p.D = a->head_dim;
  p.causal = a->causal; p.scale = a->scale;
  if (a->q_len == 1) {
    p.splits = decode_splits(*a);
    p.keys_per_split = p.splits == 1 ? a->kv_len : 512;
    if (p.splits > 1) {
      const int64_t need = aoto_sm100_attention_scratch_bytes(a);
      if (!a->scratch || a->scratch_bytes < need) return AOTO_ERR_ARGUMENT;
    }
    const int tpr = a->head_dim / 2;
    const int parts = DECODE_THREADS / tpr;
    const size_t smem = ((size_t)a->head_dim + p.keys_per_split + 32 + (size_t)parts * a->head_dim) * 4;
    int status = launch_kernel(attention_decode_kernel, dim3(a->query_heads, p.splits),
                               dim3(DECODE_THREADS), smem, stream, false, p);
    if (status != AOTO_OK || p.splits == 1) return status;
    return launch_kernel(attention_combine_kernel, dim3(a->query_heads), dim3(128), 0, stream, false, p);
  }
  p.splits = 1;
  p.keys_per_split = 0;
  const int64_t rows = (int64_t)a->query_heads * a->q_len;
  const size_t smem = (size_t)PREFILL_WARPS * a->head_dim * 4;
  return launch_kernel(attention_prefill_kernel, dim3((unsigned)((rows + PREFILL_WARPS - 1) / PREFILL_WARPS)),
                       dim3(PREFILL_WARPS * 32), smem, stream, false, p);
}
