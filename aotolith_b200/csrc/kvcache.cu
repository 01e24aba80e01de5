// Decode-step KV-cache update: rotate the step's query and key, shift one
// layer's window by one slot and append the new key/value row.
//
// The operation is functional (the incoming cache is never written); the new
// pair may be placed directly inside a larger [L,2,...] buffer so the caller can
// assemble the next cache without a second copy.
#include "common.cuh"

namespace aoto {

struct KvParams {
  const bf16* cache;
  const bf16* row;
  const bf16* key;
  const bf16* cos_row;
  const bf16* sin_row;
  bf16* q_out;
  bf16* new_pair;
  int layer, kv_heads, capacity, D;
  int query_heads, query_start, key_start, value_start;
  int rotate;
};

// bf16 op-by-op rotation of element d of a head that starts at `head` in the row
__device__ __forceinline__ float rotate_element(const bf16* head, const bf16* cos_row,
                                                const bf16* sin_row, int d, int D) {
  const int half = D >> 1;
  const float v = __bfloat162float(head[d]);
  const float partner = d < half ? -__bfloat162float(head[d + half]) : __bfloat162float(head[d - half]);
  return round_bf16(round_bf16(v * __bfloat162float(cos_row[d])) +
                    round_bf16(partner * __bfloat162float(sin_row[d])));
}

// VEC elements per thread along D (8 = one 16-byte access; needs D % 16 == 0).
template <int VEC>
__global__ void __launch_bounds__(256)
kv_cache_append_kernel(const KvParams p) {
  pdl_wait_for_producers();
  pdl_release_dependents();
  const int D = p.D, C = p.capacity, H = p.kv_heads;
  const int dv = D / VEC;
  const int64_t window_vecs = (int64_t)2 * H * C * dv;
  const int64_t query_vecs = p.rotate ? (int64_t)p.query_heads * dv : 0;
  const int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= window_vecs + query_vecs) return;

  if (idx >= window_vecs) {
    // query rotation: q_out[0, head, 0, :]
    const int64_t qi = idx - window_vecs;
    const int head = (int)(qi / dv), d0 = (int)(qi % dv) * VEC;
    const bf16* src = p.row + p.query_start + (size_t)head * D;
    bf16* dst = p.q_out + (size_t)head * D + d0;
#pragma unroll
    for (int i = 0; i < VEC; ++i)
      dst[i] = __float2bfloat16_rn(rotate_element(src, p.cos_row, p.sin_row, d0 + i, D));
    return;
  }

  const int d0 = (int)(idx % dv) * VEC;
  int64_t r = idx / dv;
  const int slot = (int)(r % C);
  r /= C;
  const int head = (int)(r % H);
  const int kv = (int)(r / H);
  bf16* dst = p.new_pair + (((size_t)kv * H + head) * C + slot) * D + d0;
  if (slot < C - 1) {
    const bf16* src = p.cache + ((((size_t)p.layer * 2 + kv) * H + head) * C + slot + 1) * D + d0;
    if (VEC == 8) {
      *reinterpret_cast<uint4*>(dst) = *reinterpret_cast<const uint4*>(src);
    } else {
#pragma unroll
      for (int i = 0; i < VEC; ++i) dst[i] = src[i];
    }
    return;
  }
  if (kv == 1) {
    const bf16* src = p.row + p.value_start + (size_t)head * D + d0;
#pragma unroll
    for (int i = 0; i < VEC; ++i) dst[i] = src[i];
  } else if (p.rotate) {
    const bf16* src = p.row + p.key_start + (size_t)head * D;
#pragma unroll
    for (int i = 0; i < VEC; ++i)
      dst[i] = __float2bfloat16_rn(rotate_element(src, p.cos_row, p.sin_row, d0 + i, D));
  } else {
    const bf16* src = p.key + (size_t)head * D + d0;
#pragma unroll
    for (int i = 0; i < VEC; ++i) dst[i] = src[i];
  }
}

}  // namespace aoto

using namespace aoto;

extern "C" int aoto_sm100_kv_cache_append(const aoto_kv_append_args* a, void* stream) {
  if (!a || !a->cache || !a->row || !a->new_pair) return AOTO_ERR_ARGUMENT;
  if (a->layers <= 0 || a->layer < 0 || a->layer >= a->layers || a->kv_heads <= 0 ||
      a->capacity <= 0 || a->head_dim <= 0 || (a->head_dim & 1))
    return AOTO_ERR_ARGUMENT;
  if (a->rotate) {
    if (!a->cos_row || !a->sin_row || !a->q_out || a->query_heads <= 0) return AOTO_ERR_ARGUMENT;
  } else if (!a->key) {
    return AOTO_ERR_ARGUMENT;
  }
  KvParams p;
  p.cache = (const bf16*)a->cache;
  p.row = (const bf16*)a->row;
  p.key = (const bf16*)a->key;
  p.cos_row = (const bf16*)a->cos_row;
  p.sin_row = (const bf16*)a->sin_row;
  p.q_out = (bf16*)a->q_out;
  p.new_pair = (bf16*)a->new_pair;
  p.layer = a->layer; p.kv_heads = a->kv_heads; p.capacity = a->capacity; p.D = a->head_dim;
  p.query_heads = a->query_heads; p.query_start = a->query_start; p.key_start = a->key_start;
  p.value_start = a->value_start; p.rotate = a->rotate;
  const bool vec = (a->head_dim % 16 == 0) && aligned_to(a->cache, 16) && aligned_to(a->new_pair, 16);
  const int dv = vec ? a->head_dim / 8 : a->head_dim;
  const int64_t total = (int64_t)2 * a->kv_heads * a->capacity * dv +
                        (a->rotate ? (int64_t)a->query_heads * dv : 0);
  const dim3 grid((unsigned)((total + 255) / 256)), block(256);
  if (vec) return launch_kernel(kv_cache_append_kernel<8>, grid, block, 0, (cudaStream_t)stream, false, p);
  return launch_kernel(kv_cache_append_kernel<1>, grid, block, 0, (cudaStream_t)stream, false, p);
}
