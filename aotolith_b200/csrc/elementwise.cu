// Small streaming kernels of the decoder path: dequantize, RMS norm (+residual),
// rotary embedding, row gathers, mask conversion, greedy argmax.
#include "common.cuh"

namespace aoto {

// --------------------------------------------------------------------------
// dequantize_i4: one thread per packed word, eight bf16 out (one 16-byte store)
// --------------------------------------------------------------------------
__global__ void __launch_bounds__(256)
dequantize_i4_kernel(const uint32_t* __restrict__ packed, const bf16* __restrict__ scales,
                     bf16* __restrict__ out, int64_t words_total, int words_per_row, int group) {
  const int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= words_total) return;
  const int64_t row = idx / words_per_row;
  const int j = (int)(idx - row * words_per_row);
  const uint32_t word = __ldg(packed + idx);
  const int groups_per_row = (words_per_row * 8) / group;
  const bf16 scale = scales[row * groups_per_row + (j * 8) / group];
  uint32_t o[4];
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int c0 = ((int)(word << (28 - 8 * i))) >> 28;
    const int c1 = ((int)(word << (24 - 8 * i))) >> 28;
    // bf16(code) is exact; the product is rounded once to bf16
    const bf16 v0 = __hmul(__int2bfloat16_rn(c0), scale);
    const bf16 v1 = __hmul(__int2bfloat16_rn(c1), scale);
    o[i] = (uint32_t)__bfloat16_as_ushort(v0) | ((uint32_t)__bfloat16_as_ushort(v1) << 16);
  }
  reinterpret_cast<uint4*>(out)[idx] = make_uint4(o[0], o[1], o[2], o[3]);
}

// --------------------------------------------------------------------------
// rms_norm (+ residual): one CTA per row
// --------------------------------------------------------------------------
__global__ void __launch_bounds__(256)
rms_norm_kernel(const bf16* __restrict__ x, const bf16* __restrict__ residual,
                const bf16* __restrict__ weight, bf16* __restrict__ out, bf16* __restrict__ sum_out,
                int H, float eps) {
  extern __shared__ float row_cache[];  // H floats + 32
  float* red = row_cache + H;
  pdl_wait_for_producers();
  pdl_release_dependents();
  const size_t base = (size_t)blockIdx.x * H;
  float ss = 0.f;
  for (int i = threadIdx.x; i < H; i += blockDim.x) {
    float v = __bfloat162float(x[base + i]);
    if (residual != nullptr) {
      // the sum is a bf16 value in the graph (add in the model dtype), so round it
      v = round_bf16(v + __bfloat162float(residual[base + i]));
      if (sum_out != nullptr) sum_out[base + i] = __float2bfloat16_rn(v);
    }
    row_cache[i] = v;
    ss = fmaf(v, v, ss);
  }
  const float total = block_sum(ss, red);
  const float inv = rsqrtf(total / (float)H + eps);
  for (int i = threadIdx.x; i < H; i += blockDim.x) {
    float v = row_cache[i] * inv;
    if (weight != nullptr) v *= __bfloat162float(weight[i]);
    out[base + i] = __float2bfloat16_rn(v);
  }
}

// --------------------------------------------------------------------------
// rope: out = bf16(bf16(x*cos) + bf16(rot(x)*sin)), as three bf16 operations
// --------------------------------------------------------------------------
__global__ void __launch_bounds__(256)
rope_kernel(const bf16* __restrict__ x, const bf16* __restrict__ cos_t, const bf16* __restrict__ sin_t,
            bf16* __restrict__ out, int heads, int T, int D, int64_t sb, int64_t sh, int64_t st,
            int64_t total) {
  const int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= total) return;
  const int d = (int)(idx % D);
  const int64_t r = idx / D;
  const int t = (int)(r % T);
  const int64_t r2 = r / T;
  const int h = (int)(r2 % heads);
  const int64_t b = r2 / heads;
  const bf16* src = x + b * sb + h * sh + t * st;
  const int half = D >> 1;
  const float v = __bfloat162float(src[d]);
  const float partner = d < half ? -__bfloat162float(src[d + half]) : __bfloat162float(src[d - half]);
  const float c = __bfloat162float(cos_t[(size_t)t * D + d]);
  const float s = __bfloat162float(sin_t[(size_t)t * D + d]);
  out[idx] = __float2bfloat16_rn(round_bf16(v * c) + round_bf16(partner * s));
}

// --------------------------------------------------------------------------
// embedding: one CTA per gathered row
// --------------------------------------------------------------------------
__global__ void __launch_bounds__(128)
embedding_kernel(const bf16* __restrict__ table, const int64_t* __restrict__ ids, bf16* __restrict__ out,
                 int64_t* __restrict__ bad_index, int rows, int width) {
  pdl_wait_for_producers();
  pdl_release_dependents();
  const int i = blockIdx.x;
  const int64_t id = ids[i];
  const bool ok = id >= 0 && id < rows;
  if (!ok && bad_index != nullptr && threadIdx.x == 0) {
    // keep the lowest offending position (0 = none seen yet)
    unsigned long long* slot = reinterpret_cast<unsigned long long*>(bad_index);
    const unsigned long long mine = (unsigned long long)(i + 1);
    unsigned long long seen = *slot;
    while (seen == 0ull || seen > mine) {
      const unsigned long long prior = atomicCAS(slot, seen, mine);
      if (prior == seen) break;
      seen = prior;
    }
  }
  bf16* dst = out + (size_t)i * width;
  const bf16* src = table + (size_t)(ok ? id : 0) * width;
  if ((width & 7) == 0 && aligned_ptr16(src) && aligned_ptr16(dst)) {
    const uint4* s4 = reinterpret_cast<const uint4*>(src);
    uint4* d4 = reinterpret_cast<uint4*>(dst);
    for (int c = threadIdx.x; c < (width >> 3); c += blockDim.x)
      d4[c] = ok ? s4[c] : make_uint4(0u, 0u, 0u, 0u);
  } else {
    for (int c = threadIdx.x; c < width; c += blockDim.x)
      dst[c] = ok ? src[c] : __float2bfloat16_rn(0.f);
  }
}

__global__ void __launch_bounds__(256)
mask_select_kernel(const uint8_t* __restrict__ mask, bf16* __restrict__ out, int64_t count,
                   float on_true, float on_false) {
  const int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx < count) out[idx] = __float2bfloat16_rn(mask[idx] ? on_true : on_false);
}

// --------------------------------------------------------------------------
// argmax / greedy pick: the row is cut into parts, one CTA per part; every CTA
// leaves its (value, index) in scratch and the last one to arrive picks the
// winner - first maximum wins (torch / numpy tie rule), NaN ranks highest as in
// torch.argmax - and, for the greedy pick, appends the token and advances the
// loop counters. The arrival counter is left at zero for the next launch.
// --------------------------------------------------------------------------
struct PickParams {
  const bf16* logits;
  int64_t* out;        // argmax: out[row]; greedy: token[0]
  int64_t* generated;  // greedy only
  int32_t* counters;   // greedy only
  float* part_value;   // scratch: [rows][parts]
  int* part_index;     // scratch: [rows][parts]
  int* arrivals;       // scratch: [rows]
  int width, parts, generated_capacity;
};

__device__ __forceinline__ void better(float& bv, int& bi, float ov, int oi) {
  if (ov > bv || (ov == bv && oi < bi)) { bv = ov; bi = oi; }
}

__device__ __forceinline__ void block_best(float& bv, int& bi, float* sv, int* si) {
#pragma unroll
  for (int offset = 16; offset > 0; offset >>= 1)
    better(bv, bi, __shfl_xor_sync(0xffffffffu, bv, offset), __shfl_xor_sync(0xffffffffu, bi, offset));
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  __syncthreads();
  if (lane == 0) { sv[warp] = bv; si[warp] = bi; }
  __syncthreads();
  const int warps = blockDim.x >> 5;
  bv = lane < warps ? sv[lane] : -INFINITY;
  bi = lane < warps ? si[lane] : 0x7fffffff;
#pragma unroll
  for (int offset = 16; offset > 0; offset >>= 1)
    better(bv, bi, __shfl_xor_sync(0xffffffffu, bv, offset), __shfl_xor_sync(0xffffffffu, bi, offset));
}

template <bool GREEDY>
__global__ void __launch_bounds__(256)
pick_kernel(const PickParams p) {
  __shared__ float sv[32];
  __shared__ int si[32];
  __shared__ int is_last;
  pdl_wait_for_producers();
  pdl_release_dependents();
  const int row = blockIdx.y, part = blockIdx.x;
  const bf16* logits = p.logits + (size_t)row * p.width;
  const int span = ((p.width + p.parts - 1) / p.parts + 7) & ~7;  // multiple of 8
  const int begin = part * span, end = min(p.width, begin + span);
  float bv = -INFINITY;
  int bi = 0x7fffffff;
  auto see = [&](float v, int i) {
    if (v != v) v = INFINITY;
    if (bi == 0x7fffffff || v > bv) { bv = v; bi = i; }
  };
  if (aligned_ptr16(logits)) {
    for (int i = begin + threadIdx.x * 8; i < end; i += blockDim.x * 8) {
      if (i + 8 <= end) {
        const uint4 v = *reinterpret_cast<const uint4*>(logits + i);
        see(bf16x2_lo(v.x), i); see(bf16x2_hi(v.x), i + 1); see(bf16x2_lo(v.y), i + 2); see(bf16x2_hi(v.y), i + 3);
        see(bf16x2_lo(v.z), i + 4); see(bf16x2_hi(v.z), i + 5); see(bf16x2_lo(v.w), i + 6); see(bf16x2_hi(v.w), i + 7);
      } else {
        for (int j = i; j < end; ++j) see(__bfloat162float(logits[j]), j);
      }
    }
  } else {
    for (int i = begin + threadIdx.x; i < end; i += blockDim.x) see(__bfloat162float(logits[i]), i);
  }
  block_best(bv, bi, sv, si);
  if (p.parts > 1) {
    if (threadIdx.x == 0) {
      p.part_value[row * p.parts + part] = bv;
      p.part_index[row * p.parts + part] = bi;
      __threadfence();
      const int arrived = atomicAdd(p.arrivals + row, 1);
      is_last = arrived == p.parts - 1;
      if (is_last) p.arrivals[row] = 0;
    }
    __syncthreads();
    if (!is_last) return;
    __threadfence();
    bv = -INFINITY;
    bi = 0x7fffffff;
    for (int q = threadIdx.x; q < p.parts; q += blockDim.x)
      better(bv, bi, __ldcg(p.part_value + row * p.parts + q), __ldcg(p.part_index + row * p.parts + q));
    block_best(bv, bi, sv, si);
  }
  if (threadIdx.x == 0) {
    p.out[GREEDY ? 0 : row] = (int64_t)bi;
    if (GREEDY) {
      const int step = p.counters[1];
      if (step < p.generated_capacity) p.generated[step] = (int64_t)bi;
      p.counters[0] += 1;
      p.counters[1] = step + 1;
    }
  }
}

static int pick_parts(int rows, int width) {
  if (width < 8192 || rows > SCRATCH_MAX_COUNTERS) return 1;
  int parts = (width + 2047) / 2048;
  return parts > 64 ? 64 : parts;
}

static int launch_pick(bool greedy, PickParams p, int rows, void* scratch, int64_t scratch_bytes,
                       cudaStream_t stream) {
  p.parts = pick_parts(rows, p.width);
  if (p.parts > 1) {
    const int64_t need = SCRATCH_HEADER_BYTES + (int64_t)rows * p.parts * 8;
    if (!scratch || scratch_bytes < need || !aligned_to(scratch, 4)) return AOTO_ERR_ARGUMENT;
    p.arrivals = reinterpret_cast<int*>(scratch);
    p.part_value = reinterpret_cast<float*>(reinterpret_cast<char*>(scratch) + SCRATCH_HEADER_BYTES);
    p.part_index = reinterpret_cast<int*>(p.part_value + (size_t)rows * p.parts);
  }
  const dim3 grid(p.parts, rows), block(256);
  if (greedy) return launch_kernel(pick_kernel<true>, grid, block, 0, stream, false, p);
  return launch_kernel(pick_kernel<false>, grid, block, 0, stream, false, p);
}

// --------------------------------------------------------------------------
// device-resident greedy loop: per-step inputs and the pick that closes a step
// --------------------------------------------------------------------------
__global__ void __launch_bounds__(256)
step_inputs_kernel(const int32_t* __restrict__ counters, int64_t* __restrict__ position,
                   uint8_t* __restrict__ mask, int capacity) {
  pdl_wait_for_producers();
  pdl_release_dependents();
  const int valid = counters[0];
  const int idx = blockIdx.x * blockDim.x + threadIdx.x;
  if (idx == 0) position[0] = (int64_t)(valid - 1);
  if (idx < capacity) mask[idx] = idx >= capacity - valid ? 1 : 0;
}

}  // namespace aoto

using namespace aoto;

extern "C" int aoto_sm100_step_inputs(const aoto_step_inputs_args* a, void* stream) {
  if (!a || !a->counters || !a->position || !a->mask || a->capacity <= 0) return AOTO_ERR_ARGUMENT;
  return launch_kernel(step_inputs_kernel, dim3((a->capacity + 255) / 256), dim3(256), 0,
                       (cudaStream_t)stream, false, a->counters, a->position, a->mask, (int)a->capacity);
}

extern "C" int aoto_sm100_greedy_pick(const aoto_greedy_pick_args* a, void* stream) {
  if (!a || !a->logits || !a->token || !a->generated || !a->counters || a->width <= 0 ||
      a->generated_capacity <= 0)
    return AOTO_ERR_ARGUMENT;
  PickParams p = {};
  p.logits = (const bf16*)a->logits;
  p.out = a->token;
  p.generated = a->generated;
  p.counters = a->counters;
  p.width = a->width;
  p.generated_capacity = a->generated_capacity;
  return launch_pick(true, p, 1, a->scratch, a->scratch_bytes, (cudaStream_t)stream);
}

extern "C" int aoto_sm100_dequantize_i4(const aoto_dequantize_args* a, void* stream) {
  if (!a || !a->packed || !a->scales || !a->out) return AOTO_ERR_ARGUMENT;
  if (a->N <= 0 || a->K <= 0 || a->group_size <= 0 || a->group_size % 8 != 0 ||
      a->K % a->group_size != 0)
    return AOTO_ERR_ARGUMENT;
  if (!aligned_to(a->out, 16)) return AOTO_ERR_ARGUMENT;
  const int words_per_row = a->K / 8;
  const int64_t words = (int64_t)a->N * words_per_row;
  const int64_t blocks = (words + 255) / 256;
  dequantize_i4_kernel<<<(unsigned)blocks, 256, 0, (cudaStream_t)stream>>>(
      (const uint32_t*)a->packed, (const bf16*)a->scales, (bf16*)a->out, words, words_per_row,
      a->group_size);
  return launch_status();
}

extern "C" int aoto_sm100_rms_norm(const aoto_rms_norm_args* a, void* stream) {
  if (!a || !a->x || !a->out || a->rows <= 0 || a->H <= 0) return AOTO_ERR_ARGUMENT;
  const size_t smem = (size_t)a->H * 4 + 32 * 4;
  if (smem > 48 * 1024) return AOTO_ERR_UNSUPPORTED;
  return launch_kernel(rms_norm_kernel, dim3(a->rows), dim3(256), smem, (cudaStream_t)stream, false,
                       (const bf16*)a->x, (const bf16*)a->residual, (const bf16*)a->weight,
                       (bf16*)a->out, (bf16*)a->sum_out, (int)a->H, a->eps);
}

extern "C" int aoto_sm100_rope(const aoto_rope_args* a, void* stream) {
  if (!a || !a->x || !a->cos_table || !a->sin_table || !a->out) return AOTO_ERR_ARGUMENT;
  if (a->B <= 0 || a->heads <= 0 || a->T <= 0 || a->D <= 0 || (a->D & 1)) return AOTO_ERR_ARGUMENT;
  const int64_t total = (int64_t)a->B * a->heads * a->T * a->D;
  const int64_t blocks = (total + 255) / 256;
  rope_kernel<<<(unsigned)blocks, 256, 0, (cudaStream_t)stream>>>(
      (const bf16*)a->x, (const bf16*)a->cos_table, (const bf16*)a->sin_table, (bf16*)a->out,
      a->heads, a->T, a->D, a->stride_b, a->stride_h, a->stride_t, total);
  return launch_status();
}

extern "C" int aoto_sm100_embedding(const aoto_embedding_args* a, void* stream) {
  if (!a || !a->table || !a->ids || !a->out || a->rows <= 0 || a->width <= 0 || a->count <= 0)
    return AOTO_ERR_ARGUMENT;
  return launch_kernel(embedding_kernel, dim3(a->count), dim3(128), 0, (cudaStream_t)stream, false,
                       (const bf16*)a->table, a->ids, (bf16*)a->out, a->bad_index, (int)a->rows,
                       (int)a->width);
}

extern "C" int aoto_sm100_mask_select(const aoto_mask_select_args* a, void* stream) {
  if (!a || !a->mask || !a->out || a->count <= 0) return AOTO_ERR_ARGUMENT;
  const int64_t blocks = (a->count + 255) / 256;
  mask_select_kernel<<<(unsigned)blocks, 256, 0, (cudaStream_t)stream>>>(
      a->mask, (bf16*)a->out, a->count, a->on_true, a->on_false);
  return launch_status();
}

extern "C" int64_t aoto_sm100_argmax_scratch_bytes(int32_t rows, int32_t width) {
  if (rows <= 0 || width <= 0) return 0;
  const int parts = pick_parts(rows, width);
  return parts > 1 ? SCRATCH_HEADER_BYTES + (int64_t)rows * parts * 8 : 0;
}

extern "C" int aoto_sm100_argmax(const aoto_argmax_args* a, void* stream) {
  if (!a || !a->logits || !a->out || a->rows <= 0 || a->width <= 0) return AOTO_ERR_ARGUMENT;
  PickParams p = {};
  p.logits = (const bf16*)a->logits;
  p.out = a->out;
  p.width = a->width;
  return launch_pick(false, p, a->rows, a->scratch, a->scratch_bytes, (cudaStream_t)stream);
}
