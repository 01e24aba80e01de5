// Device helpers shared by the packed-GEMV kernels: activation staging with the
// fused RMS norm, the epilogue, the mma wrapper and the nibble decode.
#pragma once

#include "common.cuh"

namespace aoto {

struct GemvParams {
  const bf16* x;
  const uint32_t* w0;
  const bf16* s0;
  const uint32_t* w1;
  const bf16* s1;
  const bf16* addend;
  const bf16* gate;
  const bf16* norm_w;
  bf16* out;
  int N, K, group;
  int addend_kind, epilogue;
  float alpha, beta, eps;
};

__device__ __forceinline__ void unpack8(const uint4 v, float (&f)[8]) {
  f[0] = bf16x2_lo(v.x); f[1] = bf16x2_hi(v.x);
  f[2] = bf16x2_lo(v.y); f[3] = bf16x2_hi(v.y);
  f[4] = bf16x2_lo(v.z); f[5] = bf16x2_hi(v.z);
  f[6] = bf16x2_lo(v.w); f[7] = bf16x2_hi(v.w);
}

// Stage one activation row (K bf16, K % 8 == 0) into shared memory, applying
// the fused RMS norm if asked. With PERMUTE each run of eight values is stored
// as [0,4,1,5,2,6,3,7], the order the mma B fragments want, and the sum of the
// staged (rounded) values of every run of eight is written to `chunk_sum`.
template <bool PERMUTE>
__device__ __forceinline__ void stage_activation(const GemvParams& p, const bf16* x, uint4* xs,
                                                 float* chunk_sum, float* red) {
  const int chunks = p.K >> 3;
  const uint4* xv = reinterpret_cast<const uint4*>(x);
  const uint4* wv = reinterpret_cast<const uint4*>(p.norm_w);
  float inv = 1.f;
  if (p.norm_w != nullptr) {
    float ss = 0.f;
    for (int c = threadIdx.x; c < chunks; c += blockDim.x) {
      float f[8];
      unpack8(xv[c], f);
#pragma unroll
      for (int i = 0; i < 8; ++i) ss = fmaf(f[i], f[i], ss);
    }
    const float total = block_sum(ss, red);
    inv = rsqrtf(total / (float)p.K + p.eps);
  }
  for (int c = threadIdx.x; c < chunks; c += blockDim.x) {
    float f[8];
    unpack8(xv[c], f);
    if (p.norm_w != nullptr) {
      float w[8];
      unpack8(wv[c], w);
#pragma unroll
      for (int i = 0; i < 8; ++i) f[i] = round_bf16((f[i] * inv) * w[i]);
    }
    uint4 o;
    if (PERMUTE) {
      o.x = pack_bf16x2(f[0], f[4]);
      o.y = pack_bf16x2(f[1], f[5]);
      o.z = pack_bf16x2(f[2], f[6]);
      o.w = pack_bf16x2(f[3], f[7]);
      chunk_sum[c] = ((f[0] + f[1]) + (f[2] + f[3])) + ((f[4] + f[5]) + (f[6] + f[7]));
    } else {
      o.x = pack_bf16x2(f[0], f[1]);
      o.y = pack_bf16x2(f[2], f[3]);
      o.z = pack_bf16x2(f[4], f[5]);
      o.w = pack_bf16x2(f[6], f[7]);
    }
    xs[c] = o;
  }
  __syncthreads();
}

// y = beta*addend + alpha*total, then the epilogue. `total2` is the second
// (up) projection of the paired form.
__device__ __forceinline__ float finish_output(const GemvParams& p, int m, int n, float total,
                                               float total2) {
  float y = p.alpha * total;
  if (p.addend_kind == AOTO_ADDEND_VECTOR) {
    y = fmaf(p.beta, ldcg_bf16(p.addend + n), y);
  } else if (p.addend_kind == AOTO_ADDEND_FULL) {
    y = fmaf(p.beta, ldcg_bf16(p.addend + (size_t)m * p.N + n), y);
  }
  if (p.epilogue == AOTO_EPILOGUE_SILU_MUL_PAIRED) {
    const float g = round_bf16(y);
    y = (p.alpha * total2) * (g / (1.f + expf(-g)));
  } else if (p.epilogue == AOTO_EPILOGUE_SILU_MUL) {
    const float g = ldcg_bf16(p.gate + (size_t)m * p.N + n);
    y = y * (g / (1.f + expf(-g)));
  }
  return y;
}

__device__ __forceinline__ void mma_16816(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2,
                                          uint32_t a3, uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, "
      "{%8,%9}, {%0,%1,%2,%3};\n"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// (nibble k, nibble k+4) of a word -> two bf16 holding 136 + code (exact):
// 0x4300 is 128.0 in bf16 with a unit ulp, and code + 8 == nibble ^ 8.
#define AOTO_NIB(word, shift) ((((word) >> (shift)) & 0x000F000Fu) ^ 0x43084308u)

struct WeightItem {
  uint4 lo, hi;      // 32 codes of row g and of row g+8
  uint32_t slo, shi; // the two group scales (bf16 pair) of each row
};

// Where a lane reads its B fragments. B column parity separates the two groups of a
// block: a lane either always reads the staged activation (`stride` 1) or always reads
// zeros (`stride` 0, `base` a zeroed 16-byte word), so no per-fragment select is needed.
struct BSource {
  const uint4* base;
  int stride;
};

__device__ __forceinline__ BSource b_source(const uint4* xs, const uint4* zero16, int lane) {
  const int g = lane >> 2, t = lane & 3;
  const bool keep = ((g & 1) == (t >> 1));
  BSource b;
  b.base = keep ? xs + t * 4 : zero16;
  b.stride = keep ? 1 : 0;
  return b;
}

// One 16-row x 128-column block: eight mma into one C tile that starts at minus the
// 136*sum(x) offsets of the two groups, then the per-row group scales. `lo` / `hi` are the
// contributions to rows g and g+8 (identical on the four lanes of a quad).
__device__ __forceinline__ void mma_block(const WeightItem& it, const BSource& bs, int kb,
                                          const float* xsum, float& lo, float& hi) {
  const uint4* bp = bs.base + kb * 16 * bs.stride;
  const float2 off = *reinterpret_cast<const float2*>(xsum + kb * 2);
  // One accumulator tile for the eight mma: the kernels built on this are bound by the number of
  // instructions they issue, not by the length of this chain (other warps fill its gaps).
  float c[4] = {-off.x, -off.y, -off.x, -off.y};
  const uint32_t wl[4] = {it.lo.x, it.lo.y, it.lo.z, it.lo.w};
  const uint32_t wh[4] = {it.hi.x, it.hi.y, it.hi.z, it.hi.w};
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    const uint4 b = bp[j * bs.stride];
    mma_16816(c, AOTO_NIB(wl[j], 0), AOTO_NIB(wh[j], 0), AOTO_NIB(wl[j], 4), AOTO_NIB(wh[j], 4), b.x, b.y);
    mma_16816(c, AOTO_NIB(wl[j], 8), AOTO_NIB(wh[j], 8), AOTO_NIB(wl[j], 12), AOTO_NIB(wh[j], 12), b.z, b.w);
  }
  lo = fmaf(bf16x2_lo(it.slo), c[0], bf16x2_hi(it.slo) * c[1]);
  hi = fmaf(bf16x2_lo(it.shi), c[2], bf16x2_hi(it.shi) * c[3]);
}

}  // namespace aoto
