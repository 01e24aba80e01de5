// Packed 4-bit GEMM on the fifth-generation tensor cores (prefill): y[M,N] = x[M,K] . W[N,K]^T.
//
// One CTA computes a 128 (activation rows) x 128 (weight rows) tile of y:
//   warp 0      one lane issues TMA tile loads of x (128 rows x 64 columns, 128-byte swizzle),
//   warp 1      allocates tensor memory; one lane issues tcgen05.mma (M=128, N=128, K=16) with
//               both operands in shared memory and the fp32 accumulator in tensor memory,
//   warps 2-9   turn packed codes into bf16 weights - bf16(code * scale), the very weight the
//               reference materialises - and store them into shared memory in the same swizzled
//               K-major layout the TMA produces (two warps per 32 weight rows, each half a k
//               block); afterwards they read the accumulator back with tcgen05.ld (a warp may
//               read its own 32-lane quadrant), turn each chunk through shared memory so that
//               stores, addend and gate run along output rows, and run the epilogue.
// A ring of four stages decouples the three roles; every hand-over is an mbarrier (TMA bytes,
// 256 dequantising threads, tcgen05.commit). Every wait is bounded: a wait that runs out sets a
// status word, the roles fall through to the common exit and tensor memory is released.
#include <cuda.h>

#include "qgemv_core.cuh"

namespace aoto {

constexpr int TC_BM = 128, TC_BN = 128, TC_BK = 64;
constexpr int TC_STAGES = 4;
constexpr int TC_DEQUANT_WARPS = 8;                // two per weight row: each converts half a k block
constexpr int TC_THREADS = 64 + TC_DEQUANT_WARPS * 32;
constexpr int TC_TILE_BYTES = TC_BM * TC_BK * 2;  // 16 KiB: one 128-row operand tile of one stage
constexpr int TC_WAIT_LIMIT = 1 << 20;
constexpr int TC_AHEAD = 4;  // k blocks of packed words a dequantising thread keeps in flight
constexpr size_t tc_smem_bytes(int m_tiles) { return 1024 + (size_t)(m_tiles + 1) * TC_STAGES * TC_TILE_BYTES + 256; }

struct TcParams {
  const uint32_t* w;
  const bf16* s;
  const bf16* addend;
  const bf16* gate;
  bf16* out;
  int* status;
  unsigned char* scratch;  // split-K: arrival counters (first 4096 bytes), then fp32 partial tiles
  int M, N, K;
  int blocks_per_split;    // 64-column k blocks one CTA of a split walks
  int addend_kind, epilogue;
  float alpha, beta;
};

__device__ __forceinline__ uint32_t tc_smem(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void tc_bar_init(unsigned long long* bar, int count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(tc_smem(bar)), "r"(count) : "memory");
}
__device__ __forceinline__ void tc_bar_expect(unsigned long long* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(tc_smem(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ void tc_bar_arrive(unsigned long long* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(tc_smem(bar)) : "memory");
}
// Bounded wait for the phase with the given parity; false if it never completed.
__device__ __forceinline__ bool tc_bar_wait(unsigned long long* bar, uint32_t parity) {
  for (int spin = 0; spin < TC_WAIT_LIMIT; ++spin) {
    uint32_t done;
    asm volatile(
        "{\n.reg .pred p;\nmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\nselp.u32 %0, 1, 0, p;\n}\n"
        : "=r"(done) : "r"(tc_smem(bar)), "r"(parity) : "memory");
    if (done) return true;
  }
  return false;
}

// Shared-memory operand descriptor: K-major tile, 128-byte swizzle, rows 128 bytes apart, groups
// of eight rows 1024 bytes apart.
__device__ __forceinline__ uint64_t tc_operand_descriptor(uint32_t smem_address) {
  uint64_t d = 0;
  d |= (uint64_t)((smem_address & 0x3FFFFu) >> 4);  // start address
  d |= (uint64_t)1 << 16;                            // leading byte offset (unused with this swizzle)
  d |= (uint64_t)(1024 >> 4) << 32;                  // stride byte offset: eight rows
  d |= (uint64_t)1 << 46;                            // descriptor version of this architecture
  d |= (uint64_t)2 << 61;                            // 128-byte swizzle
  return d;
}

// Instruction descriptor of kind::f16: fp32 accumulate, bf16 x bf16, both operands K-major.
__device__ __forceinline__ uint32_t tc_instruction_descriptor(int m, int n) {
  return (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(n >> 3) << 17) | ((uint32_t)(m >> 4) << 24);
}

__device__ __forceinline__ void tc_mma(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n.reg .pred p;\nsetp.ne.b32 p, %4, 0;\n"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n}\n"
      ::"r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate) : "memory");
}
// The mbarrier gets one arrival once every tcgen05.mma this thread issued so far has finished.
__device__ __forceinline__ void tc_commit(unsigned long long* bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(tc_smem(bar)) : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }

__device__ __forceinline__ void tc_tma_load(void* smem_dst, const CUtensorMap* map, int x, int y, unsigned long long* bar) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
      ::"r"(tc_smem(smem_dst)), "l"(map), "r"(x), "r"(y), "r"(tc_smem(bar)) : "memory");
}

// 32 consecutive accumulator columns of this thread's tensor-memory lane.
__device__ __forceinline__ void tc_load_32(uint32_t taddr, uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
        "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
        "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
        "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr) : "memory");
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}

// (136 + code) pairs -> bf16(code * scale) pairs
__device__ __forceinline__ uint32_t tc_scaled_pair(uint32_t biased, __nv_bfloat162 scale2) {
  __nv_bfloat162 v = *reinterpret_cast<__nv_bfloat162*>(&biased);
  v = __hmul2(__hsub2(v, __float2bfloat162_rn(136.f)), scale2);
  return *reinterpret_cast<uint32_t*>(&v);
}

// MT = 128-row activation tiles a CTA multiplies against every weight tile it converts (the
// conversion is the scarce resource: with MT = 2 it is shared by twice the tensor-core work).
template <int MT>
__global__ void __launch_bounds__(TC_THREADS, 1)
qgemm_tc_kernel(const __grid_constant__ CUtensorMap x_map, const TcParams p) {
  constexpr int A_BYTES = MT * TC_TILE_BYTES;
  extern __shared__ unsigned char tc_smem_raw[];
  // operand tiles need 1024-byte alignment for the 128-byte swizzle
  unsigned char* base = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(tc_smem_raw) + 1023) & ~(uintptr_t)1023);
  unsigned char* tile_a = base;
  unsigned char* tile_b = base + (size_t)TC_STAGES * A_BYTES;
  unsigned long long* full_a = reinterpret_cast<unsigned long long*>(tile_b + (size_t)TC_STAGES * TC_TILE_BYTES);
  unsigned long long* full_b = full_a + TC_STAGES;
  unsigned long long* empty = full_b + TC_STAGES;
  unsigned long long* accumulated = empty + TC_STAGES;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(accumulated + 1);
  volatile int* last_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int n0 = blockIdx.x * TC_BN, m0 = blockIdx.y * TC_BM * MT;
  // Split-K: blockIdx.z walks its own range of k blocks; partial tiles meet in scratch and the
  // CTA that arrives last adds them in a fixed order and runs the epilogue.
  const int splits = gridDim.z;
  const int kb_first = blockIdx.z * p.blocks_per_split;
  const int blocks = min(p.blocks_per_split, p.K / TC_BK - kb_first);
  bool ok = true;

  if (threadIdx.x == 0) {
    for (int s = 0; s < TC_STAGES; ++s) {
      tc_bar_init(full_a + s, 1);
      tc_bar_init(full_b + s, TC_DEQUANT_WARPS * 32);
      tc_bar_init(empty + s, 1);
    }
    tc_bar_init(accumulated, 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(tc_smem(tmem_slot)), "r"(TC_BN * MT) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *reinterpret_cast<volatile uint32_t*>(tmem_slot);
  // Launched as a programmatic dependent, this grid may start while its producer still runs: the
  // packed weights are constants, so their conversion goes ahead; whatever the producer writes
  // (the activations, addend and gate) and whatever this grid writes is touched only behind a wait
  // for the producer's completion. The grid after this one may start as early in turn.
  pdl_release_dependents();

  if (warp == 0) {
    // ---- activation tiles by TMA ----
    if (lane == 0) {
      pdl_wait_for_producers();
      for (int kb = 0; kb < blocks && ok; ++kb) {
        const int s = kb % TC_STAGES;
        const uint32_t round = (uint32_t)(kb / TC_STAGES);
        ok = tc_bar_wait(empty + s, (round & 1u) ^ 1u);  // a fresh barrier passes the first round
        if (!ok) break;
        tc_bar_expect(full_a + s, A_BYTES);
        tc_tma_load(tile_a + (size_t)s * A_BYTES, &x_map, (kb_first + kb) * TC_BK, m0, full_a + s);
      }
    }
  } else if (warp == 1) {
    // ---- tensor-core issue ----
    if (lane == 0) {
      pdl_wait_for_producers();  // nothing to multiply before the producer is done: wait here, not in bounded polls
      const uint32_t idesc = tc_instruction_descriptor(TC_BM, TC_BN);
      for (int kb = 0; kb < blocks && ok; ++kb) {
        const int s = kb % TC_STAGES;
        const uint32_t round = (uint32_t)(kb / TC_STAGES);
        ok = tc_bar_wait(full_a + s, round & 1u) && tc_bar_wait(full_b + s, round & 1u);
        if (!ok) break;
        tc_fence_after();
        const uint64_t desc_b = tc_operand_descriptor(tc_smem(tile_b + (size_t)s * TC_TILE_BYTES));
#pragma unroll
        for (int mt = 0; mt < MT; ++mt) {  // activation tile mt accumulates in its own 128 columns
          const uint64_t desc_a = tc_operand_descriptor(tc_smem(tile_a + (size_t)s * A_BYTES + (size_t)mt * TC_TILE_BYTES));
#pragma unroll
          for (int k = 0; k < TC_BK / 16; ++k)  // 16 columns = 32 bytes further along the swizzled row
            tc_mma(tmem_base + (uint32_t)(mt * TC_BN), desc_a + (uint64_t)(k * 2), desc_b + (uint64_t)(k * 2), idesc,
                   (kb | k) != 0 ? 1u : 0u);
        }
        tc_commit(empty + s);  // the stage is free once these mma have read it
      }
      if (ok) tc_commit(accumulated);
    }
  } else {
    // ---- weight tiles: packed codes -> bf16 in swizzled shared memory; then the epilogue ----
    const int r = (threadIdx.x - 64) & 127;   // weight row of the tile
    const int half = (threadIdx.x - 64) >> 7;  // which 32 codes of the row's k block
    const int n = n0 + r;
    const bool row_valid = n < p.N;
    const uint4* wq = reinterpret_cast<const uint4*>(p.w) + (size_t)(row_valid ? n : 0) * (p.K >> 5);
    const bf16* sc = p.s + (size_t)(row_valid ? n : 0) * (p.K >> 6);
    // The packed words of the next TC_AHEAD k blocks are always in flight (a register ring with
    // static slots: the loop below is unrolled by TC_AHEAD).
    uint4 q0[TC_AHEAD];
    uint32_t scale_bits[TC_AHEAD];
    auto request = [&](int slot, int kb) {
      q0[slot] = make_uint4(0u, 0u, 0u, 0u);
      scale_bits[slot] = 0u;
      if (row_valid && kb < blocks) {
        q0[slot] = ldg_nc_u4(wq + (size_t)(kb_first + kb) * 2 + half);
        unsigned short raw;
        asm volatile("ld.global.nc.u16 %0, [%1];" : "=h"(raw) : "l"(sc + kb_first + kb));
        scale_bits[slot] = raw;
      }
    };
#pragma unroll
    for (int a = 0; a < TC_AHEAD; ++a) request(a, a);
    for (int kb0 = 0; kb0 < blocks && ok; kb0 += TC_AHEAD) {
#pragma unroll
      for (int a = 0; a < TC_AHEAD; ++a) {
      const int kb = kb0 + a;
      if (kb >= blocks || !ok) break;
      const int s = kb % TC_STAGES;
      const uint32_t round = (uint32_t)(kb / TC_STAGES);
      const uint4 c0 = q0[a];
      const __nv_bfloat162 scale2 = __bfloat162bfloat162(__ushort_as_bfloat16((unsigned short)scale_bits[a]));
      request(a, kb + TC_AHEAD);
      ok = tc_bar_wait(empty + s, (round & 1u) ^ 1u);
      if (!ok) break;
      unsigned char* row = tile_b + (size_t)s * TC_TILE_BYTES + (size_t)r * 128;
      const uint32_t words[4] = {c0.x, c0.y, c0.z, c0.w};
#pragma unroll
      for (int w = 0; w < 4; ++w) {  // word i = codes 8i..8i+7 = 16-byte chunk i of the row
        const int i = half * 4 + w;
        uint4 o = make_uint4(0u, 0u, 0u, 0u);
        if (row_valid) {
          const uint32_t v04 = tc_scaled_pair(AOTO_NIB(words[w], 0), scale2);
          const uint32_t v15 = tc_scaled_pair(AOTO_NIB(words[w], 4), scale2);
          const uint32_t v26 = tc_scaled_pair(AOTO_NIB(words[w], 8), scale2);
          const uint32_t v37 = tc_scaled_pair(AOTO_NIB(words[w], 12), scale2);
          o.x = __byte_perm(v04, v15, 0x5410);
          o.y = __byte_perm(v26, v37, 0x5410);
          o.z = __byte_perm(v04, v15, 0x7632);
          o.w = __byte_perm(v26, v37, 0x7632);
        }
        *reinterpret_cast<uint4*>(row + ((i ^ (r & 7)) << 4)) = o;
      }
      asm volatile("fence.proxy.async.shared::cta;" ::: "memory");  // the tensor core reads through the async proxy
      tc_bar_arrive(full_b + s);
      }
    }

    // epilogue: warp q of a warpgroup may read tensor-memory lanes 32q..32q+31; two warps share
    // a lane quadrant and each takes half of the 128 columns of every tile
    pdl_wait_for_producers();  // addend, gate, the output and the split-K workspace belong to the stream's order
    if (ok) ok = tc_bar_wait(accumulated, 0u);
    ok = __all_sync(0xffffffffu, ok);  // the epilogue below synchronises the warp: all lanes or none
    const int quadrant = warp & 3;
    // A warp holds its chunk of the accumulator with one output ROW per lane; written that way
    // every store instruction would touch 32 rows with 4 bytes each. The chunk is turned through
    // shared memory instead (the operand stages are idle once `accumulated` has completed; each
    // warp owns 32 rows of 33 floats there), so that a half-warp covers 32 neighbouring columns of
    // one row: 64-byte runs for the output and for the addend and gate that come the same way.
    float* turn = reinterpret_cast<float*>(tile_b) + (size_t)(warp - 2) * 32 * 33;
    auto emit = [&](const float (&acc)[32], int m_first, int nbase) {  // called by the whole warp
#pragma unroll
      for (int j = 0; j < 32; ++j) turn[lane * 33 + j] = acc[j];
      __syncwarp();
      const int col = nbase + 2 * (lane & 15);
      const bool pairs = (p.N & 1) == 0;  // then (m * N + col) is even: 4-byte accesses are aligned
      float bias0 = 0.f, bias1 = 0.f;
      if (p.addend_kind == AOTO_ADDEND_VECTOR) {
        if (col < p.N) bias0 = __bfloat162float(p.addend[col]);
        if (col + 1 < p.N) bias1 = __bfloat162float(p.addend[col + 1]);
      }
#pragma unroll 4
      for (int it = 0; it < 16; ++it) {
        const int row = 2 * it + (lane >> 4);
        const int m = m_first + row;
        if (m >= p.M || col >= p.N) continue;
        const bool both = col + 1 < p.N;
        float y0 = p.alpha * turn[row * 33 + 2 * (lane & 15)];
        float y1 = p.alpha * turn[row * 33 + 2 * (lane & 15) + 1];
        const size_t at = (size_t)m * p.N + col;
        auto fetch = [&](const bf16* src, float& v0, float& v1) {
          if (pairs) {
            const uint32_t two = *reinterpret_cast<const uint32_t*>(src + at);
            v0 = __uint_as_float(two << 16);
            v1 = __uint_as_float(two & 0xFFFF0000u);
          } else {
            v0 = __bfloat162float(src[at]);
            v1 = both ? __bfloat162float(src[at + 1]) : 0.f;
          }
        };
        if (p.addend_kind == AOTO_ADDEND_VECTOR) {
          y0 = fmaf(p.beta, bias0, y0);
          y1 = fmaf(p.beta, bias1, y1);
        } else if (p.addend_kind == AOTO_ADDEND_FULL) {
          float a0, a1;
          fetch(p.addend, a0, a1);
          y0 = fmaf(p.beta, a0, y0);
          y1 = fmaf(p.beta, a1, y1);
        }
        if (p.epilogue == AOTO_EPILOGUE_SILU_MUL) {
          float g0, g1;
          fetch(p.gate, g0, g1);
          y0 = y0 * (g0 / (1.f + expf(-g0)));
          y1 = y1 * (g1 / (1.f + expf(-g1)));
        }
        const uint32_t packed_pair = float_to_bf16_bits(y0) | (float_to_bf16_bits(y1) << 16);
        if (pairs) {
          *reinterpret_cast<uint32_t*>(p.out + at) = packed_pair;
        } else {
          p.out[at] = __ushort_as_bfloat16((unsigned short)(packed_pair & 0xffffu));
          if (both) p.out[at + 1] = __ushort_as_bfloat16((unsigned short)(packed_pair >> 16));
        }
      }
      __syncwarp();  // the next chunk overwrites the rows
    };
    // fp32 partial tiles: [split][padded row][padded column]
    const size_t padded_cols = (size_t)gridDim.x * TC_BN, padded_rows = (size_t)gridDim.y * TC_BM * MT;
    float* partials = reinterpret_cast<float*>(p.scratch + SCRATCH_HEADER_BYTES);
    if (ok) {
      tc_fence_after();
#pragma unroll 1
      for (int cc = 0; cc < MT * 2; ++cc) {
        const int mt = cc >> 1;
        const int c = half * 2 + (cc & 1);
        const int m = m0 + mt * TC_BM + quadrant * 32 + lane;
        uint32_t raw[32];
        tc_load_32(tmem_base + ((uint32_t)(quadrant * 32) << 16) + (uint32_t)(mt * TC_BN + c * 32), raw);
        if (splits == 1) {
          float acc[32];
#pragma unroll
          for (int j = 0; j < 32; ++j) acc[j] = __uint_as_float(raw[j]);
          emit(acc, m - lane, n0 + c * 32);
        } else {
          float4* dst = reinterpret_cast<float4*>(partials + ((size_t)blockIdx.z * padded_rows + m) * padded_cols + n0 + c * 32);
#pragma unroll
          for (int j = 0; j < 8; ++j)
            dst[j] = make_float4(__uint_as_float(raw[4 * j]), __uint_as_float(raw[4 * j + 1]),
                                 __uint_as_float(raw[4 * j + 2]), __uint_as_float(raw[4 * j + 3]));
        }
      }
    }
    if (splits > 1) {
      // the converting warps (256 threads) meet on their own barrier; one of them counts the arrival
      int* counter = reinterpret_cast<int*>(p.scratch) + blockIdx.y * gridDim.x + blockIdx.x;
      __threadfence();
      asm volatile("bar.sync 1, 256;" ::: "memory");
      if (threadIdx.x == 64) {
        const int arrived = atomicAdd(counter, 1);
        const int last = arrived == splits - 1;
        if (last) *counter = 0;  // counters are zero between launches
        *last_flag = last;
      }
      asm volatile("bar.sync 1, 256;" ::: "memory");
      if (*last_flag && ok) {
        __threadfence();
#pragma unroll 1
        for (int cc = 0; cc < MT * 2; ++cc) {
          const int mt = cc >> 1;
          const int c = half * 2 + (cc & 1);
          const int m = m0 + mt * TC_BM + quadrant * 32 + lane;
          float acc[32];
#pragma unroll
          for (int j = 0; j < 32; ++j) acc[j] = 0.f;
          for (int z = 0; z < splits && m < p.M; ++z) {  // fixed order: the result does not depend on arrival order
            const float4* src = reinterpret_cast<const float4*>(partials + ((size_t)z * padded_rows + m) * padded_cols + n0 + c * 32);
#pragma unroll
            for (int j = 0; j < 8; ++j) {
              const float4 v = __ldcg(src + j);
              acc[4 * j] += v.x; acc[4 * j + 1] += v.y; acc[4 * j + 2] += v.z; acc[4 * j + 3] += v.w;
            }
          }
          emit(acc, m - lane, n0 + c * 32);
        }
      }
    }
  }

  if (!ok && p.status != nullptr) atomicExch(p.status, 1);
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(TC_BN * MT) : "memory");
  }
}

// ---------------------------------------------------------------------------
// host side
// ---------------------------------------------------------------------------
static __device__ int tc_timeout_flag;

namespace {

using EncodeTiled = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                 const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                 CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

// The tensor-map encoder lives in the driver; it is looked up through the runtime so that the
// library does not link against the driver library.
EncodeTiled tensor_map_encoder() {
  static EncodeTiled cached = nullptr;
  if (cached == nullptr) {
    void* fn = nullptr;
    cudaDriverEntryPointQueryResult result;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &result) != cudaSuccess ||
        result != cudaDriverEntryPointSuccess) {
      (void)cudaGetLastError();
      return nullptr;
    }
    cached = reinterpret_cast<EncodeTiled>(fn);
  }
  return cached;
}

constexpr int MAX_DEVICES = 64;
int* timeout_flag_address[MAX_DEVICES] = {};

int* timeout_flag_on_current_device() {
  int device = -1;
  if (cudaGetDevice(&device) != cudaSuccess || device < 0 || device >= MAX_DEVICES) {
    (void)cudaGetLastError();
    return nullptr;
  }
  if (timeout_flag_address[device] == nullptr) {
    void* address = nullptr;
    if (cudaGetSymbolAddress(&address, tc_timeout_flag) != cudaSuccess) {
      (void)cudaGetLastError();
      return nullptr;
    }
    timeout_flag_address[device] = static_cast<int*>(address);
  }
  return timeout_flag_address[device];
}

}  // namespace

bool qgemm_tc_applies(const aoto_qmatmul_args& a) {
  // a 128-row tile is the smallest the tensor core takes: worth it from 64 rows on, or from 8 rows
  // when the weight is large enough (many rows, or a long K) that converting it dominates
  return (a.M >= 64 || (a.M >= 8 && (a.N >= 4096 || a.K >= 2048))) && a.N >= 64 && a.group_size == 64 && (a.K % TC_BK) == 0 && a.norm_weight == nullptr &&
         a.epilogue != AOTO_EPILOGUE_SILU_MUL_PAIRED && (reinterpret_cast<uintptr_t>(a.x) & 15) == 0 &&
         (reinterpret_cast<uintptr_t>(a.packed) & 15) == 0;
}

// Grid of a request: activation tiles per CTA, output tiles, and - for outputs too narrow to
// occupy the GPU - how many ways K is split (each split at least sixteen k blocks: below that the
// fixed cost of a CTA and of the meeting in scratch outweighs the shorter loop; at most eight
// splits, about one CTA per SM in total).
struct TcPlan {
  int m_tiles, grid_x, grid_y, splits, blocks_per_split;
  int64_t scratch_bytes;
};

static TcPlan tc_plan(const aoto_qmatmul_args& a) {
  TcPlan plan;
  plan.m_tiles = a.M > TC_BM ? 2 : 1;
  plan.grid_x = (a.N + TC_BN - 1) / TC_BN;
  plan.grid_y = (a.M + TC_BM * plan.m_tiles - 1) / (TC_BM * plan.m_tiles);
  const int tiles = plan.grid_x * plan.grid_y, blocks = a.K / TC_BK;
  int splits = 148 / tiles;
  if (splits > 8) splits = 8;
  if (splits > blocks / 16) splits = blocks / 16;
  // with many activation rows the partial tiles cost more to write and re-read than the split saves
  if (splits < 1 || tiles > SCRATCH_MAX_COUNTERS || a.M > 256) splits = 1;
  plan.blocks_per_split = (blocks + splits - 1) / splits;
  plan.splits = (blocks + plan.blocks_per_split - 1) / plan.blocks_per_split;
  plan.scratch_bytes = plan.splits > 1
      ? SCRATCH_HEADER_BYTES + (int64_t)plan.splits * plan.grid_y * TC_BM * plan.m_tiles * plan.grid_x * TC_BN * 4
      : 0;
  return plan;
}

int64_t qgemm_tc_scratch_bytes(const aoto_qmatmul_args& a) { return tc_plan(a).scratch_bytes; }

int qgemm_tc_launch(const aoto_qmatmul_args& a, cudaStream_t stream) {
  EncodeTiled encode = tensor_map_encoder();
  if (encode == nullptr) return AOTO_ERR_UNSUPPORTED;
  // x as a [M rows, K columns] bf16 tensor; boxes of 128 rows x 64 columns, rows past M read as zero
  CUtensorMap map;
  const cuuint64_t dims[2] = {(cuuint64_t)a.K, (cuuint64_t)a.M};
  const cuuint64_t strides[1] = {(cuuint64_t)a.K * 2};
  TcPlan plan = tc_plan(a);
  if (plan.splits > 1 && (a.scratch == nullptr || a.scratch_bytes < plan.scratch_bytes ||
                          (reinterpret_cast<uintptr_t>(a.scratch) & 15) != 0)) {
    plan.splits = 1;  // no workspace given: one CTA walks all of K
    plan.blocks_per_split = a.K / TC_BK;
  }
  const int m_tiles = plan.m_tiles;
  const cuuint32_t box[2] = {(cuuint32_t)TC_BK, (cuuint32_t)(TC_BM * m_tiles)};
  const cuuint32_t element_strides[2] = {1, 1};
  if (encode(&map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(a.x), dims, strides, box, element_strides,
             CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
             CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
    return AOTO_ERR_ARGUMENT;

  static PerDeviceOnce raised1, raised2;
  if (raise_dynamic_smem(qgemm_tc_kernel<1>, tc_smem_bytes(1), raised1) != AOTO_OK ||
      raise_dynamic_smem(qgemm_tc_kernel<2>, tc_smem_bytes(2), raised2) != AOTO_OK)
    return AOTO_ERR_LAUNCH;
  TcParams p;
  p.w = (const uint32_t*)a.packed;
  p.s = (const bf16*)a.scales;
  p.addend = (const bf16*)a.addend;
  p.gate = (const bf16*)a.gate;
  p.out = (bf16*)a.out;
  p.status = timeout_flag_on_current_device();
  p.scratch = static_cast<unsigned char*>(a.scratch);
  p.blocks_per_split = plan.blocks_per_split;
  p.M = a.M; p.N = a.N; p.K = a.K;
  p.addend_kind = a.addend_kind; p.epilogue = a.epilogue;
  p.alpha = a.alpha; p.beta = a.beta;
  dim3 grid(plan.grid_x, plan.grid_y, plan.splits), block(TC_THREADS);
  const bool pdl = (a.flags & AOTO_FLAG_PDL) != 0;
  if (m_tiles == 2) return launch_kernel(qgemm_tc_kernel<2>, grid, block, tc_smem_bytes(2), stream, pdl, map, p);
  return launch_kernel(qgemm_tc_kernel<1>, grid, block, tc_smem_bytes(1), stream, pdl, map, p);
}

// Reads and clears the flag a timed-out wait of the tensor-core GEMM sets. Synchronises the
// device: a diagnostic for tests and for a caller that saw wrong results, not part of a step.
int qgemm_tc_take_timeout_flag() {
  int* flag = timeout_flag_on_current_device();
  if (flag == nullptr) return -1;
  int value = 0;
  if (cudaMemcpy(&value, flag, sizeof(int), cudaMemcpyDeviceToHost) != cudaSuccess) { (void)cudaGetLastError(); return -1; }
  if (value != 0) {
    const int zero = 0;
    if (cudaMemcpy(flag, &zero, sizeof(int), cudaMemcpyHostToDevice) != cudaSuccess) { (void)cudaGetLastError(); return -1; }
  }
  return value;
}

}  // namespace aoto
