// Small all-reduce over peer memory for tensor-parallel decode (one launch, no library call).
//
// A decode step all-reduces a hidden-state row (a few KB) twice per layer; at that size a
// collective is pure latency. Every rank owns a receive buffer that its peers can write
// (symmetric memory, mapped into each process): world x words 8-byte slots, twice (two sets that
// alternate between calls). A call on rank r
//   1. packs its partial row into stamped words (two bf16 values + the call's 32-bit epoch) and
//      stores word i into slot [r][i] of EVERY rank's buffer - plain 8-byte stores over NVLink;
//   2. polls its own buffer until slot [q][i] carries the epoch for every rank q, adds the values
//      in rank order in fp32 and writes the bf16 sum.
// The 8-byte store carries data and flag together, so no fence is needed. A rank can be at most
// one call ahead of a peer (it needs the peer's contribution to finish a call), so two slot sets
// are enough for a fast rank never to overwrite words a slow rank still has to read. The epoch
// lives in device memory and is advanced by the kernel, so a recorded launch can be replayed.
// Every poll is bounded; a poll that runs out stores 1 in `status` and the kernel returns.
#include "common.cuh"

namespace aoto {

constexpr int PEER_MAX_RANKS = 8;
constexpr int PEER_THREADS = 1024;
constexpr int PEER_POLL_LIMIT = 1 << 22;

struct PeerSumParams {
  unsigned char* buffers[PEER_MAX_RANKS];  // receive buffer of every rank, as mapped in this process
  const bf16* partial;                     // this rank's addend, `count` values
  bf16* out;                               // the sum, `count` values (may alias `partial`)
  unsigned int* epoch;                     // device word: epoch of the previous call
  int* status;
  int world, rank, count, capacity_words;  // capacity_words: words of one rank's slot row
};

__global__ void __launch_bounds__(PEER_THREADS, 1)
peer_sum_kernel(const PeerSumParams p) {
  const unsigned int epoch = *reinterpret_cast<volatile unsigned int*>(p.epoch) + 1u;
  const int words = (p.count + 1) >> 1;
  const size_t set_offset = (size_t)(epoch & 1u) * p.world * p.capacity_words * 8;
  const uint32_t* mine = reinterpret_cast<const uint32_t*>(p.partial);
  bool failed = false;
  for (int i = threadIdx.x; i < words; i += PEER_THREADS) {
    uint32_t data;
    if (2 * i + 1 < p.count) data = mine[i];
    else data = (uint32_t)__bfloat16_as_ushort(p.partial[2 * i]);
    for (int q = 0; q < p.world; ++q) {
      unsigned char* slot = p.buffers[q] + set_offset + ((size_t)p.rank * p.capacity_words + i) * 8;
      asm volatile("st.volatile.global.v2.u32 [%0], {%1, %2};" ::"l"(slot), "r"(data), "r"(epoch) : "memory");
    }
  }
  for (int i = threadIdx.x; i < words; i += PEER_THREADS) {
    float lo = 0.f, hi = 0.f;
    for (int q = 0; q < p.world && !failed; ++q) {
      const unsigned char* slot = p.buffers[p.rank] + set_offset + ((size_t)q * p.capacity_words + i) * 8;
      uint32_t data = 0, stamp = 0;
      int polls = 0;
      while (true) {
        asm volatile("ld.volatile.global.v2.u32 {%0, %1}, [%2];" : "=r"(data), "=r"(stamp) : "l"(slot) : "memory");
        if (stamp == epoch) break;
        if (++polls > PEER_POLL_LIMIT) { failed = true; break; }
      }
      lo += bf16x2_lo(data);
      hi += bf16x2_hi(data);
    }
    if (!failed) {
      if (2 * i + 1 < p.count) reinterpret_cast<uint32_t*>(p.out)[i] = pack_bf16x2(lo, hi);
      else p.out[2 * i] = __float2bfloat16_rn(lo);
    }
  }
  if (__syncthreads_or(failed) && threadIdx.x == 0 && p.status != nullptr) *p.status = 1;
  if (threadIdx.x == 0) *p.epoch = epoch;
}

}  // namespace aoto

using namespace aoto;

extern "C" int aoto_sm100_peer_sum(const aoto_peer_sum_args* a, void* stream) {
  if (!a || !a->partial || !a->out || !a->epoch || !a->buffers) return AOTO_ERR_ARGUMENT;
  if (a->world < 1 || a->world > PEER_MAX_RANKS || a->rank < 0 || a->rank >= a->world) return AOTO_ERR_ARGUMENT;
  if (a->count <= 0 || ((a->count + 1) >> 1) > a->capacity_words) return AOTO_ERR_ARGUMENT;
  if ((reinterpret_cast<uintptr_t>(a->partial) & 3) || (reinterpret_cast<uintptr_t>(a->out) & 3)) return AOTO_ERR_ARGUMENT;
  PeerSumParams p;
  for (int q = 0; q < PEER_MAX_RANKS; ++q) p.buffers[q] = q < a->world ? static_cast<unsigned char*>(a->buffers[q]) : nullptr;
  for (int q = 0; q < a->world; ++q)
    if (p.buffers[q] == nullptr || (reinterpret_cast<uintptr_t>(p.buffers[q]) & 7)) return AOTO_ERR_ARGUMENT;
  p.partial = static_cast<const bf16*>(a->partial);
  p.out = static_cast<bf16*>(a->out);
  p.epoch = static_cast<unsigned int*>(a->epoch);
  p.status = static_cast<int*>(a->status);
  p.world = a->world; p.rank = a->rank; p.count = a->count; p.capacity_words = a->capacity_words;
  return launch_kernel(peer_sum_kernel, dim3(1), dim3(PEER_THREADS), 0, (cudaStream_t)stream, false, p);
}

extern "C" int64_t aoto_sm100_peer_sum_buffer_bytes(int32_t world, int32_t capacity_words) {
  if (world < 1 || world > PEER_MAX_RANKS || capacity_words <= 0) return 0;
  return (int64_t)2 * world * capacity_words * 8;
}
