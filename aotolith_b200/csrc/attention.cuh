// Parameters shared by the attention kernels.
#pragma once

#include "common.cuh"

namespace aoto {

struct AttnParams {
  const bf16* q;
  const bf16* k;
  const bf16* v;
  const bf16* mask;
  bf16* out;
  float* scratch;
  const unsigned char* tile_classes;  // prefill: class of every (query tile, key tile) of the mask, or nullptr
  int key_tiles;                      // prefill: key tiles per query tile in tile_classes
  int QH, KVH, Lq, Lk, D;
  int causal, splits, keys_per_split;
  float scale;
};

// Tiled tensor-pipe prefill attention (attention_prefill.cu).
bool attention_prefill_mma_applies(const AttnParams& p);
int64_t attention_prefill_scratch_bytes(const AttnParams& p);
int attention_prefill_mma_launch(const AttnParams& p, int64_t scratch_bytes, cudaStream_t stream);

}  // namespace aoto
