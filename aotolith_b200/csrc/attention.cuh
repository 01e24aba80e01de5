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
  int QH, KVH, Lq, Lk, D;
  int causal, splits, keys_per_split;
  float scale;
};

// Tiled tensor-pipe prefill attention (attention_prefill.cu).
bool attention_prefill_mma_applies(const AttnParams& p);
int attention_prefill_mma_launch(const AttnParams& p, cudaStream_t stream);

}  // namespace aoto
