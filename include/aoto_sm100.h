/*
 * aoto_sm100.h - C ABI of the sm_100a (B200) kernel library behind the
 * "cuda-sm100" compile target.
 *
 * Every entry point has the same shape:
 *
 *     int aoto_sm100_<kernel>(const aoto_<kernel>_args* args, void* stream);
 *
 * `stream` is a cudaStream_t passed as an opaque pointer (NULL = legacy default
 * stream). All tensor pointers are DEVICE pointers owned by the caller; the
 * library never allocates, frees, synchronises or throws. The return value is
 * AOTO_OK (0) or one of the negative status codes below; a launch error leaves
 * the CUDA error state cleared (it is consumed and reported as
 * AOTO_ERR_LAUNCH). Entry points are re-entrant across streams and host
 * threads. Element type of every activation / scale / table tensor is bfloat16
 * unless a field says otherwise; packed weights are 32-bit words; indices are
 * int64.
 *
 * Each entry point replaces one per-operation runtime of the reference
 * compiler (paths are relative to the reference project root,
 * src/aotolith/...). The reference dispatches an operation either to a Metal
 * kernel emitted by `codegen/*` or to `runtime/mlx_ops/_evaluate_mlx_op`; the
 * citation names both where both exist.
 */
#ifndef AOTO_SM100_H
#define AOTO_SM100_H

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define AOTO_ABI_VERSION 1

/* status codes */
#define AOTO_OK 0
#define AOTO_ERR_ARGUMENT (-1)    /* null pointer, non-positive size, misaligned buffer */
#define AOTO_ERR_UNSUPPORTED (-2) /* a legal request this library has no variant for     */
#define AOTO_ERR_LAUNCH (-3)      /* the CUDA runtime refused the launch                 */
#define AOTO_ERR_TIMEOUT (-4)     /* a bounded device-side wait ran out                  */
#define AOTO_ERR_TOO_LARGE (-5)   /* the request exceeds a fixed capacity of the library */

/* Library identity: ABI version and the SM architecture it was compiled for. */
int aoto_sm100_abi_version(void);
int aoto_sm100_compiled_arch(void); /* 100 */
const char* aoto_sm100_status_string(int status);

/* ------------------------------------------------------------------------- */
/* Packed 4-bit matmul / addmm                                               */
/* ------------------------------------------------------------------------- */

/* what `addend` is */
#define AOTO_ADDEND_NONE 0
#define AOTO_ADDEND_VECTOR 1 /* [N], broadcast over rows (a bias)        */
#define AOTO_ADDEND_FULL 2   /* [M,N], same shape as the output (residual) */

/* epilogue */
#define AOTO_EPILOGUE_NONE 0
#define AOTO_EPILOGUE_SILU_MUL 1        /* out = y * silu(gate[M,N])                   */
#define AOTO_EPILOGUE_SILU_MUL_PAIRED 2 /* out = y2 * silu(y), y from packed, y2 packed2 */

/*
 * y[M,N] = beta*addend + alpha * (x_hat[M,K] . W[N,K]^T), W given as signed
 * 4-bit codes (eight per 32-bit word, code k of a word at bit 4k, word j of a
 * row = codes 8j..8j+7, two's complement) with one scale per `group_size`
 * codes along K; x_hat = x, or rms_norm(x)*norm_weight rounded to bf16 when
 * `norm_weight` is given.
 *
 * Replaces: packed `matmul` / `addmm` evaluation,
 * runtime/mlx_ops/__init__.py:569-619 with runtime/mlx_ops/matmul.py:17-37,
 * and the int4 streaming GEMV codegen/matmul.py:542-739. For M > 1 it
 * replaces the `dequantize_i4` + dense `matmul`/`addmm{transpose_b}` pair
 * (passes/quantize.py:62-71 keeps them apart when M != 1): the weight is
 * rounded to bf16 as code*scale before it is multiplied, as
 * codegen/quantize.py:41-63 materialises it.
 */
typedef struct aoto_qmatmul_args {
  const void* x;            /* [M,K] bf16                                        */
  const void* packed;       /* [N,K/8] int32 words                               */
  const void* scales;       /* [N,K/group_size] bf16                             */
  const void* packed2;      /* second weight for SILU_MUL_PAIRED, else NULL      */
  const void* scales2;
  const void* addend;       /* per addend_kind, else NULL                        */
  const void* gate;         /* [M,N] bf16 for SILU_MUL, else NULL                */
  const void* norm_weight;  /* [K] bf16: fused RMS-norm prologue, else NULL      */
  void* out;                /* [M,N] bf16                                        */
  void* scratch;            /* optional split-K workspace (see *_scratch_bytes)  */
  int64_t scratch_bytes;
  int32_t M, N, K;
  int32_t group_size;
  int32_t addend_kind;
  int32_t epilogue;
  float alpha, beta;
  float rms_norm_eps;
  int32_t flags;            /* AOTO_FLAG_* */
} aoto_qmatmul_args;

#define AOTO_FLAG_PDL 1 /* launch with programmatic dependent launch enabled */
/*
 * The weight is packed with EIGHT bits a code: four codes per 32-bit word, code k of a word at
 * bit 8k, word j of a row = codes 4j..4j+3, two's complement; `packed` is [N,K/4] (and 8-byte
 * aligned), scales as before. Every weight is rounded to bf16 as code*scale before it is
 * multiplied. K and group_size must be multiples of 8 and K <= 32768; the norm prologue and the
 * paired epilogue need M == 1; no workspace. Variants "qgemv_i8" (M == 1) and "qgemm_i8_rows".
 * Replaces: packed `matmul`/`addmm` with weight_bits == 8, runtime/mlx_ops/__init__.py:569-619
 * (unpack by quantize.py:250-262), and the int8 GEMV codegen/matmul.py:742-929.
 */
#define AOTO_FLAG_WEIGHT_BITS_8 2
/*
 * The weight is NOT packed: `packed` (and `packed2`) are dense bf16 matrices [N,K] as the model
 * stores them, `scales` and `group_size` are ignored. K must be a multiple of 8 and at most 32768;
 * no norm prologue (dense graphs keep the norm as its own operation); the paired epilogue needs
 * M == 1; no workspace; operands on 16-byte boundaries. Variants "dgemv_mma" (M == 1, K a multiple
 * of 32, N >= 16: the multiply-add on the tensor pipe), "dgemv" (other single rows) and
 * "dgemm_rows". Replaces: dense
 * `matmul`/`addmm{transpose_b}`, runtime/mlx_ops/__init__.py:587-619, and the transposed GEMV with
 * its paired epilogue codegen/matmul.py:269-457.
 */
#define AOTO_FLAG_WEIGHT_DENSE 4

int aoto_sm100_qmatmul(const aoto_qmatmul_args* args, void* stream);
/*
 * The tensor-core variant (several activation rows) waits on hardware barriers with a bound; a
 * wait that runs out sets a flag on the device and the kernel exits with its tile unwritten.
 * This call returns that flag (1 = a wait ran out since the last call, 0 = none, -1 = the
 * query itself failed) and clears it. It synchronises the device: a diagnostic, not part of a
 * step. No counterpart in the reference.
 */
int aoto_sm100_qmatmul_take_timeout_flag(void);
/* 1 if a native variant exists for these shapes/flags, 0 if not (pointers ignored). */
int aoto_sm100_qmatmul_supported(const aoto_qmatmul_args* args);
/* Bytes of scratch the split-K variant wants for this shape (0 = none needed). */
int64_t aoto_sm100_qmatmul_scratch_bytes(const aoto_qmatmul_args* args);
/* Name of the kernel variant `aoto_sm100_qmatmul` would launch (static string). */
const char* aoto_sm100_qmatmul_variant(const aoto_qmatmul_args* args);

/*
 * W[n, 8j+i] = bf16(code) * bf16(scale[n, (8j+i)/group]) rounded once to bf16.
 * Replaces: `dequantize_i4`, models/quantized.py:61-76, quantize.py:216-234,
 * codegen/quantize.py:27-63.
 */
typedef struct aoto_dequantize_args {
  const void* packed; /* [N,K/8] int32 */
  const void* scales; /* [N,K/group] bf16 */
  void* out;          /* [N,K] bf16 */
  int32_t N, K, group_size;
} aoto_dequantize_args;
int aoto_sm100_dequantize_i4(const aoto_dequantize_args* args, void* stream);
/*
 * The same for eight-bit codes: packed [N,K/4] int32 (8-byte aligned), K and group_size
 * multiples of 8 (AOTO_ERR_UNSUPPORTED otherwise).
 * Replaces: `dequantize_i8`, models/quantized.py:90-105, quantize.py:250-262.
 */
int aoto_sm100_dequantize_i8(const aoto_dequantize_args* args, void* stream);

/* ------------------------------------------------------------------------- */
/* Normalisation, rotary embedding, gathers                                  */
/* ------------------------------------------------------------------------- */

/*
 * out[r,:] = bf16( (x[r,:] (+ residual[r,:])) * rsqrt(mean(.^2)+eps) * weight ),
 * fp32 statistics, one rounding. With `residual`, `sum_out` (optional) receives
 * bf16(x+residual), the value the norm was taken of.
 * Replaces: `rms_norm`, runtime/mlx_ops/normalization.py:73-119,
 * codegen/norm.py:75-313.
 */
typedef struct aoto_rms_norm_args {
  const void* x;        /* [rows, H] */
  const void* residual; /* [rows, H] or NULL */
  const void* weight;   /* [H] or NULL */
  void* out;            /* [rows, H] */
  void* sum_out;        /* [rows, H] or NULL */
  int32_t rows, H;
  float eps;
} aoto_rms_norm_args;
int aoto_sm100_rms_norm(const aoto_rms_norm_args* args, void* stream);

/*
 * out = x*cos + rotate_half(x)*sin over the last axis, x [B,heads,T,D] given
 * with explicit element strides (so a transposed view of a projection row can
 * be read in place), tables [T,D] (row t for step t, already gathered).
 * Each product and the sum are rounded to bf16, as three separate bf16
 * operations would. Output is contiguous [B,heads,T,D].
 * Replaces: `rope`, runtime/mlx_ops/__init__.py:276-280, codegen/index.py:22-67.
 */
typedef struct aoto_rope_args {
  const void* x;
  const void* cos_table; /* [T,D] */
  const void* sin_table; /* [T,D] */
  void* out;
  int32_t B, heads, T, D;
  int64_t stride_b, stride_h, stride_t; /* element strides of x; last axis is unit */
} aoto_rope_args;
int aoto_sm100_rope(const aoto_rope_args* args, void* stream);

/*
 * out[i,:] = table[ids[i],:] for int64 ids. `bad_index` (optional, one int64
 * on the device, caller-zeroed) receives 1 + the first offending position when
 * an id is outside [0, rows); such rows are written as zeros, never read.
 * Replaces: `embedding`, runtime/mlx_ops/__init__.py:281-283 with the bounds
 * contract of runtime/bounds.py:96-106.
 */
typedef struct aoto_embedding_args {
  const void* table;  /* [rows, width] bf16 */
  const int64_t* ids; /* [count] */
  void* out;          /* [count, width] */
  int64_t* bad_index;
  int32_t rows, width, count;
} aoto_embedding_args;
int aoto_sm100_embedding(const aoto_embedding_args* args, void* stream);

/*
 * out[i] = mask[i] ? on_true : on_false for a bool (uint8) mask, bf16 output.
 * Replaces: the `fused_elementwise{scalar_tensor, scalar_tensor, where}` that
 * turns the boolean attention mask into an additive one,
 * runtime/mlx_ops/pointwise.py:38-42,101-102.
 */
typedef struct aoto_mask_select_args {
  const uint8_t* mask;
  void* out;
  int64_t count;
  float on_true, on_false;
} aoto_mask_select_args;
int aoto_sm100_mask_select(const aoto_mask_select_args* args, void* stream);

/*
 * out[r] = index of the first maximum of logits[r,:] (int64), the greedy
 * token. Replaces the host `argmax(logits[:, -1, :])` of
 * models/decoder.py:1054-1087.
 */
typedef struct aoto_argmax_args {
  const void* logits; /* [rows, width] bf16 */
  int64_t* out;       /* [rows] */
  void* scratch;      /* aoto_sm100_argmax_scratch_bytes(rows, width) bytes, or NULL when 0 */
  int64_t scratch_bytes;
  int32_t rows, width;
} aoto_argmax_args;
int aoto_sm100_argmax(const aoto_argmax_args* args, void* stream);
/* Wide rows are scanned by several CTAs that meet in scratch (same zero-before-first-use,
 * self-restoring contract as the attention scratch). 0 for narrow rows. */
int64_t aoto_sm100_argmax_scratch_bytes(int32_t rows, int32_t width);

/* ------------------------------------------------------------------------- */
/* Device-resident greedy loop                                               */
/* ------------------------------------------------------------------------- */

/*
 * The two pieces of host logic of the reference's greedy loop that sit between
 * decode steps, as kernels, so that a whole step can be one recorded graph with
 * no host round trip. `counters` is int32[2] on the device: counters[0] =
 * valid_length (tokens the cache holds after the coming step), counters[1] =
 * number of tokens generated so far by the loop.
 *
 * step_inputs: position[0] = valid_length - 1; mask[c] = (c >= capacity -
 * valid_length) for c in [0, capacity). Replaces `decode_mask` and the position
 * tensor of `decode_token` (models/decoder.py:889-932, :960-979).
 *
 * greedy_pick: token[0] = first argmax of logits[0..width); generated[counters[1]]
 * = token (if counters[1] < generated_capacity); then counters[0] += 1 and
 * counters[1] += 1. Replaces the argmax / append / `valid_length += 1` of
 * `_greedy_tokens` (models/decoder.py:1054-1087).
 */
typedef struct aoto_step_inputs_args {
  const int32_t* counters;
  int64_t* position; /* [1] */
  uint8_t* mask;     /* [capacity] bool */
  int32_t capacity;
} aoto_step_inputs_args;
int aoto_sm100_step_inputs(const aoto_step_inputs_args* args, void* stream);

typedef struct aoto_greedy_pick_args {
  const void* logits; /* [width] bf16 */
  int64_t* token;     /* [1] */
  int64_t* generated; /* [generated_capacity] */
  int32_t* counters;
  void* scratch;      /* aoto_sm100_argmax_scratch_bytes(1, width) bytes */
  int64_t scratch_bytes;
  int32_t width, generated_capacity;
} aoto_greedy_pick_args;
int aoto_sm100_greedy_pick(const aoto_greedy_pick_args* args, void* stream);

/* ------------------------------------------------------------------------- */
/* Static KV cache                                                           */
/* ------------------------------------------------------------------------- */

/*
 * One layer's decode-step cache update. `row` is the packed q/k/v projection
 * of the step, [1,1,(QH+2*KVH)*D]. Rotates the QH query heads (starting at
 * query_start) and the KVH key heads (key_start) with the step's cos/sin row,
 * copies the layer's window shifted left by one slot and writes the rotated
 * key and the value (value_start) into the last slot.
 *
 * cache is [L,2,1,KVH,C,D]; new_pair is [2,1,KVH,C,D] (it may point into a
 * slice of a larger [L,2,...] buffer); q_out is [1,QH,1,D]. With
 * `rotate == 0` the key is taken from `key` ([1,KVH,1,D], already rotated) and
 * no query is produced (`kv_cache_append`).
 *
 * Replaces: `rope_kv_cache_append` / `kv_cache_append`,
 * runtime/mlx_ops/__init__.py:189-236, codegen/kv_cache.py:43-215.
 */
typedef struct aoto_kv_append_args {
  const void* cache;
  const void* row;
  const void* key;       /* only when rotate == 0 */
  const void* cos_row;   /* [D] */
  const void* sin_row;   /* [D] */
  void* q_out;
  void* new_pair;
  int32_t layer, layers, kv_heads, capacity, head_dim;
  int32_t query_heads, query_start, key_start, value_start;
  int32_t rotate;
} aoto_kv_append_args;
int aoto_sm100_kv_cache_append(const aoto_kv_append_args* args, void* stream);

/* ------------------------------------------------------------------------- */
/* Attention                                                                 */
/* ------------------------------------------------------------------------- */

/*
 * Grouped-query scaled-dot-product attention, out = softmax(q.k^T*scale +
 * mask).v with fp32 softmax statistics; a row whose keys are all masked
 * yields zeros. q [1,QH,Lq,D], k/v [1,KVH,Lk,D] contiguous, mask additive
 * bf16 [Lq,Lk] (0 / -inf) or NULL, `causal` adds the top-left aligned causal
 * rule. out [1,QH,Lq,D]. Lq == 1 selects the split-KV decode kernel, which
 * needs `scratch` of aoto_sm100_attention_scratch_bytes() when it splits.
 * Lq > 1 with a mask over 256 or more keys can use a workspace of the same
 * query's size: a small first kernel classifies every 64 x 64 tile of the mask
 * (no key admitted / adds zero everywhere / mixed) and the attention kernel
 * passes over the first kind and reads no mask in the second. That workspace is
 * optional: with scratch NULL or too small the result is the same, every tile
 * is visited and the mask is read element by element.
 *
 * Scratch contract (the same for every entry point that takes `scratch`): the
 * first 4096 bytes hold arrival counters and must be zero before the FIRST use;
 * every launch leaves them at zero again, and the rest is payload that needs no
 * initialisation. One buffer can therefore serve different kernels and shapes
 * without clearing, as long as the launches that share it are ordered on one
 * stream (two launches that overlap on the device must not share it).
 *
 * Replaces: `attention`, runtime/mlx_ops/attention.py:52-85,
 * codegen/attention.py:447-657 (decode) and :68-422 (prefill),
 * `_zero_fully_masked_rows` codegen/attention.py:660-667.
 */
typedef struct aoto_attention_args {
  const void* q;
  const void* k;
  const void* v;
  const void* mask;
  void* out;
  void* scratch;
  int64_t scratch_bytes;
  int32_t query_heads, kv_heads, q_len, kv_len, head_dim;
  int32_t causal;
  float scale;
} aoto_attention_args;
int aoto_sm100_attention(const aoto_attention_args* args, void* stream);
int64_t aoto_sm100_attention_scratch_bytes(const aoto_attention_args* args);

/*
 * Single-query (decode) attention for callers that cannot allocate device memory.
 *
 * This entry point has no counterpart in the reference; it exists for hosts that are not allowed
 * to call cudaMalloc (or any allocating library routine) once they are running - a serving
 * process with a sealed memory budget, a runtime that embeds this library without a channel for
 * workspaces, a latency-critical loop where allocator calls are banned because they may
 * synchronise the device. It runs the same split-KV kernel as aoto_sm100_attention with
 * q_len == 1, but takes the scratch for the per-split partial results from a fixed array inside
 * the library instead of from `args->scratch` (which is ignored, as is `scratch_bytes`). The
 * caller still passes q, k, v, mask and out. It allocates nothing and frees nothing.
 *
 * Limits and rules:
 *  - the array is AOTO_STATIC_SCRATCH_BYTES (1 MiB) per GPU, held from the moment the library is
 *    loaded on that GPU until the process exits; a request whose
 *    aoto_sm100_attention_scratch_bytes() exceeds it returns AOTO_ERR_TOO_LARGE and launches
 *    nothing (roughly: query_heads * ceil(kv_len / 64) * (head_dim + 2) * 4 bytes must fit);
 *  - the first call on each device looks up the array's device address (a one-time, blocking
 *    set-up call into the CUDA runtime); make that first call during start-up, before any stream
 *    capture begins on that device;
 *  - every call on a device shares the one array and the array keeps the previous call's
 *    contents; the entry point clears the part that must start at zero on the given stream, but
 *    two calls whose kernels can overlap on the GPU (different streams, no dependency) race on
 *    it and must be serialised by the caller;
 *  - q_len must be 1 (AOTO_ERR_UNSUPPORTED otherwise: the multi-query kernel runs without a
 *    workspace through aoto_sm100_attention).
 */
#define AOTO_STATIC_SCRATCH_BYTES (1 << 20)
int aoto_sm100_attention_decode_static(const aoto_attention_args* args, void* stream);
int64_t aoto_sm100_attention_static_scratch_limit(void);

/* ------------------------------------------------------------------------- */
/* Small all-reduce over peer memory (tensor-parallel decode)                 */
/* ------------------------------------------------------------------------- */

/*
 * Sum of one bf16 row per rank, delivered to every rank, in one launch per rank and with no
 * library collective: each rank stores its row as 8-byte stamped words (two values + the call's
 * epoch) into a receive buffer of every peer and polls its own buffer for all contributions,
 * which it adds in rank order in fp32. No counterpart in the reference (it has no multi-device
 * path); it replaces an NCCL all-reduce where the payload is a few KB and latency is everything.
 *
 *  - `buffers[q]` is rank q's receive buffer AS MAPPED IN THE CALLING PROCESS (peer-accessible
 *    memory, e.g. torch symmetric memory); every buffer is aoto_sm100_peer_sum_buffer_bytes()
 *    long, 8-byte aligned, and zero before the first call;
 *  - `epoch` is a device word, zero before the first call, that the kernel advances: all ranks
 *    must make the same sequence of calls with the same `count`;
 *  - every poll is bounded; when one runs out `*status` is set to 1 and the output is undefined;
 *  - the ranks' kernels wait on one another: one rank per GPU, never several ranks on one GPU.
 */
typedef struct aoto_peer_sum_args {
  void* const* buffers;   /* `world` device pointers (a host array)                 */
  const void* partial;    /* bf16 [count], this rank's addend                        */
  void* out;              /* bf16 [count], may alias partial                         */
  void* epoch;            /* uint32 device word                                      */
  void* status;           /* int32 device word or NULL                               */
  int32_t world, rank, count, capacity_words;
} aoto_peer_sum_args;

int aoto_sm100_peer_sum(const aoto_peer_sum_args* args, void* stream);
int64_t aoto_sm100_peer_sum_buffer_bytes(int32_t world, int32_t capacity_words);

/* ------------------------------------------------------------------------- */
/* A whole decode step as one persistent kernel                              */
/* ------------------------------------------------------------------------- */

/*
 * A decode step of the lowered graph is a chain of ~120 tiny operations, each
 * depending on the previous one; launched one by one, launch latency and the
 * cold start of every kernel dominate the step. aoto_sm100_decode_step runs the
 * whole chain in ONE cooperative launch: the caller describes the step as a
 * program of stages (below) and every CTA of the grid walks the program.
 *
 * Stages are NOT separated by barriers. Every intermediate vector lives in the
 * arena as 8-byte words {two bf16 values, 32-bit stamp}; a producer stores each
 * word with one 8-byte store carrying the launch's `epoch` as stamp, and a
 * consumer simply polls the words it needs until they carry that stamp. A stage
 * therefore starts on a CTA as soon as ITS inputs have landed, one L2 round
 * trip after they were produced, and the weights of a projection are requested
 * before its input row is polled, so the HBM stream does not stop at stage
 * boundaries. Polls are bounded: one that runs out stores 1 + the stage index
 * in `status` and the CTA leaves the kernel (its consumers then run out too).
 *
 * `epoch` must be non-zero and differ from the epoch of every earlier launch
 * that used the same arena (count launches). The arena needs no clearing.
 *
 * The program is what the reference's unrolled plan runner executes operation
 * by operation (runtime/plan.py:554-733) for the decode graph of
 * models/decoder.py:565-615; each stage kind covers the operations named in its
 * comment. All pointers in a stage are device pointers; `stages` itself is a
 * device array.
 */
#define AOTO_STAGE_GEMV 1      /* packed matmul / addmm, M = 1 (+ embedding gather of its input) */
#define AOTO_STAGE_ATTENTION 2 /* rope_kv_cache_append + mask conversion + attention of one layer */
#define AOTO_STAGE_PICK 3      /* greedy token from the per-CTA maxima of the preceding GEMV       */

#define AOTO_STAGE_FLAG_ARGMAX 2   /* GEMV: every CTA leaves its (max, index) in scratch for PICK  */
#define AOTO_STAGE_FLAG_WINDOW 4   /* ATTENTION: position and mask come from `counters`            */
#define AOTO_STAGE_FLAG_OUT_PLAIN 8 /* GEMV: `out` is a plain bf16 vector (a graph output)         */
#define AOTO_STAGE_FLAG_X_GATHER 16 /* GEMV: `x` is a bf16 table [x_rows, K]; its row x_index[0] is
                                       the input (an embedding folded into the projection)          */

/* how a GEMV stage reads its addend */
/* Tensor-parallel forms (streamed step kernel only). An exchanged vector of N values is `world`
 * rows of N/2 stamped words, row r written by rank r; every GPU holds all rows in a buffer its
 * peers can store into. */
#define AOTO_STAGE_FLAG_TO_PEERS 32   /* GEMV: `out` is row 0 of an exchanged vector: this rank's result goes
                                         to row `rank` of the vector on EVERY rank (peer stores)            */
#define AOTO_STAGE_FLAG_X_SUM 64      /* GEMV: `x` is an exchanged vector: the input is the sum of its rows  */
#define AOTO_STAGE_FLAG_ADDEND_SUM 128 /* GEMV: the stamped addend is an exchanged vector: sum of its rows   */
#define AOTO_STAGE_ADDEND_NONE 0
#define AOTO_STAGE_ADDEND_PLAIN 1   /* constant bf16 vector (a bias)                                */
#define AOTO_STAGE_ADDEND_STAMPED 2 /* an intermediate in the arena                                 */
#define AOTO_STAGE_ADDEND_GATHER 3  /* row x_index[0] of the bf16 table `addend` (width N)          */

typedef struct aoto_step_stage {
  /* GEMV */
  const void* x;             /* stamped [K], or the table of AOTO_STAGE_FLAG_X_GATHER                */
  const int64_t* x_index;    /* [1]: row index of the gathered input and/or of a gathered addend     */
  const void* packed;
  const void* scales;
  const void* packed2;
  const void* scales2;
  const void* addend;
  const void* norm_weight;
  void* out;                 /* stamped [N] (or plain bf16 with AOTO_STAGE_FLAG_OUT_PLAIN)            */
  /* ATTENTION */
  const void* row;           /* stamped packed q/k/v projection of the step, [(QH+2*KVH)*D]        */
  const void* cos_table;     /* bf16 [table_rows, D]; the row used is the step's position           */
  const void* sin_table;
  const int64_t* position;   /* [1] (ignored with AOTO_STAGE_FLAG_WINDOW)                           */
  const void* cache_in;      /* this layer's pair [2,1,KVH,C,D] in the incoming cache              */
  void* cache_out;           /* this layer's pair in the next cache                                 */
  const uint8_t* mask;       /* bool [C], true = attend (ignored with AOTO_STAGE_FLAG_WINDOW)       */
  void* attn_out;            /* stamped [QH*D] */
  /* PICK, and the window of ATTENTION */
  int64_t* token;            /* [1] */
  int64_t* generated;
  int32_t* counters;         /* int32[2]: valid_length of the step, tokens generated so far         */
  int64_t x_rows;
  int32_t kind, flags;
  int32_t N, K, group_size, addend_mode, epilogue;
  int32_t query_heads, kv_heads, capacity, head_dim;
  int32_t query_start, key_start, value_start, table_rows;
  int32_t generated_capacity, reserved;
  float alpha, beta, rms_norm_eps, scale;
} aoto_step_stage;

typedef struct aoto_decode_step_args {
  const aoto_step_stage* stages; /* device array */
  int32_t stage_count;
  int32_t ctas;                  /* 0 = one per SM */
  uint32_t epoch;                /* stamp of this launch, see above */
  int32_t reserved;
  int32_t* status;               /* device int32, zero = no error                                   */
  void* scratch;                 /* same contract as the other entry points                         */
  int64_t scratch_bytes;
  uint64_t* trace;               /* optional, device uint64[stage_count * 8]: CTA 0's %globaltimer
                                    (ns) per stage at: 0 stage reached, 1 input complete, 2 input
                                    staged, 3 first weight batch multiplied, 4 first round reduced,
                                    5 first round stored, 6 work done, 7 results out (stages other
                                    than GEMV fill 0, 1, 6, 7)                                       */
} aoto_decode_step_args;

int aoto_sm100_decode_step(const aoto_decode_step_args* args, void* stream);
/* Scratch bytes a program needs (host copy of the stages). */
int64_t aoto_sm100_decode_step_scratch_bytes(const aoto_step_stage* host_stages, int32_t stage_count);
/* 1 if every stage of the host copy is within the kernel's limits, else 0. */
int aoto_sm100_decode_step_supported(const aoto_step_stage* host_stages, int32_t stage_count);
int aoto_sm100_decode_step_stage_size(void); /* sizeof(aoto_step_stage), for binding checks */
/* Bytes of a stamped vector of `count` bf16 values (count even). */
int64_t aoto_sm100_stamped_bytes(int64_t count);

/* ------------------------------------------------------------------------- */
/* A whole decode step, weights streamed ahead of the dependency chain        */
/* ------------------------------------------------------------------------- */

/*
 * aoto_sm100_stream_step runs the same chain of stages as aoto_sm100_decode_step (same
 * stamped-word exchange between stages, same bounded polls, same replacement of
 * runtime/plan.py:554-733 over the decode graph of models/decoder.py:565-615), but takes the
 * weights from a STREAM the caller lays out once per model for the grid it will launch:
 *
 *  - the grid is one CTA of AOTO_STREAM_WARPS warps per SM; the caller decides, per stage, which
 *    contiguous range of 16-row weight tiles every CTA owns (`cta_table`) and cuts the CTA's
 *    blocks of the stage - (tile, matrix, 128-column block), tile-major - into one contiguous
 *    share per warp;
 *  - every warp has its own byte stream: the blocks of all its shares, stage after stage, in
 *    the order it will multiply them, cut into pieces of at most AOTO_STREAM_PIECE_BLOCKS
 *    blocks. A piece is a 16-byte header (aoto_stream_piece) followed by its blocks;
 *  - a block is AOTO_STREAM_BLOCK_BYTES of the packed weight in the order the tensor-core
 *    fragments want it (below), so one bulk copy brings a piece into the warp's ring in shared
 *    memory and the warp multiplies it from there with conflict-free 128-bit loads.
 *
 * A warp keeps `ring_depth` pieces in flight at all times, ACROSS stage boundaries: the weights
 * of a stage have normally been resident for several stages when its input row arrives, so a
 * stage on the critical path costs one poll, the staging of the row and a few blocks per warp.
 * Nothing but the warp itself touches its ring: no CTA-wide synchronisation manages it.
 *
 * Block layout (16 rows r0..r0+15 of one matrix, columns c0..c0+127, group size 64):
 *   bytes [0,512)     lane L = 4g+t (g = 0..7, t = 0..3): four 32-bit words for row r0+g;
 *   bytes [512,1024)  the same for row r0+g+8;
 *   bytes [1024,1088) row r: bf16 scale of columns c0..c0+63, then of c0+64..c0+127.
 *   Nibble n (bits 4n..4n+3) of word j holds the two's-complement code of column
 *   c0 + 16*(2j + ((n & 3) >> 1)) + 2t + 8*(n & 1) + (n >> 2): the k-th m16n8k16 step of a
 *   block (k = 0..7) covers columns c0+16k..c0+16k+15, so steps 0-3 belong to the first scale
 *   group and steps 4-7 to the second. Rows past N are zero.
 *
 * Layer-wise attention (rope_kv_cache_append + mask + attention). A window of at most 256 slots
 * whose buffers fit is handled by one CTA per query head, which takes the cache window the same
 * way: every warp bulk-copies its share of the keys and values of the NEXT layer while the current
 * one is still being computed. A longer window is cut into slices: CTA (kv head, slice) scores
 * all query heads of the group against its slice, and CTA h merges head h's partial results
 * (which travel through `scratch`, see aoto_sm100_stream_step_scratch_bytes_for).
 */
#define AOTO_STREAM_WARPS 16
#define AOTO_STREAM_BLOCK_BYTES 1088
#define AOTO_STREAM_PIECE_BLOCKS 3
#define AOTO_STREAM_SLOT_BYTES (16 + AOTO_STREAM_PIECE_BLOCKS * AOTO_STREAM_BLOCK_BYTES)
#define AOTO_STREAM_MAX_RING 3
#define AOTO_STREAM_PART_SLOTS 32   /* partial sums of tiles shared between warps, per CTA and stage */
#define AOTO_STREAM_NO_STAGE 0xFFFFu

#define AOTO_PIECE_SEG_END 1  /* last piece of this warp's share of the tile                      */
#define AOTO_PIECE_WHOLE 2    /* the share is the whole tile: the warp finishes it by itself      */
#define AOTO_PIECE_MAT1 4     /* the blocks belong to the second matrix of the paired form        */

/* 16 bytes in front of the blocks of every piece, in the form the kernel consumes them. */
typedef struct aoto_stream_piece {
  uint16_t next_stage;   /* stage of the warp's next piece, AOTO_STREAM_NO_STAGE after the last    */
  uint8_t nblocks;       /* 1..AOTO_STREAM_PIECE_BLOCKS                                            */
  uint8_t flags;         /* AOTO_PIECE_*                                                           */
  uint32_t column_bytes; /* 256 * (first 128-column block): where the blocks' columns start in the
                            staged row                                                             */
  uint16_t part_bytes;   /* SEG_END: 128 * (slot of this share's partial sums). Shares of a tile cut
                            across warps have consecutive slots below AOTO_STREAM_PART_SLOTS; a whole
                            tile uses slot AOTO_STREAM_PART_SLOTS + warp                            */
  uint16_t tile;         /* tile, counted from the first tile the CTA owns in this stage           */
  uint32_t ahead_bytes;  /* size of the piece `ring_depth` pieces later in this stream, 0 = none   */
} aoto_stream_piece;

/*
 * One entry per (stage, CTA, warp): the tile shared between warps that this warp finishes once
 * all shares have met (it holds the tile's last block), or 0.
 */
#define AOTO_STREAM_DUTY(tile, first_slot, nparts) \
  ((uint32_t)(tile) | 0x8000u | ((uint32_t)(first_slot) << 16) | ((uint32_t)(nparts) << 24))

typedef struct aoto_stream_warp_start {
  uint32_t offset16;     /* where the warp's stream starts in `stream`, in units of 16 bytes       */
  uint16_t size16[3];    /* sizes / 16 of its first pieces (0 = the stream has fewer)              */
  uint16_t first_stage;  /* stage of its first piece, AOTO_STREAM_NO_STAGE for an empty stream     */
  uint32_t reserved;
} aoto_stream_warp_start;

/* One entry per (stage, CTA): tile range of the CTA and whether it shares a tile between warps. */
#define AOTO_STREAM_CTA_ENTRY(tile0, tiles, shared) \
  ((uint32_t)(tile0) | ((uint32_t)(tiles) << 16) | ((uint32_t)((shared) ? 1u : 0u) << 31))

typedef struct aoto_stream_stage {
  const void* x;           /* GEMV: stamped [K] (or the table of AOTO_STAGE_FLAG_X_GATHER)
                              ATTENTION: stamped packed q/k/v projection of the step              */
  void* out;               /* GEMV: stamped [N] (plain bf16 with AOTO_STAGE_FLAG_OUT_PLAIN)
                              ATTENTION: stamped [query_heads * head_dim]                          */
  const void* addend;      /* GEMV: per addend_mode; ATTENTION: this layer's pair in the incoming cache */
  const void* norm_weight; /* GEMV: [K] or NULL;     ATTENTION: this layer's pair in the next cache */
  int32_t N, K;            /* GEMV                                                                 */
  float alpha, beta, rms_norm_eps;
  uint8_t kind;            /* AOTO_STAGE_GEMV / ATTENTION / PICK                                   */
  uint8_t epilogue;        /* AOTO_EPILOGUE_NONE or AOTO_EPILOGUE_SILU_MUL_PAIRED                  */
  uint8_t addend_mode;     /* AOTO_STAGE_ADDEND_*                                                  */
  uint8_t flags;           /* AOTO_STAGE_FLAG_*                                                    */
  int32_t next_attention;  /* ATTENTION: index of the next ATTENTION stage, -1 after the last      */
  int32_t ordinal;         /* ATTENTION: how many ATTENTION stages come before this one            */
} aoto_stream_stage;

typedef struct aoto_stream_step_args {
  const aoto_stream_stage* stages;      /* device array [stage_count]                              */
  const uint32_t* cta_table;            /* device [stage_count * ctas], AOTO_STREAM_CTA_ENTRY      */
  const uint32_t* duties;               /* device [stage_count * ctas * AOTO_STREAM_WARPS], AOTO_STREAM_DUTY */
  const aoto_stream_warp_start* starts; /* device [ctas * AOTO_STREAM_WARPS]                       */
  const void* stream;                   /* device, 16-byte aligned                                 */
  int64_t stream_bytes;
  int32_t stage_count;
  int32_t ctas;                         /* the grid the stream was laid out for                    */
  int32_t ring_depth;                   /* 2..AOTO_STREAM_MAX_RING, as the piece headers assume    */
  int32_t max_k;                        /* largest K of a GEMV stage                               */
  /* attention geometry, the same for every layer */
  int32_t query_heads, kv_heads, capacity, head_dim;
  int32_t query_start, key_start, value_start, table_rows;
  float scale;
  int32_t first_attention;              /* index of the first ATTENTION stage, -1 = none           */
  const void* cos_table;                /* bf16 [table_rows, head_dim]                             */
  const void* sin_table;
  const int64_t* position;              /* [1], ignored with `window`                              */
  const uint8_t* mask;                  /* bool [capacity], ignored with `window`                  */
  /* the step's token: row index of the gathered input / addend                                    */
  const int64_t* x_index;
  int64_t x_rows;
  /* greedy pick */
  int64_t* token;
  int64_t* generated;
  int32_t* counters;                    /* int32[2]: valid_length of the step, tokens generated    */
  int32_t generated_capacity;
  int32_t window;                       /* 1: position and mask come from `counters`               */
  uint32_t epoch;                       /* as for aoto_sm100_decode_step                           */
  int32_t attention_stages;             /* how many ATTENTION stages the program has               */
  int32_t* status;
  void* scratch;                        /* per-CTA maxima of the ARGMAX stage (16 bytes per CTA), then, with a
                                           long window, every ATTENTION stage's partial results (a region per
                                           stage: stamps cannot tell the layers of one launch apart)      */
  int64_t scratch_bytes;
  /* tensor parallelism: one process per GPU runs the same program over its shard. `world` = 1 and
     everything below zero for a single GPU. peer_delta[q] = (base of rank q's exchange buffer as
     mapped in this process) - (base of this rank's), so that a local address of the buffer plus
     peer_delta[q] is the same place on rank q; peer_delta[rank] = 0. Plain stores, no multimem.  */
  int32_t world, rank;
  int64_t peer_delta[8];
  void* pick_exchange;                  /* in the exchange buffer: `world` slots of 16 bytes, slot r = rank
                                           r's best (logit, global index) of the step                 */
  int32_t vocab_offset;                 /* index of this rank's first logit in the whole vocabulary   */
  int32_t reserved2;
  uint64_t* trace;                      /* optional, uint64[ctas * stage_count * 8]: every CTA's
                                           %globaltimer (ns) at eight points of every stage it works in
                                           (GEMV: 0 reached, 1-2 row complete, 3 row staged, 4 first piece
                                           multiplied, 5 all pieces, 6 shares met, 7 done; ATTENTION: 0
                                           reached, 1 row polled, 2 rotated, 3 window landed, 4 keys
                                           attended, 5 warps met, 6 merged, 7 done). Slows the kernel.  */
} aoto_stream_step_args;

int aoto_sm100_stream_step(const aoto_stream_step_args* args, void* stream);
/*
 * Dynamic shared memory the kernel needs for this geometry, or -1 if it has no form for it
 * (K not a multiple of 128 or above 16384, head_dim not 64/128, or a long window with more than
 * 512 stamped words of queries, key and value per kv head). Pointers of `args` are ignored.
 */
int64_t aoto_sm100_stream_step_smem_bytes(const aoto_stream_step_args* args);
int64_t aoto_sm100_stream_step_scratch_bytes(int32_t ctas);
/*
 * The same for a given geometry (pointers of `args` are ignored): with a window too long for the
 * per-warp buffers the kernel spreads every kv head's window over many CTAs and keeps their partial
 * results in scratch as well. This is the size `scratch_bytes` must cover; -1 if the kernel has
 * no form for the geometry.
 */
int64_t aoto_sm100_stream_step_scratch_bytes_for(const aoto_stream_step_args* args);
int aoto_sm100_stream_stage_size(void); /* sizeof(aoto_stream_stage), for binding checks */
int aoto_sm100_stream_args_size(void);  /* sizeof(aoto_stream_step_args), for binding checks */

#ifdef __cplusplus
}
#endif
#endif /* AOTO_SM100_H */
