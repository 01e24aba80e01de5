// Library identity and the packed-matmul entry point, which picks between the
// GEMV kernels (one activation row per grid slice) and the tensor-core GEMM.
#include "common.cuh"

namespace aoto {
int qgemv_launch(const aoto_qmatmul_args& a, cudaStream_t stream);
int qgemv_check(const aoto_qmatmul_args& a, bool pointers);
const char* qgemv_variant(const aoto_qmatmul_args& a);
bool qgemm_applies(const aoto_qmatmul_args& a);
bool qgemm_tc_applies(const aoto_qmatmul_args& a);
bool qgemm_rows_applies(const aoto_qmatmul_args& a);
int qgemm_rows_launch(const aoto_qmatmul_args& a, cudaStream_t stream);
bool qgemv_stream_applies(const aoto_qmatmul_args& a);
int qgemv_stream_launch(const aoto_qmatmul_args& a, cudaStream_t stream);
int qgemm_tc_launch(const aoto_qmatmul_args& a, cudaStream_t stream);
int qgemm_tc_take_timeout_flag();
int64_t qgemm_tc_scratch_bytes(const aoto_qmatmul_args& a);
int qgemm_launch(const aoto_qmatmul_args& a, cudaStream_t stream);
bool qmatmul_i8_supported(const aoto_qmatmul_args& a);
int qmatmul_i8_launch(const aoto_qmatmul_args& a, cudaStream_t stream);
const char* qmatmul_i8_variant(const aoto_qmatmul_args& a);
bool dmatmul_supported(const aoto_qmatmul_args& a);
int dmatmul_launch(const aoto_qmatmul_args& a, cudaStream_t stream);
const char* dmatmul_variant(const aoto_qmatmul_args& a);
int dequantize_i8_launch(const aoto_dequantize_args& a, cudaStream_t stream);
}  // namespace aoto

using namespace aoto;

extern "C" int aoto_sm100_abi_version(void) { return AOTO_ABI_VERSION; }

extern "C" int aoto_sm100_compiled_arch(void) { return 100; }

extern "C" const char* aoto_sm100_status_string(int status) {
  switch (status) {
    case AOTO_OK: return "ok";
    case AOTO_ERR_ARGUMENT: return "invalid argument (null pointer, bad size or misaligned buffer)";
    case AOTO_ERR_UNSUPPORTED: return "no kernel variant for this request";
    case AOTO_ERR_LAUNCH: return "the CUDA runtime refused the launch";
    case AOTO_ERR_TIMEOUT: return "a bounded device-side wait ran out";
    case AOTO_ERR_TOO_LARGE: return "the request exceeds a fixed capacity of the library";
    default: return "unknown status";
  }
}

extern "C" int aoto_sm100_qmatmul_supported(const aoto_qmatmul_args* a) {
  if (!a) return 0;
  if (qgemv_check(*a, false) != AOTO_OK) return 0;
  if (a->flags & AOTO_FLAG_WEIGHT_DENSE) return dmatmul_supported(*a) ? 1 : 0;
  if (a->flags & AOTO_FLAG_WEIGHT_BITS_8) return qmatmul_i8_supported(*a) ? 1 : 0;
  if (a->K > 49152) return 0;
  return 1;
}

extern "C" int64_t aoto_sm100_qmatmul_scratch_bytes(const aoto_qmatmul_args* a) {
  if (!a || (a->flags & (AOTO_FLAG_WEIGHT_BITS_8 | AOTO_FLAG_WEIGHT_DENSE))) return 0;
  if (qgemm_rows_applies(*a)) return 0;
  if (qgemm_tc_applies(*a)) return qgemm_tc_scratch_bytes(*a);  // split-K partial tiles
  return 0;
}

extern "C" const char* aoto_sm100_qmatmul_variant(const aoto_qmatmul_args* a) {
  if (!a) return "none";
  if (a->flags & AOTO_FLAG_WEIGHT_DENSE) return dmatmul_supported(*a) ? dmatmul_variant(*a) : "none";
  if (a->flags & AOTO_FLAG_WEIGHT_BITS_8) return qmatmul_i8_supported(*a) ? qmatmul_i8_variant(*a) : "none";
  if (qgemm_rows_applies(*a)) return "qgemm_rows";
  if (qgemm_tc_applies(*a)) return "gemm_tcgen05";
  if (qgemv_stream_applies(*a)) return "qgemv_stream";
  if (qgemm_applies(*a)) return "gemm_mma";
  return qgemv_variant(*a);
}

extern "C" int aoto_sm100_qmatmul(const aoto_qmatmul_args* a, void* stream) {
  if (!a) return AOTO_ERR_ARGUMENT;
  const int status = qgemv_check(*a, true);
  if (status != AOTO_OK) return status;
  if (a->flags & AOTO_FLAG_WEIGHT_DENSE) return dmatmul_launch(*a, (cudaStream_t)stream);
  if (a->flags & AOTO_FLAG_WEIGHT_BITS_8) return qmatmul_i8_launch(*a, (cudaStream_t)stream);
  if (qgemm_rows_applies(*a)) return qgemm_rows_launch(*a, (cudaStream_t)stream);
  if (qgemm_tc_applies(*a)) return qgemm_tc_launch(*a, (cudaStream_t)stream);
  if (qgemv_stream_applies(*a)) return qgemv_stream_launch(*a, (cudaStream_t)stream);
  if (qgemm_applies(*a)) return qgemm_launch(*a, (cudaStream_t)stream);
  return qgemv_launch(*a, (cudaStream_t)stream);
}

extern "C" int aoto_sm100_qmatmul_take_timeout_flag(void) { return qgemm_tc_take_timeout_flag(); }

extern "C" int aoto_sm100_dequantize_i8(const aoto_dequantize_args* a, void* stream) {
  if (!a || !a->packed || !a->scales || !a->out) return AOTO_ERR_ARGUMENT;
  if (a->N <= 0 || a->K <= 0 || a->group_size <= 0 || a->K % a->group_size != 0) return AOTO_ERR_ARGUMENT;
  if (!aligned_to(a->out, 16) || !aligned_to(a->packed, 8)) return AOTO_ERR_ARGUMENT;
  return dequantize_i8_launch(*a, (cudaStream_t)stream);
}
