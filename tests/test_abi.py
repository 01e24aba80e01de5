"""The C ABI without a GPU: the library loads and exports what the header declares.

No kernel is launched here. The checks are: every function declared in
``include/aoto_sm100.h`` is an exported symbol of the built library and is bound
by the ctypes stub; the structs of the stub have the layout the header gives
them; the pure host-side queries (support, variant, scratch sizes, status
strings) answer as documented; argument checks refuse bad requests before any
CUDA call.
"""

import ctypes
import re
from pathlib import Path

import pytest

from aotolith_b200 import _native as N

HEADER = Path(__file__).resolve().parent.parent / "include" / "aoto_sm100.h"


def _declared_functions() -> list[str]:
    text = re.sub(r"/\*.*?\*/", "", HEADER.read_text(), flags=re.S)
    return sorted(set(re.findall(r"\b(aoto_sm100_\w+)\s*\(", text)))


def _header_struct_fields(name: str) -> list[str]:
    text = re.sub(r"/\*.*?\*/", "", HEADER.read_text(), flags=re.S)
    body = re.search(r"typedef struct " + name + r"\s*\{(.*?)\}\s*" + name + r"\s*;", text, flags=re.S).group(1)
    fields = []
    for statement in body.split(";"):
        statement = statement.strip()
        if not statement:
            continue
        # "const void* x", "int32_t kind, flags, N"
        first, *rest = statement.split(",")
        fields.append(re.findall(r"(\w+)\s*(?:\[\d+\])?$", first.strip())[0])
        fields.extend(r.strip().lstrip("*").strip() for r in rest)
    return fields


def test_library_exports_every_declared_function():
    declared = _declared_functions()
    assert len(declared) >= 25
    lib = N.load()
    for name in declared:
        assert hasattr(lib, name), f"{name} is declared in the header but not exported"
    assert sorted(N.EXPORTS) == declared, "the ctypes stub and the header list different functions"


@pytest.mark.parametrize("c_name,struct", [
    ("aoto_qmatmul_args", N.QMatmulArgs), ("aoto_attention_args", N.AttentionArgs),
    ("aoto_step_stage", N.StepStage), ("aoto_decode_step_args", N.DecodeStepArgs),
    ("aoto_dequantize_args", N.DequantizeArgs), ("aoto_rms_norm_args", N.RmsNormArgs),
    ("aoto_rope_args", N.RopeArgs), ("aoto_embedding_args", N.EmbeddingArgs),
    ("aoto_kv_append_args", N.KvAppendArgs), ("aoto_peer_sum_args", N.PeerSumArgs),
])
def test_struct_fields_follow_the_header(c_name, struct):
    assert [name for name, _ in struct._fields_] == _header_struct_fields(c_name)


def test_identity_and_status_strings():
    lib = N.load()
    assert lib.aoto_sm100_abi_version() == N.ABI_VERSION
    assert lib.aoto_sm100_compiled_arch() == 100
    assert lib.aoto_sm100_decode_step_stage_size() == ctypes.sizeof(N.StepStage)
    seen = {N.status_string(code) for code in (0, -1, -2, -3, -4, -5)}
    assert len(seen) == 6 and "unknown status" not in seen
    assert N.status_string(-99) == "unknown status"


def _qargs(M, n_rows, K, group, epilogue=N.EPILOGUE_NONE):
    args = N.QMatmulArgs()
    args.M, args.N, args.K, args.group_size, args.epilogue = M, n_rows, K, group, epilogue
    args.alpha = args.beta = 1.0
    return args


def test_qmatmul_queries_are_host_only():
    lib = N.load()
    assert lib.aoto_sm100_qmatmul_supported(ctypes.byref(_qargs(1, 1152, 896, 64))) == 1
    assert lib.aoto_sm100_qmatmul_supported(ctypes.byref(_qargs(1, 16, 128, 48))) == 0   # 48 does not divide 128
    assert lib.aoto_sm100_qmatmul_supported(ctypes.byref(_qargs(0, 16, 128, 64))) == 0
    assert lib.aoto_sm100_qmatmul_supported(None) == 0
    assert lib.aoto_sm100_qmatmul_variant(ctypes.byref(_qargs(1, 1152, 896, 64))) == b"qgemv_mma"
    assert lib.aoto_sm100_qmatmul_variant(ctypes.byref(_qargs(16, 1152, 896, 64))) == b"qgemm_rows"   # 2..16 rows
    assert lib.aoto_sm100_qmatmul_variant(ctypes.byref(_qargs(24, 1152, 896, 64))) == b"gemm_mma"
    assert lib.aoto_sm100_qmatmul_variant(ctypes.byref(_qargs(8, 4096, 14336, 64))) == b"gemm_tcgen05"  # staged rows too long
    assert lib.aoto_sm100_qmatmul_scratch_bytes(ctypes.byref(_qargs(16, 896, 4864, 64))) == 0
    assert lib.aoto_sm100_qmatmul_variant(ctypes.byref(_qargs(1, 24, 64, 16))) == b"qgemv_generic"
    assert lib.aoto_sm100_qmatmul_scratch_bytes(ctypes.byref(_qargs(1, 1152, 896, 64))) == 0
    # narrow prefill products split K over several CTAs and ask for a workspace of partial tiles:
    # 7 output tiles, 76 k blocks -> 4 splits of 128 x 896 fp32 behind the 4096-byte counter header
    assert lib.aoto_sm100_qmatmul_scratch_bytes(ctypes.byref(_qargs(128, 896, 4864, 64))) == 4096 + 4 * 128 * 896 * 4
    assert lib.aoto_sm100_qmatmul_scratch_bytes(ctypes.byref(_qargs(128, 896, 896, 64))) == 0      # 14 k blocks: too short to split
    assert lib.aoto_sm100_qmatmul_scratch_bytes(ctypes.byref(_qargs(128, 151936, 896, 64))) == 0   # 1187 tiles fill the GPU
    # eight-bit words (four codes a word) select their own kernels and never ask for a workspace
    eight = _qargs(1, 1152, 896, 64)
    eight.flags = N.FLAG_WEIGHT_BITS_8
    assert lib.aoto_sm100_qmatmul_supported(ctypes.byref(eight)) == 1
    assert lib.aoto_sm100_qmatmul_variant(ctypes.byref(eight)) == b"qgemv_i8"
    eight.M = 128
    assert lib.aoto_sm100_qmatmul_variant(ctypes.byref(eight)) == b"qgemm_i8_rows"
    assert lib.aoto_sm100_qmatmul_scratch_bytes(ctypes.byref(eight)) == 0
    eight.epilogue = N.EPILOGUE_SILU_MUL_PAIRED                       # the paired form needs a single row
    assert lib.aoto_sm100_qmatmul_supported(ctypes.byref(eight)) == 0
    assert lib.aoto_sm100_dequantize_i8(None, None) == N.ERR_ARGUMENT
    # a dense bf16 weight (no scales, no groups): rows of whole 16-byte units, one row for the paired form
    dense = _qargs(1, 1152, 896, 896)
    dense.flags = N.FLAG_WEIGHT_DENSE
    assert lib.aoto_sm100_qmatmul_supported(ctypes.byref(dense)) == 1
    assert lib.aoto_sm100_qmatmul_variant(ctypes.byref(dense)) == b"dgemv_mma"      # one row, K a multiple of 32
    narrow = _qargs(1, 1152, 72, 72)
    narrow.flags = N.FLAG_WEIGHT_DENSE
    assert lib.aoto_sm100_qmatmul_variant(ctypes.byref(narrow)) == b"dgemv"         # other K: a warp per weight row
    assert lib.aoto_sm100_qmatmul_scratch_bytes(ctypes.byref(dense)) == 0
    dense.M = 24
    assert lib.aoto_sm100_qmatmul_variant(ctypes.byref(dense)) == b"dgemm_rows"
    dense.epilogue = N.EPILOGUE_SILU_MUL_PAIRED
    assert lib.aoto_sm100_qmatmul_supported(ctypes.byref(dense)) == 0
    odd = _qargs(1, 16, 100, 100)                                      # 100 weights are not whole units
    odd.flags = N.FLAG_WEIGHT_DENSE
    assert lib.aoto_sm100_qmatmul_supported(ctypes.byref(odd)) == 0
    assert lib.aoto_sm100_qmatmul_variant(ctypes.byref(odd)) == b"none"
    assert lib.aoto_sm100_qmatmul(ctypes.byref(dense), None) == N.ERR_ARGUMENT
    # null pointers are refused before anything reaches the CUDA runtime
    assert lib.aoto_sm100_qmatmul(ctypes.byref(_qargs(1, 1152, 896, 64)), None) == N.ERR_ARGUMENT
    assert lib.aoto_sm100_qmatmul(None, None) == N.ERR_ARGUMENT


def test_peer_sum_refuses_bad_requests_on_the_host():
    lib = N.load()
    assert lib.aoto_sm100_peer_sum_buffer_bytes(2, 2048) == 2 * 2 * 2048 * 8
    assert lib.aoto_sm100_peer_sum_buffer_bytes(9, 2048) == 0      # at most eight ranks
    assert lib.aoto_sm100_peer_sum(None, None) == N.ERR_ARGUMENT
    args = N.PeerSumArgs()
    args.world, args.rank, args.count, args.capacity_words = 2, 0, 4096, 2048
    assert lib.aoto_sm100_peer_sum(ctypes.byref(args), None) == N.ERR_ARGUMENT   # null pointers


def test_scratch_size_queries():
    lib = N.load()
    args = N.AttentionArgs()
    args.query_heads, args.kv_heads, args.q_len, args.kv_len, args.head_dim = 14, 2, 1, 192, 64
    assert lib.aoto_sm100_attention_scratch_bytes(ctypes.byref(args)) == 4096 + 14 * 3 * 66 * 4
    args.kv_len = 64
    assert lib.aoto_sm100_attention_scratch_bytes(ctypes.byref(args)) == 0      # one split: no merge
    args.q_len, args.kv_len = 128, 128
    assert lib.aoto_sm100_attention_scratch_bytes(ctypes.byref(args)) == 0      # short prefill uses none
    # a long masked prefill classifies the 64 x 64 tiles of its mask: one byte per tile behind the header
    args.q_len, args.kv_len, args.mask = 1000, 1024, 4096
    assert lib.aoto_sm100_attention_scratch_bytes(ctypes.byref(args)) == 4096 + 16 * 16
    args.mask = None
    assert lib.aoto_sm100_attention_scratch_bytes(ctypes.byref(args)) == 0      # nothing to classify
    assert lib.aoto_sm100_attention_static_scratch_limit() == 1 << 20
    assert lib.aoto_sm100_argmax_scratch_bytes(1, 151936) > 4096
    assert lib.aoto_sm100_stamped_bytes(896) == 896 * 4                          # 2 values per 8-byte word
    # requests the static-scratch entry point refuses without touching the device
    args.q_len, args.kv_len, args.query_heads, args.head_dim = 1, 1 << 20, 64, 128
    assert lib.aoto_sm100_attention_decode_static(ctypes.byref(args), None) == N.ERR_TOO_LARGE
    args.q_len = 2
    assert lib.aoto_sm100_attention_decode_static(ctypes.byref(args), None) == N.ERR_UNSUPPORTED
    assert lib.aoto_sm100_attention_decode_static(None, None) == N.ERR_ARGUMENT
