"""The decode-attention entry point for callers that must not allocate.

Some hosts cannot hand this library a workspace: their device memory is carved up once at
start-up and allocation afterwards is forbidden (or there is simply no channel to pass a buffer
through). ``aoto_sm100_attention_decode_static`` serves them: it is the split-KV decode kernel
with its scratch in a fixed 1 MiB array inside the library. This file checks, through the C ABI,
that it gives the same answer as the ordinary entry point (which takes caller-allocated scratch)
on two calls in a row - the array is shared and keeps the first call's contents, so the second
call is the one that would expose a counter left dirty - and that a request too large for the
array is refused before anything is launched.

It is named to be collected last: every other test has already run when this one starts.
"""

import ctypes

import pytest
import torch

from tests.helpers import activations

pytestmark = pytest.mark.gpu

TOL = 1e-2  # the tolerance of the other attention parity tests (relative to max|expected|)


def _args(N, q, k, v, mask, out, scale):
    args = N.AttentionArgs()
    args.q, args.k, args.v, args.out = q.data_ptr(), k.data_ptr(), v.data_ptr(), out.data_ptr()
    args.mask = mask.data_ptr() if mask is not None else None
    _, qh, lq, d = q.shape
    args.query_heads, args.kv_heads, args.q_len, args.kv_len, args.head_dim = qh, k.shape[1], lq, k.shape[2], d
    args.causal, args.scale = 0, scale
    return args


def test_static_scratch_entry_point_matches_the_allocating_one(cuda):
    import aotolith_b200._native as N
    import aotolith_b200.ops as ops

    lib = N.load()
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    assert lib.aoto_sm100_attention_static_scratch_limit() == 1 << 20
    for round_index, (qh, kvh, kv_len, d, valid) in enumerate([(32, 8, 1280, 128, 1025), (14, 2, 700, 64, 700)]):
        q = activations(200 + round_index, 1, qh, 1, d).to(cuda)
        k = activations(210 + round_index, 1, kvh, kv_len, d).to(cuda)
        v = activations(220 + round_index, 1, kvh, kv_len, d).to(cuda)
        keep = (torch.arange(kv_len) >= kv_len - valid).reshape(1, 1, 1, kv_len).to(cuda)
        mask = ops.mask_select(keep, 0.0, float("-inf"))
        expected = ops.attention(q, k, v, mask, scale=d ** -0.5)  # caller-allocated scratch
        probe = _args(N, q, k, v, mask, expected, d ** -0.5)
        assert lib.aoto_sm100_attention_scratch_bytes(ctypes.byref(probe)) > 0  # the case does use scratch
        for call in range(2):  # twice in a row on the shared array
            out = torch.full_like(expected, float("nan"))
            args = _args(N, q, k, v, mask, out, d ** -0.5)
            status = lib.aoto_sm100_attention_decode_static(ctypes.byref(args), stream)
            assert status == N.OK, N.status_string(status)
            torch.cuda.synchronize()
            error = float((out.float() - expected.float()).abs().max()) / float(expected.float().abs().max())
            assert error <= TOL, f"shape {round_index}, call {call}: relative error {error}"
            assert torch.equal(out, expected)  # same kernel, same split order: bit-identical


def test_static_scratch_entry_point_refuses_what_does_not_fit(cuda):
    import aotolith_b200._native as N

    lib = N.load()
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    qh, kvh, kv_len, d = 32, 8, 8192, 128  # 32 heads x 128 splits x 130 floats: about 2 MiB of partials
    q = torch.zeros((1, qh, 1, d), dtype=torch.bfloat16, device=cuda)
    k = torch.zeros((1, kvh, kv_len, d), dtype=torch.bfloat16, device=cuda)
    out = torch.full_like(q, 7.0)
    args = _args(N, q, k, k, None, out, 1.0)
    assert lib.aoto_sm100_attention_scratch_bytes(ctypes.byref(args)) > lib.aoto_sm100_attention_static_scratch_limit()
    assert lib.aoto_sm100_attention_decode_static(ctypes.byref(args), stream) == N.ERR_TOO_LARGE
    torch.cuda.synchronize()
    assert bool((out == 7.0).all())  # nothing ran
    prefill = _args(N, torch.zeros((1, qh, 4, d), dtype=torch.bfloat16, device=cuda), k, k, None, out, 1.0)
    assert lib.aoto_sm100_attention_decode_static(ctypes.byref(prefill), stream) == N.ERR_UNSUPPORTED
