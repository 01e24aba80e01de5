"""The algorithmic-byte accounting the roofline figures of bench.py rest on.

Weights of one Qwen2.5-0.5B-shaped layer are 7 926 528 bytes and the LM head is
72 321 536 bytes in the packed format (codes at half a byte plus one bf16 scale
per 64 codes); the per-projection figures of the packed-matmul sweep follow the
same formula. These are the numbers the reference's own accounting of ~250 MB
per step rounds (``README.md:222`` of the reference).
"""

import importlib.util
from pathlib import Path
from types import SimpleNamespace

ROOT = Path(__file__).resolve().parent.parent
spec = importlib.util.spec_from_file_location("bench_module", ROOT / "bench.py")
bench = importlib.util.module_from_spec(spec)
spec.loader.exec_module(bench)


def _weights(n, k):
    return n * k // 2 + n * (k // 64) * 2


def test_projection_bytes_match_the_sweep_table():
    assert bench.projection_bytes(1152, 896, bias=True) == 554_752
    assert bench.projection_bytes(896, 896) == 430_080
    assert bench.projection_bytes(4864, 896) == 2_326_784
    assert bench.projection_bytes(896, 4864) == 2_326_784
    assert bench.projection_bytes(151936, 896) == 72_627_200
    assert bench.projection_bytes(1152, 896, bias=True, m=128) == 1_074_944
    assert bench.projection_bytes(151936, 896, m=128) == 111_446_528


def test_step_bytes_of_the_qwen_shape():
    config = SimpleNamespace(hidden_size=896, intermediate_size=4864, num_hidden_layers=24, num_attention_heads=14,
                             num_key_value_heads=2, head_dim=64, vocab_size=151936)
    layer_weights = (_weights(1152, 896) + _weights(896, 896) + 2 * _weights(4864, 896) + _weights(896, 4864)
                     + 1152 * 2 + 2 * 896 * 2)  # packed matrices, q/k/v bias, two norm weights
    assert layer_weights == 7_926_528
    assert _weights(151936, 896) == 72_321_536
    total = bench.step_bytes(config, 160)
    weights = 24 * layer_weights + 72_321_536
    assert weights == 262_558_208
    # activations, norms, bias, KV window and logits add about one per cent
    assert weights < total < weights * 1.02
    assert total == 265_669_120


def test_step_bytes_of_the_llama_shape():
    config = SimpleNamespace(hidden_size=4096, intermediate_size=14336, num_hidden_layers=32, num_attention_heads=32,
                             num_key_value_heads=8, head_dim=128, vocab_size=128256)
    layer_weights = (_weights(6144, 4096) + _weights(4096, 4096) + 2 * _weights(14336, 4096) + _weights(4096, 14336)
                     + 2 * 4096 * 2)  # packed matrices and two norm weights (no bias)
    assert layer_weights == 115_884_032
    assert _weights(128256, 4096) == 279_085_056
    total = bench.step_bytes(config, 1152)
    assert 32 * layer_weights + 279_085_056 < total < (32 * layer_weights + 279_085_056) * 1.05


def test_dense_step_bytes_of_the_qwen_shape():
    """Two bytes a weight: the ~991 MB a step the reference's bf16 rows stream (``README.md:147-152``)."""

    config = SimpleNamespace(hidden_size=896, intermediate_size=4864, num_hidden_layers=24, num_attention_heads=14,
                             num_key_value_heads=2, head_dim=64, vocab_size=151936)
    weights = 2 * (24 * (1152 * 896 + 896 * 896 + 3 * 4864 * 896) + 151936 * 896)
    assert weights == 987_922_432
    total = bench.dense_step_bytes(config, 160)
    assert weights < total < weights * 1.01
