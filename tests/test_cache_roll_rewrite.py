"""The KV-cache roll rewrite: what it folds, what it leaves alone, and what it computes.

After the reference's tests/test_passes_cache.py. The roll is one statement written as a dozen
operations; the pass must fire on the spelling the decode adapter emits, must not fire on a
chain that only looks similar (a window that drops two slots, a pair with a third reader, a pair
that is a graph result), and the operation it produces must compute the same window, bit for
bit, as the concatenate it replaced - here through the oracle's evaluation of the rewritten graph.
"""

import torch

from aotolith_b200.capture import capture_fx
from aotolith_b200.passes.cache import fuse_kv_cache_update
from oracle.interp import run_graph

LAYERS, CAPACITY, HEADS, HEAD_DIM = 3, 12, 2, 8
PACKED = HEADS * HEAD_DIM * 3


class Roll(torch.nn.Module):
    """The decode adapter's spelling: drop the oldest slot, append the new pair, read it back."""

    def __init__(self, drop: int = 1, extra_reader: bool = False, return_pair: bool = False) -> None:
        super().__init__()
        self.drop, self.extra_reader, self.return_pair = drop, extra_reader, return_pair

    def forward(self, cache, projected, key):
        pairs, key_windows, value_windows, extras = [], [], [], []
        for layer in range(LAYERS):
            window = cache[layer][:, :, :, self.drop:, :]
            value = projected[:, :, 2 * HEADS * HEAD_DIM:].view(1, 1, HEADS, HEAD_DIM).transpose(1, 2)
            fresh = torch.stack((key[layer], value), dim=0)
            if self.drop == 2:
                fresh = torch.cat((fresh, fresh), dim=3)          # keeps the capacity, drops two slots
            new_pair = torch.cat((window, fresh), dim=3)
            pairs.append(new_pair)
            key_windows.append(new_pair[0])
            value_windows.append(new_pair[1])
            if self.extra_reader:
                extras.append(new_pair + new_pair)                 # a third reader of the pair
        outputs = [torch.stack(pairs, dim=0), torch.stack(key_windows, dim=0), torch.stack(value_windows, dim=0)]
        if self.extra_reader:
            outputs.append(torch.stack(extras, dim=0))
        if self.return_pair:
            outputs.append(pairs[0])
        return tuple(outputs)


def _inputs(seed: int = 0):
    generator = torch.Generator().manual_seed(seed)
    return (
        torch.randn((LAYERS, 2, 1, HEADS, CAPACITY, HEAD_DIM), generator=generator).bfloat16(),
        torch.randn((1, 1, PACKED), generator=generator).bfloat16(),
        torch.randn((LAYERS, 1, HEADS, 1, HEAD_DIM), generator=generator).bfloat16(),
    )


def _lowered(module):
    graph = capture_fx(module.eval(), _inputs())
    return graph, fuse_kv_cache_update(graph)


def _appends(graph):
    return [op for op in graph.ops if op.op == "kv_cache_append"]


def test_the_roll_becomes_one_operation_per_layer():
    graph, rewritten = _lowered(Roll())
    appends = _appends(rewritten)
    assert len(appends) == LAYERS
    assert [op.attrs["layer"] for op in appends] == list(range(LAYERS))
    assert all(op.attrs["value_start"] == 2 * HEADS * HEAD_DIM for op in appends)
    # the window slice, the pair slice, the squeezes, the concatenate and the value's
    # slice / reshape / transpose all go away with it
    assert len(graph.ops) - len(rewritten.ops) >= LAYERS * 6
    rewritten.validate()


def test_the_rewritten_graph_computes_the_same_window():
    for seed in (0, 7):
        inputs = _inputs(seed)
        expected = Roll()(*inputs)
        _, rewritten = _lowered(Roll())
        actual = run_graph(rewritten, list(inputs))
        assert len(actual) == len(expected)
        for got, want in zip(actual, expected):
            assert got.dtype == want.dtype and tuple(got.shape) == tuple(want.shape)
            assert torch.equal(got, want)


def test_the_unrewritten_graph_and_the_rewritten_one_agree():
    inputs = _inputs(3)
    graph, rewritten = _lowered(Roll())
    for got, want in zip(run_graph(rewritten, list(inputs)), run_graph(graph, list(inputs))):
        assert torch.equal(got, want)


def test_a_window_that_drops_two_slots_is_left_alone():
    graph, rewritten = _lowered(Roll(drop=2))
    assert _appends(rewritten) == []
    inputs = _inputs(1)
    for got, want in zip(run_graph(rewritten, list(inputs)), Roll(drop=2)(*inputs)):
        assert torch.equal(got, want)


def test_a_value_that_is_not_the_projection_row_is_left_alone():
    class Shaped(torch.nn.Module):
        def forward(self, cache, projected, key):
            pairs = []
            for layer in range(LAYERS):
                window = cache[layer][:, :, :, 1:, :]
                value = key[layer] + key[layer]                    # not a slice of the projected row
                pairs.append(torch.cat((window, torch.stack((key[layer], value), 0)), 3))
            return torch.stack(pairs)

    graph = capture_fx(Shaped().eval(), _inputs())
    rewritten = fuse_kv_cache_update(graph)
    assert _appends(rewritten) == []
    inputs = _inputs(5)
    (got,) = run_graph(rewritten, list(inputs))
    assert torch.equal(got, Shaped()(*inputs))


def test_other_readers_of_the_new_pair_read_the_operation_result():
    """The fused operation yields the pair itself as its first result, so a third reader of the
    pair (or the graph returning it) does not block the rewrite and sees the same values."""

    for module in (Roll(extra_reader=True), Roll(return_pair=True)):
        _, rewritten = _lowered(module)
        assert len(_appends(rewritten)) == LAYERS
        rewritten.validate()
        inputs = _inputs(2)
        for got, want in zip(run_graph(rewritten, list(inputs)), module(*inputs)):
            assert torch.equal(got, want)


def test_the_old_pair_may_have_other_readers():
    """The layer slice of the incoming cache is not deleted by the rewrite (dead operations are
    swept afterwards), so returning it or reading it elsewhere strands nobody."""

    class Exported(torch.nn.Module):
        def forward(self, cache, projected, key):
            pairs, keys, values = [], [], []
            for layer in range(LAYERS):
                pair = cache[layer]
                value = projected[:, :, 2 * HEADS * HEAD_DIM:].view(1, 1, HEADS, HEAD_DIM).transpose(1, 2)
                new_pair = torch.cat((pair[:, :, :, 1:, :], torch.stack((key[layer], value), 0)), dim=3)
                pairs.append(new_pair)
                keys.append(new_pair[0])
                values.append(new_pair[1])
            return torch.stack(pairs), torch.stack(keys), torch.stack(values), cache[0], cache[1] + cache[1]

    graph = capture_fx(Exported().eval(), _inputs())
    rewritten = fuse_kv_cache_update(graph)
    rewritten.validate()
    assert len(_appends(rewritten)) == LAYERS
    inputs = _inputs(6)
    for got, want in zip(run_graph(rewritten, list(inputs)), Exported()(*inputs)):
        assert torch.equal(got, want)
