"""The weight streams of the streamed decode-step kernel, read back on the CPU.

``aotolith_b200/runtime/stream_plan.py`` cuts every packed projection of a decode step into
per-warp byte streams. This file walks those streams the way the kernel does - start record,
piece after piece, headers telling what a piece is and how large the piece ``ring_depth``
ahead will be - decodes every block by the layout the C header documents, multiplies, and
compares with the exact product of the same packed weights. It also checks the partition
itself: every block of every stage is multiplied exactly once, partial-sum slots of a tile are
consecutive and the warp with the tile's last block has the duty of finishing it.
"""

import numpy as np
import pytest
import torch

from aotolith_b200.runtime import stream_plan as sp
from tests.helpers import activations, exact_packed_matmul, packed_weight


def block_weights(block: np.ndarray) -> np.ndarray:
    """``float64 [16, 128]`` weights of one 1088-byte block, by the layout of the C header."""

    words = block[:1024].view("<u4").reshape(2, 32, 4)          # [half][lane][word]
    scales = torch.from_numpy(block[1024:].view("<i2").copy()).view(torch.bfloat16).double().numpy().reshape(16, 2)
    out = np.zeros((16, 128))
    for half in range(2):
        for lane in range(32):
            g, t = lane >> 2, lane & 3
            for j in range(4):
                word = int(words[half, lane, j])
                for n in range(8):
                    nibble = (word >> (4 * n)) & 0xF
                    code = nibble - 16 if nibble >= 8 else nibble
                    col = 16 * (2 * j + ((n & 3) >> 1)) + 2 * t + 8 * (n & 1) + (n >> 2)
                    out[g + 8 * half, col] = code * scales[g + 8 * half, col // 64]
    return out


def run_stage(layout, stream: np.ndarray, stage: int, shape: sp.GemvShape, x: np.ndarray, cursors: dict) -> np.ndarray:
    """What the kernel's GEMV stage computes from the stream: ``[mats, tiles * 16]`` sums."""

    tiles = -(-shape.n_rows // 16)
    result = np.full((shape.mats, tiles * 16), np.nan)
    covered = np.zeros((shape.mats, tiles, shape.K // 128), dtype=np.int64)
    for cta in range(layout.ctas):
        entry = int(layout.table[stage, cta])
        tile0, count, shared = entry & 0xFFFF, (entry >> 16) & 0x7FFF, entry >> 31
        parts: dict[int, np.ndarray] = {}
        for warp in range(sp.WARPS):
            state = cursors[(cta, warp)]
            acc = np.zeros((2, 16))
            while state["next_stage"] == stage:
                assert count > 0, "a CTA without tiles has no pieces"
                at = state["offset"]
                header = stream[at: at + 16].view(sp.PIECE_DTYPE)[0]
                size = 16 + int(header["nblocks"]) * sp.BLOCK_BYTES
                assert state["sizes"].pop(0) == size  # what the ring was told to fetch
                flags = int(header["flags"])
                mat = 1 if flags & sp.MAT1 else 0
                assert int(header["column_bytes"]) % 256 == 0
                for b in range(int(header["nblocks"])):
                    block = stream[at + 16 + b * sp.BLOCK_BYTES: at + 16 + (b + 1) * sp.BLOCK_BYTES]
                    kb = int(header["column_bytes"]) // 256 + b
                    acc[mat] += block_weights(block) @ x[kb * 128:(kb + 1) * 128]
                    covered[mat, tile0 + int(header["tile"]), kb] += 1
                if header["ahead_bytes"]:
                    state["sizes"].append(int(header["ahead_bytes"]))
                state["offset"] += size
                state["next_stage"] = int(header["next_stage"])
                if flags & sp.SEG_END:
                    assert int(header["tile"]) < count
                    slot, rest = divmod(int(header["part_bytes"]), 128)
                    assert rest == 0 and slot not in parts
                    parts[slot] = acc.copy()
                    if flags & sp.WHOLE:
                        assert slot == sp.PART_SLOTS + warp  # the warp's own slot
                        tile = tile0 + int(header["tile"])
                        result[:, tile * 16:(tile + 1) * 16] = acc[: shape.mats]
                        del parts[slot]
                    else:
                        assert shared and slot < sp.PART_SLOTS
                    acc = np.zeros((2, 16))
            assert not acc.any(), "a share ended without SEG_END"
        finished = 0
        for warp in range(sp.WARPS):  # after the CTA barrier: every warp looks up its duty
            duty = int(layout.duties[stage, cta, warp])
            if duty == 0:
                continue
            assert shared and duty & 0x8000
            tile, first, nparts = tile0 + (duty & 0x7FFF), (duty >> 16) & 0xFF, duty >> 24
            total = sum(parts.pop(first + i) for i in range(nparts))
            result[:, tile * 16:(tile + 1) * 16] = total[: shape.mats]
            finished += 1
        assert not parts, "every partial sum belongs to a tile somebody finishes"
        if not shared:
            assert finished == 0
    assert (covered == 1).all(), "every block of the stage is multiplied exactly once"
    return result


def start_cursors(layout, depth):
    cursors = {}
    for cta in range(layout.ctas):
        for warp in range(sp.WARPS):
            start = layout.starts[cta * sp.WARPS + warp]
            sizes = [int(s) * 16 for s in start["size16"][:depth] if s]
            cursors[(cta, warp)] = {"offset": int(start["offset16"]) * 16, "next_stage": int(start["first_stage"]),
                                    "sizes": sizes}
    return cursors


@pytest.mark.parametrize("ctas,depth", [(148, 3), (5, 2), (37, 3)])
def test_streams_reproduce_the_products(ctas, depth):
    """A miniature step: four projections (one paired, one with N not a multiple of 16)."""

    specs = [  # (N, K, mats)
        (1152, 896, 1), (40, 256, 1), (608, 896, 2), (896, 1280, 1), (3000, 128, 1),
    ]
    shapes, weights, inputs = [], {}, {}
    for index, (n_rows, K, mats) in enumerate(specs):
        stage = 2 * index  # odd stages are not GEMV: they have no pieces
        shapes.append(sp.GemvShape(stage, n_rows, K, mats))
        weights[stage] = [packed_weight(100 + 10 * index + m, n_rows, K, 64) for m in range(mats)]
        inputs[stage] = activations(200 + index, K).double().numpy()
    stage_count = 2 * len(specs)
    layout = sp.layout_streams(shapes, stage_count, ctas, depth)
    stream = sp.fill_stream(layout, shapes, weights, layout.table, torch.device("cpu")).numpy()
    assert stream.size == layout.stream_bytes
    cursors = start_cursors(layout, depth)
    for shape in shapes:
        got = run_stage(layout, stream, shape.stage, shape, inputs[shape.stage], cursors)
        for m, (packed, scales) in enumerate(weights[shape.stage]):
            want = exact_packed_matmul(torch.from_numpy(inputs[shape.stage])[None, :], packed, scales, 64)[0].numpy()
            np.testing.assert_allclose(got[m, : shape.n_rows], want, rtol=1e-9, atol=1e-12)
            assert not got[m, shape.n_rows:].any()  # rows past N are zero weights
    for state in cursors.values():  # every stream was read to its end
        assert state["next_stage"] == sp.NO_STAGE and not state["sizes"]


def test_stage_partition_keeps_the_critical_path_short():
    """Stages with fewer tiles than CTAs use as few CTAs as the busiest warp allows."""

    assert sp.tiles_per_cta(72, 7, 148) == 2      # q/k/v of the 0.5B shape: 14 of 16 warps, one block each
    assert sp.tiles_per_cta(56, 38, 148) == 1     # down: 38 blocks over 16 warps is already three a warp
    table, _, pieces = sp.plan_stage(0, 304, 7, 2, 148, 0)  # gate/up: 304 paired tiles over 148 CTAs
    counts = (table >> 16) & 0x7FFF
    assert counts.sum() == 304 and counts.max() == 3 and counts.min() == 2
    per_warp = {}
    for cta, warp, *_rest in pieces:
        per_warp[(cta, warp)] = per_warp.get((cta, warp), 0) + _rest[3]
    assert max(per_warp.values()) == 3  # ceil(42 / 16)
    table, _, _ = sp.plan_stage(0, 9496, 7, 1, 148, 0)  # LM head
    counts = (table >> 16) & 0x7FFF
    assert counts.sum() == 9496 and counts.max() - counts.min() <= 1


def test_small_stages_take_turns_over_the_grid():
    shapes = [sp.GemvShape(0, 1152, 896, 1), sp.GemvShape(1, 896, 896, 1), sp.GemvShape(2, 896, 4864, 1)]
    layout = sp.layout_streams(shapes, 3, 148, 3)
    busy = [(layout.table[s] >> 16) & 0x7FFF for s in range(3)]
    assert not np.any((busy[0] > 0) & (busy[1] > 0))  # q/k/v and o do not land on the same CTAs
    assert [int(np.count_nonzero(b)) for b in busy] == [36, 28, 56]
