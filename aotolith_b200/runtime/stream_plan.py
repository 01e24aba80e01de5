"""Stage program -> per-warp weight streams of the streamed decode-step kernel.

``aoto_sm100_stream_step`` (``include/aoto_sm100.h``) multiplies packed weights that
reach each warp as a byte stream laid out once per model. This module does the
laying out, on the host:

* ``plan_stage``   which CTA owns which 16-row tiles of a GEMV stage and how a CTA's
                   blocks - (tile, matrix, 128-column block), tile-major - are cut into
                   one contiguous share per warp, shares into pieces of at most three
                   blocks;
* ``retile``       the packed ``int32 [N, K/8]`` words and ``bf16 [N, K/64]`` scales of
                   the reference format (``src/aotolith/quantize.py:95-152``) as
                   1088-byte blocks in tensor-core fragment order;
* ``build``        piece headers, per-warp start records, the per-(stage, CTA) table
                   and the stream itself for a whole stage program.

Everything here is index arithmetic and tensor permutation (torch is the array
library); nothing is multiplied. ``tests/test_stream_plan.py`` reads a stream back
the way the kernel does and checks it against the oracle on the CPU.
"""

from __future__ import annotations

import ctypes
from dataclasses import dataclass

import numpy as np
import torch

from .. import _native as N

WARPS = 16
BLOCK_BYTES = 1088
PIECE_BLOCKS = 3
HEADER_BYTES = 16
SLOT_BYTES = HEADER_BYTES + PIECE_BLOCKS * BLOCK_BYTES
PART_SLOTS = 32
NO_STAGE = 0xFFFF
SEG_END, WHOLE, MAT1 = 1, 2, 4

PIECE_DTYPE = np.dtype([
    ("next_stage", "<u2"), ("nblocks", "u1"), ("flags", "u1"), ("column_bytes", "<u4"),
    ("part_bytes", "<u2"), ("tile", "<u2"), ("ahead_bytes", "<u4"),
])
START_DTYPE = np.dtype([("offset16", "<u4"), ("size16", "<u2", (3,)), ("first_stage", "<u2"), ("reserved", "<u4")])
assert PIECE_DTYPE.itemsize == 16 and START_DTYPE.itemsize == 16


# ---------------------------------------------------------------------------
# tiles -> CTAs -> warps -> pieces
# ---------------------------------------------------------------------------

def tiles_per_cta(tiles: int, per_tile: int, ctas: int) -> int:
    """Tiles a participating CTA takes when a stage has fewer tiles than the grid has CTAs.

    A stage is as slow as its busiest warp, which multiplies ``ceil(t * per_tile / 16)``
    blocks when a CTA owns ``t`` tiles. Fewer CTAs poll fewer copies of the input row, so
    take the largest ``t`` that does not lengthen that critical path.
    """

    floor = -(-per_tile // WARPS)
    t = 1
    while (t + 1) * per_tile <= floor * WARPS and t + 1 <= tiles:
        t += 1
    return t


def assign_tiles(tiles: int, per_tile: int, ctas: int, first_cta: int, reserved: int = 0) -> list[tuple[int, int]]:
    """``[(tile0, count)]`` per CTA: contiguous, balanced ranges; idle CTAs get ``(0, 0)``.

    The first ``reserved`` CTAs get nothing: they are the attention stage's (one per query
    head). A CTA that runs both the attention code and the projection code cycles through more
    instructions per layer than the SM's instruction cache holds (32 KB on this part, measured)
    and runs every stage cold; kept apart, each kind of CTA stays inside the cache.
    """

    ranges = [(0, 0)] * ctas
    workers = ctas - reserved
    if tiles >= workers:
        for c in range(workers):
            lo, hi = c * tiles // workers, (c + 1) * tiles // workers
            ranges[reserved + c] = (lo, hi - lo)
        return ranges
    t = tiles_per_cta(tiles, per_tile, workers)
    used = -(-tiles // t)
    for i in range(used):
        lo, hi = i * tiles // used, (i + 1) * tiles // used
        ranges[reserved + (first_cta + i) % workers] = (lo, hi - lo)
    return ranges


def plan_stage(stage: int, tiles: int, nb: int, mats: int, ctas: int, first_cta: int, reserved: int = 0):
    """Pieces of one GEMV stage.

    Returns ``(table_row, duties, pieces)``: the ``uint32[ctas]`` entries of the stage, the
    ``uint32[ctas, 16]`` finishing duties, and a list of
    ``(cta, warp, tile_local, mat, kb0, nblocks, flags, part_slot)`` in the order every warp
    multiplies its pieces. A tile cut across warps gets consecutive partial slots in block
    order and is finished by the warp that holds its last block; a tile held by one warp uses
    that warp's own slot (``PART_SLOTS + warp``) and is finished as soon as it is multiplied.
    """

    per_tile = mats * nb
    ranges = assign_tiles(tiles, per_tile, ctas, first_cta, reserved)
    table = np.zeros(ctas, dtype=np.uint32)
    duties = np.zeros((ctas, WARPS), dtype=np.uint32)
    pieces: list[tuple] = []
    for cta, (tile0, count) in enumerate(ranges):
        if count == 0:
            continue
        total = count * per_tile
        # segments: (warp, tile_local, first block of the tile, blocks)
        segments = []
        for warp in range(WARPS):
            lo, hi = warp * total // WARPS, (warp + 1) * total // WARPS
            while lo < hi:
                tile_local, inside = divmod(lo, per_tile)
                take = min(hi - lo, per_tile - inside)
                segments.append((warp, tile_local, inside, take))
                lo += take
        parts_of_tile: dict[int, int] = {}
        for _, tile_local, _, take in segments:
            if take != per_tile:
                parts_of_tile[tile_local] = parts_of_tile.get(tile_local, 0) + 1
        next_slot = 0
        first_slot: dict[int, int] = {}
        seen: dict[int, int] = {}
        for warp, tile_local, inside, take in segments:
            whole = take == per_tile
            flags_end = SEG_END | (WHOLE if whole else 0)
            part_slot = PART_SLOTS + warp
            if not whole:
                if tile_local not in first_slot:
                    first_slot[tile_local] = next_slot
                    next_slot += parts_of_tile[tile_local]
                    seen[tile_local] = 0
                part_slot = first_slot[tile_local] + seen[tile_local]
                seen[tile_local] += 1
                if inside + take == per_tile:
                    if duties[cta, warp]:
                        raise ValueError(f"stage {stage}: warp {warp} of CTA {cta} would finish two shared tiles")
                    duties[cta, warp] = (tile_local | 0x8000 | (first_slot[tile_local] << 16)
                                         | (parts_of_tile[tile_local] << 24))
            # pieces never cross a matrix boundary and hold at most PIECE_BLOCKS blocks
            at, end = inside, inside + take
            while at < end:
                mat, kb0 = divmod(at, nb)
                n = min(PIECE_BLOCKS, end - at, nb - kb0)
                last = at + n == end
                pieces.append((cta, warp, tile_local, mat, kb0, n, flags_end if last else 0, part_slot))
                at += n
        if next_slot > PART_SLOTS:
            raise ValueError(f"stage {stage}: {next_slot} shared-tile partial sums in one CTA exceed {PART_SLOTS}")
        if tile0 > 0xFFFF or count > 0x7FFF:
            raise ValueError(f"stage {stage}: tile range ({tile0}, {count}) does not fit the table entry")
        table[cta] = tile0 | (count << 16) | ((1 << 31) if next_slot else 0)
    return table, duties, pieces


# ---------------------------------------------------------------------------
# packed words -> blocks in fragment order
# ---------------------------------------------------------------------------

def _fragment_map() -> tuple[torch.Tensor, torch.Tensor]:
    """(row, column) within a 16 x 128 block of every nibble of its 256 code words.

    Word ``w = half*128 + lane*4 + j`` (half 0: rows 0-7, half 1: rows 8-15; lane ``4g + t``),
    nibble ``n``: row ``g + 8*half``, column ``16*(2j + ((n & 3) >> 1)) + 2t + 8*(n & 1) + (n >> 2)``.
    """

    half, lane, j, n = np.meshgrid(np.arange(2), np.arange(32), np.arange(4), np.arange(8), indexing="ij")
    g, t = lane >> 2, lane & 3
    row = g + 8 * half
    col = 16 * (2 * j + ((n & 3) >> 1)) + 2 * t + 8 * (n & 1) + (n >> 2)
    return torch.from_numpy(row.reshape(-1)), torch.from_numpy(col.reshape(-1))


def retile(packed: torch.Tensor, scales: torch.Tensor) -> torch.Tensor:
    """``uint8 [tiles, K/128, 1088]``: the blocks of one packed matrix (group size 64)."""

    n_rows, words = packed.shape
    K = words * 8
    if K % 128 or scales.shape != (n_rows, K // 64):
        raise ValueError("retile needs K % 128 == 0 and one scale per 64 columns")
    tiles, nb = -(-n_rows // 16), K // 128
    device = packed.device
    shifts = torch.arange(8, device=device, dtype=torch.int32) * 4
    nibbles = ((packed.unsqueeze(-1) >> shifts) & 0xF).to(torch.uint8).reshape(n_rows, K)
    if tiles * 16 != n_rows:
        nibbles = torch.cat((nibbles, nibbles.new_zeros(tiles * 16 - n_rows, K)))
        scales = torch.cat((scales, scales.new_zeros(tiles * 16 - n_rows, K // 64)))
    grid = nibbles.reshape(tiles, 16, nb, 128).permute(0, 2, 1, 3)           # [tiles, nb, 16, 128]
    row, col = (index.to(device) for index in _fragment_map())
    ordered = grid[:, :, row, col].reshape(tiles, nb, 256, 8).to(torch.int64)  # nibbles of every word
    weights = (torch.ones(8, dtype=torch.int64, device=device) << (4 * torch.arange(8, device=device)))
    code_words = (ordered * weights).sum(dim=-1)
    code_words = torch.where(code_words >= 2 ** 31, code_words - 2 ** 32, code_words).to(torch.int32)
    code_bytes = code_words.contiguous().view(torch.uint8).reshape(tiles, nb, 1024)
    scale_bytes = (scales.reshape(tiles, 16, nb, 2).permute(0, 2, 1, 3).contiguous()
                   .view(torch.uint8).reshape(tiles, nb, 64))
    return torch.cat((code_bytes, scale_bytes), dim=-1).contiguous()


# ---------------------------------------------------------------------------
# the whole program
# ---------------------------------------------------------------------------

@dataclass(slots=True)
class GemvShape:
    """What the planner needs to know of a GEMV stage."""

    stage: int
    n_rows: int
    K: int
    mats: int


@dataclass(slots=True)
class StreamLayout:
    """Host description of a stream: tables, piece records and where every block goes."""

    ctas: int
    ring_depth: int
    stage_count: int
    table: np.ndarray            # uint32 [stage_count, ctas]
    duties: np.ndarray           # uint32 [stage_count, ctas, WARPS]
    starts: np.ndarray           # START_DTYPE [ctas * WARPS]
    headers: np.ndarray          # PIECE_DTYPE [pieces], in stream order
    piece_stage: np.ndarray      # what the headers no longer say: stage, matrix and first block
    piece_mat: np.ndarray
    piece_kb0: np.ndarray
    piece_offset16: np.ndarray   # int64 [pieces]
    piece_cta: np.ndarray
    piece_warp: np.ndarray
    stream_bytes: int


def layout_streams(shapes: list[GemvShape], stage_count: int, ctas: int, ring_depth: int,
                   attention_ctas: int = 0, last_attention: int = -1) -> StreamLayout:
    """Plan every GEMV stage and lay the pieces out as one stream per (CTA, warp).

    ``attention_ctas`` CTAs (the first ones) take no projection work in the stages up to
    ``last_attention`` (see :func:`assign_tiles`); after the last attention stage every CTA works.
    """

    table = np.zeros((stage_count, ctas), dtype=np.uint32)
    duties = np.zeros((stage_count, ctas, WARPS), dtype=np.uint32)
    records: list[tuple] = []
    cursor = 0
    for shape in shapes:
        tiles, nb = -(-shape.n_rows // 16), shape.K // 128
        reserved = attention_ctas if shape.stage < last_attention else 0
        row, duty, pieces = plan_stage(shape.stage, tiles, nb, shape.mats, ctas, cursor, reserved)
        table[shape.stage], duties[shape.stage] = row, duty
        used = int(np.count_nonzero(row))
        if used < ctas - reserved:
            cursor = (cursor + used) % (ctas - attention_ctas)  # small stages take turns over the grid
        records.extend((shape.stage, *piece) for piece in pieces)
    if not records:
        raise ValueError("a stage program without packed projections has no stream")
    fields = np.array(records, dtype=np.int64)
    stage, cta, warp, tile, mat, kb0, nblocks, flags, part_slot = fields.T
    # stream order: by (cta, warp), stages ascending, planning order within a stage (stable sort)
    order = np.lexsort((np.arange(len(stage)), stage, warp, cta))
    stage, cta, warp, tile, mat, kb0, nblocks, flags, part_slot = (
        column[order] for column in (stage, cta, warp, tile, mat, kb0, nblocks, flags, part_slot))
    size16 = 1 + nblocks * (BLOCK_BYTES // 16)
    offset16 = np.concatenate(([0], np.cumsum(size16)[:-1]))
    owner = cta * WARPS + warp
    count = len(stage)
    index = np.arange(count)
    first_of_owner = np.concatenate(([True], owner[1:] != owner[:-1]))
    headers = np.zeros(count, dtype=PIECE_DTYPE)
    headers["nblocks"], headers["flags"] = nblocks, flags | np.where(mat == 1, MAT1, 0)
    headers["column_bytes"], headers["tile"] = kb0 * 256, tile
    headers["part_bytes"] = part_slot * 128
    same_next = np.concatenate((owner[1:] == owner[:-1], [False]))
    headers["next_stage"] = np.where(same_next, np.concatenate((stage[1:], [0])), NO_STAGE)
    ahead = index + ring_depth
    valid = ahead < count
    ahead_owner = np.where(valid, owner[np.minimum(ahead, count - 1)], -1)
    headers["ahead_bytes"] = np.where(ahead_owner == owner, size16[np.minimum(ahead, count - 1)] * 16, 0)

    starts = np.zeros(ctas * WARPS, dtype=START_DTYPE)
    starts["first_stage"] = NO_STAGE
    firsts = index[first_of_owner]
    for at in firsts:
        who = owner[at]
        starts["offset16"][who] = offset16[at]
        starts["first_stage"][who] = stage[at]
        for i in range(3):
            if at + i < count and owner[at + i] == who:
                starts["size16"][who, i] = size16[at + i]
    if offset16[-1] + size16[-1] >= 2 ** 32:
        raise ValueError("the stream exceeds 64 GiB")
    return StreamLayout(
        ctas=ctas, ring_depth=ring_depth, stage_count=stage_count, table=table, duties=duties, starts=starts,
        headers=headers, piece_stage=stage, piece_mat=mat, piece_kb0=kb0, piece_offset16=offset16, piece_cta=cta,
        piece_warp=warp, stream_bytes=int((offset16[-1] + size16[-1]) * 16),
    )


def fill_stream(layout: StreamLayout, shapes: list[GemvShape], weights: dict[int, list[tuple[torch.Tensor, torch.Tensor]]],
                table: np.ndarray, device: torch.device) -> torch.Tensor:
    """The stream bytes on ``device``: headers, then every stage's blocks copied to their pieces."""

    stream = torch.zeros(layout.stream_bytes, dtype=torch.uint8, device=device)
    rows = stream.view(torch.int32).view(-1, 4)  # 16-byte rows
    header_rows = torch.from_numpy(layout.headers.view(np.int32).reshape(-1, 4).copy()).to(device)
    rows.index_copy_(0, torch.from_numpy(layout.piece_offset16.astype(np.int64)).to(device), header_rows)
    per_block = BLOCK_BYTES // 16
    headers = layout.headers
    for shape in shapes:
        selected = np.nonzero(layout.piece_stage == shape.stage)[0]
        if len(selected) == 0:
            continue
        tiles, nb = -(-shape.n_rows // 16), shape.K // 128
        blocks = torch.stack([retile(packed.to(device), scales.to(device)) for packed, scales in weights[shape.stage]])
        block_rows = blocks.view(torch.int32).view(-1, 4)  # [mats * tiles * nb * 68, 4]
        tile0 = (table[shape.stage][layout.piece_cta[selected]] & 0xFFFF).astype(np.int64)
        counts = headers["nblocks"][selected].astype(np.int64)
        repeat = np.repeat(np.arange(len(selected)), counts)
        within = np.arange(counts.sum()) - np.repeat(np.cumsum(counts) - counts, counts)
        source = ((layout.piece_mat[selected][repeat] * tiles + tile0[repeat]
                   + headers["tile"][selected][repeat].astype(np.int64)) * nb
                  + layout.piece_kb0[selected][repeat] + within)
        target = layout.piece_offset16[selected][repeat] + 1 + within * per_block
        lanes = torch.arange(per_block, device=device)
        source_rows = (torch.from_numpy(source).to(device)[:, None] * per_block + lanes).reshape(-1)
        target_rows = (torch.from_numpy(target.astype(np.int64)).to(device)[:, None] + lanes).reshape(-1)
        rows.index_copy_(0, target_rows, block_rows.index_select(0, source_rows))
        del blocks, block_rows, source_rows, target_rows
    return stream


# ---------------------------------------------------------------------------
# binding a stage program
# ---------------------------------------------------------------------------

def gemv_shapes(program) -> list[GemvShape]:
    shapes = []
    for index, spec in enumerate(program.stages):
        if spec.kind == N.STAGE_GEMV:
            shapes.append(GemvShape(index, spec.ints["N"], spec.ints["K"],
                                    2 if spec.ints["epilogue"] == N.EPILOGUE_SILU_MUL_PAIRED else 1))
    return shapes


def geometry(program) -> dict | None:
    """Attention geometry shared by every layer, or None if the layers disagree."""

    found = None
    for spec in program.stages:
        if spec.kind != N.STAGE_ATTENTION:
            continue
        here = {k: spec.ints[k] for k in ("query_heads", "kv_heads", "capacity", "head_dim",
                                          "query_start", "key_start", "value_start", "table_rows")}
        here["scale"] = spec.floats["scale"]
        here["cos_table"], here["sin_table"] = spec.refs["cos_table"], spec.refs["sin_table"]
        here["position"], here["mask"] = spec.refs["position"], spec.refs["mask"]
        if found is not None and found != here:
            return None
        found = here
    return found


def base_args(program, ctas: int, ring_depth: int) -> N.StreamStepArgs:
    """Geometry fields of the launch arguments (pointers unset): what the support query reads."""

    args = N.StreamStepArgs()
    shapes = gemv_shapes(program)
    args.stage_count = len(program.stages) + 1  # the greedy pick closes every program
    args.ctas, args.ring_depth = ctas, ring_depth
    args.max_k = max((shape.K for shape in shapes), default=0)
    geo = geometry(program)
    attention_stages = [i for i, spec in enumerate(program.stages) if spec.kind == N.STAGE_ATTENTION]
    args.first_attention = attention_stages[0] if attention_stages else -1
    args.attention_stages = len(attention_stages)
    if geo is not None:
        for key in ("query_heads", "kv_heads", "capacity", "head_dim", "query_start", "key_start", "value_start",
                    "table_rows"):
            setattr(args, key, geo[key])
        args.scale = geo["scale"]
    return args


def choose_ring_depth(program, ctas: int, smem_limit: int) -> int:
    """The deepest ring whose shared memory fits, or 0 if the kernel has no form for the program."""

    if any(spec.kind == N.STAGE_GEMV and (spec.ints["K"] % 128 or spec.ints["group_size"] != 64 or spec.ints["N"] % 2)
           for spec in program.stages):
        return 0
    if geometry(program) is None and any(spec.kind == N.STAGE_ATTENTION for spec in program.stages):
        return 0
    lib = N.load()
    for depth in (3, 2):
        need = int(lib.aoto_sm100_stream_step_smem_bytes(ctypes.byref(base_args(program, ctas, depth))))
        if 0 < need <= smem_limit:
            return depth
    return 0


def stage_array(program, resolve):
    """ctypes array of ``aoto_stream_stage`` (plus the closing pick) for one cache direction."""

    count = len(program.stages) + 1
    array = (N.StreamStage * count)()
    attention = [i for i, spec in enumerate(program.stages) if spec.kind == N.STAGE_ATTENTION]
    following = {a: b for a, b in zip(attention, attention[1:])}
    for slot, spec in enumerate(program.stages):
        stage = array[slot]
        stage.kind = spec.kind
        stage.flags = spec.flags
        if spec.kind == N.STAGE_GEMV:
            stage.x = resolve(spec.refs["x"])
            stage.out = resolve(spec.refs["out"])
            stage.addend = resolve(spec.refs["addend"]) if "addend" in spec.refs else None
            stage.norm_weight = resolve(spec.refs["norm_weight"]) if "norm_weight" in spec.refs else None
            stage.N, stage.K = spec.ints["N"], spec.ints["K"]
            stage.alpha, stage.beta = spec.floats["alpha"], spec.floats["beta"]
            stage.rms_norm_eps = spec.floats.get("rms_norm_eps", 0.0)
            stage.epilogue, stage.addend_mode = spec.ints["epilogue"], spec.ints["addend_mode"]
        else:
            stage.x = resolve(spec.refs["row"])
            stage.out = resolve(spec.refs["attn_out"])
            stage.addend = resolve(spec.refs["cache_in"])
            stage.norm_weight = resolve(spec.refs["cache_out"])
            stage.next_attention = following.get(slot, -1)
            stage.ordinal = attention.index(slot)
    last = array[len(program.stages) - 1]
    last.flags |= N.STAGE_FLAG_ARGMAX
    array[count - 1].kind = N.STAGE_PICK
    return array


# ---------------------------------------------------------------------------
# device side of a bound program
# ---------------------------------------------------------------------------

_STREAMS: dict[tuple, tuple] = {}
_STREAM_CACHE_ENTRIES = 4


def device_stream(program, tensors: dict, device: torch.device, ctas: int, ring_depth: int):
    """``(layout, stream, table, starts, duties)`` on ``device`` for the program's packed weights.

    Laying out a stream costs a pass over every packed weight, and the result depends only on
    the weights and the grid, so programs over the same weights (the buckets of one model, the
    sessions of one runtime) share it. The cache holds the weight tensors it was built from,
    which keeps their addresses from being reused while an entry lives.
    """

    shapes = gemv_shapes(program)
    weights: dict[int, list[tuple[torch.Tensor, torch.Tensor]]] = {}
    for shape in shapes:
        refs = program.stages[shape.stage].refs
        pairs = [(tensors[refs["packed"].key], tensors[refs["scales"].key])]
        if shape.mats == 2:
            pairs.append((tensors[refs["packed2"].key], tensors[refs["scales2"].key]))
        weights[shape.stage] = pairs
    key = (str(device), ctas, ring_depth, len(program.stages), tuple(i for i, spec in enumerate(program.stages)
                                                              if spec.kind == N.STAGE_ATTENTION),
           tuple((shape.stage, shape.n_rows, shape.K, *(t.data_ptr() for pair in weights[shape.stage] for t in pair))
                 for shape in shapes))
    hit = _STREAMS.get(key)
    if hit is not None:
        _STREAMS[key] = _STREAMS.pop(key)  # most recently used last
        return hit[:5]
    attention = [i for i, spec in enumerate(program.stages) if spec.kind == N.STAGE_ATTENTION]
    geo = geometry(program)
    heads = geo["query_heads"] if geo is not None else 0
    # Head CTAs that take no projection work until the last attention stage shorten every layer's
    # chain when the heads are few; with many heads the idle multipliers cost more than that saves.
    dedicated = heads if attention and ctas >= 8 * heads else 0
    layout = layout_streams(shapes, len(program.stages) + 1, ctas, ring_depth, dedicated,
                            attention[-1] if attention else -1)
    stream = fill_stream(layout, shapes, weights, layout.table, device)
    table = torch.from_numpy(layout.table.view(np.int32).copy()).to(device)
    starts = torch.from_numpy(layout.starts.view(np.uint8).copy()).to(device)
    duties = torch.from_numpy(layout.duties.view(np.int32).copy()).to(device)
    _STREAMS[key] = (layout, stream, table, starts, duties, weights)
    while len(_STREAMS) > _STREAM_CACHE_ENTRIES:
        _STREAMS.pop(next(iter(_STREAMS)))
    return layout, stream, table, starts, duties


def launch(args: "N.StreamStepArgs", epoch: int, trace: torch.Tensor | None = None) -> None:
    """One decode step; ``epoch`` as for :func:`aotolith_b200.runtime.step_program.launch`."""

    args.epoch = epoch & 0xFFFFFFFF or 1
    args.trace = trace.data_ptr() if trace is not None else None
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    N.check(N.load().aoto_sm100_stream_step(ctypes.byref(args), stream), "aoto_sm100_stream_step")
