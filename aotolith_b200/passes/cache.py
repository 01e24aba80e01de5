"""KV-cache passes: recognise the rolling-window update and absorb the rotations.

``fuse_kv_cache_update`` matches the frontend's spelling of one layer's decode
cache update,

    cat((pair[:, :, :, 1:, :], cat(unsqueeze(key, 0), unsqueeze(value, 0), dim=0)), dim=3)

with ``pair = squeeze(slice(cache, dim 0, layer:layer+1))`` on a rank-6 cache
whose axis 1 has extent 2, ``value = transpose(1, 2)(reshape(slice(row, dim 2,
start:start + KVH*D)))`` and the two halves read back by ``slice`` + ``squeeze``,
and emits ``kv_cache_append(cache, key, row) -> (new_pair, keys, values)``
with ``{layer, value_start}``.

``fuse_rope_into_kv_cache_update`` then folds the key rotation that feeds it and
the query rotation that reads the same projection row into
``rope_kv_cache_append(cache, row, cos, sin) -> (query, new_pair, keys, values)``
with ``{layer, query_start, key_start, value_start, query_heads}``.

Behavioural counterparts of ``src/aotolith/passes/cache.py:193-495``.
"""

from __future__ import annotations

from ..ir import Graph, Operation
from .rewriter import Rewriter


def _slice_bounds(op: Operation, extent: int) -> tuple[int, int, int]:
    start, end = int(op.attrs["start"]), int(op.attrs["end"])
    if start < 0:
        start += extent
    if end < 0:
        end += extent
    return max(start, 0), min(end, extent), int(op.attrs.get("step", 1))


def _row_slice(rw: Rewriter, value_id: str):
    """``value_id`` as ``layout*(slice(row, dim 2, start:end))`` -> ``(row, start, end)``."""

    seen = 0
    while seen < 4:
        op = rw.producer(value_id)
        if op is None:
            return None
        if op.op in ("reshape", "transpose", "unsqueeze", "squeeze"):
            if op.op == "transpose":
                shape = rw.shape(op.inputs[0])
                rank = len(shape)
                dims = sorted((int(op.attrs["dim0"]) % rank, int(op.attrs["dim1"]) % rank))
                # only a swap of the step axis (extent 1) with the head axis keeps row order
                if shape[dims[0]] != 1 and shape[dims[1]] != 1:
                    return None
            value_id = op.inputs[0]
            seen += 1
            continue
        if op.op == "slice":
            row = op.inputs[0]
            shape = rw.shape(row)
            if len(shape) != 3 or int(op.attrs["dim"]) % 3 != 2:
                return None
            start, end, step = _slice_bounds(op, shape[2])
            if step != 1:
                return None
            return row, start, end
        return None
    return None


def fuse_kv_cache_update(graph: Graph) -> Graph:
    rw = Rewriter(graph)
    for op in list(rw.ops):
        if op.op != "cat" or len(op.inputs) != 2:
            continue
        out = op.outputs[0]
        out_shape = rw.shape(out)
        if len(out_shape) != 5 or int(op.attrs["dim"]) % 5 != 3 or out_shape[0] != 2:
            continue
        window, rows = (rw.producer(v) for v in op.inputs)
        if window is None or rows is None or window.op != "slice" or rows.op != "cat":
            continue
        # window = pair[:, :, :, 1:, :]
        pair_id = window.inputs[0]
        pair_shape = rw.shape(pair_id)
        if int(window.attrs["dim"]) % 5 != 3 or pair_shape != out_shape:
            continue
        if _slice_bounds(window, pair_shape[3]) != (1, pair_shape[3], 1):
            continue
        squeeze = rw.producer(pair_id)
        if squeeze is None or squeeze.op != "squeeze" or int(squeeze.attrs["dim"]) != 0:
            continue
        pick = rw.producer(squeeze.inputs[0])
        if pick is None or pick.op != "slice" or int(pick.attrs["dim"]) != 0:
            continue
        cache_id = pick.inputs[0]
        cache_shape = rw.shape(cache_id)
        if len(cache_shape) != 6 or cache_shape[1] != 2:
            continue
        layer, layer_end, step = _slice_bounds(pick, cache_shape[0])
        if layer_end != layer + 1 or step != 1:
            continue
        # rows = cat(unsqueeze(key, 0), unsqueeze(value, 0), dim 0)
        if len(rows.inputs) != 2 or int(rows.attrs["dim"]) % 5 != 0:
            continue
        lifted = [rw.producer(v) for v in rows.inputs]
        if any(l is None or l.op != "unsqueeze" or int(l.attrs["dim"]) != 0 for l in lifted):
            continue
        key_id, value_id = lifted[0].inputs[0], lifted[1].inputs[0]
        heads, head_dim = cache_shape[3], cache_shape[5]
        if rw.shape(key_id) != (cache_shape[2], heads, 1, head_dim):
            continue
        source = _row_slice(rw, value_id)
        if source is None:
            continue
        row_id, value_start, value_end = source
        if value_end - value_start != heads * head_dim or rw.shape(row_id)[1] != 1:
            continue
        # read-backs: squeeze(slice(cat, dim 0, i:i+1)) for i = 0, 1
        halves: dict[int, Operation] = {}
        for user in rw.users(out):
            if user.op != "slice" or int(user.attrs["dim"]) != 0:
                continue
            lo, hi, st = _slice_bounds(user, 2)
            if hi != lo + 1 or st != 1 or not rw.single_use(user.outputs[0]):
                continue
            follower = rw.users(user.outputs[0])[0]
            if follower.op == "squeeze" and int(follower.attrs["dim"]) == 0:
                halves[lo] = follower
        if set(halves) != {0, 1}:
            continue
        fused = Operation(
            "kv_cache_append",
            (cache_id, key_id, row_id),
            (out, halves[0].outputs[0], halves[1].outputs[0]),
            {"layer": layer, "value_start": value_start},
        )
        rw.erase(halves[0], halves[1])
        rw.replace(op, fused)
    return rw.finish()


def fuse_rope_into_kv_cache_update(graph: Graph) -> Graph:
    rw = Rewriter(graph)
    for op in list(rw.ops):
        if op.op != "kv_cache_append":
            continue
        cache_id, key_id, row_id = op.inputs
        key_rope = rw.producer(key_id)
        if key_rope is None or key_rope.op != "rope" or not rw.single_use(key_id):
            continue
        cache_shape = rw.shape(cache_id)
        heads, head_dim = cache_shape[3], cache_shape[5]
        row_shape = rw.shape(row_id)
        if len(row_shape) != 3 or row_shape[1] != 1:
            continue
        key_source = _row_slice(rw, key_rope.inputs[0])
        if key_source is None or key_source[0] != row_id:
            continue
        key_start = key_source[1]
        if key_source[2] - key_start != heads * head_dim:
            continue
        cosine, sine = key_rope.inputs[1], key_rope.inputs[2]
        if rw.type(cosine).numel != head_dim or rw.type(sine).numel != head_dim:
            continue
        keys_out, values_out = op.outputs[1], op.outputs[2]
        # the attention that reads this layer's window, and the rope feeding its query
        chosen = None
        for attention in rw.users(keys_out):
            if attention.op != "attention" or attention.inputs[1] != keys_out:
                continue
            if attention.inputs[2] != values_out:
                continue
            query_rope = rw.producer(attention.inputs[0])
            if query_rope is None or query_rope.op != "rope":
                continue
            if query_rope.inputs[1:] != (cosine, sine) or not rw.single_use(attention.inputs[0]):
                continue
            query_source = _row_slice(rw, query_rope.inputs[0])
            if query_source is None or query_source[0] != row_id:
                continue
            width = query_source[2] - query_source[1]
            if width % head_dim:
                continue
            chosen = (query_rope, query_source[1], width // head_dim)
            break
        if chosen is None:
            continue
        query_rope, query_start, query_heads = chosen
        if rw.shape(query_rope.outputs[0]) != (cache_shape[2], query_heads, 1, head_dim):
            continue
        fused = Operation(
            "rope_kv_cache_append",
            (cache_id, row_id, cosine, sine),
            (query_rope.outputs[0],) + op.outputs,
            {
                "layer": int(op.attrs["layer"]),
                "query_start": query_start,
                "key_start": key_start,
                "value_start": int(op.attrs["value_start"]),
                "query_heads": query_heads,
            },
        )
        rw.erase(query_rope, key_rope)
        rw.replace(op, fused)
    return rw.finish()
