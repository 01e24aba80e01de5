"""Versioned ``.aoto`` artifacts for compiled plans of the ``cuda-sm100`` target.

The container follows the reference's artifact (``src/aotolith/artifact.py:82-421``):
one zip archive holding a canonical-JSON ``manifest.json`` (format name and
version, ABI version, compiler version, target, entry point, compile options,
device profile, digests), the captured and the lowered graph, the kernel table,
the selection records, the storage plan, and one raw payload per distinct state
tensor (tensors that alias in memory share a payload and alias again after
loading). What differs from the reference is what a kernel entry holds: there
is no shader source to store - an entry names the C-ABI entry point and variant
(``aoto_sm100_qmatmul[qgemv_mma]``) the selection bound, and loading re-runs the
backend on the stored lowered graph and refuses the artifact if the rebuilt
selections differ from the stored ones.

Loading needs no GPU for validation; binding the state to a device does. On a
host without CUDA the state stays on the CPU and the plan can be inspected but
not called, as with ``compile_module``.
"""

from __future__ import annotations

import hashlib
import json
import os
import tempfile
import zipfile
from pathlib import Path
from typing import Any

import numpy as np
import torch

from ._version import __version__
from .errors import ArtifactCompatibilityError
from .ir import DType, Graph, Operation, TensorType, Value
from .planning import BufferSlot, StoragePlan, ValueLifetime
from .runtime.plan import KernelArtifact
from .selection import KernelSelection

ARTIFACT_FORMAT = "aotolith"
FORMAT_VERSION = 5
SUPPORTED_FORMAT_VERSIONS = (5,)
ABI_VERSION = "1.3"
SUPPORTED_ABI_VERSIONS = ("1.3",)

_TORCH_OF = {
    "bfloat16": torch.bfloat16, "float16": torch.float16, "float32": torch.float32,
    "int32": torch.int32, "int64": torch.int64, "bool": torch.bool, "uint8": torch.uint8,
}
_NAME_OF = {dtype: name for name, dtype in _TORCH_OF.items()}


# ---------------------------------------------------------------------------
# canonical JSON of the pieces
# ---------------------------------------------------------------------------

def _canonical(payload: Any) -> bytes:
    return json.dumps(payload, sort_keys=True, separators=(",", ":"), allow_nan=False).encode()


def _digest(payload: bytes) -> str:
    return "sha256:" + hashlib.sha256(payload).hexdigest()


def _encode_attr(value: Any) -> Any:
    """Attributes are scalars, strings, None, tuples/lists of those, dtypes, or nested graphs."""

    if isinstance(value, DType):
        return {"$dtype": value.value}
    if isinstance(value, (bool, int, str)) or value is None:
        return value
    if isinstance(value, float):
        if value != value or value in (float("inf"), float("-inf")):
            return {"$float": repr(value)}
        return {"$float": value.hex()}
    if isinstance(value, tuple):
        return {"$tuple": [_encode_attr(v) for v in value]}
    if isinstance(value, list):
        return [_encode_attr(v) for v in value]
    if isinstance(value, Graph):
        return {"$graph": encode_graph(value)}
    if isinstance(value, Operation):
        return {"$op": _encode_op(value)}
    if isinstance(value, dict):
        return {"$dict": {str(k): _encode_attr(v) for k, v in value.items()}}
    if isinstance(value, torch.dtype):
        return {"$torch_dtype": _NAME_OF[value]}
    raise ArtifactCompatibilityError(f"attribute of type {type(value).__name__} cannot be stored in an artifact")


def _decode_attr(value: Any) -> Any:
    if isinstance(value, list):
        return [_decode_attr(v) for v in value]
    if not isinstance(value, dict):
        return value
    if "$dtype" in value:
        return DType(value["$dtype"])
    if "$float" in value:
        text = value["$float"]
        return float.fromhex(text) if text.startswith(("0x", "-0x")) else float(text)
    if "$tuple" in value:
        return tuple(_decode_attr(v) for v in value["$tuple"])
    if "$graph" in value:
        return decode_graph(value["$graph"])
    if "$op" in value:
        return _decode_op(value["$op"])
    if "$dict" in value:
        return {k: _decode_attr(v) for k, v in value["$dict"].items()}
    if "$torch_dtype" in value:
        return _TORCH_OF[value["$torch_dtype"]]
    raise ArtifactCompatibilityError("artifact attribute encoding is not recognised")


def _encode_op(op: Operation) -> dict:
    return {"op": op.op, "inputs": list(op.inputs), "outputs": list(op.outputs),
            "attrs": {name: _encode_attr(v) for name, v in op.attrs.items()}}


def _decode_op(entry: dict) -> Operation:
    return Operation(str(entry["op"]), tuple(entry["inputs"]), tuple(entry["outputs"]),
                     {name: _decode_attr(v) for name, v in entry["attrs"].items()})


def encode_graph(graph: Graph) -> dict:
    return {
        "inputs": list(graph.inputs),
        "outputs": list(graph.outputs),
        "values": [{"id": v.id, "shape": list(v.type.shape), "dtype": v.type.dtype.value} for v in graph.values.values()],
        "ops": [_encode_op(op) for op in graph.ops],
    }


def decode_graph(entry: dict) -> Graph:
    values = {
        str(v["id"]): Value(str(v["id"]), TensorType(tuple(int(d) for d in v["shape"]), DType(v["dtype"])))
        for v in entry["values"]
    }
    graph = Graph(tuple(entry["inputs"]), values, tuple(_decode_op(op) for op in entry["ops"]), tuple(entry["outputs"]))
    graph.validate()
    return graph


def _encode_selection(selection: KernelSelection) -> dict:
    return {
        "op_index": selection.op_index, "op": selection.op, "output_id": selection.output_id,
        "implementation": selection.implementation, "kind": selection.kind, "reason": selection.reason,
        "artifact_name": selection.artifact_name, "autotuned": selection.autotuned,
        "device_name": selection.device_name, "device_architecture": selection.device_architecture,
    }


def _decode_selection(entry: dict) -> KernelSelection:
    return KernelSelection(
        op_index=int(entry["op_index"]), op=str(entry["op"]), output_id=str(entry["output_id"]),
        implementation=str(entry["implementation"]), kind=str(entry["kind"]), reason=str(entry["reason"]),
        artifact_name=entry.get("artifact_name"), autotuned=bool(entry.get("autotuned", False)),
        device_name=entry.get("device_name"), device_architecture=entry.get("device_architecture"),
    )


def _encode_kernel(kernel: KernelArtifact) -> dict:
    entry = {}
    for name in getattr(kernel, "__slots__", None) or vars(kernel):
        value = getattr(kernel, name)
        if isinstance(value, dict):
            value = {str(k): _encode_attr(v) for k, v in value.items()}
        else:
            value = _encode_attr(value)
        entry[name] = value
    return entry


def _encode_storage(plan: StoragePlan) -> dict:
    return {
        "lifetimes": [
            {"value_id": l.value_id, "shape": list(l.tensor_type.shape), "dtype": l.tensor_type.dtype.value,
             "start": l.start, "end": l.end, "size_bytes": l.size_bytes, "is_input": l.is_input, "is_output": l.is_output}
            for l in plan.lifetimes
        ],
        "slots": [
            {"slot_id": s.slot_id, "offset_bytes": s.offset_bytes, "size_bytes": s.size_bytes,
             "alignment_bytes": s.alignment_bytes, "value_ids": list(s.value_ids)}
            for s in plan.slots
        ],
        "release_after_op": [list(values) for values in plan.release_after_op],
        "peak_live_bytes": plan.peak_live_bytes,
        "arena_size_bytes": plan.arena_size_bytes,
    }


def _decode_storage(entry: dict) -> StoragePlan:
    return StoragePlan(
        lifetimes=tuple(
            ValueLifetime(str(l["value_id"]), TensorType(tuple(l["shape"]), DType(l["dtype"])), int(l["start"]),
                          int(l["end"]), int(l["size_bytes"]), bool(l["is_input"]), bool(l["is_output"]))
            for l in entry["lifetimes"]
        ),
        slots=tuple(
            BufferSlot(int(s["slot_id"]), int(s["offset_bytes"]), int(s["size_bytes"]), int(s["alignment_bytes"]),
                       tuple(s["value_ids"]))
            for s in entry["slots"]
        ),
        release_after_op=tuple(tuple(values) for values in entry["release_after_op"]),
        peak_live_bytes=int(entry["peak_live_bytes"]),
        arena_size_bytes=int(entry["arena_size_bytes"]),
    )


# ---------------------------------------------------------------------------
# state payloads
# ---------------------------------------------------------------------------

def _tensor_bytes(tensor: torch.Tensor) -> bytes:
    host = tensor.detach().to("cpu").contiguous().reshape(-1)  # a 0-dim tensor has no byte view
    return host.view(torch.uint8).numpy().tobytes() if host.numel() else b""


def _tensor_from_bytes(payload: bytes, shape: tuple[int, ...], dtype: torch.dtype) -> torch.Tensor:
    flat = torch.from_numpy(np.frombuffer(payload, dtype=np.uint8).copy())
    expected = int(np.prod(shape, dtype=np.int64)) * torch.empty((), dtype=dtype).element_size()
    if flat.numel() != expected:
        raise ArtifactCompatibilityError("a state payload does not have the size its entry declares")
    return flat.view(dtype).reshape(shape)


# ---------------------------------------------------------------------------
# save
# ---------------------------------------------------------------------------

def _device_profile() -> dict:
    if torch.cuda.is_available():
        index = torch.cuda.current_device()
        major, minor = torch.cuda.get_device_capability(index)
        return {"device_name": torch.cuda.get_device_name(index), "architecture": f"sm_{major}{minor}"}
    return {"device_name": None, "architecture": None}


def save_compiled(compiled: Any, path: str | os.PathLike[str]) -> Path:
    """Write a ``CompilationResult`` or ``CompiledModulePlan`` to one ``.aoto`` archive.

    The archive is written to a temporary file beside the destination and moved
    into place, so a crash never leaves a half-written artifact under the final
    name. Every payload but the device profile is canonical: saving the same
    plan twice gives the same bytes.
    """

    from .compiler import CompiledModulePlan

    is_module = isinstance(compiled, CompiledModulePlan)
    result = compiled.compilation if is_module else compiled
    plan = result.plan
    state_names = tuple(compiled.state_names) if is_module else ()
    state_values = tuple(compiled._state_values) if is_module else ()
    kwarg_names = tuple(compiled.tensor_kwarg_names) if is_module else ()
    input_count = compiled.input_count if is_module else len(plan.graph.inputs)
    if len(state_names) != len(state_values):
        raise ValueError(f"{len(state_names)} state names for {len(state_values)} state tensors")
    if len(plan.graph.inputs) != input_count + len(kwarg_names) + len(state_values):
        raise ValueError("graph inputs do not match public inputs, tensor keyword inputs and module state")

    # one payload per distinct storage: aliases share it
    payload_of: dict[tuple, str] = {}
    payloads: list[tuple[str, bytes]] = []
    state_entries = []
    for name, tensor in zip(state_names, state_values):
        key = (tensor.data_ptr(), tuple(tensor.shape), tuple(tensor.stride()), tensor.dtype)
        file_name = payload_of.get(key)
        if file_name is None:
            file_name = f"state/{len(payloads):05d}.bin"
            data = _tensor_bytes(tensor)
            payloads.append((file_name, data))
            payload_of[key] = file_name
        else:
            data = next(d for f, d in payloads if f == file_name)
        state_entries.append({
            "name": name, "file": file_name, "shape": list(tensor.shape), "dtype": _NAME_OF[tensor.dtype],
            "digest": _digest(data),
        })

    input_graph_bytes = _canonical(encode_graph(result.input_graph))
    lowered_graph_bytes = _canonical(encode_graph(result.lowered_graph))
    kernels_bytes = _canonical([_encode_kernel(k) for k in plan.kernels])
    selections_bytes = _canonical([_encode_selection(s) for s in plan.selections])
    storage_bytes = _canonical(_encode_storage(plan.storage_plan))
    manifest = {
        "format": ARTIFACT_FORMAT,
        "format_version": FORMAT_VERSION,
        "abi_version": ABI_VERSION,
        "compiler_version": __version__,
        "target": result.target,
        "entrypoint": {
            "kind": "module" if is_module else "callable",
            "input_count": input_count,
            "kwargs": [{"name": name, "index": i} for i, name in enumerate(kwarg_names)],
            "state": state_entries,
        },
        "compile_options": {
            "codegen_matmul": result.codegen_matmul, "codegen_attention": result.codegen_attention,
            "autotune": result.autotune, "autotune_warmup": result.autotune_warmup,
            "autotune_iterations": result.autotune_iterations,
        },
        "profile": _device_profile(),
        "graph": {
            "input_digest": _digest(input_graph_bytes), "lowered_digest": _digest(lowered_graph_bytes),
            "inputs": list(plan.graph.inputs), "outputs": list(plan.graph.outputs),
        },
        "payload_digests": {
            "kernels": _digest(kernels_bytes), "selections": _digest(selections_bytes),
            "storage_plan": _digest(storage_bytes),
        },
        "payloads": {
            "input_graph": "input_graph.json", "lowered_graph": "lowered_graph.json", "kernels": "kernels.json",
            "selections": "selections.json", "storage_plan": "storage_plan.json",
        },
    }

    destination = Path(path)
    destination.parent.mkdir(parents=True, exist_ok=True)
    handle, temporary_name = tempfile.mkstemp(dir=destination.parent, suffix=".tmp")
    os.close(handle)
    temporary = Path(temporary_name)
    try:
        with zipfile.ZipFile(temporary, "w", compression=zipfile.ZIP_STORED) as archive:
            def put(name: str, data: bytes) -> None:
                info = zipfile.ZipInfo(name, date_time=(1980, 1, 1, 0, 0, 0))  # fixed stamp: canonical bytes
                archive.writestr(info, data)

            put("manifest.json", _canonical(manifest))
            put("input_graph.json", input_graph_bytes)
            put("lowered_graph.json", lowered_graph_bytes)
            put("kernels.json", kernels_bytes)
            put("selections.json", selections_bytes)
            put("storage_plan.json", storage_bytes)
            for name, data in payloads:
                put(name, data)
        os.replace(temporary, destination)
    finally:
        if temporary.exists():
            temporary.unlink()
    return destination


# ---------------------------------------------------------------------------
# load
# ---------------------------------------------------------------------------

def _open(path: Path) -> zipfile.ZipFile:
    try:
        return zipfile.ZipFile(path, "r")
    except (OSError, zipfile.BadZipFile) as error:
        raise ArtifactCompatibilityError(f"{path} is not a readable artifact: {error}") from error


def _safe_payload_name(name: Any) -> str:
    """A payload name from the manifest: a relative path inside the archive, nothing else."""

    if (not isinstance(name, str) or not name or name.startswith(("/", "\\")) or "\\" in name or ":" in name
            or any(part in ("", ".", "..") for part in name.split("/"))):
        raise ArtifactCompatibilityError(f"artifact payload name {name!r} is not a plain relative path")
    return name


def _read(archive: zipfile.ZipFile, name: str) -> bytes:
    name = _safe_payload_name(name)
    try:
        return archive.read(name)
    except KeyError as error:
        raise ArtifactCompatibilityError(f"artifact payload {name!r} is missing") from error


def _check_digest(payload: bytes, expected: Any, label: str) -> None:
    if not isinstance(expected, str) or _digest(payload) != expected:
        raise ArtifactCompatibilityError(f"artifact {label} digest mismatch: the file was modified or is truncated")


def _validate_manifest(manifest: Any, *, require_device_match: bool) -> None:
    from .backends import TARGETS

    if not isinstance(manifest, dict) or manifest.get("format") != ARTIFACT_FORMAT:
        raise ArtifactCompatibilityError(f"not an {ARTIFACT_FORMAT} artifact")
    if manifest.get("format_version") not in SUPPORTED_FORMAT_VERSIONS:
        raise ArtifactCompatibilityError(
            f"artifact format version must be one of {list(SUPPORTED_FORMAT_VERSIONS)}, "
            f"got {manifest.get('format_version')!r}"
        )
    if manifest.get("abi_version") not in SUPPORTED_ABI_VERSIONS:
        raise ArtifactCompatibilityError(
            f"artifact ABI version must be one of {list(SUPPORTED_ABI_VERSIONS)}, got {manifest.get('abi_version')!r}"
        )
    if manifest.get("target") not in TARGETS:
        raise ArtifactCompatibilityError(f"artifact target {manifest.get('target')!r} is not one of {list(TARGETS)}")
    for key in ("entrypoint", "compile_options", "graph", "payload_digests", "payloads"):
        if not isinstance(manifest.get(key), dict):
            raise ArtifactCompatibilityError(f"artifact manifest has no {key!r} section")
    if require_device_match:
        profile, here = manifest.get("profile") or {}, _device_profile()
        if profile.get("device_name") != here["device_name"]:
            raise ArtifactCompatibilityError(
                f"artifact was compiled on {profile.get('device_name')!r}, this device is {here['device_name']!r}"
            )


def read_artifact_manifest(path: str | os.PathLike[str]) -> dict:
    """The validated manifest of an artifact, without touching its payloads."""

    with _open(Path(path)) as archive:
        manifest = _json(_read(archive, "manifest.json"), "manifest")
    _validate_manifest(manifest, require_device_match=False)
    return manifest


def _json(payload: bytes, label: str) -> Any:
    try:
        return json.loads(payload)
    except (ValueError, UnicodeDecodeError) as error:
        raise ArtifactCompatibilityError(f"artifact {label} is not valid JSON: {error}") from error


def load_compiled_module(
    path: str | os.PathLike[str],
    *,
    require_device_match: bool = False,
    device: Any = None,
):
    """Load, validate and rebuild a module plan saved by :func:`save_compiled`.

    Kernels are rebuilt by running the backend the manifest names over the
    stored lowered graph; the result must select what the stored records say
    (same implementation, kind and kernel variant per operation), else the
    artifact is refused: it was produced by a library whose selection rules differ.
    A malformed artifact (broken JSON, a missing key, a field of the wrong type) is
    refused with :class:`ArtifactCompatibilityError` like any other mismatch.
    """

    try:
        return _load_compiled_module(path, require_device_match=require_device_match, device=device)
    except ArtifactCompatibilityError:
        raise
    except (KeyError, TypeError, ValueError, IndexError, AttributeError) as error:
        raise ArtifactCompatibilityError(
            f"{path} is malformed: {type(error).__name__}: {error}",
            hint="the artifact was truncated, edited or written by an incompatible library",
        ) from error


def _load_compiled_module(path, *, require_device_match: bool, device: Any):

    from .compiler import CompilationResult, CompiledModulePlan, _to_device_once, backend_for

    with _open(Path(path)) as archive:
        manifest = _json(_read(archive, "manifest.json"), "manifest")
        _validate_manifest(manifest, require_device_match=require_device_match)
        names = manifest["payloads"]
        lowered_bytes = _read(archive, names["lowered_graph"])
        input_bytes = _read(archive, names["input_graph"])
        kernels_bytes = _read(archive, names["kernels"])
        selections_bytes = _read(archive, names["selections"])
        storage_bytes = _read(archive, names["storage_plan"])
        _check_digest(lowered_bytes, manifest["graph"].get("lowered_digest"), "lowered graph")
        _check_digest(input_bytes, manifest["graph"].get("input_digest"), "input graph")
        _check_digest(kernels_bytes, manifest["payload_digests"].get("kernels"), "kernel table")
        _check_digest(selections_bytes, manifest["payload_digests"].get("selections"), "selections")
        _check_digest(storage_bytes, manifest["payload_digests"].get("storage_plan"), "storage plan")
        lowered = decode_graph(_json(lowered_bytes, "lowered graph"))
        captured = decode_graph(_json(input_bytes, "input graph"))
        if list(lowered.inputs) != manifest["graph"].get("inputs") or list(lowered.outputs) != manifest["graph"].get("outputs"):
            raise ArtifactCompatibilityError("manifest graph inputs or outputs do not match the stored graph")
        entry = manifest["entrypoint"]
        state_entries = entry.get("state", [])
        loaded: dict[str, torch.Tensor] = {}
        state_values = []
        for item in state_entries:
            file_name = str(item["file"])
            tensor = loaded.get(file_name)
            if tensor is None:
                payload = _read(archive, file_name)
                _check_digest(payload, item.get("digest"), f"state {item.get('name')!r}")
                dtype = _TORCH_OF.get(str(item["dtype"]))
                if dtype is None:
                    raise ArtifactCompatibilityError(f"state dtype {item['dtype']!r} is not supported")
                tensor = _tensor_from_bytes(payload, tuple(int(d) for d in item["shape"]), dtype)
                loaded[file_name] = tensor
            state_values.append(tensor)

    stored_selections = tuple(_decode_selection(s) for s in _json(selections_bytes, "selections"))
    stored_storage = _decode_storage(_json(storage_bytes, "storage plan"))
    options = manifest["compile_options"]
    target = str(manifest["target"])
    backend = backend_for(target, codegen_matmul=bool(options.get("codegen_matmul")),
                          codegen_attention=bool(options.get("codegen_attention")))
    plan = backend.compile(lowered)
    if len(plan.selections) != len(stored_selections):
        raise ArtifactCompatibilityError("the rebuilt plan has a different number of operations than the artifact")
    for rebuilt, stored in zip(plan.selections, stored_selections):
        same = (rebuilt.op, rebuilt.output_id, rebuilt.implementation, rebuilt.kind, rebuilt.artifact_name) == (
            stored.op, stored.output_id, stored.implementation, stored.kind, stored.artifact_name)
        if not same:
            raise ArtifactCompatibilityError(
                f"operation {stored.op_index} ({stored.op}) was bound to {stored.artifact_name!r} when the artifact "
                f"was written; this library selects {rebuilt.artifact_name!r}"
            )
    if plan.storage_plan.arena_size_bytes != stored_storage.arena_size_bytes:
        raise ArtifactCompatibilityError("the rebuilt storage plan differs from the stored one")
    plan.selections = stored_selections

    input_count = int(entry["input_count"])
    kwarg_names = tuple(str(k["name"]) for k in entry.get("kwargs", []))
    if len(lowered.inputs) != input_count + len(kwarg_names) + len(state_values):
        raise ArtifactCompatibilityError("artifact entry point does not match the graph inputs")
    for value_id, tensor, item in zip(lowered.inputs[input_count + len(kwarg_names):], state_values, state_entries):
        spec = lowered.value(value_id).type
        if tuple(tensor.shape) != spec.shape or _NAME_OF[tensor.dtype] != spec.dtype.value:
            raise ArtifactCompatibilityError(f"state {item['name']!r} does not have the type of graph input {value_id}")

    where = torch.device(device) if device is not None else torch.device(plan.device)
    bound = _to_device_once(state_values, where) if torch.cuda.is_available() else tuple(state_values)
    plan.device = str(where)
    plan.dynamic_inputs = input_count + len(kwarg_names)
    compilation = CompilationResult(
        plan=plan, input_graph=captured, lowered_graph=lowered,
        codegen_matmul=bool(options.get("codegen_matmul")), codegen_attention=bool(options.get("codegen_attention")),
        autotune=bool(options.get("autotune", False)), autotune_warmup=int(options.get("autotune_warmup", 2)),
        autotune_iterations=int(options.get("autotune_iterations", 7)), target=target,
    )
    return CompiledModulePlan(
        compilation=compilation, input_count=input_count,
        state_names=tuple(str(item["name"]) for item in state_entries), _state_values=bound,
        tensor_kwarg_names=kwarg_names, tensor_kwarg_templates=(),
    )


__all__ = [
    "ABI_VERSION", "ARTIFACT_FORMAT", "FORMAT_VERSION", "load_compiled_module", "read_artifact_manifest",
    "save_compiled", "encode_graph", "decode_graph",
]
