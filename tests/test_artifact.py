"""Artifact round trip for the cuda-sm100 target.

CPU part: a compiled module plan is written and read back on a host without a
GPU (state stays on the host, the plan is rebuilt and validated); the manifest
carries the format/ABI/target fields the reference's loader checks
(``src/aotolith/artifact.py:437-487``), and tampering is refused. GPU part: the
loaded plan computes what the saved one did.
"""

import json
import zipfile

import pytest
import torch

import aotolith_b200 as aoto
from aotolith_b200.artifact import decode_graph, encode_graph
from aotolith_b200.errors import ArtifactCompatibilityError
from aotolith_b200.models.synthetic import tiny_decoder


def _runtime():
    model = tiny_decoder("qwen2", seed=4)
    return aoto.compile_qwen2_static_cache(model, prompt_length=8, max_new_tokens=4, quantize=16)


def test_graph_json_round_trip_is_exact():
    runtime = _runtime()
    for plan in (runtime.prefill, runtime.decode):
        graph = plan.plan.graph
        again = decode_graph(json.loads(json.dumps(encode_graph(graph))))
        assert again.inputs == graph.inputs and again.outputs == graph.outputs
        assert [(o.op, o.inputs, o.outputs) for o in again.ops] == [(o.op, o.inputs, o.outputs) for o in graph.ops]
        for a, b in zip(again.ops, graph.ops):
            assert repr(a.attrs) == repr(b.attrs)
        assert {k: (v.type.shape, v.type.dtype) for k, v in again.values.items()} == \
               {k: (v.type.shape, v.type.dtype) for k, v in graph.values.items()}


def test_save_and_load_without_a_gpu(tmp_path):
    runtime = _runtime()
    prefill_path, decode_path = runtime.save(tmp_path / "tiny")
    assert prefill_path.name == "tiny.prefill.aoto" and decode_path.name == "tiny.decode.aoto"
    manifest = aoto.read_artifact_manifest(decode_path)
    assert manifest["format"] == "aotolith" and manifest["format_version"] == aoto.FORMAT_VERSION
    assert manifest["abi_version"] == aoto.ABI_VERSION and manifest["target"] == "cuda-sm100"
    assert manifest["entrypoint"]["kind"] == "module" and manifest["entrypoint"]["input_count"] == 4
    names = [entry["name"] for entry in manifest["entrypoint"]["state"]]
    assert names == list(runtime.decode.state_names)
    # tensors that alias in memory (tied embeddings, shared packed buffers) share a payload
    files = [entry["file"] for entry in manifest["entrypoint"]["state"]]
    assert len(set(files)) <= len(files)

    loaded = aoto.load_compiled_module(decode_path)
    assert loaded.state_names == runtime.decode.state_names and loaded.input_count == 4
    assert loaded.target == "cuda-sm100"
    assert [s.artifact_name for s in loaded.plan.selections] == [s.artifact_name for s in runtime.decode.plan.selections]
    for a, b in zip(loaded._state_values, runtime.decode._state_values):
        assert a.dtype == b.dtype and tuple(a.shape) == tuple(b.shape)
        assert torch.equal(a.cpu().view(torch.uint8), b.cpu().contiguous().view(torch.uint8))
    # aliasing survives the round trip
    pointers = {}
    for name, tensor in zip(runtime.decode.state_names, runtime.decode._state_values):
        pointers.setdefault(tensor.data_ptr(), []).append(name)
    loaded_pointers = {}
    for name, tensor in zip(loaded.state_names, loaded._state_values):
        loaded_pointers.setdefault(tensor.data_ptr(), []).append(name)
    assert sorted(map(tuple, pointers.values())) == sorted(map(tuple, loaded_pointers.values()))
    # saving twice gives the same bytes
    again = runtime.decode.save(tmp_path / "again.aoto")
    assert again.read_bytes() == decode_path.read_bytes()


def _rewrite(path, out, edit):
    with zipfile.ZipFile(path) as src, zipfile.ZipFile(out, "w") as dst:
        for item in src.infolist():
            data = src.read(item.filename)
            data = edit(item.filename, data)
            if data is not None:
                dst.writestr(item, data)


def test_tampered_or_foreign_artifacts_are_refused(tmp_path):
    runtime = _runtime()
    path = runtime.decode.save(tmp_path / "d.aoto")

    def manifest_edit(**changes):
        def edit(name, data):
            if name != "manifest.json":
                return data
            manifest = json.loads(data)
            manifest.update(changes)
            return json.dumps(manifest).encode()
        return edit

    for changes in ({"format": "other"}, {"format_version": 99}, {"abi_version": "0.1"}, {"target": "vulkan"}):
        bad = tmp_path / "bad.aoto"
        _rewrite(path, bad, manifest_edit(**changes))
        with pytest.raises(ArtifactCompatibilityError):
            aoto.load_compiled_module(bad)

    def flip_state(name, data):
        if name == "state/00000.bin":
            return bytes([data[0] ^ 1]) + data[1:]
        return data

    bad = tmp_path / "flipped.aoto"
    _rewrite(path, bad, flip_state)
    with pytest.raises(ArtifactCompatibilityError, match="digest"):
        aoto.load_compiled_module(bad)

    def other_kernel(name, data):
        if name == "selections.json":
            return data.replace(b"qgemv_generic", b"qgemv_other")
        return data

    bad = tmp_path / "selection.aoto"
    _rewrite(path, bad, other_kernel)
    with pytest.raises(ArtifactCompatibilityError):
        aoto.load_compiled_module(bad)

    with pytest.raises(ArtifactCompatibilityError):
        (tmp_path / "junk.aoto").write_bytes(b"not a zip")
        aoto.load_compiled_module(tmp_path / "junk.aoto")


@pytest.mark.gpu
def test_loaded_plan_computes_what_the_saved_one_did(cuda, tmp_path):
    runtime = _runtime()
    prefill_path, decode_path = runtime.save(tmp_path / "tiny")
    prefill = aoto.load_compiled_module(prefill_path)
    decode = aoto.load_compiled_module(decode_path)
    prompt = torch.randint(0, 64, (1, 8), generator=torch.Generator().manual_seed(2)).to(cuda)
    positions = torch.arange(8, device=cuda)[None, :]
    mask = runtime._prefill_mask
    want_logits, want_cache = runtime.prefill(prompt, positions, mask)
    got_logits, got_cache = prefill(prompt, positions, mask)
    assert torch.equal(got_logits, want_logits) and torch.equal(got_cache, want_cache)
    cache = runtime.pad_cache(want_cache)
    token = want_logits[:, -1, :].float().argmax(-1, keepdim=True)
    dmask = runtime.decode_mask(9)
    position = torch.tensor([[8]], device=cuda)
    want = runtime.decode(token, position, dmask, cache)
    got = decode(token, position, dmask, cache)
    assert torch.equal(got[0], want[0]) and torch.equal(got[1], want[1])


def _edit_manifest(path, out, edit):
    def apply(name, data):
        if name != "manifest.json":
            return data
        manifest = json.loads(data)
        edit(manifest)
        return json.dumps(manifest).encode()

    _rewrite(path, out, apply)


def test_state_that_does_not_fit_its_graph_input_is_refused(tmp_path):
    """A manifest whose state entry claims another shape or dtype than the graph input it binds
    (tests/test_artifact.py:333-387 of the reference)."""

    path = _runtime().decode.save(tmp_path / "d.aoto")
    manifest = aoto.read_artifact_manifest(path)
    index = next(i for i, item in enumerate(manifest["entrypoint"]["state"]) if item["name"] == "final_norm")

    def other_shape(m):
        m["entrypoint"]["state"][index]["shape"] = [32, 2]           # same bytes, another shape

    def other_dtype(m):
        m["entrypoint"]["state"][index]["dtype"] = "float16"          # same bytes, another dtype

    def unknown_dtype(m):
        m["entrypoint"]["state"][index]["dtype"] = "float8"

    def short_payload(m):
        m["entrypoint"]["state"][index]["shape"] = [65]               # one element more than the payload holds

    for edit in (other_shape, other_dtype, unknown_dtype, short_payload):
        bad = tmp_path / f"{edit.__name__}.aoto"
        _edit_manifest(path, bad, edit)
        with pytest.raises(ArtifactCompatibilityError):
            aoto.load_compiled_module(bad)


def test_tampered_tables_and_missing_payloads_are_refused(tmp_path):
    path = _runtime().decode.save(tmp_path / "d.aoto")
    for member, needle in (("kernels.json", b"aoto_sm100_embedding"), ("lowered_graph.json", b"addmm"),
                           ("input_graph.json", b"arg0"), ("storage_plan.json", b"arena_size_bytes")):
        def edit(name, data, member=member, needle=needle):
            if name == member:
                assert needle in data
                return data.replace(needle, needle[:-1] + b"_", 1)
            return data

        bad = tmp_path / f"tampered_{member}.aoto"
        _rewrite(path, bad, edit)
        with pytest.raises(ArtifactCompatibilityError, match="digest"):
            aoto.load_compiled_module(bad)

        def drop(name, data, member=member):
            return None if name == member else data

        bad = tmp_path / f"without_{member}.aoto"
        _rewrite(path, bad, drop)
        with pytest.raises(ArtifactCompatibilityError, match="missing"):
            aoto.load_compiled_module(bad)


def test_a_manifest_that_disagrees_with_its_graph_is_refused(tmp_path):
    path = _runtime().decode.save(tmp_path / "d.aoto")

    def fewer_inputs(m):
        m["entrypoint"]["input_count"] = 3

    def other_outputs(m):
        m["graph"]["outputs"] = list(reversed(m["graph"]["outputs"]))

    for edit in (fewer_inputs, other_outputs):
        bad = tmp_path / f"{edit.__name__}.aoto"
        _edit_manifest(path, bad, edit)
        with pytest.raises(ArtifactCompatibilityError):
            aoto.load_compiled_module(bad)


def test_malformed_artifacts_are_refused_with_the_coded_error(tmp_path):
    """Broken JSON, missing keys, wrong field types and unsafe payload names never escape as raw
    KeyError / TypeError / JSONDecodeError."""

    path = _runtime().decode.save(tmp_path / "d.aoto")

    def truncated_manifest(name, data):
        return data[: len(data) // 2] if name == "manifest.json" else data

    def broken_selections(name, data):
        return b"[{" if name == "selections.json" else data

    for index, edit in enumerate((truncated_manifest, broken_selections)):
        bad = tmp_path / f"broken_{index}.aoto"
        _rewrite(path, bad, edit)
        with pytest.raises(ArtifactCompatibilityError):
            aoto.load_compiled_module(bad)

    def no_state_file(m):
        del m["entrypoint"]["state"][0]["file"]

    def no_input_count(m):
        del m["entrypoint"]["input_count"]

    def shape_of_wrong_type(m):
        m["entrypoint"]["state"][0]["shape"] = "wide"

    def escaping_payload(m):
        m["payloads"]["kernels"] = "../kernels.json"

    def no_payload_table(m):
        del m["payloads"]

    for edit in (no_state_file, no_input_count, shape_of_wrong_type, escaping_payload, no_payload_table):
        bad = tmp_path / f"{edit.__name__}.aoto"
        _edit_manifest(path, bad, edit)
        with pytest.raises(ArtifactCompatibilityError):
            aoto.load_compiled_module(bad)


def test_scalar_state_has_a_byte_payload():
    from aotolith_b200.artifact import _tensor_bytes, _tensor_from_bytes

    for value in (torch.tensor(1.5, dtype=torch.bfloat16), torch.tensor(-2.0), torch.zeros((), dtype=torch.int64)):
        data = _tensor_bytes(value)
        assert len(data) == value.element_size()
        assert torch.equal(_tensor_from_bytes(data, (), value.dtype), value)


def test_an_artifact_loads_in_a_new_process(tmp_path):
    """Nothing of the compiling process is needed to read an artifact back: a fresh interpreter
    rebuilds the plan and finds the same selections and state."""

    import subprocess
    import sys
    from pathlib import Path

    runtime = _runtime()
    path = runtime.decode.save(tmp_path / "d.aoto")
    expected = [s.artifact_name for s in runtime.decode.plan.selections]
    script = (
        "import json, sys, aotolith_b200 as aoto\n"
        f"plan = aoto.load_compiled_module({str(path)!r})\n"
        "print(json.dumps({'names': list(plan.state_names), 'inputs': plan.input_count, 'target': plan.target,\n"
        "                  'selections': [s.artifact_name for s in plan.plan.selections]}))\n"
    )
    root = Path(__file__).resolve().parent.parent
    done = subprocess.run([sys.executable, "-c", script], capture_output=True, text=True, cwd=root, timeout=300)
    assert done.returncode == 0, done.stderr[-2000:]
    report = json.loads(done.stdout.strip().splitlines()[-1])
    assert report["names"] == list(runtime.decode.state_names) and report["inputs"] == 4
    assert report["target"] == "cuda-sm100" and report["selections"] == expected
