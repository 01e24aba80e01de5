"""Benchmark of the static-KV-cache decoder path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--workload NAME]

Workload (default ``qwen25_05b``): a Qwen2.5-0.5B-shaped decoder (hidden 896,
MLP 4864, 24 layers, 14/2 heads, head dim 64, vocab 151936, tied embeddings,
q/k/v bias, bf16), random-init from a seed, 4-bit group-64 packed, compiled
through ``compile_qwen2_static_cache``; prompt = 128 uniform-random token ids,
64 greedy tokens at batch 1. One *step* of the benchmark is one such request:
prefill, then 63 decode steps on the device-resident stepper.

The printed JSON line reports

* ``value``    decode tok/s, whole job: decode steps of all ranks / device time of
               the decode loops (CUDA events; prompt and weights resident in HBM);
* ``e2e``      generated tok/s through ``runtime.greedy_generate`` from pinned host
               prompt ids to host tokens (prefill, copies and the final read-back
               inside the timed region);
* ``roofline`` the dominant kernel - the persistent decode-step kernel, one launch
               per token: algorithmic bytes of a step over the CUDA-event duration of
               a launch inside the timed region, against the measured HBM peak;
* ``lm_head_roofline`` the largest single projection (the LM-head GEMV over the packed
               vocabulary matrix) alone, on rotating weight copies larger than L2;
* ``bf16``     the same decoder with dense bf16 weights (``quantize=None``), one GPU only;
* ``rows``     one decode step over eight tokens (``decode_rows=8``) against eight one-token
               plan calls, one GPU only;
* ``cpu_baseline`` the same decoder evaluated eagerly by PyTorch on the host cores
               for a bounded sample (prefill + a few decode steps).

``--impl reference`` times only that CPU arm. With ``--gpus N`` (launched by
``torch.distributed.run``) every rank serves its own request stream on its own
GPU - the path has no exchange step at this model size - and the line is the
sum over ranks with the slowest rank's time.
"""

from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time
from pathlib import Path

import torch

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

PROMPT, NEW_TOKENS, GROUP = 128, 64, 64

WORKLOADS = {
    "qwen25_05b": dict(builder="qwen25_05b_shaped", family="qwen2", layers=24,
                       description="Qwen2.5-0.5B-shaped, 4-bit g64, prompt 128, 64 greedy tokens, batch 1"),
    "llama3_8b": dict(builder="llama3_8b_shaped", family="llama", layers=32, prompt=1024, new_tokens=256,
                      description="Llama-3-8B-shaped, 4-bit g64, prompt 1024, 256 greedy tokens, batch 1"),
    "llama3_8b_tp": dict(builder="llama3_8b_shaped", family="llama", layers=32, prompt=1024, new_tokens=256,
                         description="Llama-3-8B-shaped, 4-bit g64, prompt 1024, 256 greedy tokens, batch 1, "
                                     "tensor parallel over the GPUs of the run"),
    "qwen25_05b_bucketed": dict(builder="qwen25_05b_shaped", family="qwen2", layers=24,
                                description="bucketed Qwen2.5-0.5B-shaped runtime, buckets {32,64,128,256}, "
                                            "prompt lengths uniform in [1,256], 64 greedy tokens per request"),
}
BUCKETS = (32, 64, 128, 256)


def measured_peaks() -> tuple[float, str]:
    path = ROOT / "MEASURED_PEAKS.json"
    if path.exists():
        try:
            return float(json.loads(path.read_text())["hbm_gbs"]), "measured"
        except Exception:  # noqa: BLE001
            pass
    return 6650.0, "fallback"


def tensor_peak() -> float | None:
    """Measured dense bf16 TFLOP/s of this pool's B200 (burst), if the driver wrote it."""

    try:
        return float(json.loads((ROOT / "MEASURED_PEAKS.json").read_text())["bf16_tflops"])
    except Exception:
        return None


def projection_bytes(n: int, k: int, *, bias=False, norm=False, residual=False, m: int = 1) -> int:
    """Algorithmic bytes of one packed projection (codes, scales, x, y and optional operands)."""

    total = n * k // 2 + n * (k // GROUP) * 2 + m * k * 2 + m * n * 2
    total += n * 2 if bias else 0
    total += k * 2 if norm else 0
    total += m * n * 2 if residual else 0
    return total


def step_bytes(config, valid_length: int) -> int:
    """Algorithmic HBM bytes of one decode step (weights once, KV window read, logits, cache write)."""

    h, i, layers = config.hidden_size, config.intermediate_size, config.num_hidden_layers
    qh, kvh, d, v = config.num_attention_heads, config.num_key_value_heads, config.head_dim, config.vocab_size
    qkv = projection_bytes((qh + 2 * kvh) * d, h, bias=True, norm=True)
    o = projection_bytes(h, qh * d, residual=True)
    gate_up = 2 * (i * h // 2 + i * (h // GROUP) * 2) + h * 2 + h * 2 + i * 2
    down = projection_bytes(h, i, residual=True)
    head = projection_bytes(v, h, norm=True)
    kv_read = 2 * kvh * d * 2 * valid_length
    kv_write = 2 * kvh * d * 2
    return layers * (qkv + o + gate_up + down + kv_read + kv_write) + head + h * 2


def dense_step_bytes(config, valid_length: int) -> int:
    """Algorithmic HBM bytes of one decode step over dense bf16 weights (two bytes a weight)."""

    h, i, layers = config.hidden_size, config.intermediate_size, config.num_hidden_layers
    qh, kvh, d, v = config.num_attention_heads, config.num_key_value_heads, config.head_dim, config.vocab_size

    def dense(n, k, extra=0):
        return n * k * 2 + k * 2 + n * 2 + extra

    qkv = dense((qh + 2 * kvh) * d, h, extra=(qh + 2 * kvh) * d * 2 + 2 * h * 2)   # bias; the norm reads and writes x
    o = dense(h, qh * d, extra=h * 2)                                              # residual
    gate_up = 2 * i * h * 2 + h * 2 + i * 2 + 2 * h * 2
    down = dense(h, i, extra=h * 2)
    head = dense(v, h, extra=2 * h * 2)
    kv_read = 2 * kvh * d * 2 * valid_length
    kv_write = 2 * kvh * d * 2
    return layers * (qkv + o + gate_up + down + kv_read + kv_write) + head + h * 2


def measure_rows(model, prompt_host, device, rows: int = 8, repeats: int = 10) -> dict:
    """One decode step over ``rows`` tokens (``decode_rows=rows``) against ``rows`` one-token plan calls.

    The proposed tokens are the greedy ones, so row j of the step must confirm token j + 1. CUDA
    events over ``repeats`` steps after three untimed ones; weights larger than L2.
    """

    import aotolith_b200 as aoto

    runtime = aoto.compile_qwen2_static_cache(model, prompt_length=PROMPT, max_new_tokens=NEW_TOKENS,
                                              quantize=GROUP, decode_rows=rows)
    prompt = prompt_host.to(device)
    greedy = runtime.greedy_generate(prompt)                       # the tokens a host would propose
    logits, compact = runtime.prefill_ids(prompt)
    cache = runtime.pad_cache(compact)
    proposed = greedy[:, :rows].contiguous()
    for _ in range(3):
        step_logits, _ = runtime.decode_tokens(proposed, cache, PROMPT + rows, verify_tokens=False)
    torch.cuda.synchronize()
    marks = [torch.cuda.Event(enable_timing=True) for _ in range(3)]
    marks[0].record()
    for _ in range(repeats):
        step_logits, _ = runtime.decode_tokens(proposed, cache, PROMPT + rows, verify_tokens=False)
    marks[1].record()
    for _ in range(repeats):
        single, valid = cache, PROMPT
        for j in range(rows):
            valid += 1
            one_logits, single = runtime.decode_token(proposed[:, j : j + 1], single, valid, verify_token=False)
    marks[2].record()
    torch.cuda.synchronize()
    rows_us = marks[0].elapsed_time(marks[1]) * 1e3 / repeats
    singles_us = marks[1].elapsed_time(marks[2]) * 1e3 / repeats
    # row j predicts the token after proposed token j: the greedy continuation, when the proposal was the greedy one
    predicted = step_logits[0].float().argmax(dim=-1)
    agree = int((predicted[:-1] == greedy[0, 1:rows]).sum())
    last_gap = float((step_logits[0, -1].float() - one_logits[0, -1].float()).abs().max() / one_logits.float().abs().max())
    return {"workload": f"Qwen2.5-0.5B-shaped, 4-bit g64, prompt 128: one step over {rows} tokens",
            "rows": rows, "rows_step_us": round(rows_us, 1), "us_per_token": round(rows_us / rows, 1),
            "value": round(rows * 1e6 / rows_us, 1), "unit": "tok/s verified per step",
            "one_token_plan_calls_us": round(singles_us, 1),
            "greedy_tokens_confirmed": f"{agree} of {rows - 1}", "last_row_vs_one_token_step": last_gap,
            "kernels": sorted({s.artifact_name for s in runtime.rows.plan.selections
                               if s.kind in ("matmul", "addmm", "attention")})}


def measure_dense(model, prompt_host, device, peak: float, peak_kind: str, requests: int = 3) -> dict:
    """The same decoder with its bf16 weights as they are (``quantize=None``): the ``bf16`` record.

    One request = prefill + NEW_TOKENS - 1 decode steps through the per-operation plan under a
    recorded graph; CUDA events around the prompt pass and around whole requests, weights (about
    1 GB a step) larger than L2.
    """

    import aotolith_b200 as aoto

    runtime = aoto.models.compile_decoder_static_cache(model, prompt_length=PROMPT, max_new_tokens=NEW_TOKENS,
                                                       target="cuda-sm100")
    prompt = prompt_host.to(device)
    for _ in range(3):
        tokens = runtime.greedy_generate(prompt)
    torch.cuda.synchronize()
    marks = [torch.cuda.Event(enable_timing=True) for _ in range(3)]
    marks[0].record()
    for _ in range(requests):
        runtime.prefill_ids(prompt)
    marks[1].record()
    for _ in range(requests):
        tokens = runtime.greedy_generate(prompt)
    marks[2].record()
    torch.cuda.synchronize()
    prefill_ms = marks[0].elapsed_time(marks[1]) / requests
    request_ms = marks[1].elapsed_time(marks[2]) / requests
    decode_us = (request_ms - prefill_ms) * 1e3 / (NEW_TOKENS - 1)
    nbytes = dense_step_bytes(model.config, PROMPT + 1 + (NEW_TOKENS - 1) // 2)
    achieved = nbytes / (decode_us * 1e-6) / 1e9
    kinds = sorted({s.artifact_name for s in runtime.decode.plan.selections if s.kind in ("matmul", "addmm")})
    return {"workload": "the same decoder with dense bf16 weights (quantize=None), prompt 128, 64 greedy tokens",
            "value": 1e6 / decode_us, "unit": "tok/s", "decode_us_per_token": decode_us,
            "prefill": {"ms": prefill_ms, "tok_s": PROMPT / prefill_ms * 1e3},
            "roofline": {"kernel": "per-operation decode plan over " + ", ".join(kinds), "bound": "hbm", "achieved": achieved,
                         "peak": peak, "unit": "GB/s", "frac": achieved / peak, "bytes_per_step": nbytes, "peak_source": peak_kind},
            "tokens": int(tokens.numel())}


class ClockSampler:
    """Samples ``nvidia-smi`` clocks and throttle reasons while the timed region runs."""

    FIELDS = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
              "clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int) -> None:
        self.index = index
        self.rows: list[list[str]] = []
        self.proc = None
        self.thread = None

    def start(self) -> None:
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--id={self.index}", f"--query-gpu={self.FIELDS}",
                 "--format=csv,noheader,nounits", "-lms", "100"],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            self.proc = None
            return

        def pump():
            for line in self.proc.stdout:
                parts = [p.strip() for p in line.split(",")]
                if len(parts) == 6:
                    self.rows.append(parts)

        self.thread = threading.Thread(target=pump, daemon=True)
        self.thread.start()

    def stop(self) -> dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        clocks, reasons, peak = [], set(), None
        for sm, sm_max, hw, hw_thermal, sw_thermal, power in self.rows:
            try:
                clocks.append(float(sm))
                peak = float(sm_max)
            except ValueError:
                continue
            for name, flag in (("hw_slowdown", hw), ("hw_thermal_slowdown", hw_thermal),
                               ("sw_thermal_slowdown", sw_thermal), ("sw_power_cap", power)):
                if flag.lower().startswith("active"):
                    reasons.add(name)
        return {
            "sm_mhz": statistics.median(clocks) if clocks else None,
            "sm_max_mhz": peak,
            "reasons": sorted(reasons),
            "samples": len(clocks),
        }


def build_model(workload: str, seed: int, device="cpu", **options):
    """The workload's seeded model. ``device``: where it is drawn (the 8B shape takes minutes on the
    host and seconds on a GPU; the values depend on the device kind, not on which GPU)."""

    from aotolith_b200.models import synthetic

    spec = WORKLOADS[workload]
    return getattr(synthetic, spec["builder"])(seed=seed, device=device, **options), spec


def seeded_prompt(vocab: int, seed: int, length: int | None = None) -> torch.Tensor:
    return torch.randint(0, vocab, (1, length or PROMPT), generator=torch.Generator().manual_seed(seed), dtype=torch.int64)


# ---------------------------------------------------------------------------
# CPU arm
# ---------------------------------------------------------------------------

def cpu_sample(model, prompt, decode_steps: int) -> dict:
    from oracle.eager import EagerCpuDecoder

    threads = os.cpu_count() or 1
    torch.set_num_threads(threads)
    decoder = EagerCpuDecoder(model, PROMPT, NEW_TOKENS, GROUP)
    _, prefill_s, decode_s = decoder.run(prompt, decode_steps)
    return {
        "value": decode_steps / decode_s,
        "unit": "tok/s",
        "cores": torch.get_num_threads(),
        "kind": "port",
        "sample": f"prefill of {PROMPT} tokens ({prefill_s:.2f} s, not counted) then {decode_steps} "
                  f"decode steps of the same decoder, PyTorch CPU bf16 eager ({decode_s:.2f} s)",
        "prefill_tok_s": PROMPT / prefill_s,
    }


def run_reference(args) -> None:
    """The CPU arm alone: one step = one greedy decode step on the host cores."""

    from oracle.eager import EagerCpuDecoder

    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    model, spec = build_model(args.workload, seed=0)
    prompt = seeded_prompt(model.config.vocab_size, 1)
    torch.set_num_threads(os.cpu_count() or 1)
    decoder = EagerCpuDecoder(model, PROMPT, NEW_TOKENS, GROUP)
    prefill_s = decoder.start(prompt)
    for _ in range(args.warmup):
        decoder.step()
    seconds = [decoder.step() for _ in range(args.steps)]
    value = len(seconds) / sum(seconds)
    baseline = {
        "value": value, "unit": "tok/s", "cores": torch.get_num_threads(), "kind": "port",
        "sample": f"{args.steps} decode steps after a {PROMPT}-token prefill ({prefill_s:.2f} s, not counted), "
                  "PyTorch CPU bf16 eager over the same adapter modules",
        "prefill_tok_s": PROMPT / prefill_s,
    }
    print(json.dumps({
        "impl": "reference",
        "metric": "batch-1 decode tok/s (4-bit g64 static cache)",
        "value": value, "unit": "tok/s", "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": sum(seconds) * 1e3 / len(seconds), "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": {"workload": spec["description"], "arm": "host CPU cores, PyTorch eager",
                   "step": "one decode step (one token) on the host"},
        "cpu_baseline": baseline,
        "e2e": {"value": value, "unit": "tok/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }))


# ---------------------------------------------------------------------------
# GPU arm
# ---------------------------------------------------------------------------

def time_lm_head(runtime, peak_gbs: float, peak_kind: str) -> dict:
    """The LM-head GEMV alone, on rotating copies of its weight so every launch streams from HBM."""

    from aotolith_b200 import ops

    state = dict(zip(runtime.decode.state_names, runtime.decode._state_values))
    packed, scales, norm = state["lm_head_0_packed"], state["lm_head_0_scales"], state["final_norm"]
    n, words = packed.shape
    k = words * 8
    copies = max(3, int(400e6 // (packed.numel() * 4)) + 1)
    packs = [packed.clone() for _ in range(copies)]
    scale_copies = [scales.clone() for _ in range(copies)]
    x = torch.randn(1, k, device=packed.device).bfloat16()
    out = torch.empty(1, n, dtype=torch.bfloat16, device=packed.device)
    for i in range(copies):
        ops.qmatmul(x, packs[i], scale_copies[i], group_size=GROUP, norm_weight=norm, rms_norm_eps=1e-6, out=out)
    torch.cuda.synchronize()
    iterations = 60
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    start.record()
    for i in range(iterations):
        j = i % copies
        ops.qmatmul(x, packs[j], scale_copies[j], group_size=GROUP, norm_weight=norm, rms_norm_eps=1e-6, out=out)
    stop.record()
    torch.cuda.synchronize()
    seconds = start.elapsed_time(stop) / 1e3 / iterations
    algorithmic = projection_bytes(n, k, norm=True)
    achieved = algorithmic / seconds / 1e9
    return {
        "kernel": f"{ops.qmatmul_variant(1, n, k, GROUP)} (LM head, N={n}, K={k})", "bound": "hbm", "achieved": achieved,
        "peak": peak_gbs, "unit": "GB/s", "frac": achieved / peak_gbs,
        # dram__bytes_read.sum + dram__bytes_write.sum of one launch of this shape under ncu
        "traffic": 72_360_000 + 1_420_000,
        "peak_source": peak_kind, "bytes_per_launch": algorithmic, "us_per_launch": seconds * 1e6,
        "note": f"{iterations} launches over {copies} weight copies ({copies * packed.numel() * 4 / 1e6:.0f} MB > L2)",
    }


SWEEP_SHAPES = [(896, 1152, True), (896, 896, False), (896, 4864, False), (4864, 896, False), (896, 151936, False)]
SWEEP_ROWS = (1, 16, 128)


def qmatmul_sweep(device, hbm_peak: float, tensor_peak: float | None) -> list[dict]:
    """The packed-matmul sweep on the Qwen2.5-0.5B projection shapes, M in {1, 16, 128}.

    Every point is timed as 24 launches recorded in one CUDA graph over rotating weight copies
    (more than L2 in total), replayed four times between two CUDA events: the small shapes
    take 3-20 us, below what a host can launch back to back.
    """

    from aotolith_b200 import ops

    results = []
    for K, N, bias in SWEEP_SHAPES:
        generator = torch.Generator().manual_seed(K + N)
        packed = torch.randint(-2**31, 2**31 - 1, (N, K // 8), dtype=torch.int32, generator=generator).to(device)
        scales = (torch.rand(N, K // 64, generator=generator) * 0.01 + 0.001).bfloat16().to(device)
        copies = min(64, max(3, int(400e6 // (N * K // 2)) + 1))
        packs = [packed.clone() for _ in range(copies)]
        scale_copies = [scales.clone() for _ in range(copies)]
        addend = torch.randn(N, generator=generator).bfloat16().to(device) if bias else None
        for M in SWEEP_ROWS:
            x = torch.randn(M, K, generator=generator).bfloat16().to(device)
            out = torch.empty(M, N, dtype=torch.bfloat16, device=device)

            def launch(i):
                ops.qmatmul(x, packs[i % copies], scale_copies[i % copies], group_size=GROUP, addend=addend, out=out)

            for i in range(copies):
                launch(i)
            torch.cuda.synchronize()
            side = torch.cuda.Stream()
            side.wait_stream(torch.cuda.current_stream())
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph, stream=side):
                for i in range(24):
                    launch(i)
            graph.replay()
            torch.cuda.synchronize()
            begin, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            begin.record()
            for _ in range(4):
                graph.replay()
            end.record()
            torch.cuda.synchronize()
            us = begin.elapsed_time(end) * 1e3 / 96
            nbytes = projection_bytes(N, K, bias=bias, m=M)
            point = {
                "K": K, "N": N, "M": M, "variant": ops.qmatmul_variant(M, N, K, GROUP), "us": round(us, 2),
                "gbs": round(nbytes / us / 1e3, 1), "frac_hbm_measured": round(nbytes / us / 1e3 / hbm_peak, 4),
                "frac_hbm_8tbs": round(nbytes / us / 1e3 / 8000.0, 4),
                "tflops": round(2.0 * M * N * K / us / 1e6, 2),
            }
            if tensor_peak:
                point["frac_tensor_measured"] = round(point["tflops"] / tensor_peak, 4)
            results.append(point)
            del graph
    return results


def run_ours(args) -> None:
    import torch.distributed as dist

    import aotolith_b200 as aoto
    from aotolith_b200.models.session import decode_session

    world, rank, device = start_ranks()
    local = device.index

    # the 8B shape is drawn on the GPU (seconds instead of minutes on the host); its CPU arm is left out
    on_device = WORKLOADS[args.workload]["family"] == "llama"
    model, spec = build_model(args.workload, seed=0, device=device if on_device else "cpu")
    compile_fn = aoto.compile_qwen2_static_cache if spec["family"] == "qwen2" else aoto.compile_llama_static_cache
    runtime = compile_fn(model, prompt_length=PROMPT, max_new_tokens=NEW_TOKENS, quantize=GROUP)
    config = model.config
    if on_device:
        model = None  # the bf16 original is not needed once the packed runtime exists
        torch.cuda.empty_cache()
    prompt_host = seeded_prompt(config.vocab_size, 1 + rank).pin_memory()
    prompt_dev = prompt_host.to(device)
    session = decode_session(runtime)
    decode_steps = NEW_TOKENS - 1
    # kernel mode: the whole step is one launch of the persistent step kernel; otherwise the
    # per-operation plan plus the step-input and greedy-pick kernels
    kernel_mode, kernel_name = session.mode == "kernel", session.kernel_name
    if kernel_mode:
        kernels_per_token = 1
    else:
        kernels_per_token = sum(1 for s in runtime.decode.plan.selections if s.is_native) + 2
    kernels_prefill = sum(1 for s in runtime.prefill.plan.selections
                          if s.is_native and "weight operand" not in (s.artifact_name or "")) + 1

    def request(ids):
        """One request with device-resident inputs; returns (tokens, decode-loop milliseconds)."""
        logits, compact = runtime.prefill_ids(ids)
        cache = runtime.pad_cache(compact)
        from aotolith_b200 import ops
        token = ops.argmax(logits[:, -1, :]).reshape(1, 1)
        begin, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        begin.record()
        rest = session.run(token, cache, PROMPT, decode_steps)
        end.record()
        return rest, begin, end

    for _ in range(max(args.warmup, 3)):
        request(prompt_dev)
        runtime.greedy_generate(prompt_host).cpu()
    torch.cuda.synchronize()

    # prefill alone (128 tokens through the prefill plan), CUDA events, after the warm-up above
    begin, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    begin.record()
    for _ in range(5):
        runtime.prefill_ids(prompt_dev)
    end.record()
    torch.cuda.synchronize()
    prefill_ms = begin.elapsed_time(end) / 5
    prefill_stats = {"ms": prefill_ms, "tok_s": PROMPT / (prefill_ms / 1e3), "tokens": PROMPT,
                     "launches": kernels_prefill}

    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize()
    wall_start = time.perf_counter()
    events = []
    torch.cuda.nvtx.range_push("aoto_timed_requests")  # lets a profiler list exactly the timed launches
    for _ in range(args.steps):
        _, begin, end = request(prompt_dev)
        events.append((begin, end))
    torch.cuda.synchronize()
    torch.cuda.nvtx.range_pop()
    wall = time.perf_counter() - wall_start
    decode_ms = sum(b.elapsed_time(e) for b, e in events)

    # end to end through the public call: pinned host ids in, host tokens out
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize()
    e2e_start = time.perf_counter()
    for _ in range(args.steps):
        tokens_host = runtime.greedy_generate(prompt_host).cpu()
    e2e_wall = time.perf_counter() - e2e_start
    clocks = sampler.stop() if rank == 0 else None

    from aotolith_b200 import replicas

    group_device = device if world > 1 else None
    decode_job = replicas.job_throughput(args.steps * decode_steps, decode_ms, group_device)
    e2e_job = replicas.job_throughput(args.steps * NEW_TOKENS, e2e_wall * 1e3, group_device)
    wall = replicas.job_throughput(0, wall * 1e3, group_device).milliseconds / 1e3
    if world > 1:
        dist.barrier()
    decode_ms = decode_job.milliseconds

    # With more than one GPU the same command also reports the two workloads that use them
    # together or at volume: the 8B shape sharded over the ranks (after a checked comparison of the
    # sharded decoder with the unsharded one) and the bucketed runtime under many requests.
    extra = {}
    if world > 1 and args.workload == "qwen25_05b" and not args.skip_multi:
        del session
        runtime = None
        torch.cuda.empty_cache()
        # a record that cannot be made (a shape a kernel declines at this N, say) is reported as such and does
        # not take the line with it; a failed parity check still ends the run
        def guarded(name, make):
            try:
                extra[name] = make()
            except Exception as error:  # noqa: BLE001
                extra[name] = {"error": f"{type(error).__name__}: {error}"[:500]} if rank == 0 else None

        guarded("bucketed", lambda: measure_bucketed(world, rank, device, per_rank=512, warmup=3, with_clocks=False,
                                                      in_child=True))
        guarded("tp_parity", lambda: check_tp_parity(world, rank, device))
        # the sharded decoder is timed only behind a passed check (every rank knows the verdict)
        if parity_passed(extra.get("tp_parity"), rank, device):
            guarded("tp", lambda: measure_tp(world, rank, device, steps=2, warmup=1, with_clocks=False))
        elif rank == 0:
            extra["tp"] = {"error": "not timed: the tensor-parallel parity check did not pass"}

    if rank == 0:
        peak, peak_kind = measured_peaks()
        value = decode_job.per_second
        per_token_us = decode_ms * 1e3 / (args.steps * decode_steps)
        mean_valid = PROMPT + 1 + decode_steps // 2
        bytes_step = step_bytes(config, mean_valid)
        achieved_step = bytes_step / (per_token_us * 1e-6) / 1e9
        line = {
            "metric": "batch-1 decode tok/s (4-bit g64 static cache)",
            "value": value, "unit": "tok/s", "n_gpus": world, "steps": args.steps, "warmup": max(args.warmup, 3),
            "ms_per_step": wall * 1e3 / args.steps, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            "config": {
                "workload": spec["description"],
                "step": f"one request: prefill({PROMPT}) + {decode_steps} decode steps; value counts the decode loop only",
                "parallelism": f"{world} independent request stream(s), one runtime per GPU",
                "l2": f"inputs larger than L2: {bytes_step / 1e6:.0f} MB of packed weights are streamed per token",
                "e2e_definition": f"{NEW_TOKENS} generated tokens / wall time of greedy_generate(host ids) -> host tokens",
            },
            "decode_us_per_token": per_token_us,
            "e2e": {"value": e2e_job.per_second, "unit": "tok/s",
                    "h2d_bytes_per_step": PROMPT * 8, "d2h_bytes_per_step": NEW_TOKENS * 8},
            "gpu_launches": args.steps * (kernels_prefill + decode_steps * kernels_per_token),
            "clocks": clocks,
        }
        step_roofline = {
            "kernel": f"{kernel_name} (one launch = one decode step)" if kernel_mode
            else "per-operation decode plan (CUDA graph of one step)",
            "bound": "hbm", "achieved": achieved_step, "peak": peak, "unit": "GB/s",
            "frac": achieved_step / peak,
            # ncu on the same kernel over a 4-layer cut of the 0.5B shape moved 110.06 MB of DRAM (105.67 read
            # + 4.39 written) for 104.0 MB of algorithmic bytes; traffic grows with the layers like the bytes
            "traffic": int(bytes_step * 110.06 / 104.0) if args.workload == "qwen25_05b" and kernel_name == "stream_step_kernel" else None,
            "bytes_per_launch": bytes_step, "us_per_launch": per_token_us,
            "frac_of_8tbs": achieved_step / 8000.0, "peak_source": peak_kind,
            "note": "launch duration = CUDA-event time of the decode loop / launches, inside the timed region",
        }
        line["roofline"] = step_roofline
        if world == 1:
            lm_head = time_lm_head(runtime, peak, peak_kind)
            if kernel_mode:
                line["lm_head_roofline"] = lm_head
            else:
                line["roofline"], line["step_roofline"] = lm_head, step_roofline
        line["prefill"] = prefill_stats
        line.update(extra)
        if world == 1 and args.workload == "qwen25_05b":
            line["qmatmul_sweep"] = qmatmul_sweep(device, peak, tensor_peak())
            try:
                line["bf16"] = measure_dense(model, prompt_host, device, peak, peak_kind)
            except Exception as error:  # noqa: BLE001 - a sub-record must not lose the line
                line["bf16"] = {"error": f"{type(error).__name__}: {error}"[:500]}
            try:
                line["rows"] = measure_rows(model, prompt_host, device)
            except Exception as error:  # noqa: BLE001
                line["rows"] = {"error": f"{type(error).__name__}: {error}"[:500]}
        if world == 1 and not args.skip_cpu and not on_device:
            line["cpu_baseline"] = cpu_sample(model, prompt_host, 3)
        print(json.dumps(line))
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


def print_stage_trace(runtime, session, token, cache) -> None:
    """One step with the kernel's trace on, printed stage by stage.

    The streamed kernel records every CTA on the global timer: per stage, when the last CTA had
    its input, had it staged, had multiplied, and was done - and from those the exchange time
    (last input minus the previous stage's last `done`) and the work time. The in-place kernel
    records CTA 0 only.
    """

    import numpy as np

    streamed = session.kernel_name == "stream_step_kernel"
    ctas = torch.cuda.get_device_properties(session.device).multi_processor_count if streamed else 1
    trace = torch.zeros(ctas * session.stage_count * 8, dtype=torch.int64, device=session.device)
    session.token.copy_(token)
    session.caches[0].copy_(cache)
    session.counters.copy_(torch.tensor([PROMPT + 1, 0], dtype=torch.int32))
    for step in range(6):
        session.launch_step(step & 1, trace=trace if step == 5 else None)
    torch.cuda.synchronize()
    kinds = [stage.kind for stage in runtime.decode.plan.step_program.stages] + [3]
    names = {1: "gemv", 2: "attention", 3: "pick"}
    if not streamed:
        table = trace.cpu().reshape(-1, 8).tolist()
        origin, previous_end = table[0][0], table[0][0]
        for index, row in enumerate(table):
            print(f"stage {index:3d} {names[kinds[index]]:9s} at {row[0] - origin:7d} ns  gap {row[0] - previous_end:5d} | "
                  f"poll {row[1] - row[0]:5d} work {row[7] - row[1]:6d}")
            previous_end = row[7]
        print(f"total {table[-1][7] - origin} ns, status {int(session.status.item())}")
        return
    times = trace.cpu().numpy().reshape(ctas, session.stage_count, 8).astype(np.float64)
    times[times == 0] = np.nan
    times -= np.nanmin(times)
    print("stage kind      ctas | last input  staged  multiplied  done | exchange  work   (ns, 256 ns timer)")
    previous_done = 0.0
    for index in range(session.stage_count):
        rows = times[:, index, :]
        busy = ~np.isnan(rows[:, 2] if kinds[index] == 2 else rows[:, 1])
        if kinds[index] == 3 or not busy.any():
            continue
        rows = rows[busy]
        last_input, done = np.nanmax(rows[:, 1]), np.nanmax(rows[:, 7])
        print(f"{index:5d} {names[kinds[index]]:9s} {int(busy.sum()):4d} | {last_input:10.0f} {np.nanmax(rows[:, 3]):7.0f} "
              f"{np.nanmax(rows[:, 5]):11.0f} {done:5.0f} | {last_input - previous_done:8.0f} {done - last_input:5.0f}")
        if kinds[index] == 2:  # the last CTA at each of the stage's eight marks, and the median CTA
            print("      marks (last CTA)  ", " ".join(f"{np.nanmax(rows[:, m]):7.0f}" for m in range(8)))
            print("      marks (median CTA)", " ".join(f"{np.nanmedian(rows[:, m]):7.0f}" for m in range(8)))
        previous_done = done
    print(f"total {np.nanmax(times):.0f} ns, status {int(session.status.item())}")


def start_ranks():
    """``(world, rank, device)`` of this process; joins the NCCL group when there is more than one rank."""

    import torch.distributed as dist

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device; the cuda-sm100 target has no CPU path")
    torch.cuda.set_device(local)
    device = torch.device("cuda", local)
    # the peer exchange of this library uses plain stores into mapped peer buffers, never multimem:
    # keep the symmetric-memory buffers off NVLink multicast objects
    os.environ.setdefault("TORCH_SYMM_MEM_DISABLE_MULTICAST", "1")
    if world > 1 and not dist.is_initialized():
        from datetime import timedelta

        # a rank that died must not keep the others waiting for the default ten minutes
        dist.init_process_group("nccl", device_id=device, timeout=timedelta(minutes=5))
    return world, rank, device


def measure_tp(world: int, rank: int, device, steps: int, warmup: int, with_clocks: bool = True,
               streamed: bool = True) -> dict | None:
    """One request stream, the Llama-3-8B shape sharded over all ranks (strong scaling).

    Every rank draws the same seeded model on its own GPU and packs only its shard. A step is
    one request: prefill of 1024 tokens (per-operation kernels, NCCL all-reduces of the prompt
    rows), then 255 decode steps. ``streamed``: a step is ONE launch per rank of the streamed step
    kernel, which stores the partial o/down rows into every peer's exchange buffer and adds them
    where they are consumed; otherwise the recorded per-operation step with two peer-memory sums
    per layer. Returns the record on rank 0.
    """

    import torch.distributed as dist

    from aotolith_b200 import replicas
    from aotolith_b200.tensor_parallel import StreamedTensorParallelDecoder, TensorParallelDecoder

    spec = WORKLOADS["llama3_8b_tp"]
    prompt_length, new_tokens = spec["prompt"], spec["new_tokens"]
    model, _ = build_model("llama3_8b_tp", seed=0, device=device)
    kind = StreamedTensorParallelDecoder if streamed else TensorParallelDecoder
    decoder = kind(model, prompt_length=prompt_length, max_new_tokens=new_tokens, group_size=GROUP,
                   world=world, rank=rank, device=device)
    config = model.config
    del model
    torch.cuda.empty_cache()
    prompt = seeded_prompt(config.vocab_size, 1, prompt_length).pin_memory()
    decode_steps = new_tokens - 1
    for _ in range(warmup):
        decoder.greedy_generate(prompt).cpu()
    torch.cuda.synchronize()
    sampler = ClockSampler(device.index)
    if rank == 0 and with_clocks:
        sampler.start()
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize()
    decode_ms = prefill_ms = 0.0
    e2e_start = time.perf_counter()
    for _ in range(steps):
        marks = [torch.cuda.Event(enable_timing=True) for _ in range(3)]
        marks[0].record()
        logits = decoder.prefill(prompt)
        first = decoder.ops.argmax(logits).reshape(1, 1)
        marks[1].record()
        rest = decoder.decode_after_prefill(first, decode_steps)
        marks[2].record()
        tokens_host = rest.cpu()
        prefill_ms += marks[0].elapsed_time(marks[1])
        decode_ms += marks[1].elapsed_time(marks[2])
    e2e_wall = time.perf_counter() - e2e_start
    clocks = sampler.stop() if rank == 0 and with_clocks else None
    group_device = device if world > 1 else None
    decode_ms = replicas.job_throughput(0, decode_ms, group_device).milliseconds
    prefill_ms = replicas.job_throughput(0, prefill_ms, group_device).milliseconds
    e2e_ms = replicas.job_throughput(0, e2e_wall * 1e3, group_device).milliseconds
    if world > 1:
        dist.barrier()
    decoder.close()
    del decoder
    torch.cuda.empty_cache()
    if rank != 0:
        return None
    peak, peak_kind = measured_peaks()
    per_token_us = decode_ms * 1e3 / (steps * decode_steps)
    bytes_step = step_bytes(config, prompt_length + 1 + decode_steps // 2)
    achieved = bytes_step / (per_token_us * 1e-6) / 1e9
    return {
        "metric": "batch-1 decode tok/s (4-bit g64 static cache)", "value": steps * decode_steps / (decode_ms / 1e3),
        "unit": "tok/s", "n_gpus": world, "steps": steps, "warmup": warmup,
        "ms_per_step": e2e_ms / steps, "higher_is_better": True, "scaling": "strong",
        "vs_baseline": None, "dtype": "bf16", "data": "synthetic (model drawn on the device from a seed)",
        "config": {"workload": spec["description"], "parallelism": f"tp{world}: column-split q/k/v, gate, up and LM head; row-split o and down; "
                   + ("decode step = one streamed-step kernel per rank with peer stores of the partial rows, "
                      if streamed else "two peer-memory sums per layer inside the recorded step, ") + "NCCL in prefill",
                   "step": f"one request: prefill({prompt_length}) + {decode_steps} decode steps; value counts the decode loop only",
                   "l2": f"inputs larger than L2: {bytes_step / world / 1e6:.0f} MB of packed weights per GPU and token"},
        "decode_us_per_token": per_token_us,
        "prefill": {"ms": prefill_ms / steps, "tok_s": prompt_length / (prefill_ms / steps / 1e3), "tokens": prompt_length},
        "e2e": {"value": steps * new_tokens / (e2e_ms / 1e3), "unit": "tok/s",
                "h2d_bytes_per_step": prompt_length * 8, "d2h_bytes_per_step": new_tokens * 8},
        "clocks": clocks,
        "roofline": {"kernel": "stream_step_kernel with peer stores (one launch per rank and token)" if streamed
                     else "recorded decode step (per-operation kernels + peer-memory sums)", "bound": "hbm",
                     "achieved": achieved, "peak": peak * world, "unit": "GB/s", "frac": achieved / (peak * world),
                     "traffic": None, "bytes_per_launch": bytes_step, "us_per_launch": per_token_us,
                     "peak_source": peak_kind, "note": "whole-job bytes over whole-job peak (all GPUs)"},
    }


def check_tp_parity(world: int, rank: int, device) -> dict | None:
    """The sharded decoder against the same decoder on one rank, before anything sharded is timed.

    A 2-layer cut of the Llama-3-8B shape (prompt 128, 16 greedy tokens), drawn from one seed on
    every rank. All ranks run the sharded decoder (per-operation prefill, streamed step kernel with
    peer stores for the steps); rank 0 also runs the unsharded per-operation one step by step
    and compares: the prompt's logits within 2e-2 of max|logit|, and token for token - a differing
    token must be a near-tie of the unsharded logits (gap within the same 2e-2), after which the
    sequences are no longer comparable. Why 2e-2: both sides are bf16 evaluations of the same
    packed model that differ in where partial sums are rounded (a sharded o/down product is rounded
    once per rank before the sum), each is held to 1e-2 against the exact evaluation, and one bf16
    step at max|logit| is already up to 0.8e-2 of it. After a failed check nothing sharded is timed.
    """

    import torch.distributed as dist

    from aotolith_b200.tensor_parallel import StreamedTensorParallelDecoder, TensorParallelDecoder

    prompt_length, new_tokens, tolerance = 128, 16, 2e-2
    model, _ = build_model("llama3_8b", seed=3, device=device, layers=2)
    sharded = StreamedTensorParallelDecoder(model, prompt_length=prompt_length, max_new_tokens=new_tokens,
                                            group_size=GROUP, world=world, rank=rank, device=device)
    prompt = seeded_prompt(model.config.vocab_size, 5, prompt_length)
    got_logits = sharded.prefill(prompt).float().clone()
    got = sharded.greedy_generate(prompt).reshape(-1).tolist()
    torch.cuda.synchronize()
    dist.barrier()
    sharded.close()
    record = None
    if rank == 0:
        single = TensorParallelDecoder(model, prompt_length=prompt_length, max_new_tokens=new_tokens, group_size=GROUP,
                                       world=1, rank=0, device=device, peer_exchange=False)
        raw = single.prefill(prompt)
        logits = raw.float().clone()
        scale = float(logits.abs().max())
        prefill_error = float((got_logits - logits).abs().max()) / scale
        single.token.copy_(single.ops.argmax(raw).reshape(1, 1))
        single.counters.copy_(torch.tensor([prompt_length + 1, 0], dtype=torch.int32, device=device))
        matched, tie_gap = 0, None
        for step in range(new_tokens):
            want = int(single.token.item())
            if got[step] != want:
                tie_gap = float(logits.reshape(-1)[want] - logits.reshape(-1)[got[step]]) / scale
                break
            matched += 1
            if step + 1 < new_tokens:
                single._step(step & 1)
                logits = single.logits.float().clone()
        ok = prefill_error <= tolerance and (tie_gap is None or tie_gap <= tolerance)
        record = {"workload": f"2-layer cut of the Llama-3-8B shape, prompt {prompt_length}, {new_tokens} greedy tokens, "
                              f"tp{world} (streamed step kernel with peer stores) against one rank (per-operation kernels)",
                  "prefill_logits_error": prefill_error, "tolerance": tolerance, "tokens_compared": new_tokens,
                  "tokens_matched": matched, "near_tie_gap_at_first_difference": tie_gap, "ok": ok}
        single.close()
        del single
    del sharded, model
    torch.cuda.empty_cache()
    if rank == 0 and not record["ok"]:
        print(json.dumps({"tp_parity": record}), file=sys.stderr)
    return record


def parity_passed(record, rank: int, device) -> bool:
    """Rank 0's verdict on the parity record, on every rank."""

    import torch.distributed as dist

    ok = 1 if rank != 0 or (isinstance(record, dict) and record.get("ok")) else 0
    verdict = torch.tensor([ok], dtype=torch.int32, device=device)
    dist.broadcast(verdict, src=0)
    return bool(int(verdict.item()))


def run_tp(args) -> None:
    import torch.distributed as dist

    world, rank, device = start_ranks()
    line = measure_tp(world, rank, device, args.steps, max(args.warmup, 3))
    if rank == 0:
        print(json.dumps(line))
    if world > 1:
        dist.destroy_process_group()


def serve_bucketed(shard_world: int, shard_rank: int, device, per_rank: int, warmup: int, model=None) -> dict:
    """One GPU's share of the bucketed workload, in this process: ``{generated, prompt_tokens, ms}``.

    The request list (prompt lengths uniform in [1, 256], ids uniform over the vocabulary) is the
    same seeded list of ``per_rank * shard_world`` requests wherever it is built; this process serves
    requests ``shard_rank, shard_rank + shard_world, ...`` through the public call
    ``greedy_generate(host ids) -> host tokens`` and times them with CUDA events.
    """

    import aotolith_b200 as aoto
    from aotolith_b200 import replicas

    if model is None:
        model, _ = build_model("qwen25_05b_bucketed", seed=0)
    runtime = aoto.compile_qwen2_bucketed(model, prompt_lengths=BUCKETS, max_new_tokens=NEW_TOKENS, quantize=GROUP)
    vocab = model.config.vocab_size
    generator = torch.Generator().manual_seed(7)
    lengths = torch.randint(1, BUCKETS[-1] + 1, (per_rank * shard_world,), generator=generator).tolist()
    requests = [torch.randint(0, vocab, (1, n), generator=generator, dtype=torch.int64).pin_memory() for n in lengths]
    mine = replicas.shard(requests, shard_world, shard_rank)
    for ids in requests[: warmup * 4]:
        runtime.greedy_generate(ids).cpu()
    for bucket in BUCKETS:  # every bucket's stepper is recorded before the clock starts
        runtime.greedy_generate(torch.randint(0, vocab, (1, bucket), dtype=torch.int64)).cpu()
    torch.cuda.synchronize()
    begin, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    begin.record()
    generated = 0
    for ids in mine:
        generated += int(runtime.greedy_generate(ids).cpu().numel())
    end.record()
    torch.cuda.synchronize()
    return {"generated": generated, "prompt_tokens": sum(int(r.numel()) for r in mine), "ms": begin.elapsed_time(end)}


def serve_bucketed_in_child(world: int, rank: int, device, per_rank: int, warmup: int) -> dict:
    """The same share served by a child process that owns this rank's GPU and joins no process group.

    Independent request streams are deployed as plain single-GPU processes, and that is what is
    measured: the child is this file run with ``--bucketed-share rank/world``; it sees only this
    rank's GPU, builds its own runtime and prints ``serve_bucketed``'s figures as one JSON line.
    """

    visible = os.environ.get("CUDA_VISIBLE_DEVICES")
    physical = visible.split(",")[device.index].strip() if visible else str(device.index)
    env = {k: v for k, v in os.environ.items()
           if k not in ("RANK", "LOCAL_RANK", "WORLD_SIZE", "MASTER_ADDR", "MASTER_PORT", "GROUP_RANK", "ROLE_RANK",
                        "LOCAL_WORLD_SIZE", "ROLE_WORLD_SIZE", "TORCHELASTIC_RUN_ID", "TORCHELASTIC_RESTART_COUNT",
                        "TORCHELASTIC_MAX_RESTARTS", "TORCHELASTIC_USE_AGENT_STORE", "TORCH_NCCL_ASYNC_ERROR_HANDLING")}
    env["CUDA_VISIBLE_DEVICES"] = physical
    command = [sys.executable, str(Path(__file__).resolve()), "--bucketed-share", f"{rank}/{world}",
               "--requests-per-gpu", str(per_rank), "--warmup", str(warmup)]
    done = subprocess.run(command, env=env, capture_output=True, text=True, timeout=1800)
    if done.returncode != 0:
        raise SystemExit(f"the bucketed child of rank {rank} failed ({done.returncode}):\n{done.stderr[-2000:]}")
    return json.loads(done.stdout.strip().splitlines()[-1])


def measure_bucketed(world: int, rank: int, device, per_rank: int, warmup: int, with_clocks: bool = True,
                     model=None, in_child: bool = False) -> dict | None:
    """Independent request streams over a bucketed runtime, one runtime per GPU; the record on rank 0.

    ``in_child``: every rank hands its share to a single-GPU child process (see
    ``serve_bucketed_in_child``) and only the figures cross the process group.
    """

    import torch.distributed as dist

    from aotolith_b200 import replicas

    spec = WORKLOADS["qwen25_05b_bucketed"]
    sampler = ClockSampler(device.index)
    if rank == 0 and with_clocks:
        sampler.start()
    if world > 1:
        dist.barrier()
    if in_child:
        share = serve_bucketed_in_child(world, rank, device, per_rank, warmup)
    else:
        share = serve_bucketed(world, rank, device, per_rank, warmup, model)
    clocks = sampler.stop() if rank == 0 and with_clocks else None
    group_device = device if world > 1 else None
    job = replicas.job_throughput(share["generated"], share["ms"], group_device)
    prompt_tokens = replicas.job_throughput(share["prompt_tokens"], share["ms"], group_device).units
    if world > 1:
        dist.barrier()
    torch.cuda.empty_cache()
    if rank != 0:
        return None
    return {
        "metric": "bucketed runtime generated tok/s (4-bit g64 static cache, independent request streams)",
        "value": job.per_second, "unit": "tok/s", "n_gpus": world, "warmup": warmup,
        "ms_per_request": job.milliseconds / max(per_rank, 1), "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": {"workload": spec["description"], "requests": per_rank * world, "requests_per_gpu": per_rank,
                   "request": "prefill (left-padded to its bucket) + 64 greedy tokens",
                   "parallelism": f"{world} independent request stream(s), one bucketed runtime per GPU"
                                  + (", each in a single-GPU process of its own" if in_child else ""),
                   "timing": "CUDA events around each GPU's whole share (clock samples cover runtime construction too); "
                             "job = all generated tokens / slowest GPU",
                   "l2": "inputs larger than L2: 262 MB of packed weights are streamed per token"},
        "e2e": {"value": job.per_second, "unit": "tok/s",
                "h2d_bytes_per_request": int(8 * prompt_tokens / max(per_rank * world, 1)),
                "d2h_bytes_per_request": NEW_TOKENS * 8},
        "prompt_tok_s": prompt_tokens / (job.milliseconds / 1e3),
        "clocks": clocks,
    }


def run_bucketed(args) -> None:
    import torch.distributed as dist

    world, rank, device = start_ranks()
    line = measure_bucketed(world, rank, device, 16 * args.steps, max(args.warmup, 3), in_child=world > 1)
    if rank == 0:
        line.update(steps=args.steps, ms_per_step=line["ms_per_request"] * 16)
        line["config"]["step"] = "16 requests per GPU"
        print(json.dumps(line))
    if world > 1:
        dist.destroy_process_group()


def run_bucketed_share(args) -> None:
    """Child of ``serve_bucketed_in_child``: one GPU, no process group, one JSON line."""

    shard_rank, shard_world = (int(v) for v in args.bucketed_share.split("/"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device; the cuda-sm100 target has no CPU path")
    torch.cuda.set_device(0)
    share = serve_bucketed(shard_world, shard_rank, torch.device("cuda", 0), args.requests_per_gpu, max(args.warmup, 3))
    print(json.dumps(share))


def run_probe(name: str, probe_prompt: int = 0) -> None:
    """Small fixed cases for a profiler: a handful of launches of one kernel, a few GB at most.

    ``lm_head``  six packed GEMV launches over three copies of a [151936, 896] weight (RMS norm fused);
    ``rows_gemm`` six launches of the packed product with 16 rows over three copies of a [151936, 896] weight;
    ``gemm``     six packed GEMM launches, K=4096 N=14336 M=1024, over five weight copies;
    ``attention`` six launches of prefill attention, 32 query / 8 kv heads, 1024 x 1024, D = 128, causal mask;
    ``i8``       eight-bit packed projections of the 0.5B shape, timed with CUDA events;
    ``i8_decoder`` one request of the default workload with the decoder packed with eight bits;
    ``rows``     one decode step over eight tokens (``decode_rows=8``) against eight one-token plan calls;
    ``dense_lm_head`` six dense GEMV launches over two copies of a [151936, 896] bf16 weight;
    ``dense``    dense bf16 projections of the 0.5B and 8B shapes, timed with CUDA events;
    ``dense_decoder`` one request of the default workload with the decoder's bf16 weights as they are;
    ``step``     a 4-layer Qwen2.5-0.5B-shaped decoder: prefill, then six launches of the step kernel;
    ``trace``    the same, then one more step with the kernel's own per-stage timeline printed;
    ``trace_llama`` the timeline for a 2-layer cut of the Llama-3-8B shape (prompt 128);
    ``trace_llama_long`` the same with the configuration's window (prompt 1024, 256 new tokens).
    """

    global PROMPT, NEW_TOKENS

    from aotolith_b200 import ops

    device = torch.device("cuda", 0)
    generator = torch.Generator().manual_seed(1)
    if name == "lm_head":
        N, K = 151936, 896
        packs = [torch.randint(-2**31, 2**31 - 1, (N, K // 8), dtype=torch.int32, generator=generator).to(device) for _ in range(3)]
        scales = [(torch.rand(N, K // 64, generator=generator) * 0.01 + 0.001).bfloat16().to(device) for _ in range(3)]
        x = torch.randn(1, K, generator=generator).bfloat16().to(device)
        norm = (torch.randn(K, generator=generator) * 0.1 + 1).bfloat16().to(device)
        out = torch.empty(1, N, dtype=torch.bfloat16, device=device)
        for i in range(6):
            ops.qmatmul(x, packs[i % 3], scales[i % 3], group_size=GROUP, norm_weight=norm, rms_norm_eps=1e-6, out=out)
        torch.cuda.synchronize()
        print(json.dumps({"probe": name, "variant": ops.qmatmul_variant(1, N, K, GROUP), "max": float(out.float().abs().max())}))
    elif name == "rows_gemm":
        # six launches of the packed product with 16 activation rows over three copies of a [151936, 896] weight
        N, K, M = 151936, 896, 16
        packs = [torch.randint(-2**31, 2**31 - 1, (N, K // 8), dtype=torch.int32, generator=generator).to(device) for _ in range(3)]
        scales = [(torch.rand(N, K // 64, generator=generator) * 0.01 + 0.001).bfloat16().to(device) for _ in range(3)]
        x = torch.randn(M, K, generator=generator).bfloat16().to(device)
        out = torch.empty(M, N, dtype=torch.bfloat16, device=device)
        for i in range(6):
            ops.qmatmul(x, packs[i % 3], scales[i % 3], group_size=GROUP, out=out)
        torch.cuda.synchronize()
        print(json.dumps({"probe": name, "variant": ops.qmatmul_variant(M, N, K, GROUP), "max": float(out.float().abs().max())}))
    elif name == "attention":
        heads, kv_heads, length, dim = 32, 8, 1024, 128
        q = torch.randn(1, heads, length, dim, generator=generator).bfloat16().to(device)
        k = torch.randn(1, kv_heads, length, dim, generator=generator).bfloat16().to(device)
        v = torch.randn(1, kv_heads, length, dim, generator=generator).bfloat16().to(device)
        causal = torch.ones((length, length), dtype=torch.bool).tril()[None, None].to(device)
        mask = ops.mask_select(causal, 0.0, float("-inf"))
        start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        for i in range(6):
            if i == 1:
                start.record()
            out = ops.attention(q, k, v, mask, scale=dim ** -0.5)
        stop.record()
        torch.cuda.synchronize()
        us = start.elapsed_time(stop) * 1e3 / 5
        flops = 4.0 * heads * length * length * dim
        print(json.dumps({"probe": name, "us": us, "tflops_dense": flops / us / 1e6, "tflops_causal_half": flops / 2 / us / 1e6,
                          "max": float(out.float().abs().max())}))
    elif name == "i8":
        # eight-bit words (four codes a word): the Qwen-0.5B projections of one decode step, and the prompt rows
        results = []
        for K, N, M in ((896, 1152, 1), (896, 4864, 1), (4864, 896, 1), (896, 151936, 1), (896, 4864, 128)):
            copies = max(3, min(48, int(300e6 // (N * K)) + 1))
            packs = [torch.randint(-2**31, 2**31 - 1, (N, K // 4), dtype=torch.int32, generator=generator).to(device)
                     for _ in range(copies)]
            scales = [(torch.rand(N, K // GROUP, generator=generator) * 0.001 + 0.0001).bfloat16().to(device) for _ in range(copies)]
            x = torch.randn(M, K, generator=generator).bfloat16().to(device)
            out = torch.empty(M, N, dtype=torch.bfloat16, device=device)
            start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            rounds = 4
            for i in range(copies * (rounds + 1)):
                if i == copies:
                    start.record()
                ops.qmatmul(x, packs[i % copies], scales[i % copies], group_size=GROUP, out=out, weight_bits=8)
            stop.record()
            torch.cuda.synchronize()
            us = start.elapsed_time(stop) * 1e3 / (copies * rounds)
            nbytes = N * K + N * (K // GROUP) * 2 + M * K * 2 + M * N * 2
            results.append({"K": K, "N": N, "M": M, "variant": ops.qmatmul_variant(M, N, K, GROUP, weight_bits=8),
                            "us": round(us, 2), "gbs": round(nbytes / us / 1e3, 1)})
        print(json.dumps({"probe": name, "note": "back-to-back launches over rotating weight copies larger than L2", "results": results}))
    elif name == "dense_lm_head":
        # six launches of the dense GEMV over two copies of a [151936, 896] bf16 weight (544 MB, larger than L2)
        N, K = 151936, 896
        weights = [torch.randn(N, K, device=device, dtype=torch.bfloat16) * 0.02 for _ in range(2)]
        x = torch.randn(1, K, generator=generator).bfloat16().to(device)
        out = torch.empty(1, N, dtype=torch.bfloat16, device=device)
        for i in range(6):
            ops.dmatmul(x, weights[i % 2], out=out)
        torch.cuda.synchronize()
        print(json.dumps({"probe": name, "variant": ops.dmatmul_variant(1, N, K), "max": float(out.float().abs().max())}))
    elif name == "dense":
        # dense bf16 weights: the projections of one decode step at the 0.5B and 8B shapes, and prompt rows
        results = []
        for K, N, M, paired in ((896, 151936, 1, False), (896, 4864, 1, True), (4864, 896, 1, False), (4096, 14336, 1, True),
                                (14336, 4096, 1, False), (4096, 6144, 1, False), (896, 4864, 8, False), (896, 4864, 128, False)):
            nbytes = N * K * 2 * (2 if paired else 1)
            copies = max(2, int(400e6 // nbytes) + 1)
            weights = [(torch.randn(N, K, device=device, dtype=torch.bfloat16) * 0.02) for _ in range(copies * (2 if paired else 1))]
            x = torch.randn(M, K, generator=generator).bfloat16().to(device)
            out = torch.empty(M, N, dtype=torch.bfloat16, device=device)
            start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            rounds = 4
            for i in range(copies * (rounds + 1)):
                if i == copies:
                    start.record()
                ops.dmatmul(x, weights[i % copies], weight2=weights[copies + i % copies] if paired else None, out=out)
            stop.record()
            torch.cuda.synchronize()
            us = start.elapsed_time(stop) * 1e3 / (copies * rounds)
            results.append({"K": K, "N": N, "M": M, "paired": paired, "variant": ops.dmatmul_variant(M, N, K, paired),
                            "us": round(us, 2), "gbs": round((nbytes + M * K * 2 + M * N * 2) / us / 1e3, 1)})
            del weights
        print(json.dumps({"probe": name, "note": "back-to-back launches over rotating weight copies larger than L2", "results": results}))
    elif name == "dense_decoder":
        # the whole decoder with its bf16 weights as they are: one request of the default workload, CUDA events
        import aotolith_b200 as aoto
        from aotolith_b200.models.synthetic import qwen25_05b_shaped

        model = qwen25_05b_shaped(seed=0)
        runtime = aoto.compile_qwen2_static_cache(model, prompt_length=PROMPT, max_new_tokens=NEW_TOKENS)
        prompt = seeded_prompt(model.config.vocab_size, 1).to(device)
        runtime.greedy_generate(prompt)
        torch.cuda.synchronize()
        marks = [torch.cuda.Event(enable_timing=True) for _ in range(3)]
        marks[0].record()
        logits, compact = runtime.prefill_ids(prompt)
        cache = runtime.pad_cache(compact)
        marks[1].record()
        tokens = runtime.greedy_generate(prompt)
        marks[2].record()
        torch.cuda.synchronize()
        prefill_ms = marks[0].elapsed_time(marks[1])
        request_ms = marks[1].elapsed_time(marks[2])
        decode_us = (request_ms - prefill_ms) * 1e3 / (NEW_TOKENS - 1)
        print(json.dumps({"probe": name, "workload": "Qwen2.5-0.5B-shaped, dense bf16, prompt 128, 64 greedy tokens",
                          "prefill_ms": round(prefill_ms, 3), "request_ms": round(request_ms, 3),
                          "decode_us_per_token": round(decode_us, 1), "decode_tok_s": round(1e6 / decode_us, 1),
                          "tokens": int(tokens.numel())}))
    elif name == "rows":
        # a step over eight tokens against eight one-token steps, default workload, CUDA events
        from aotolith_b200.models.synthetic import qwen25_05b_shaped

        model = qwen25_05b_shaped(seed=0)
        record = measure_rows(model, seeded_prompt(model.config.vocab_size, 1), device)
        print(json.dumps({"probe": name, **record}))
    elif name == "i8_decoder":
        # the whole decoder packed with eight bits: one request of the default workload, timed with CUDA events
        import aotolith_b200 as aoto
        from aotolith_b200.models.synthetic import qwen25_05b_shaped

        model = qwen25_05b_shaped(seed=0)
        runtime = aoto.compile_qwen2_static_cache(model, prompt_length=PROMPT, max_new_tokens=NEW_TOKENS,
                                                  quantize=GROUP, quantize_bits=8)
        prompt = seeded_prompt(model.config.vocab_size, 1).to(device)
        runtime.greedy_generate(prompt)
        torch.cuda.synchronize()
        marks = [torch.cuda.Event(enable_timing=True) for _ in range(3)]
        marks[0].record()
        logits, compact = runtime.prefill_ids(prompt)
        cache = runtime.pad_cache(compact)
        marks[1].record()
        tokens = runtime.greedy_generate(prompt)
        marks[2].record()
        torch.cuda.synchronize()
        prefill_ms = marks[0].elapsed_time(marks[1])
        request_ms = marks[1].elapsed_time(marks[2])
        decode_us = (request_ms - prefill_ms) * 1e3 / (NEW_TOKENS - 1)
        print(json.dumps({"probe": "i8_decoder", "workload": "Qwen2.5-0.5B-shaped, 8-bit g64, prompt 128, 64 greedy tokens",
                          "prefill_ms": round(prefill_ms, 3), "request_ms": round(request_ms, 3),
                          "decode_us_per_token": round(decode_us, 1), "decode_tok_s": round(1e6 / decode_us, 1),
                          "tokens": int(tokens.numel())}))
    elif name == "gemm":
        K, N, M = 4096, 14336, 1024
        packs = [torch.randint(-2**31, 2**31 - 1, (N, K // 8), dtype=torch.int32, generator=generator).to(device) for _ in range(5)]
        scales = [(torch.rand(N, K // 64, generator=generator) * 0.01 + 0.001).bfloat16().to(device) for _ in range(5)]
        x = torch.randn(M, K, generator=generator).bfloat16().to(device)
        out = torch.empty(M, N, dtype=torch.bfloat16, device=device)
        for i in range(6):
            ops.qmatmul(x, packs[i % 5], scales[i % 5], group_size=GROUP, out=out)
        torch.cuda.synchronize()
        print(json.dumps({"probe": name, "variant": ops.qmatmul_variant(M, N, K, GROUP), "max": float(out.float().abs().max())}))
    else:
        import aotolith_b200 as aoto
        from aotolith_b200.models.session import decode_session
        from aotolith_b200.models.synthetic import qwen25_05b_shaped

        if name in ("trace_llama", "trace_llama_long"):
            from aotolith_b200.models.synthetic import llama3_8b_shaped

            if name == "trace_llama_long":
                PROMPT, NEW_TOKENS = (probe_prompt or 1024), 256
            model = llama3_8b_shaped(seed=0, layers=2, device=device)
            runtime = aoto.compile_llama_static_cache(model, prompt_length=PROMPT, max_new_tokens=NEW_TOKENS, quantize=GROUP)
        else:
            model = qwen25_05b_shaped(seed=0, layers=4)
            runtime = aoto.compile_qwen2_static_cache(model, prompt_length=PROMPT, max_new_tokens=NEW_TOKENS, quantize=GROUP)
        prompt = seeded_prompt(model.config.vocab_size, 1).to(device)
        logits, compact = runtime.prefill_ids(prompt)
        cache = runtime.pad_cache(compact)
        token = ops.argmax(logits[:, -1, :]).reshape(1, 1)
        session = decode_session(runtime)
        tokens = session.run(token, cache, PROMPT, 6)
        torch.cuda.synchronize()
        print(json.dumps({"probe": name, "mode": session.mode, "tokens": tokens.tolist()}))
        if name in ("trace", "trace_llama", "trace_llama_long") and session.mode == "kernel":
            print_stage_trace(runtime, session, token, cache)


def main() -> None:
    parser = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    parser.add_argument("--gpus", type=int, default=1)
    parser.add_argument("--steps", type=int, default=20)
    parser.add_argument("--warmup", type=int, default=3)
    parser.add_argument("--impl", choices=("ours", "reference"), default="ours")
    parser.add_argument("--workload", choices=sorted(WORKLOADS), default="qwen25_05b")
    parser.add_argument("--skip-cpu", action="store_true", help="leave the cpu_baseline object out")
    parser.add_argument("--skip-multi", action="store_true",
                        help="with more than one GPU: leave the tensor-parallel and bucketed records out")
    parser.add_argument("--probe", choices=("lm_head", "rows_gemm", "gemm", "attention", "i8", "i8_decoder", "dense", "dense_lm_head", "dense_decoder", "rows", "step", "trace", "trace_llama",
                                            "trace_llama_long"), default=None,
                        help="run a small fixed case of one kernel for a profiler instead of the benchmark")
    parser.add_argument("--probe-prompt", type=int, default=0, help="with --probe trace_llama_long: another prompt length")
    parser.add_argument("--bucketed-share", default=None, metavar="RANK/WORLD",
                        help="internal: serve one GPU's share of the bucketed workload and print its figures")
    parser.add_argument("--requests-per-gpu", type=int, default=512, help="with --bucketed-share")
    args = parser.parse_args()
    if args.bucketed_share is not None:
        run_bucketed_share(args)
        return
    if args.probe is not None:
        run_probe(args.probe, args.probe_prompt)
        return
    global PROMPT, NEW_TOKENS
    PROMPT = WORKLOADS[args.workload].get("prompt", PROMPT)
    NEW_TOKENS = WORKLOADS[args.workload].get("new_tokens", NEW_TOKENS)
    if args.impl == "reference":
        run_reference(args)
    elif args.workload == "qwen25_05b_bucketed":
        run_bucketed(args)
    elif args.workload == "llama3_8b_tp":
        run_tp(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
