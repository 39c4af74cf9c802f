#!/usr/bin/env python3
"""Decode and prefill throughput of the engine at Llama-3.1-8B layer sizes on one B200.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--impl ours|reference]

One JSON line on stdout.  ``value`` is decoded tokens a second at batch 8 (device-timed over exactly K
decode steps after W warm-up steps, prompts of 2,048 random ids, decoding on from there; when K is small the
K steps are timed several times over, decoding on, and the median counts); ``e2e`` is the same through the
Python entry point with host tokens in and out; ``prefill`` is one 2,048-token prompt; ``points`` holds
decoding at batch 1 and 64 and the two serving workloads of the smaller sizes (64 mixed requests at the
Llama-3.2-1B sizes, 16 long-context requests at the Llama-3.2-3B sizes) through the Python entry point;
``roofline`` relates the decode step to the measured HBM bandwidth.  Weights are random (N(0, 0.02), norm weights 1) and token ids synthetic: there is no
network for checkpoints or datasets.  Several GPUs are not supported: one line says so, exit code 2.

The reference has no single-GPU Llama-3.1-8B number; its own harness times ``generate`` on random
prompts with a device synchronisation on both sides (src/torchinferno/benchmarks/torchinferno_llama.py:169-194,
347-348), which is what ``--impl reference`` does with the unmodified reference from ``baseline/_ref``.
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

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

# Layer sizes of Llama-3.1-8B (the third configuration of BASELINE.json).
LLAMA_8B = {
    "architectures": ["LlamaForCausalLM"], "model_type": "llama", "vocab_size": 128256, "hidden_size": 4096,
    "intermediate_size": 14336, "num_hidden_layers": 32, "num_attention_heads": 32, "num_key_value_heads": 8,
    "head_dim": 128, "max_position_embeddings": 131072, "rope_theta": 500000.0,
    "rope_scaling": {"rope_type": "llama3", "factor": 8.0, "low_freq_factor": 1.0, "high_freq_factor": 4.0,
                     "original_max_position_embeddings": 8192},
    "rms_norm_eps": 1e-5, "tie_word_embeddings": False, "torch_dtype": "bfloat16",
}
FULL_LAYERS = 32
PROMPT_LEN = 2048
CONTEXT = 4096
PAGE_SIZE = 16
METRIC = "decode tok/s at batch 8 (Llama-3.1-8B bf16, 2048-token prompts, decode towards 4096 context)"


def load_peaks() -> dict:
    path = ROOT / "MEASURED_PEAKS.json"
    if path.is_file():
        data = json.loads(path.read_text())
        return {"hbm_gbs": float(data["hbm_gbs"]), "bf16_tflops": float(data["bf16_tflops"]),
                "bf16_tflops_sustained": float(data.get("bf16_tflops_sustained", data["bf16_tflops"])), "source": "measured"}
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0, "source": "fallback"}


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs (every 200 ms), and once
    more through NVML at a moment the caller chooses (``snap``: while the timed steps are still running on the GPU),
    so that a region shorter than the sampling period has a sample too.  Reading only: nothing is set."""
    QUERY = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
             "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
             "clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int = 0) -> None:
        self.lines: list[str] = []
        self.proc = None
        self.nvml = None
        try:
            import pynvml
            pynvml.nvmlInit()
            self.nvml = (pynvml, pynvml.nvmlDeviceGetHandleByIndex(index))
        except Exception:      # (no NVML binding: the periodic samples remain)
            self.nvml = None
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--id={index}", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits", "-lms", "200"],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None

    def _read(self) -> None:
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def mark(self) -> int:
        return len(self.lines)

    def snap(self) -> None:
        """One sample now, in the format of the periodic ones."""
        if self.nvml is None:
            return
        nv, handle = self.nvml
        try:
            sm = nv.nvmlDeviceGetClockInfo(handle, nv.NVML_CLOCK_SM)
            top = nv.nvmlDeviceGetMaxClockInfo(handle, nv.NVML_CLOCK_SM)
            watts = nv.nvmlDeviceGetPowerUsage(handle) / 1e3
            bits = nv.nvmlDeviceGetCurrentClocksEventReasons(handle)
            flag = lambda bit: "Active" if bits & bit else "Not Active"
            self.lines.append(", ".join([str(sm), str(top), f"{watts:.2f}", flag(nv.nvmlClocksEventReasonHwSlowdown),
                                         flag(nv.nvmlClocksEventReasonHwThermalSlowdown),
                                         flag(nv.nvmlClocksEventReasonSwThermalSlowdown),
                                         flag(nv.nvmlClocksEventReasonSwPowerCap)]))
        except Exception:
            pass

    def stop(self) -> None:
        if self.proc is not None:
            self.proc.terminate()
            try:
                self.proc.wait(timeout=5)
            except subprocess.TimeoutExpired:
                self.proc.kill()

    def summary(self, start: int = 0, end: int | None = None) -> dict:
        rows = [l.split(", ") for l in self.lines[start:end] if l.count(",") >= 6]
        if not rows:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["unsampled"]}
        clocks = [float(r[0]) for r in rows if r[0].replace(".", "").isdigit()]
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        reasons = [n for i, n in enumerate(names) if any(r[3 + i].strip().lower() == "active" for r in rows)]
        return {"sm_mhz": statistics.median(clocks) if clocks else None, "sm_max_mhz": float(rows[0][1]),
                "power_w_max": max(float(r[2]) for r in rows), "samples": len(rows), "reasons": reasons}


# ------------------------------------------------------------------- ours
def model_numbers(model, layers: int) -> dict:
    cfg = model.spec.config
    h, i, v = cfg["hidden_size"], cfg["intermediate_size"], cfg["vocab_size"]
    heads, kv, d = cfg["num_attention_heads"], cfg["num_key_value_heads"], cfg["head_dim"]
    per_layer_params = h * (heads + 2 * kv) * d + heads * d * h + 3 * h * i
    return {"matmul_params": layers * per_layer_params + v * h, "per_layer_params": per_layer_params,
            "kv_bytes_per_token": layers * 2 * kv * d * 2, "heads": heads, "head_dim": d, "layers": layers,
            "lm_head_params": v * h}


def prefill_requests(runner, ids, prompts, chunk: int) -> list[int]:
    """Run the prompts through the step function in portions; returns the first drawn token of each."""
    import torch
    from torchinferno_b200.engine.batch import StepEntry
    from torchinferno_b200.kernels import ops
    first = []
    for rid, prompt in zip(ids, prompts):
        logits = None
        for pos in range(0, len(prompt), chunk):
            part = prompt[pos:pos + chunk]
            last = pos + chunk >= len(prompt)
            logits = runner.step([StepEntry(rid, part, [len(part) - 1] if last else [])])
        out = torch.empty(1, dtype=torch.int32, device=logits.device)
        ops.sample(logits, out)
        first.append(int(out.item()))
    return first


REPEAT_TARGET_STEPS = 240     # a run of fewer timed steps than this is repeated (decoding on) until it has as many
MAX_REPEATS = 15


def timed_decode(runner, batch: int, steps: int, warmup: int, numbers: dict, sampler, seed: int) -> dict:
    """Prefill ``batch`` prompts, then time exactly ``steps`` device-side decode steps; a short run is repeated
    from where the last repeat ended and the median repeat counts (a region of 70 ms is at the mercy of one
    clock change)."""
    import torch
    from torchinferno_b200.kernels import ops
    vocab = runner.model.spec.vocab_size
    g = torch.Generator().manual_seed(seed)
    prompts = torch.randint(0, vocab, (batch, PROMPT_LEN), generator=g).tolist()
    ids = [f"b{batch}-{i}" for i in range(batch)]
    first = prefill_requests(runner, ids, prompts, PROMPT_LEN)
    temps, seeds = [0.0] * batch, list(range(batch))
    drawn = runner.decode_loop(ids, first, warmup, temperature=temps, seeds=seeds)   # captures the graph too
    torch.cuda.synchronize()
    last = drawn[-1].tolist() if warmup else first
    room = CONTEXT + PAGE_SIZE - 1 - PROMPT_LEN - warmup
    repeats = max(1, min(MAX_REPEATS, -(-REPEAT_TARGET_STEPS // steps), room // steps))
    start_context = PROMPT_LEN + warmup
    mark = sampler.mark()
    runs = []
    for r in range(repeats):
        launches_before, replays_before = ops.launch_count(), runner.graph_replays
        begin, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        begin.record()
        drawn = runner.decode_loop(ids, last, steps)
        end.record()
        sampler.snap()                   # (the steps are launched, not finished: the GPU is at work on them)
        torch.cuda.synchronize()
        last = drawn[-1].tolist()
        graph = runner._graphs[batch]
        launches = (ops.launch_count() - launches_before) + (runner.graph_replays - replays_before) * graph.launches
        runs.append((begin.elapsed_time(end), start_context + r * steps, launches))
    clocks = sampler.summary(mark, sampler.mark())
    ms, context, launches = sorted(runs)[len(runs) // 2]          # the median repeat, with its own contexts
    mean_context = context + (steps + 1) / 2                      # cached tokens a step reads, on average
    step_bytes = numbers["matmul_params"] * 2 + batch * mean_context * numbers["kv_bytes_per_token"]
    runner.end(ids)
    return {"batch": batch, "steps": steps, "ms": ms, "ms_per_step": ms / steps, "tokens_per_s": batch * steps / (ms / 1e3),
            "context_from": context, "context_to": context + steps, "step_bytes": step_bytes, "repeats": repeats,
            "repeat_ms": [round(m, 3) for m, _, _ in runs],
            "achieved_gbs": step_bytes / (ms / steps / 1e3) / 1e9, "launches": launches, "clocks": clocks}


def timed_prefill(runner, numbers: dict, iters: int, warmup: int, seed: int) -> dict:
    import torch
    from torchinferno_b200.engine.batch import StepEntry
    vocab = runner.model.spec.vocab_size
    g = torch.Generator().manual_seed(seed)
    times = []
    for it in range(warmup + iters):
        prompt = torch.randint(0, vocab, (PROMPT_LEN,), generator=g).tolist()
        begin, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        begin.record()
        runner.step([StepEntry(f"p{it}", prompt, [PROMPT_LEN - 1])])
        end.record()
        torch.cuda.synchronize()
        runner.end([f"p{it}"])
        if it >= warmup:
            times.append(begin.elapsed_time(end))
    ms = statistics.median(times)
    t = PROMPT_LEN
    linear = 2 * t * (numbers["matmul_params"] - numbers["lm_head_params"]) + 2 * numbers["lm_head_params"]
    attention = numbers["layers"] * 4 * numbers["heads"] * numbers["head_dim"] * t * (t + 1) / 2   # causal
    return {"ms": ms, "tokens": t, "flops": linear + attention, "value": t / (ms / 1e3)}


def timed_e2e(model, batch: int, steps: int, warmup: int, seed: int) -> dict:
    """Through the Python entry point: host token ids in, host token ids out, every step.  As the device-timed run,
    a short run is repeated (decoding on) and the median repeat counts."""
    import torch
    from torchinferno_b200.config.engine_config import EngineConfig
    from torchinferno_b200.engine.engine import InferenceEngine
    from torchinferno_b200.engine.types import GenerateRequest, SamplingConfig
    from torchinferno_b200.kernels import gemm
    room = CONTEXT - PROMPT_LEN - batch - warmup - 2
    repeats = max(1, min(MAX_REPEATS, -(-REPEAT_TARGET_STEPS // steps), room // steps))
    total_steps = steps * repeats
    config = EngineConfig(model="<in memory>", dtype="bfloat16", page_size=PAGE_SIZE, max_batch_size=batch, gemm_backend=gemm.get_backend(),
                          max_num_batched_tokens=PROMPT_LEN, prefill_chunk_size=PROMPT_LEN,
                          kv_cache_tokens=batch * (PROMPT_LEN + batch + warmup + total_steps + 2 * PAGE_SIZE))
    engine = InferenceEngine(model, config)
    g = torch.Generator().manual_seed(seed + 99)
    prompts = torch.randint(0, model.spec.vocab_size, (batch, PROMPT_LEN), generator=g).tolist()
    for i, prompt in enumerate(prompts):
        engine.submit(GenerateRequest(f"e{i}", prompt_token_ids=prompt,
                                      sampling=SamplingConfig(max_tokens=batch + warmup + total_steps + 2, temperature=0.0)))
    # run until every request decodes, plus the warm-up steps
    while any(r.prefilling for r in engine.scheduler.running) or engine.scheduler.waiting:
        engine.step()
    for _ in range(warmup):
        engine.step()
    torch.cuda.synchronize()
    h2d0, d2h0, ahead0 = engine.stats["h2d_bytes"], engine.stats["d2h_bytes"], engine.stats["steps_ahead"]
    runs = []
    for _ in range(repeats):
        begin, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        begin.record()
        tokens = 0
        for _ in range(steps):
            tokens += sum(1 for e in engine.step() if e.token is not None)
        end.record()
        torch.cuda.synchronize()
        if tokens != batch * steps:   # (earlier requests decode while later prompts are computed: max_tokens leaves room for that)
            raise RuntimeError(f"the end-to-end run drew {tokens} tokens, not {batch * steps}: a request ended inside the timed region")
        runs.append(begin.elapsed_time(end))
    ms = sorted(runs)[len(runs) // 2]
    for i in range(batch):
        engine.cancel(f"e{i}")
    engine.close()
    return {"value": tokens / (ms / 1e3), "unit": "tok/s", "ms_per_step": ms / steps, "tokens": tokens, "repeats": repeats,
            "h2d_bytes_per_step": (engine.stats["h2d_bytes"] - h2d0) / total_steps,
            "d2h_bytes_per_step": (engine.stats["d2h_bytes"] - d2h0) / total_steps,
            # steps launched before the host had read the tokens of the step before (async scheduling)
            "steps_launched_ahead": engine.stats["steps_ahead"] - ahead0}


# The two serving workloads of the smaller sizes (the fourth and fifth configurations of BASELINE.json), run
# through InferenceEngine as a user would: requests in, tokens out, continuous batching in between.
WORKLOADS = {
    "mixed_1b": dict(preset="llama-3.2-1b.json", requests=64, prompt_min=16, prompt_max=2048, new_tokens=256, temperature=0.0),
    "long_3b": dict(preset="llama-3.2-3b.json", requests=16, prompt_min=8192, prompt_max=8192, new_tokens=512, temperature=0.7),
}


def timed_workload(name: str, peaks: dict, gemm_backend: str) -> dict:
    """Output tokens a second of one workload, the split of its steps (those that carry prompt portions, those
    that only decode) and, for the decode steps, the bytes they must read (every weight once, the cache of the
    running requests) over their time.  The harness of the reference for such runs:
    src/torchinferno/benchmarks/torchinferno_llama.py:58-437."""
    import torch
    from torchinferno_b200.config.engine_config import EngineConfig
    from torchinferno_b200.engine.engine import InferenceEngine
    from torchinferno_b200.engine.factory import random_model
    from torchinferno_b200.engine.types import GenerateRequest, SamplingConfig
    w = WORKLOADS[name]
    config = json.loads((ROOT / "torchinferno_b200" / "config" / "presets" / w["preset"]).read_text())
    model = random_model(config, seed=0, dtype="bfloat16")
    longest = w["prompt_max"] + w["new_tokens"]
    engine = InferenceEngine(model, EngineConfig(
        model="<in memory>", dtype="bfloat16", page_size=PAGE_SIZE, max_batch_size=w["requests"], gemm_backend=gemm_backend,
        max_model_len=longest + PAGE_SIZE, kv_cache_tokens=w["requests"] * (longest + PAGE_SIZE)))
    weight_bytes, kv_bytes = model.weight_bytes(), engine.runner.cache.kv_bytes_per_token()
    result = {}
    for it in range(2):                                   # (the first pass warms up: the same requests, so that every
        g = torch.Generator().manual_seed(17)             # batch size the run meets has its decode step captured)
        lengths = torch.randint(w["prompt_min"], w["prompt_max"] + 1, (w["requests"],), generator=g).tolist()
        for i, n in enumerate(lengths):
            engine.submit(GenerateRequest(f"{name}-{it}-{i}", prompt_token_ids=torch.randint(0, model.spec.vocab_size, (n,), generator=g).tolist(),
                                          sampling=SamplingConfig(w["new_tokens"], w["temperature"], (), 1000 + i)))
        split = {"prefill": [0, 0.0], "decode": [0, 0.0]}
        decode_bytes, tokens = 0, 0
        torch.cuda.synchronize()
        begin = last = time.perf_counter()
        while engine.scheduler.has_work():
            sched, cache = engine.scheduler, engine.runner.cache
            prefilling = bool(sched.waiting) or any(r.prefilling for r in sched.running)
            held = sum(cache.length(r.request_id) for r in sched.running if r.request_id in cache)
            tokens += sum(1 for e in engine.step() if e.token is not None)
            now = time.perf_counter()
            kind = "prefill" if prefilling else "decode"
            split[kind][0] += 1
            split[kind][1] += now - last
            if not prefilling:
                decode_bytes += weight_bytes + held * kv_bytes
            last = now
        torch.cuda.synchronize()
        seconds = time.perf_counter() - begin
        split["decode"][1] += time.perf_counter() - last
        decode_seconds = max(split["decode"][1], 1e-9)
        result = {name: round(tokens / seconds, 1), f"{name}_seconds": round(seconds, 3),
                  f"{name}_prompt_tokens": sum(lengths), f"{name}_output_tokens": tokens,
                  f"{name}_prefill_steps": split["prefill"][0],
                  f"{name}_prefill_ms_per_step": round(1e3 * split["prefill"][1] / max(1, split["prefill"][0]), 3),
                  f"{name}_decode_steps": split["decode"][0],
                  f"{name}_decode_ms_per_step": round(1e3 * decode_seconds / max(1, split["decode"][0]), 3),
                  f"{name}_decode_gbs": round(decode_bytes / decode_seconds / 1e9, 1),
                  f"{name}_decode_hbm_frac": round(decode_bytes / decode_seconds / 1e9 / peaks["hbm_gbs"], 4),
                  f"{name}_preemptions": engine.scheduler.stats["preemptions"]}
    engine.close()
    del engine, model
    torch.cuda.empty_cache()
    return result


def run_ours(args) -> dict:
    import torch
    from torchinferno_b200.engine.factory import make_runner, random_model
    from torchinferno_b200.kernels.library import library_path, load_library
    from torchinferno_b200.kernels import gemm
    peaks = load_peaks()
    load_library()
    gemm.set_backend(args.gemm_backend)
    config = dict(LLAMA_8B)
    config["num_hidden_layers"] = args.layers
    sampler = ClockSampler()
    with torch.inference_mode():
        model = random_model(config, seed=0, dtype="bfloat16")
        numbers = model_numbers(model, args.layers)
        biggest = max([args.batch] + args.points)
        pool_tokens = biggest * (CONTEXT + 2 * PAGE_SIZE)
        runner = make_runner(model, page_size=PAGE_SIZE, max_tokens=pool_tokens, max_requests=biggest,
                             max_request_tokens=CONTEXT + PAGE_SIZE, check_errors=False)
        prefill = timed_prefill(runner, numbers, iters=5, warmup=3, seed=1)
        main = timed_decode(runner, args.batch, args.steps, args.warmup, numbers, sampler, seed=2)
        # (the same batch through the entry point next, in the state of the chip the device-timed run left)
        e2e = timed_e2e(model, args.batch, min(args.steps, args.e2e_steps or args.steps), args.warmup, seed=4)
        points = {}
        for b in args.points:
            r = timed_decode(runner, b, args.point_steps, args.warmup, numbers, sampler, seed=3 + b)
            points[f"decode_b{b}"] = round(r["tokens_per_s"], 1)
            points[f"decode_b{b}_ms_per_step"] = round(r["ms_per_step"], 4)
            points[f"decode_b{b}_hbm_frac"] = round(r["achieved_gbs"] / peaks["hbm_gbs"], 4)
        del runner
        torch.cuda.empty_cache()
        del model
        torch.cuda.empty_cache()
        for name in args.workloads:
            points.update(timed_workload(name, peaks, args.gemm_backend))
    sampler.stop()
    peak_flops = peaks["bf16_tflops"] * 1e12
    record = {
        "metric": METRIC, "value": round(main["tokens_per_s"], 1), "unit": "tok/s", "n_gpus": 1, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": round(main["ms_per_step"], 4), "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "bf16", "data": "synthetic token ids, random weights N(0,0.02), norm weights 1",
        "impl": "ours",
        "config": {
            "model": "Llama-3.1-8B sizes", "layers": args.layers, "layers_of_model": FULL_LAYERS, "hidden": 4096,
            "heads": 32, "kv_heads": 8, "head_dim": 128, "intermediate": 14336, "vocab": 128256, "global_batch": args.batch,
            "seq_len": CONTEXT, "prompt_len": PROMPT_LEN, "context_from": main["context_from"],
            "context_to": main["context_to"], "page_size": PAGE_SIZE, "parallelism": "single GPU",
            "l2": "inputs larger than L2 (weights of a step: %.1f GB)" % (numbers["matmul_params"] * 2 / 1e9),
            "peaks": peaks["source"], "gemm_backend": args.gemm_backend,
            "repeats": "%d runs of %d steps, decoding on; the median run counts" % (main["repeats"], args.steps),
        },
        "clocks": main["clocks"],
        "e2e": {k: (round(v, 2) if isinstance(v, float) else v) for k, v in e2e.items()},
        "gpu_launches": main["launches"],
        "prefill": {"value": round(prefill["value"], 1), "tokens": prefill["tokens"], "ms": round(prefill["ms"], 3),
                    "frac": round(prefill["flops"] / (prefill["ms"] / 1e3) / peak_flops, 4),
                    "peak_tflops": peaks["bf16_tflops"],
                    # (against the library's throughput in a seconds-long loop under the power cap, which is the
                    # state the five timed prompts run in)
                    "frac_of_sustained": round(prefill["flops"] / (prefill["ms"] / 1e3) / (peaks["bf16_tflops_sustained"] * 1e12), 4)},
        "roofline": {"bound": "hbm", "achieved": round(main["achieved_gbs"], 1), "peak": peaks["hbm_gbs"], "unit": "GB/s",
                     "frac": round(main["achieved_gbs"] / peaks["hbm_gbs"], 4), "bytes_per_step": int(main["step_bytes"])},
        "points": points,
        "library": library_path(),
    }
    return record


# -------------------------------------------------------------- reference
def run_reference(args) -> dict:
    """The unmodified reference from baseline/_ref: its Llama3PipelineForCausalLM.generate on the same sizes."""
    ref = ROOT / "baseline" / "_ref"
    if not (ref / "torchinferno").is_dir():
        return {"impl": "reference", "unavailable": "baseline/_ref is not installed (pip install --no-index --no-deps --target baseline/_ref)"}
    sys.path.insert(0, str(ref))
    os.environ.setdefault("HF_HUB_OFFLINE", "1")
    try:
        import tempfile

        import torch
        from safetensors.torch import save_file
        from torchinferno.models.llama3.pipeline import Llama3PipelineForCausalLM
    except Exception as exc:  # noqa: BLE001 - whatever stops the import is the reason
        return {"impl": "reference", "unavailable": f"reference cannot be imported: {type(exc).__name__}: {exc}"[:300]}
    from torchinferno_b200.weights.random_init import build_model, random_tensor
    config = dict(LLAMA_8B)
    config["num_hidden_layers"] = args.layers
    config.pop("head_dim")                       # not a key of the reference's configuration
    sampler = ClockSampler()
    with tempfile.TemporaryDirectory(dir=os.environ.get("TMPDIR")) as tmp, torch.inference_mode():
        folder = Path(tmp)
        spec_model = build_model({**config, "head_dim": 128}, dtype=torch.bfloat16, device="cpu")
        tensors = {name: random_tensor(ws, 0, device="cuda", dtype=torch.bfloat16).cpu()
                   for name, ws in spec_model.expected_tensors().items()}
        save_file(tensors, str(folder / "model.safetensors"))
        (folder / "model.safetensors.index.json").write_text(json.dumps(
            {"metadata": {}, "weight_map": {k: "model.safetensors" for k in tensors}}))
        (folder / "config.json").write_text(json.dumps(config))
        del tensors
        model = Llama3PipelineForCausalLM.from_pretrained(str(folder), devices=["cuda:0"], dtype=torch.bfloat16)
        g = torch.Generator().manual_seed(2)
        prompts = torch.randint(0, config["vocab_size"], (args.batch, PROMPT_LEN), generator=g).cuda()
        # the reference's generate() is one call; its decode steps are timed as (whole - prefill only)
        def timed(new_tokens):
            torch.cuda.synchronize()
            b, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            b.record()
            model.generate(prompts, max_new_tokens=new_tokens, temperature=0.0)
            e.record()
            torch.cuda.synchronize()
            return b.elapsed_time(e)
        # end to end, as a caller of generate() meets it: the prompts start in pinned host memory and the
        # generated ids end in host memory, inside the timed region
        host_prompts = prompts.cpu().pin_memory()
        def timed_e2e(new_tokens):
            torch.cuda.synchronize()
            b, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            b.record()
            out = model.generate(host_prompts.to("cuda", non_blocking=True), max_new_tokens=new_tokens, temperature=0.0)
            ids = out[:, PROMPT_LEN:].cpu()
            e.record()
            torch.cuda.synchronize()
            return b.elapsed_time(e), ids.numel() * ids.element_size()
        for _ in range(max(1, min(args.warmup, 3))):
            timed(2)
        timed(1 + args.steps)      # (the first call at a length sets up what that length needs: not part of a step's time)
        mark = sampler.mark()
        short = timed(1)
        long = timed(1 + args.steps)
        e2e_short, _ = timed_e2e(1)
        e2e_long, out_bytes = timed_e2e(1 + args.steps)
        clocks = sampler.summary(mark, sampler.mark())
    sampler.stop()
    ms = long - short
    e2e_ms = e2e_long - e2e_short
    return {"metric": METRIC, "value": round(args.batch * args.steps / (ms / 1e3), 1), "unit": "tok/s", "n_gpus": 1,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": round(ms / args.steps, 4), "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic token ids, random weights",
            "impl": "reference", "clocks": clocks,
            "e2e": {"value": round(args.batch * args.steps / (e2e_ms / 1e3), 1), "unit": "tok/s", "ms_per_step": round(e2e_ms / args.steps, 4),
                    "h2d_bytes_per_step": round(host_prompts.numel() * host_prompts.element_size() / (1 + args.steps), 1),
                    "d2h_bytes_per_step": round(out_bytes / (1 + args.steps), 1),
                    "how": "generate() with the prompts in pinned host memory and the new ids read back, (1 + steps) new tokens minus 1"},
            "config": {"model": "Llama-3.1-8B sizes", "layers": args.layers, "layers_of_model": FULL_LAYERS,
                       "global_batch": args.batch, "seq_len": CONTEXT, "prompt_len": PROMPT_LEN,
                       "path": "Llama3PipelineForCausalLM.generate (dense cache, torch ops)"},
            "prefill": {"ms": round(short, 3), "tokens": args.batch * PROMPT_LEN,
                        "value": round(args.batch * PROMPT_LEN / (short / 1e3), 1)}}


def main(argv=None) -> int:
    parser = argparse.ArgumentParser(description=__doc__.splitlines()[0])
    parser.add_argument("--gpus", type=int, default=1)
    parser.add_argument("--steps", type=int, default=2032)
    parser.add_argument("--warmup", type=int, default=8)
    parser.add_argument("--impl", choices=["ours", "reference"], default="ours")
    parser.add_argument("--batch", type=int, default=8)
    parser.add_argument("--layers", type=int, default=FULL_LAYERS, help="fewer layers than the model has (named in config)")
    parser.add_argument("--points", type=int, nargs="*", default=[1, 64], help="other batch sizes to decode at")
    parser.add_argument("--point-steps", type=int, default=None, help="decode steps of the other batch sizes (default: --steps)")
    parser.add_argument("--e2e-steps", type=int, default=None, help="steps of the end-to-end run (default: --steps, the same contexts)")
    parser.add_argument("--gemm-backend", choices=["auto", "tcgen05", "library"], default="auto")
    parser.add_argument("--workloads", nargs="*", default=list(WORKLOADS), choices=list(WORKLOADS),
                        help="serving workloads of the smaller sizes to add to points")
    args = parser.parse_args(argv)
    if args.gpus != 1 or int(os.environ.get("WORLD_SIZE", "1")) != 1:
        if int(os.environ.get("RANK", "0")) == 0:
            print(json.dumps({"metric": METRIC, "unsupported": f"this engine runs on one GPU; --gpus {args.gpus} is not supported",
                              "n_gpus": args.gpus}))
        return 2
    if args.warmup < 3:
        args.warmup = 3
    if args.point_steps is None:
        args.point_steps = args.steps
    if PROMPT_LEN + args.warmup + max(args.steps, args.point_steps) + 1 > CONTEXT + PAGE_SIZE:
        parser.error(f"--warmup + --steps must stay within the {CONTEXT}-token context after a {PROMPT_LEN}-token prompt")
    record = run_reference(args) if args.impl == "reference" else run_ours(args)
    print(json.dumps(record))
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
