"""Traces for the replay tests and two ways to run them: in this process through the engine's
step function, or through ``bin/trace_run`` as a user would."""
from __future__ import annotations

import json
import random
import subprocess
import sys
from pathlib import Path

import numpy as np
import torch

ROOT = Path(__file__).resolve().parent.parent


def round64(n: int) -> int:
    return -(-n // 64) * 64


def peak_tokens(steps) -> int:
    """The most tokens live requests hold at any time, each rounded up to a multiple of 64."""
    held, peak = {}, 0
    for step in steps:
        for e in step["entries"]:
            held[e["id"]] = held.get(e["id"], 0) + len(e["tokens"])
        peak = max(peak, sum(round64(n) for n in held.values()))
        for rid in step["end"]:
            held.pop(rid, None)
    return peak


# ------------------------------------------------------------------ traces
# Every maker returns (steps, index) where index[(step, row)] = (request name, position).
def _finish(steps):
    index = {}
    for step in steps:
        row = 0
        for e in step["entries"]:
            for w in e["want"]:
                index[(step["step"], row)] = (e["id"].split("#")[0], e["_start"] + w)
                row += 1
    for step in steps:
        for e in step["entries"]:
            e.pop("_start")
    return steps, index


def trace_whole(requests: dict[str, list[int]], tag=""):
    steps = []
    for name, toks in requests.items():
        steps.append({"step": len(steps), "entries": [
            {"id": name + tag, "tokens": toks, "want": list(range(len(toks))), "_start": 0}], "end": [name + tag]})
    return _finish(steps)


def trace_tail_decode(requests, tail=32, tag="#t"):
    steps = []
    for name, toks in requests.items():
        head = max(1, len(toks) - tail)
        steps.append({"step": len(steps), "entries": [
            {"id": name + tag, "tokens": toks[:head], "want": [head - 1], "_start": 0}], "end": []})
        for pos in range(head, len(toks)):
            steps.append({"step": len(steps), "entries": [
                {"id": name + tag, "tokens": [toks[pos]], "want": [0], "_start": pos}],
                "end": [name + tag] if pos == len(toks) - 1 else []})
        if head == len(toks):
            steps[-1]["end"] = [name + tag]
    return _finish(steps)


def trace_portions(requests, sizes=(2, 7, 16, 3, 33, 2, 5, 17, 64, 2), tag="#p"):
    steps = []
    for r, (name, toks) in enumerate(requests.items()):
        pos, i = 0, r
        while pos < len(toks):
            n = min(sizes[i % len(sizes)], len(toks) - pos)
            if len(toks) - pos - n == 1:      # no portion below two tokens, except a last single one
                n += 1
            i += 1
            steps.append({"step": len(steps), "entries": [
                {"id": name + tag, "tokens": toks[pos:pos + n], "want": list(range(n)), "_start": pos}],
                "end": [name + tag] if pos + n == len(toks) else []})
            pos += n
    return _finish(steps)


def trace_mixed(requests, seed=0, max_live=4, tag="#m"):
    """Up to ``max_live`` requests at a time: portions of some beside single tokens of others,
    a request now and then left out of a step, new requests taking the place (and pages) of ended ones."""
    rng = random.Random(seed)
    waiting = list(requests.items())
    live: dict[str, dict] = {}
    steps = []
    while waiting or live:
        while waiting and len(live) < max_live:
            name, toks = waiting.pop(0)
            live[name] = {"toks": toks, "pos": 0, "decode_from": max(2, int(len(toks) * rng.uniform(0.4, 0.8)))}
        entries, ended = [], []
        names = list(live)
        rng.shuffle(names)
        for name in names:
            st = live[name]
            if len(names) > 1 and rng.random() < 0.15:
                continue                      # left out of this step, goes on later
            remaining = len(st["toks"]) - st["pos"]
            if st["pos"] >= st["decode_from"] or remaining == 1:
                n = 1
            else:
                n = min(rng.choice([2, 3, 5, 8, 13, 16, 21, 40]), st["decode_from"] - st["pos"], remaining)
                n = max(n, min(2, remaining))
            want = list(range(n)) if n <= 3 else sorted(rng.sample(range(n), 3) + [n - 1])
            want = sorted(set(want))
            entries.append({"id": name + tag, "tokens": st["toks"][st["pos"]:st["pos"] + n], "want": want, "_start": st["pos"]})
            st["pos"] += n
            if st["pos"] == len(st["toks"]):
                ended.append(name + tag)
                del live[name]
        if entries:
            steps.append({"step": len(steps), "entries": entries, "end": ended})
    return _finish(steps)


# ----------------------------------------------------------------- runners
class InProcessReplayer:
    """Drives the engine's own model, step function, cache and kernels in this process."""

    def __init__(self, folder, dtype: str, max_tokens: int, page_size: int = 16):
        from torchinferno_b200.engine.factory import load_model, make_runner
        self.model = load_model(folder, dtype=dtype)
        self.runner = make_runner(self.model, page_size=page_size, max_tokens=max_tokens, max_requests=8)

    def run(self, steps):
        from torchinferno_b200.engine.batch import StepEntry
        out = {}
        with torch.inference_mode():
            for step in steps:
                entries = [StepEntry(e["id"], e["tokens"], e["want"]) for e in step["entries"]]
                logits = self.runner.step(entries)
                if logits.shape[0]:
                    out[step["step"]] = logits.cpu().numpy()
                self.runner.end(step["end"])
                self.runner.cache.audit()
        return out


def run_trace_program(folder, dtype: str, max_tokens: int, steps, out_dir: Path, env=None):
    """Feed ``steps`` to bin/trace_run one by one, waiting for ``done <step>`` each time."""
    out_dir.mkdir(parents=True, exist_ok=True)
    cmd = [sys.executable, str(ROOT / "bin" / "trace_run"), "--model", str(folder), "--dtype", dtype,
           "--out", str(out_dir), "--max-tokens", str(max_tokens)]
    proc = subprocess.Popen(cmd, stdin=subprocess.PIPE, stdout=subprocess.PIPE, text=True, env=env)
    try:
        for step in steps:
            proc.stdin.write(json.dumps(step) + "\n")
            proc.stdin.flush()
            line = proc.stdout.readline().strip()
            assert line == f"done {step['step']}", f"trace_run said {line!r} (exit {proc.poll()})"
        proc.stdin.close()
        assert proc.wait(timeout=120) == 0
    finally:
        if proc.poll() is None:
            proc.kill()
    vocab = json.loads((Path(folder) / "config.json").read_text())["vocab_size"]
    out = {}
    for step in steps:
        wanted = sum(len(e["want"]) for e in step["entries"])
        path = out_dir / f"{step['step']}.f32"
        if wanted:
            out[step["step"]] = np.fromfile(path, dtype="<f4").reshape(wanted, vocab)
        else:
            assert not path.exists()
    return out


def gather(results, index):
    """{(request, position): logits row} from per-step outputs."""
    rows = {}
    for (step, row), key in index.items():
        rows.setdefault(key, []).append(results[step][row])
    return rows
