"""Time single kernels of the engine in isolation and relate them to the B200's measured peaks.

    python -m torchinferno_b200.bench_kernels decode-attention --batch 8 --context 2048
    python -m torchinferno_b200.bench_kernels prefill-attention --tokens 2048
    python -m torchinferno_b200.bench_kernels gemm --rows 8
    python -m torchinferno_b200.bench_kernels elementwise --rows 2048
    python -m torchinferno_b200.bench_kernels step-timeline --layers 32 --batch 8 --context 3072

Each run prints one JSON line per case: microseconds (median of CUDA-event timings, an L2 flush
between iterations), the bytes or flops the kernel has to move or do, and the fraction of the
measured copy bandwidth or tensor throughput (``MEASURED_PEAKS.json`` at the repository root when
present).  The same commands, small, are what the ``ncu`` summaries under ``profiles/`` were taken
from.  The reference keeps such microbenchmarks as stand-alone scripts (``scripts/`` in its tree).
"""
from __future__ import annotations

import argparse
import json
import math
import statistics
from pathlib import Path

import torch

from torchinferno_b200.kernels import ops

ROOT = Path(__file__).resolve().parent.parent


def peaks() -> dict:
    path = ROOT / "MEASURED_PEAKS.json"
    if path.is_file():
        data = json.loads(path.read_text())
        return {"hbm_gbs": data["hbm_gbs"], "bf16_tflops": data["bf16_tflops"], "source": "measured"}
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "source": "fallback"}


class Timer:
    def __init__(self, iters: int, warmup: int = 3) -> None:
        self.iters, self.warmup = iters, warmup
        self.flush = torch.empty(256 << 20, dtype=torch.uint8, device="cuda")   # larger than the 126 MB L2

    def __call__(self, fn) -> float:
        for _ in range(self.warmup):
            fn()
        times = []
        for _ in range(self.iters):
            self.flush.zero_()
            begin, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            begin.record()
            fn()
            end.record()
            torch.cuda.synchronize()
            times.append(begin.elapsed_time(end) * 1e3)
        return statistics.median(times)


def report(name: str, us: float, *, bytes_moved: float | None = None, flops: float | None = None, **extra) -> None:
    p = peaks()
    line = {"kernel": name, "us": round(us, 2), **extra}
    if bytes_moved is not None:
        line["gbs"] = round(bytes_moved / us / 1e3, 1)
        line["hbm_frac"] = round(bytes_moved / us / 1e3 / p["hbm_gbs"], 4)
    if flops is not None:
        line["tflops"] = round(flops / us / 1e6, 1)
        line["tensor_frac"] = round(flops / us / 1e6 / p["bf16_tflops"], 4)
    line["peaks"] = p["source"]
    print(json.dumps(line), flush=True)


def paged_cache(batch: int, context: int, kv_heads: int, head_dim: int, page: int):
    """A filled pool with shuffled pages and the block table of ``batch`` requests of ``context`` tokens."""
    pages_per = -(-context // page)
    total = batch * pages_per
    pool = (torch.randn(total, 2, kv_heads, page, head_dim, device="cuda") * 0.5).to(torch.bfloat16)
    order = torch.randperm(total, device="cuda", dtype=torch.int32)
    table = order.view(batch, pages_per).contiguous()
    return pool, table


def run_decode_attention(args) -> None:
    h, k, d = args.heads, args.kv_heads, args.head_dim
    pool, table = paged_cache(args.batch, args.context, k, d, args.page_size)
    n = args.batch
    q = torch.randn(n, h * d, device="cuda").to(torch.bfloat16)
    out = torch.empty_like(q)
    i32 = lambda v: torch.tensor(v, dtype=torch.int32, device="cuda")
    q_start, kv_start, slots = i32(list(range(n + 1))), i32([args.context - 1] * n), i32(list(range(n)))
    timer = Timer(args.iters)
    kv_bytes = n * args.context * 2 * k * d * 2
    kernels = ["cp_async"] + (["tma"] if ops.decode_attention_tma_supports(d, h // k, args.page_size) else [])
    for forced in (args.splits or [None]):
        splits, chunk = (ops.decode_num_splits(n, h, k, args.context) if forced is None else forced), 0
        scratch = torch.empty(n * h * splits * (d + 2), dtype=torch.float32, device="cuda")
        for kernel in kernels:
            fn = lambda: ops.decode_attention(q, pool, out, q_start, kv_start, slots, table, n, h, k, d, 1 / math.sqrt(d),
                                              args.context, scratch=scratch, num_splits=splits, chunk=chunk, kernel=kernel)
            report(f"decode_attention[{kernel}]+merge", timer(fn), bytes_moved=kv_bytes, batch=n, context=args.context,
                   splits=splits, heads=h, kv_heads=k, head_dim=d)
        if "tma" in kernels:      # the same from the unrotated rows of the qkv product: rotary and the cache write inside
            qkv = torch.randn(n, (h + 2 * k) * d, device="cuda").to(torch.bfloat16)
            inv_freq = (1.0 / (500000.0 ** (torch.arange(0, d, 2, dtype=torch.float32) / d))).cuda()
            fn = lambda: ops.decode_attention_rope(qkv, pool, out, q_start, kv_start, slots, table, n, h, k, d, 1 / math.sqrt(d),
                                                   args.context, inv_freq, scratch=scratch, num_splits=splits)
            report("decode_attention[tma, rotates and stores the newest token]+merge", timer(fn), bytes_moved=kv_bytes, batch=n,
                   context=args.context, splits=splits, heads=h, kv_heads=k, head_dim=d)


def run_prefill_attention(args) -> None:
    h, k, d, t = args.heads, args.kv_heads, args.head_dim, args.tokens
    pool, table = paged_cache(args.batch, t, k, d, args.page_size)
    n = args.batch
    q = torch.randn(n * t, h * d, device="cuda").to(torch.bfloat16)
    out = torch.empty_like(q)
    i32 = lambda v: torch.tensor(v, dtype=torch.int32, device="cuda")
    q_start, kv_start, slots = i32([i * t for i in range(n + 1)]), i32([0] * n), i32(list(range(n)))
    fn = lambda: ops.prefill_attention(q, pool, out, q_start, kv_start, slots, table, n, t, h, k, d, 1 / math.sqrt(d))
    flops = n * 4 * h * d * t * (t + 1) / 2
    timer = Timer(args.iters)
    report("prefill_attention[mma.sync]", timer(fn), flops=flops, batch=n, tokens=t, heads=h, kv_heads=k, head_dim=d,
           note="causal flops")
    if ops.prefill_attention_tcgen05_supports(d, h // k, args.page_size):
        fn5 = lambda: ops.prefill_attention_tcgen05(q, pool, out, q_start, kv_start, slots, table, n, t, h, k, d, 1 / math.sqrt(d))
        report("prefill_attention[tcgen05]", timer(fn5), flops=flops, batch=n, tokens=t, heads=h, kv_heads=k, head_dim=d,
               note="causal flops")


def run_gemm(args) -> None:
    shapes = {"qkv": (6144, 4096), "o": (4096, 4096), "gate_up": (28672, 4096), "down": (4096, 14336), "lm_head": (128256, 4096)}
    timer = Timer(args.iters)
    for name, (n, k) in shapes.items():
        if args.only and name not in args.only:
            continue
        w = (torch.randn(n, k, device="cuda") * 0.02).to(torch.bfloat16)
        x = torch.randn(args.rows, k, device="cuda").to(torch.bfloat16)
        out = torch.empty(args.rows, n, dtype=torch.bfloat16, device="cuda")
        common = dict(bytes_moved=n * k * 2, flops=2 * args.rows * n * k, rows=args.rows, n=n, k=k)
        if ops.gemm_tcgen05_swapab_supports(args.rows, n, k):
            report(f"gemm_tcgen05_swapab[{name}]", timer(lambda: ops.gemm_tcgen05_swapab(x, w, out)), **common)
            w_kn = w.t().contiguous()
            for features, splits in ((256, 1), (128, 1), (128, 2), (128, 4), (128, 5)):      # the few-rows kernel's tiles
                if args.decode_config and (features, splits) != tuple(args.decode_config):
                    continue
                if ops.gemm_decode_supports(args.rows, n, k, features, splits):
                    report(f"gemm_decode[{name}, {features} features, K over {splits}]",
                           timer(lambda: ops.gemm_decode(x, w_kn, out, features=features, splits=splits)), **common)
            if name == "gate_up":      # (the columns stand for interleaved gate / up pairs: the activation in the epilogue)
                act = torch.empty(args.rows, n // 2, dtype=torch.bfloat16, device="cuda")
                for features in (256, 128):
                    if args.decode_config and features != args.decode_config[0]:
                        continue
                    report(f"gemm_decode[{name}, {features} features, SwiGLU epilogue]",
                           timer(lambda: ops.gemm_decode(x, w_kn, act, features=features, splits=1, epilogue=ops.DG_SWIGLU)), **common)
            report(f"gemm_tcgen05_swapab_kn[{name}]", timer(lambda: ops.gemm_tcgen05_swapab(x, w_kn, out, w_kn=True)), **common)
            report(f"library_gemm_kn[{name}]", timer(lambda: torch.mm(x, w_kn, out=out)), **common)
            del w_kn
        elif ops.gemm_tcgen05_supports(args.rows, n, k):
            report(f"gemm_tcgen05[{name}]", timer(lambda: ops.gemm_tcgen05(x, w, out)), **common)
            if args.rows >= 128 and ops.gemm_tcgen05_2cta_supports(args.rows, n, k):
                report(f"gemm_tcgen05_2cta[{name}]", timer(lambda: ops.gemm_tcgen05_2cta(x, w, out)), **common)
        report(f"library_gemm[{name}]", timer(lambda: torch.mm(x, w.t(), out=out)), **common)


def run_elementwise(args) -> None:
    rows, hidden, inter = args.rows, args.hidden, args.intermediate
    timer = Timer(args.iters)
    delta = torch.randn(rows, hidden, device="cuda").to(torch.bfloat16)
    residual = torch.randn(rows, hidden, device="cuda")
    weight = torch.ones(hidden, device="cuda")
    out = torch.empty_like(delta)
    report("add_rmsnorm", timer(lambda: ops.add_rmsnorm(delta, residual, weight, 1e-5, out)),
           bytes_moved=rows * hidden * (2 + 4 + 4 + 2), rows=rows, hidden=hidden)
    gate_up = torch.randn(rows, 2 * inter, device="cuda").to(torch.bfloat16)
    act = torch.empty(rows, inter, dtype=torch.bfloat16, device="cuda")
    report("swiglu", timer(lambda: ops.swiglu(gate_up, act)), bytes_moved=rows * inter * 6, rows=rows, intermediate=inter)
    h, k, d = args.heads, args.kv_heads, args.head_dim
    qkv = torch.randn(rows, (h + 2 * k) * d, device="cuda").to(torch.bfloat16)
    q_out = torch.empty(rows, h * d, dtype=torch.bfloat16, device="cuda")
    pool, table = paged_cache(1, rows, k, d, args.page_size)
    positions = torch.arange(rows, dtype=torch.int32, device="cuda")
    slot = torch.zeros(rows, dtype=torch.int32, device="cuda")
    inv_freq = (1.0 / (500000.0 ** (torch.arange(0, d, 2, dtype=torch.float32) / d))).cuda()
    report("rope_append", timer(lambda: ops.rope_append(qkv, q_out, pool, positions, slot, table, inv_freq, h, k, d)),
           bytes_moved=rows * ((h + 2 * k) * d * 2 + (h + 2 * k) * d * 2), rows=rows)


def run_step_timeline(args) -> None:
    """Which kernels a captured decode step (or, with --prompt, the step of one whole prompt of --context tokens)
    spends its time in: every kernel of one step with its start and duration as the driver's activity records
    (CUPTI, through torch.profiler) give them, summed by kernel, and one layer listed launch by launch (a
    negative gap: the kernel was placed before the one before it had ended, by programmatic dependent launch,
    and its duration includes the wait)."""
    import collections
    from torch.profiler import ProfilerActivity, profile
    from torchinferno_b200.engine.batch import StepEntry
    from torchinferno_b200.engine.factory import make_runner, random_model
    from torchinferno_b200.kernels import gemm
    gemm.set_backend(args.gemm_backend)
    config = {"architectures": ["LlamaForCausalLM"], "model_type": "llama", "vocab_size": args.vocab, "hidden_size": args.hidden,
              "intermediate_size": args.intermediate, "num_hidden_layers": args.layers, "num_attention_heads": args.heads,
              "num_key_value_heads": args.kv_heads, "head_dim": args.head_dim, "max_position_embeddings": 131072,
              "rope_theta": 500000.0, "rms_norm_eps": 1e-5, "tie_word_embeddings": False}
    model = random_model(config, seed=0, dtype="bfloat16")
    n, ctx = args.batch, args.context
    prompts = torch.randint(0, args.vocab, (n, ctx), generator=torch.Generator().manual_seed(0)).tolist()
    if args.prompt:
        runner = make_runner(model, page_size=args.page_size, max_tokens=2 * (ctx + 64), max_requests=2, check_errors=False)
        turn = [0]

        def step() -> None:      # a new request's whole prompt, alone in its step
            turn[0] += 1
            runner.step([StepEntry(turn[0], prompts[0], [ctx - 1])])
            runner.end([turn[0]])
    else:
        runner = make_runner(model, page_size=args.page_size, max_tokens=n * (ctx + 64), max_requests=n, check_errors=False)
        for i, prompt in enumerate(prompts):
            runner.step([StepEntry(i, prompt, [ctx - 1])])
        step = lambda: runner.step([StepEntry(i, [5], [0]) for i in range(n)])
    for _ in range(5):
        step()
    torch.cuda.synchronize()
    if args.plain:           # (for a launch list under ncu: no second profiler in the process)
        for _ in range(args.iters):
            step()
        torch.cuda.synchronize()
        print(json.dumps({"steps": args.iters, "batch": n, "context": ctx, "layers": args.layers}))
        return
    with profile(activities=[ProfilerActivity.CUDA]) as prof:
        for _ in range(3):
            step()
        torch.cuda.synchronize()
    kernels = sorted((e for e in prof.events() if e.device_type == torch.autograd.DeviceType.CUDA and e.time_range.end > e.time_range.start),
                     key=lambda e: e.time_range.start)
    last = kernels[-(len(kernels) // 3):]
    t0, t1 = last[0].time_range.start, max(e.time_range.end for e in last)
    total = collections.defaultdict(lambda: [0, 0.0])
    for e in last:
        total[e.name[:64]][0] += 1
        total[e.name[:64]][1] += e.time_range.end - e.time_range.start
    print(json.dumps({"step_us": round(t1 - t0, 1), "kernels": len(last), "step": "prompt" if args.prompt else "decode",
                      "batch": 1 if args.prompt else n, "context": ctx, "layers": args.layers, "gemm_backend": args.gemm_backend}))
    for name, (count, us) in sorted(total.items(), key=lambda kv: -kv[1][1]):
        print(f"{us:9.1f} us  x{count:4d}  avg {us / count:7.2f}  {name}")
    print("one layer, launch by launch (gap to the end of the kernel before, duration):")
    per_layer = max(1, (len(last) - 3) // max(1, args.layers))
    mid = len(last) // 2
    end = None
    for e in last[mid:mid + per_layer + 2]:
        gap = 0.0 if end is None else e.time_range.start - end
        print(f"  gap {gap:7.2f}  dur {e.time_range.end - e.time_range.start:7.2f}  {e.name[:70]}")
        end = e.time_range.end


def main(argv=None) -> int:
    parser = argparse.ArgumentParser(prog="python -m torchinferno_b200.bench_kernels", description=__doc__.splitlines()[0])
    parser.add_argument("--ordinary-launches", action="store_true",
                        help="launch the kernels without programmatic dependent launch (a profiler that lists kernels "
                             "by name does not see dependent launches)")
    sub = parser.add_subparsers(dest="command", required=True)

    def common(p):
        p.add_argument("--heads", type=int, default=32)
        p.add_argument("--kv-heads", type=int, default=8)
        p.add_argument("--head-dim", type=int, default=128)
        p.add_argument("--page-size", type=int, default=16)
        p.add_argument("--iters", type=int, default=20)

    p = sub.add_parser("decode-attention")
    p.add_argument("--batch", type=int, default=8)
    p.add_argument("--context", type=int, default=2048)
    p.add_argument("--splits", type=int, nargs="*", default=None, help="try these numbers of context splits")
    common(p)
    p.set_defaults(func=run_decode_attention)
    p = sub.add_parser("prefill-attention")
    p.add_argument("--batch", type=int, default=1)
    p.add_argument("--tokens", type=int, default=2048)
    common(p)
    p.set_defaults(func=run_prefill_attention)
    p = sub.add_parser("gemm")
    p.add_argument("--rows", type=int, default=8)
    p.add_argument("--only", nargs="*", default=None)
    p.add_argument("--iters", type=int, default=20)
    p.add_argument("--decode-config", type=int, nargs=2, default=None, metavar=("FEATURES", "SPLITS"),
                   help="of the few-rows kernel's configurations only this one")
    p.set_defaults(func=run_gemm)
    p = sub.add_parser("elementwise")
    p.add_argument("--rows", type=int, default=2048)
    p.add_argument("--hidden", type=int, default=4096)
    p.add_argument("--intermediate", type=int, default=14336)
    common(p)
    p.set_defaults(func=run_elementwise)
    p = sub.add_parser("step-timeline")
    p.add_argument("--layers", type=int, default=32)
    p.add_argument("--batch", type=int, default=8)
    p.add_argument("--context", type=int, default=3072)
    p.add_argument("--hidden", type=int, default=4096)
    p.add_argument("--intermediate", type=int, default=14336)
    p.add_argument("--vocab", type=int, default=128256)
    p.add_argument("--gemm-backend", choices=["auto", "tcgen05", "library"], default="auto")
    p.add_argument("--plain", action="store_true", help="run the steps without the activity profiler (for ncu)")
    p.add_argument("--prompt", action="store_true", help="the step of one whole prompt of --context tokens instead of a decode step")
    common(p)
    p.set_defaults(func=run_step_timeline, iters=3)
    args = parser.parse_args(argv)
    if not torch.cuda.is_available():
        raise SystemExit("bench_kernels needs a CUDA device")
    if args.ordinary_launches:
        ops.set_dependent_launch(False)
    with torch.inference_mode():
        args.func(args)
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
