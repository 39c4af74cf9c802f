"""Command line of the engine, in the manner of the reference's ``torchinferno`` command
(src/torchinferno/cli.py:1654-2398: one parser with sub-commands, each a ``run_*`` function
returning an exit code).

Sub-commands and where their option names come from:

``text-generate MODEL PROMPT``   src/torchinferno/cli.py:1952-1963 (``--tokenizer --device
                                 --new-tokens 16 --temperature 0.0``)
``generate MODEL --input-ids``   the same on token ids (``--input-ids`` as in ``deepseek-hf-smoke``,
                                 cli.py:1945-1950), prints ``output_ids=[...]``
``llama-bench MODEL``            cli.py:1776-1816 (``--dtype --input-len 32 --output-len 128
                                 --batch-size 8 --num-iters-warmup 1 --num-iters 3 --num-prompts
                                 --temperature 1.0 --seed 0``; ``--benchmark latency|throughput`` for its
                                 ``--benchmarks``)
``serve-smoke``                  cli.py:2095-2104 (``--page-size 16 --max-active-requests 2
                                 --new-tokens 2 --vocab-size 128 --temperature 0.0 --seed 0``)
``capture-logits`` / ``validate-logits``   cli.py:2330-2350 (``model output --input-ids`` /
                                 ``model reference --atol 1e-4 --rtol 1e-4``)
``random-model CONFIG OUT``      writes a model folder with seeded random weights (no counterpart)
"""
from __future__ import annotations

import argparse
import json
import tempfile
import time
from pathlib import Path


def _engine_options(parser: argparse.ArgumentParser) -> None:
    parser.add_argument("--device", default=None, help="CUDA device, default cuda:0")
    parser.add_argument("--dtype", default="auto", help="auto | bfloat16 | float32")
    parser.add_argument("--max-model-len", type=int, default=None)
    parser.add_argument("--page-size", type=int, default=16)
    parser.add_argument("--max-batch-size", type=int, default=64)
    parser.add_argument("--max-num-batched-tokens", type=int, default=8192, help="token budget of one step")
    parser.add_argument("--prefill-chunk-size", type=int, default=2048)
    parser.add_argument("--kv-cache-tokens", type=int, default=None, help="size of the page pool in tokens")
    parser.add_argument("--gemm-backend", choices=["auto", "tcgen05", "library"], default="auto",
                        help="bf16 projections: hand-written tcgen05 kernels, cuBLAS, or the measured mix")


def _engine(args, model: str, **extra):
    from torchinferno_b200.config.engine_config import EngineConfig
    from torchinferno_b200.engine.engine import InferenceEngine
    config = EngineConfig(
        model=model, tokenizer=getattr(args, "tokenizer", None), device=args.device, dtype=args.dtype,
        max_model_len=args.max_model_len, page_size=args.page_size, max_batch_size=args.max_batch_size,
        max_num_batched_tokens=args.max_num_batched_tokens, prefill_chunk_size=args.prefill_chunk_size,
        kv_cache_tokens=args.kv_cache_tokens, seed=getattr(args, "seed", 0),
        gemm_backend=getattr(args, "gemm_backend", "auto"), **extra)
    return InferenceEngine.from_config(config)


def run_generate(args) -> int:
    from torchinferno_b200.engine.types import GenerateRequest, SamplingConfig
    with _engine(args, args.model) as engine:
        out = engine.generate(GenerateRequest("cli-0", prompt_token_ids=args.input_ids, sampling=SamplingConfig(
            args.new_tokens, args.temperature, tuple(args.stop_token_ids), args.seed)))
    print("TorchInferno-B200 generation")
    print(f"model={args.model} dtype={args.dtype} new={args.new_tokens} finish_reason={out.finish_reason}")
    print(f"input_ids={list(args.input_ids)}")
    print(f"output_ids={list(args.input_ids) + list(out.token_ids)}")
    return 0


def run_text_generate(args) -> int:
    from torchinferno_b200.engine.types import GenerateRequest, SamplingConfig
    if args.tokenizer is None:
        args.tokenizer = args.model
    with _engine(args, args.model) as engine:
        if engine.tokenizer is None:
            raise SystemExit("text-generate needs a tokenizer.json (give --tokenizer)")
        out = engine.generate(GenerateRequest("cli-0", prompt=args.prompt, sampling=SamplingConfig(
            args.new_tokens, args.temperature, (), args.seed)))
    print("TorchInferno-B200 text generation")
    print(f"model={args.model} tokenizer={args.tokenizer}")
    print(f"output_ids={list(out.token_ids)}")
    print(out.text)
    return 0


def run_random_model(args) -> int:
    import torch
    from torchinferno_b200.weights.random_init import write_random_model
    config = json.loads(Path(args.config).read_text())
    dtype = {"bfloat16": torch.bfloat16, "float32": torch.float32}[args.dtype]
    folder = write_random_model(config, args.output, args.seed, dtype)
    print(f"wrote {folder}/config.json and {folder}/model.safetensors (seed {args.seed}, {args.dtype})")
    return 0


def run_serve_smoke(args) -> int:
    """A tiny random model through scheduler, step function and sampler; prints the tokens."""
    from torchinferno_b200.engine.types import GenerateRequest, SamplingConfig
    from torchinferno_b200.weights.random_init import write_random_model
    config = {"architectures": ["LlamaForCausalLM"], "model_type": "llama", "vocab_size": args.vocab_size,
              "hidden_size": 64, "intermediate_size": 160, "num_hidden_layers": 2, "num_attention_heads": 4,
              "num_key_value_heads": 2, "max_position_embeddings": 128, "rope_theta": 10000.0, "rms_norm_eps": 1e-5}
    with tempfile.TemporaryDirectory() as tmp:
        write_random_model(config, tmp, args.seed)
        args.max_batch_size = args.max_active_requests
        with _engine(args, tmp) as engine:
            requests = [GenerateRequest(f"smoke-{i}", prompt_token_ids=[(7 * i + j) % args.vocab_size for j in range(3 + i)],
                                        sampling=SamplingConfig(args.new_tokens, args.temperature, (), args.seed))
                        for i in range(args.max_active_requests + 1)]
            outputs = engine.generate_many(requests)
    print("TorchInferno-B200 serve smoke")
    for out in outputs:
        print(f"{out.request_id}: tokens={list(out.token_ids)} finish_reason={out.finish_reason}")
    return 0


def _last_logits(args, model: str, input_ids):
    import torch
    from torchinferno_b200.engine.batch import StepEntry
    from torchinferno_b200.engine.factory import load_model, make_runner
    with torch.inference_mode():
        loaded = load_model(model, dtype=args.dtype, device=args.device or "cuda:0")
        runner = make_runner(loaded, page_size=args.page_size, max_tokens=len(input_ids) + args.page_size, max_requests=1)
        logits = runner.step([StepEntry("capture", list(input_ids), [len(input_ids) - 1])])
        return logits[0].cpu().tolist()


def run_capture_logits(args) -> int:
    logits = _last_logits(args, args.model, args.input_ids)
    Path(args.output).write_text(json.dumps({"model": args.model, "input_ids": list(args.input_ids),
                                             "dtype": args.dtype, "logits": logits}))
    print(f"captured {len(logits)} logits of the last position to {args.output}")
    return 0


def run_validate_logits(args) -> int:
    reference = json.loads(Path(args.reference).read_text())
    logits = _last_logits(args, args.model, reference["input_ids"])
    want = reference["logits"]
    if len(want) != len(logits):
        print(f"FAIL: {len(logits)} logits, the reference has {len(want)}")
        return 1
    worst = max(abs(a - b) - (args.atol + args.rtol * abs(b)) for a, b in zip(logits, want))
    max_abs = max(abs(a - b) for a, b in zip(logits, want))
    print(f"max_abs_error={max_abs:.3e} atol={args.atol} rtol={args.rtol} -> {'ok' if worst <= 0 else 'FAIL'}")
    return 0 if worst <= 0 else 1


def _bench_engine(args):
    """The engine of a benchmark run: MODEL is a model folder, or with --random-weights a config.json whose
    model is built with seeded random weights on the device (nothing is written to disk)."""
    if not args.random_weights:
        return _engine(args, args.model)
    from torchinferno_b200.config.engine_config import EngineConfig
    from torchinferno_b200.engine.engine import InferenceEngine
    from torchinferno_b200.engine.factory import random_model
    from torchinferno_b200.kernels import gemm
    gemm.set_backend(args.gemm_backend)          # decides the layout the weights are bound in
    path = Path(args.model)
    config = json.loads((path / "config.json" if path.is_dir() else path).read_text())
    dtype = "bfloat16" if args.dtype == "auto" else args.dtype
    model = random_model(config, args.seed, dtype=dtype, device=args.device or "cuda:0")
    return InferenceEngine(model, EngineConfig(
        model=str(path), device=args.device, dtype=dtype, max_model_len=args.max_model_len, page_size=args.page_size,
        max_batch_size=args.max_batch_size, max_num_batched_tokens=args.max_num_batched_tokens,
        prefill_chunk_size=args.prefill_chunk_size, kv_cache_tokens=args.kv_cache_tokens, seed=args.seed,
        gemm_backend=args.gemm_backend))


def run_llama_bench(args) -> int:
    """``--benchmark latency``: time of ``generate`` on a batch of random prompts of one length, as
    src/torchinferno/benchmarks/torchinferno_llama.py:169-194.  ``--benchmark throughput``: ``--num-prompts``
    requests with prompt lengths uniform in ``--input-len-min .. --input-len`` submitted at once and run by the
    continuous-batching scheduler (prompt portions beside decoded tokens), as the throughput mode of
    src/torchinferno/cli.py:1776-1816; reports request, prompt and output tokens per second and the split of
    the steps."""
    import torch
    from torchinferno_b200.engine.types import GenerateRequest, SamplingConfig
    throughput = args.benchmark == "throughput"
    low = args.input_len if args.input_len_min is None else args.input_len_min
    if not 1 <= low <= args.input_len:
        raise SystemExit("--input-len-min must lie in 1 .. --input-len")
    running = min(args.max_batch_size, args.num_prompts) if throughput else args.batch_size
    args.max_batch_size = max(args.max_batch_size, running) if not throughput else args.max_batch_size
    if args.kv_cache_tokens is None:
        args.kv_cache_tokens = running * (args.input_len + args.output_len + args.page_size)
    with _bench_engine(args) as engine:
        if args.warm_up:
            engine.warm_up()          # (every batch size's decode step is captured before anything is timed)
        vocab = engine.model.spec.vocab_size
        g = torch.Generator().manual_seed(args.seed)
        count = args.num_prompts if throughput else args.batch_size
        latencies, record = [], {}
        for it in range(args.num_iters_warmup + args.num_iters):
            lengths = torch.randint(low, args.input_len + 1, (count,), generator=g).tolist()
            prompts = [torch.randint(0, vocab, (n,), generator=g).tolist() for n in lengths]
            requests = [GenerateRequest(f"bench-{it}-{i}", prompt_token_ids=p, sampling=SamplingConfig(
                args.output_len, args.temperature, (), args.seed + i)) for i, p in enumerate(prompts)]
            before = dict(engine.scheduler.stats)
            torch.cuda.synchronize()
            t0 = time.perf_counter()
            outputs = engine.generate_many(requests)
            torch.cuda.synchronize()
            if it >= args.num_iters_warmup:
                latencies.append(time.perf_counter() - t0)
                record = {k: engine.scheduler.stats[k] - before[k] for k in before}
                record["prompt_tokens"] = sum(lengths)
        tokens = sum(len(o.token_ids) for o in outputs)
    mean = sum(latencies) / len(latencies)
    line = {"benchmark": args.benchmark, "model": args.model, "dtype": args.dtype, "input_len": args.input_len,
            "output_len": args.output_len, "latency_s": round(mean, 4), "output_tokens_per_s": round(tokens / mean, 1)}
    if throughput:
        line.update({"num_prompts": count, "input_len_min": low, "max_batch_size": args.max_batch_size,
                     "requests_per_s": round(count / mean, 2),
                     "total_tokens_per_s": round((tokens + record["prompt_tokens"]) / mean, 1),
                     "steps": record["steps"], "ms_per_step": round(1e3 * mean / max(1, record["steps"]), 3),
                     "prefill_tokens": record["prefill_tokens"], "decode_tokens": record["decode_tokens"],
                     "preemptions": record["preemptions"]})
    else:
        line["batch_size"] = args.batch_size
    print(json.dumps(line))
    return 0


def build_parser() -> argparse.ArgumentParser:
    parser = argparse.ArgumentParser(prog="torchinferno-b200", description="B200-native Llama 3 inference engine")
    sub = parser.add_subparsers(dest="command", required=True)

    gen = sub.add_parser("generate", help="Generate from token ids with a model folder.")
    gen.add_argument("model", help="folder with config.json and model.safetensors")
    gen.add_argument("--input-ids", type=int, nargs="+", default=[1, 2, 3])
    gen.add_argument("--new-tokens", type=int, default=16)
    gen.add_argument("--temperature", type=float, default=0.0)
    gen.add_argument("--seed", type=int, default=0)
    gen.add_argument("--stop-token-ids", type=int, nargs="*", default=[])
    _engine_options(gen)
    gen.set_defaults(func=run_generate)

    text = sub.add_parser("text-generate", help="Tokenize text, generate, and decode.")
    text.add_argument("model")
    text.add_argument("prompt")
    text.add_argument("--tokenizer", default=None, help="tokenizer.json or its folder, defaults to model")
    text.add_argument("--new-tokens", type=int, default=16)
    text.add_argument("--temperature", type=float, default=0.0)
    text.add_argument("--seed", type=int, default=0)
    _engine_options(text)
    text.set_defaults(func=run_text_generate)

    rnd = sub.add_parser("random-model", help="Write a model folder with seeded random weights.")
    rnd.add_argument("config", help="a config.json")
    rnd.add_argument("output", help="folder to write")
    rnd.add_argument("--seed", type=int, default=0)
    rnd.add_argument("--dtype", choices=["bfloat16", "float32"], default="bfloat16")
    rnd.set_defaults(func=run_random_model)

    smoke = sub.add_parser("serve-smoke", help="Run a tiny random model through the whole engine.")
    smoke.add_argument("--max-active-requests", type=int, default=2)
    smoke.add_argument("--new-tokens", type=int, default=2)
    smoke.add_argument("--vocab-size", type=int, default=128)
    smoke.add_argument("--temperature", type=float, default=0.0)
    smoke.add_argument("--seed", type=int, default=0)
    _engine_options(smoke)
    smoke.set_defaults(func=run_serve_smoke)

    cap = sub.add_parser("capture-logits", help="Write the last position's logits to a JSON file.")
    cap.add_argument("model")
    cap.add_argument("output")
    cap.add_argument("--input-ids", type=int, nargs="+", default=[1, 2, 3])
    _engine_options(cap)
    cap.set_defaults(func=run_capture_logits)

    val = sub.add_parser("validate-logits", help="Compare the last position's logits with a captured file.")
    val.add_argument("model")
    val.add_argument("reference")
    val.add_argument("--atol", type=float, default=1e-4)
    val.add_argument("--rtol", type=float, default=1e-4)
    _engine_options(val)
    val.set_defaults(func=run_validate_logits)

    bench = sub.add_parser("llama-bench", help="Latency and throughput of generate on random prompts.")
    bench.add_argument("model")
    bench.add_argument("--input-len", type=int, default=32)
    bench.add_argument("--output-len", type=int, default=128)
    bench.add_argument("--batch-size", type=int, default=8)
    bench.add_argument("--num-iters-warmup", type=int, default=1)
    bench.add_argument("--num-iters", type=int, default=3)
    bench.add_argument("--temperature", type=float, default=1.0)
    bench.add_argument("--seed", type=int, default=0)
    bench.add_argument("--benchmark", choices=["latency", "throughput"], default="latency")
    bench.add_argument("--num-prompts", type=int, default=64, help="throughput: requests submitted at once")
    bench.add_argument("--warm-up", action="store_true", help="capture the decode step for every batch size before timing")
    bench.add_argument("--input-len-min", type=int, default=None,
                       help="prompt lengths are uniform in this .. --input-len (default: all --input-len)")
    bench.add_argument("--random-weights", action="store_true",
                       help="MODEL is a config.json (or a folder with one): build it with seeded random weights")
    _engine_options(bench)
    bench.set_defaults(func=run_llama_bench)
    return parser


def main(argv: list[str] | None = None) -> int:
    parser = build_parser()
    args = parser.parse_args(argv)
    return args.func(args)


if __name__ == "__main__":
    raise SystemExit(main())
