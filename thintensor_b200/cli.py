"""Command line: ``python -m thintensor_b200 {run,bench,validate,random} ...``

Option names and meanings follow the reference's ``thintensor`` command
(thinruntime/cli.py:165-264 for ``run``, :305-403 for ``bench``, :405-431 for
``validate``): ``--prompt``, ``--context`` (most prompt + new tokens), ``--max-new-tokens``
/ ``--steps``, ``--temperature``, ``--top-p``, ``--top-k``, ``--seed``, ``--device``,
``--dtype``, ``--tokenizer``, ``--json``; ``bench`` has ``--steps``, ``--warmup``,
``--prompt-token-ids``, ``--out``; ``validate`` has ``--require-tier``.  ``bench`` and
``validate`` also take ``--shape NAME`` in place of a model folder: random weights of a
named size.  What the reference's flags select among engines, profiles, quantisation and
residency has no counterpart here.  Unlike the reference, which refuses anything but greedy decoding
(thinruntime/cli.py:1940-1945), sampling options are honoured.
"""
from __future__ import annotations

import argparse
import json
import sys
import time
from pathlib import Path


SHAPE_NAMES = ("llama-3.2-1b", "llama-3.2-3b", "llama-3.1-8b", "tiny-a", "tiny-b")     # keys of config/shapes.json


def build_parser() -> argparse.ArgumentParser:
    parser = argparse.ArgumentParser(prog="thintensor_b200", description="Llama dense decoder on one B200")
    sub = parser.add_subparsers(dest="command", required=True)

    run = sub.add_parser("run", help="Generate tokens", formatter_class=argparse.ArgumentDefaultsHelpFormatter)
    run.add_argument("model", help="model folder (config.json + safetensors)")
    run.add_argument("--prompt", default="Hello", help="Input prompt (needs a tokenizer in the model folder or --tokenizer)")
    run.add_argument("--prompt-token-ids", action="append", help="Comma-separated prompt token ids; repeat for a batch")
    run.add_argument("--prompts-file", help="JSON file holding a list of token-id lists")
    run.add_argument("--context", type=int, default=512, help="Context length: most prompt + new tokens of a sequence")
    run.add_argument("--max-new-tokens", "--steps", dest="max_new_tokens", type=int, default=200, help="Maximum generated tokens")
    run.add_argument("--temperature", type=float, default=0.0, help="Sampling temperature; 0 is greedy")
    run.add_argument("--top-p", type=float, default=1.0, help="Nucleus mass; 1 switches it off")
    run.add_argument("--top-k", type=int, default=0, help="Keep the k most likely tokens; 0 switches it off")
    run.add_argument("--seed", type=int, default=0, help="Random seed")
    run.add_argument("--device", choices=["cuda"], default="cuda")
    run.add_argument("--dtype", choices=["bf16", "fp32"], default="bf16")
    run.add_argument("--tokenizer", help="Tokenizer directory")
    run.add_argument("--batch-size", type=int, default=8, help="Most sequences decoded together")
    run.add_argument("--ignore-eos", action="store_true", help="Always generate --max-new-tokens tokens")
    run.add_argument("--random-weights", type=int, metavar="SEED", help="Read only config.json from the folder and draw the weights from this seed")
    run.add_argument("--json", action="store_true", help="JSON output")

    bench = sub.add_parser("bench", help="Benchmark prefill and decode", formatter_class=argparse.ArgumentDefaultsHelpFormatter)
    bench.add_argument("model", nargs="?", help="model folder (or --shape)")
    bench.add_argument("--shape", choices=SHAPE_NAMES, help="Random weights of a named shape instead of a model folder")
    bench.add_argument("--steps", "--decode-steps", dest="steps", type=int, default=200, help="Timed decode steps")
    bench.add_argument("--warmup", type=int, default=10, help="Warmup decode steps")
    bench.add_argument("--prompt-token-ids", help="Comma-separated explicit prompt token ids used by every sequence")
    bench.add_argument("--prompt-len", default="128", help="Length of the synthetic prompts when no ids are given; LO:HI draws every "
                       "sequence's length uniformly from [LO, HI] with the seed (an unequal batch)")
    bench.add_argument("--batch", default="1", help="Sequences decoded together; a comma-separated list measures each")
    bench.add_argument("--context", type=int, help="Context length of a sequence (default: prompt + warm-up + steps)")
    bench.add_argument("--to-context", action="store_true", help="Decode until the longest sequence fills --context (sets --steps)")
    bench.add_argument("--peaks", help="JSON file with hbm_gbs and bf16_tflops, the denominators of the roofline fractions "
                       "(default: MEASURED_PEAKS.json in the working directory, else a stated fallback)")
    bench.add_argument("--profile-classes", action="store_true", help="Also time one decode step and one prefill step kernel class by "
                       "kernel class (CUDA events around every kernel, which then run one after another)")
    bench.add_argument("--seed", type=int, default=0)
    bench.add_argument("--device", choices=["cuda"], default="cuda")
    bench.add_argument("--dtype", choices=["bf16", "fp32"], default="bf16")
    bench.add_argument("--json", action="store_true")
    bench.add_argument("--out", help="Write JSON results to this file")

    validate = sub.add_parser("validate", help="Compare the engine's ways of running with reference logits (or its own 32-bit path)",
                              formatter_class=argparse.ArgumentDefaultsHelpFormatter)
    validate.add_argument("model", nargs="?", help="model folder (or --shape)")
    validate.add_argument("--shape", choices=SHAPE_NAMES, help="Random weights of a named shape, written to a temporary folder")
    validate.add_argument("--require-tier", choices=["ranking", "exact"], default="ranking", help="Minimum accepted correctness tier")
    validate.add_argument("--prompt-token-ids", help="Comma-separated token ids; default is a seeded synthetic sequence")
    validate.add_argument("--reference-logits", metavar="PATH", help="Logits from outside this engine to compare with: an .npz (logits [n, vocab], "
                          "optional positions [n] and tokens) or a folder of bin/trace_run output with the trace.jsonl that made it")
    validate.add_argument("--request", help="With a trace folder: the id of the request to compare (default: the trace's first)")
    validate.add_argument("--length", type=int, default=96, help="Length of the synthetic sequence")
    validate.add_argument("--seed", type=int, default=0)
    validate.add_argument("--device", choices=["cuda"], default="cuda")
    validate.add_argument("--dtype", choices=["bf16", "fp32"], default="bf16")
    validate.add_argument("--json", action="store_true")

    random = sub.add_parser("random", help="Write a model folder with random weights",
                            formatter_class=argparse.ArgumentDefaultsHelpFormatter)
    random.add_argument("out", help="folder to write config.json and model.safetensors into")
    random.add_argument("--config", required=True, help="config.json (or a folder holding one) that gives every size")
    random.add_argument("--seed", type=int, default=0)
    random.add_argument("--dtype", choices=["bfloat16", "float32"], default="bfloat16", help="stored dtype")
    return parser


def parse_ids(text: str) -> list[int]:
    try:
        return [int(part) for part in text.replace(" ", "").split(",") if part]
    except ValueError as exc:
        raise SystemExit(f"token ids must be comma-separated integers: {exc}")


def load_tokenizer(model: Path, override: str | None):
    """A tokenizer found next to the model or at ``--tokenizer``; used as a black box,
    as the reference does (thinruntime/cli.py:4661-4721)."""
    where = Path(override) if override else model
    if not any((where / name).is_file() for name in ("tokenizer.json", "tokenizer.model", "tokenizer_config.json")):
        raise SystemExit(f"no tokenizer files in {where}; pass --prompt-token-ids or --tokenizer DIR")
    from transformers import AutoTokenizer

    return AutoTokenizer.from_pretrained(str(where))


def cmd_run(args) -> int:
    import thintensor_b200

    if args.max_new_tokens <= 0:
        raise SystemExit("--max-new-tokens must be positive")
    if args.context <= 0:
        raise SystemExit("--context must be positive")
    tokenizer = None
    if args.prompts_file:
        prompts = json.loads(Path(args.prompts_file).read_text())
    elif args.prompt_token_ids:
        prompts = [parse_ids(p) for p in args.prompt_token_ids]
    else:
        tokenizer = load_tokenizer(Path(args.model), args.tokenizer)
        prompts = [tokenizer(args.prompt)["input_ids"]]
    if args.random_weights is not None:
        from thintensor_b200.config.base import read_config_json

        runtime = thintensor_b200.random_model(read_config_json(args.model), seed=args.random_weights, dtype=args.dtype, device=args.device)
    else:
        runtime = thintensor_b200.load_model(args.model, dtype=args.dtype, device=args.device)
    started = time.perf_counter()
    outputs = runtime.generate(
        prompts, max_new_tokens=args.max_new_tokens, temperature=args.temperature, top_p=args.top_p, top_k=args.top_k,
        seed=args.seed, stop_ids=() if args.ignore_eos else None, context=args.context, batch_size=args.batch_size,
    )
    elapsed = time.perf_counter() - started
    new_tokens = sum(len(o) for o in outputs)
    if args.json:
        print(json.dumps({
            "prompt_token_ids": prompts, "generated_token_ids": outputs, "new_tokens": new_tokens,
            "seconds": elapsed, "tokens_per_s": new_tokens / elapsed if elapsed > 0 else None,
            "dtype": args.dtype, "temperature": args.temperature, "top_p": args.top_p, "top_k": args.top_k, "seed": args.seed,
        }))
    else:
        for prompt, output in zip(prompts, outputs):
            print(tokenizer.decode(output) if tokenizer is not None else ",".join(str(t) for t in output))
        print(f"[{new_tokens} tokens in {elapsed:.3f} s]", file=sys.stderr)
    return 0


def cmd_bench(args) -> int:
    """Prefill and decode rates with the bytes and FLOP behind them and the fraction of the device's
    peaks they reach, after the reference's per-shape bandwidth report (scripts/thin_runtime.py:602-645)
    and its static byte model (thinruntime/gpu_runtime.py:10781-10885)."""
    import torch

    import thintensor_b200
    from thintensor_b200.benchmark import SHAPES, measure_classes, measure_decode, measure_prefill, peaks, roofline

    if (args.model is None) == (args.shape is None):
        raise SystemExit("bench needs a model folder or --shape, not both")
    pk = peaks(args.peaks)
    if args.shape:
        runtime = thintensor_b200.random_model(SHAPES[args.shape], seed=args.seed, dtype=args.dtype, device=args.device)
    else:
        runtime = thintensor_b200.load_model(args.model, dtype=args.dtype, device=args.device)
    batches = parse_ids(args.batch)
    if not batches or min(batches) <= 0:
        raise SystemExit("--batch must name positive numbers of sequences")
    vocab = runtime.model.spec.vocab_size
    g = torch.Generator().manual_seed(args.seed)

    def prompts_for(batch: int) -> list[list[int]]:
        if args.prompt_token_ids:
            return [parse_ids(args.prompt_token_ids)] * batch
        try:
            low, _, high = args.prompt_len.partition(":")
            low, high = int(low), int(high or low)
        except ValueError:
            raise SystemExit("--prompt-len takes N or LO:HI")
        if not 0 < low <= high:
            raise SystemExit("--prompt-len needs 0 < LO <= HI")
        lengths = [low] * batch if low == high else torch.randint(low, high + 1, (batch,), generator=g).tolist()
        return [torch.randint(0, vocab, (n,), generator=g).tolist() for n in lengths]

    runs = []
    for batch in batches:
        prompts = prompts_for(batch)
        longest = max(len(p) for p in prompts)
        warmup = max(args.warmup, 2)
        steps = args.steps
        if args.to_context:
            if not args.context:
                raise SystemExit("--to-context needs --context")
            steps = args.context - longest - warmup - 1
            if steps <= 0:
                raise SystemExit(f"a prompt of {longest} tokens leaves no room to decode in a context of {args.context}")
        context = args.context or longest + warmup + steps + 1
        prefill = measure_prefill(runtime, prompts, repeats=3)
        decode = measure_decode(runtime, prompts, context, warmup, steps)
        lines = roofline(decode, prefill if args.dtype == "bf16" else None, pk)
        run = {
            "batch_size": batch, "prompt_tokens": [len(p) for p in prompts] if len({len(p) for p in prompts}) > 1 else longest,
            "steps": steps, "warmup_steps": warmup, "context": context, "mean_context": decode["mean_context"],
            "tokens_per_s": decode["tokens_per_s"], "ms_per_step": decode["ms_per_step"], "launches_per_step": decode["launches_per_step"],
            "bytes_per_step": int(decode["bytes_per_step"]), "decode_gbs": lines["decode"]["achieved_gbs"],
            "decode_frac_of_hbm_peak": lines["decode"]["frac"] if args.dtype == "bf16" else None,
            "prefill_tokens": prefill["tokens"], "prefill_tokens_per_s": prefill["tokens_per_s"], "prefill_ms": prefill["ms"],
            "prefill_flops": prefill["flops"], "prefill_tflops": prefill["flops"] / (prefill["ms"] / 1e3) / 1e12,
            "prefill_frac_of_tensor_peak": lines["prefill"]["frac"] if "prefill" in lines else None,
        }
        if args.profile_classes:
            run["classes"] = measure_classes(runtime, prompts, context)
        runs.append(run)
    first = runs[0]
    result = {
        "model": str(args.model or args.shape), "dtype": args.dtype, "peaks": pk,
        "batch_size": first["batch_size"], "prompt_tokens": first["prompt_tokens"], "steps": first["steps"],
        "warmup_steps": first["warmup_steps"], "context": first["context"],
        "tokens_per_s": first["tokens_per_s"], "ms_per_token": first["ms_per_step"],
        "prefill_tokens_per_s": first["prefill_tokens_per_s"], "prefill_ms": first["prefill_ms"],
        "batches": runs,
    }
    text = json.dumps(result, indent=None if args.json else 2)
    if args.out:
        Path(args.out).write_text(text + "\n")
    print(text)
    return 0


def cmd_validate(args) -> int:
    from thintensor_b200.validate import validate_model

    ids = parse_ids(args.prompt_token_ids) if args.prompt_token_ids else None
    if (args.model is None) == (args.shape is None):
        raise SystemExit("validate needs a model folder or --shape, not both")
    if args.shape:
        import tempfile

        import thintensor_b200
        from thintensor_b200.benchmark import SHAPES

        with tempfile.TemporaryDirectory() as folder:      # both dtypes are read from the same file
            thintensor_b200.save_random_model(folder, SHAPES[args.shape], seed=args.seed, dtype="bfloat16")
            report = validate_model(folder, dtype=args.dtype, tokens=ids, length=args.length, seed=args.seed,
                                    reference_logits=args.reference_logits, request=args.request)
    else:
        report = validate_model(args.model, dtype=args.dtype, tokens=ids, length=args.length, seed=args.seed,
                                reference_logits=args.reference_logits, request=args.request)
    print(json.dumps(report) if args.json else json.dumps(report, indent=2))
    order = {"fail": 0, "ranking_pass": 1, "exact_pass": 2}
    needed = {"ranking": 1, "exact": 2}[args.require_tier]
    return 0 if order[report["tier"]] >= needed else 1


def cmd_random(args) -> int:
    import thintensor_b200
    from thintensor_b200.config.base import read_config_json

    folder = thintensor_b200.save_random_model(args.out, read_config_json(args.config), seed=args.seed, dtype=args.dtype)
    print(str(folder))
    return 0


def main(argv: list[str] | None = None) -> int:
    args = build_parser().parse_args(argv)
    handler = {"run": cmd_run, "bench": cmd_bench, "validate": cmd_validate, "random": cmd_random}[args.command]
    try:
        return handler(args)
    except (ValueError, RuntimeError) as exc:
        print(f"error: {exc}", file=sys.stderr)
        return 2


if __name__ == "__main__":
    sys.exit(main())
