"""Headline benchmark: decode tokens per second of the Llama-3.2-1B shape in bfloat16
with random weights at batch 8 and a 4,096-token context, on one B200.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--impl ours|reference]

A "step" is one decode step of the whole batch.  The run prefills 2,048-token prompts,
does W untimed decode steps, times K steps with CUDA events (no host synchronisation
inside; every step reads all weights, 2.47 GB, far more than the 126 MB L2, so steps
cannot serve each other from cache) and prints ONE JSON line.  The same line carries
the end-to-end number through ``Runtime.generate`` (host token lists in and out, a
host-to-device and a device-to-host copy every step), the prefill of 2,048 tokens, the
decode roofline, and decode at batch 1 and 64.  More than one GPU is not supported.
"""
from __future__ import annotations

import argparse
import json
import statistics
import subprocess
import sys
import threading
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

# Every size comes from the package's table of named shapes (whole config.json dicts, kept as
# data).  --shape picks another one for `--only` measurements; the headline stays the 1B shape.
SHAPES = json.loads((ROOT / "thintensor_b200" / "config" / "shapes.json").read_text(encoding="utf-8"))
SHAPE_NAMES = {"1b": "llama-3.2-1b", "3b": "llama-3.2-3b", "8b": "llama-3.1-8b"}
CONTEXT = 4096
PROMPT = 2048
BATCH = 8
METRIC = "decode tok/s at batch 8 (Llama-3.2-1B bf16, 2,048-token prompts, context 4,096)"


def peaks() -> dict:
    """Measured peaks if the driver wrote them next to this file, else the stated fallback."""
    from thintensor_b200.benchmark import peaks as read_peaks

    file = ROOT / "MEASURED_PEAKS.json"
    return read_peaks(file if file.is_file() else None)


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""

    QUERY = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self):
        self.lines: list[str] = []
        self.process = None

    def __enter__(self):
        try:
            self.process = subprocess.Popen(
                ["nvidia-smi", "-i", "0", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits", "-lms", "100"],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._read, daemon=True).start()
        except OSError:
            self.process = None
        return self

    def _read(self):
        for line in self.process.stdout:
            self.lines.append(line.strip())

    def __exit__(self, *exc):
        if self.process is not None:
            time.sleep(0.15)
            self.process.terminate()
            try:
                self.process.wait(timeout=5)
            except subprocess.TimeoutExpired:
                self.process.kill()

    def summary(self) -> dict:
        sm, top, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in self.lines:
            parts = [p.strip() for p in line.split(",")]
            if len(parts) < 6:
                continue
            try:
                sm.append(float(parts[0]))
                top.append(float(parts[1]))
            except ValueError:
                continue
            for name, value in zip(names, parts[2:6]):
                if value.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(top) if top else None,
                "reasons": sorted(reasons), "samples": len(sm)}


def reference_arm(config: dict, steps: int, warmup: int) -> int:
    """The unmodified reference from baseline/_ref on the same shape and workload."""
    sys.path.insert(0, str(ROOT / "baseline"))
    try:
        import reference_arm as arm

        line = arm.run(config, METRIC, BATCH, PROMPT, CONTEXT, steps, max(warmup, 3))
    except Exception as exc:  # noqa: BLE001 - the arm must always print a line and exit 0
        line = {"impl": "reference", "unavailable": f"the reference failed to run: {type(exc).__name__}: {str(exc)[:300]}"}
    print(json.dumps(line))
    return 0


def main() -> int:
    parser = argparse.ArgumentParser()
    parser.add_argument("--gpus", type=int, default=1)
    parser.add_argument("--steps", type=int, default=256)
    parser.add_argument("--warmup", type=int, default=8)
    parser.add_argument("--impl", choices=["ours", "reference"], default="ours")
    parser.add_argument("--layers", type=int, default=None, help="fewer layers than the configuration has (both numbers are reported)")
    parser.add_argument("--skip-points", action="store_true", help="leave out decode at batch 1 and 64")
    parser.add_argument("--only", choices=["decode", "prefill"], help="run one phase only and print its numbers (for profiling)")
    parser.add_argument("--batch", type=int, default=BATCH, help="with --only decode: sequences decoded together")
    parser.add_argument("--shape", choices=sorted(SHAPE_NAMES), default="1b", help="with --only: layer sizes of another model of the family")
    parser.add_argument("--prompt-len", type=int, default=PROMPT, help="with --only: tokens per prompt (the context is this plus room for the steps)")
    args = parser.parse_args()
    if args.impl == "reference":
        return reference_arm(dict(SHAPES[SHAPE_NAMES["1b"]]), min(args.steps, 128), args.warmup)
    if args.gpus != 1:
        print("bench.py measures one GPU only: this library does not run on several GPUs")
        return 2
    if args.warmup < 3:
        args.warmup = 3

    import torch

    import thintensor_b200
    from thintensor_b200.benchmark import class_fractions, measure_classes, measure_decode, measure_prefill
    from thintensor_b200.engine.generate import GenerationStats

    pk = peaks()
    raw = dict(SHAPES[SHAPE_NAMES[args.shape if args.only else "1b"]])
    full_layers = raw["num_hidden_layers"]
    if args.layers is not None:
        raw["num_hidden_layers"] = args.layers
    prompt_len = args.prompt_len if args.only else PROMPT
    if prompt_len != PROMPT:
        raw["max_position_embeddings"] = max(raw.get("max_position_embeddings", 0), 2 * prompt_len)
    runtime = thintensor_b200.random_model(raw, seed=0, dtype="bf16", device="cuda:0")
    vocab = raw["vocab_size"]
    g = torch.Generator().manual_seed(1)
    prompts = [torch.randint(0, vocab, (prompt_len,), generator=g).tolist() for _ in range(max(64, args.batch) if args.only == "decode" else 64)]

    if args.only == "decode":
        context = CONTEXT if prompt_len == PROMPT else prompt_len + args.warmup + args.steps + 64
        print(json.dumps(measure_decode(runtime, prompts[:args.batch], context, args.warmup, args.steps)))
        return 0
    if args.only == "prefill":
        print(json.dumps(measure_prefill(runtime, prompts[0], repeats=max(1, args.steps), warmup=args.warmup)))
        return 0

    with ClockSampler() as clocks:
        decode = measure_decode(runtime, prompts[:BATCH], CONTEXT, args.warmup, args.steps)
    points = {}
    if not args.skip_points:
        for batch in (1, 64):
            steps = min(args.steps, 128)
            points[f"decode_b{batch}"] = round(measure_decode(runtime, prompts[:batch], CONTEXT, args.warmup, steps)["tokens_per_s"], 1)
    prefill = measure_prefill(runtime, prompts[0], repeats=3, warmup=2)

    # end to end through the public entry point: host token lists in, host token lists out,
    # tokens copied up from pinned memory and read back every step (a stop id that no
    # token equals keeps the loop on the path that looks at every token)
    e2e_steps = min(args.steps, 128)
    stats = GenerationStats()
    runtime.generate(prompts[:BATCH], max_new_tokens=e2e_steps + 1, stop_ids=(-1,), batch_size=BATCH, context=CONTEXT)  # warm-up, same shape
    runtime.generate(prompts[:BATCH], max_new_tokens=e2e_steps + 1, stop_ids=(-1,), batch_size=BATCH, context=CONTEXT, stats=stats)
    e2e_value = stats.decoded_tokens / stats.decode_seconds if stats.decode_seconds > 0 else None

    # where the two steps' time goes, by class of kernel, each against its own bound
    spans = measure_classes(runtime, prompts[:BATCH], CONTEXT, prefill_prompts=prompts[:1])
    classes = class_fractions(runtime.model, spans, pk, prompts[:1], BATCH, spans["mean_context"])

    achieved = decode["bytes_per_step"] / (decode["ms_per_step"] / 1e3) / 1e9
    line = {
        "metric": METRIC,
        "value": round(decode["tokens_per_s"], 1),
        "unit": "tokens/s",
        "n_gpus": 1,
        "steps": args.steps,
        "warmup": args.warmup,
        "ms_per_step": round(decode["ms_per_step"], 4),
        "higher_is_better": True,
        "scaling": "weak",
        "vs_baseline": None,
        "dtype": "bf16",
        "data": "synthetic: random weights N(0, 0.02) from a seed, token ids uniform in [0, vocab)",
        "impl": "ours",
        "config": {
            "model": "Llama-3.2-1B shape", "layers": raw["num_hidden_layers"], "layers_of_configuration": full_layers,
            "hidden_size": raw["hidden_size"], "heads": raw["num_attention_heads"], "kv_heads": raw["num_key_value_heads"],
            "head_dim": raw["head_dim"], "intermediate_size": raw["intermediate_size"], "vocab_size": vocab,
            "tied_embeddings": True, "rope": "llama3 factor 32", "global_batch": BATCH, "prompt_len": PROMPT,
            "seq_len": CONTEXT, "parallelism": "none (1 GPU)",
            "l2": "every step reads all weights (2.47 GB > 126 MB L2)", "peaks": pk["source"],
        },
        "clocks": clocks.summary(),
        "e2e": {"value": None if e2e_value is None else round(e2e_value, 1), "unit": "tokens/s", "steps": e2e_steps,
                "h2d_bytes_per_step": 4 * BATCH, "d2h_bytes_per_step": 4 * BATCH},
        "gpu_launches": int(decode["launches_per_step"] * args.steps),
        "prefill": {"value": round(prefill["tokens_per_s"], 1), "tokens": prefill["tokens"], "ms": round(prefill["ms"], 3),
                    "frac": round(prefill["flops"] / (prefill["ms"] / 1e3) / (pk["bf16_tflops"] * 1e12), 4)},
        "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": pk["hbm_gbs"], "unit": "GB/s",
                     "frac": round(achieved / pk["hbm_gbs"], 4), "of": pk["source"]},
        "points": points,
        "classes": classes,
    }
    print(json.dumps(line))
    return 0


if __name__ == "__main__":
    sys.exit(main())
