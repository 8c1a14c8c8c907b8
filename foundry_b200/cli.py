"""The `foundry` command line: `run` and `bench`, with the reference's option
names and meanings (src/cli/mod.rs:29-136).

    foundry run   --model DIR --prompt-ids 1,2,3 --max-new-tokens N
    foundry bench --model DIR --prompt-tokens P --new-tokens N --out DIR [...]

Differences: `--model` is a folder holding config.json and model.safetensors
(the reference resolves `owner/name` in the local Hugging Face cache,
src/cli/command.rs:314-347); `--prompt-ids` may be repeated for a batch;
`--temperature`, `--seed`, `--dtype` are added. The reference's `eval`
subcommand compares with other engines' recorded activations; its place is
taken by `bin/trace_run`.
"""
from __future__ import annotations

import argparse
import datetime
import json
import logging
import os
import subprocess
import sys
from typing import List, Optional

log = logging.getLogger("foundry")


def _ids(text: str) -> List[int]:
    try:
        ids = [int(t) for t in text.split(",") if t.strip() != ""]
    except ValueError:
        raise argparse.ArgumentTypeError(f"not a comma-separated list of token ids: {text!r}")
    if not ids or any(i < 0 for i in ids):
        raise argparse.ArgumentTypeError("prompt ids must be non-negative and not empty")
    return ids


def build_parser() -> argparse.ArgumentParser:
    parser = argparse.ArgumentParser(prog="foundry", description="Foundry LLM inference engine (B200).")
    sub = parser.add_subparsers(dest="command", required=True)
    run = sub.add_parser("run", help="Generate token IDs from prompt token IDs and print them as JSON.")
    run.add_argument("--model", required=True, help="Model folder (config.json, model.safetensors).")
    run.add_argument("--prompt-ids", required=True, type=_ids, action="append",
                     help="Prompt token IDs, comma-separated. Repeat for a batch.")
    run.add_argument("--max-new-tokens", required=True, type=int,
                     help="Maximum number of generated tokens.")
    run.add_argument("--temperature", type=float, default=0.0, help="0 selects greedily.")
    run.add_argument("--seed", type=int, default=0, help="Seed of temperature sampling.")
    run.add_argument("--dtype", default="bfloat16", choices=["bfloat16", "float32"])
    run.add_argument("--ignore-eos", action="store_true")

    bench = sub.add_parser("bench", help="Benchmark prefill and greedy decode on random token IDs "
                                         "and write report.json.")
    bench.add_argument("--model", required=True)
    bench.add_argument("--prompt-tokens", required=True, type=int,
                       help="Prompt tokens processed in one prefill; 0 benchmarks generation only.")
    bench.add_argument("--new-tokens", required=True, type=int,
                       help="Exactly N new tokens, including the prefill output; 0 measures only "
                            "prompt processing.")
    bench.add_argument("--timing-scope", default="generation", choices=["forward", "generation"],
                       help="Time forwards through logits or generation through host token "
                            "availability.")
    bench.add_argument("--depth", type=int, default=0,
                       help="Tokens filled into the cache before each measured run.")
    bench.add_argument("--warmup-runs", type=int, default=1, help="Minimum number of warmup runs.")
    bench.add_argument("--warmup-ms", type=int, default=0,
                       help="Minimum warmup duration in milliseconds.")
    bench.add_argument("--runs", type=int, default=10, help="Number of measured runs.")
    bench.add_argument("--batch-size", type=int, default=1,
                       help="Sequences generated together, each with its own random prompt of "
                            "the same length.")
    bench.add_argument("--seed", type=int, default=0, help="Seed of the random token IDs.")
    bench.add_argument("--profile", choices=["steps", "kernels"], default=None,
                       help="Record device dispatches, allocations and GPU busy time per step; "
                            "steps keeps execution unchanged, kernels also times each kernel with "
                            "one launch at a time (no graph replay), which slows wall times.")
    bench.add_argument("--dtype", default="bfloat16", choices=["bfloat16", "float32"])
    bench.add_argument("--out", required=True, help="Directory that receives report.json.")
    return parser


def check_token_ids(prompts, vocab_size: int) -> None:
    """Every prompt id must be inside the vocabulary (src/cli/command.rs:362-378)."""
    for prompt in prompts:
        for t in prompt:
            if not 0 <= t < vocab_size:
                raise SystemExit(f"token id {t} is outside the vocabulary of {vocab_size}")


def write_token_ids(out, token_ids) -> None:
    """`[1,2,3]` and a newline (src/cli/command.rs:493-503)."""
    out.write("[" + ",".join(str(t) for t in token_ids) + "]\n")


def _git_commit() -> Optional[str]:
    try:
        root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
        return subprocess.run(["git", "-C", root, "rev-parse", "HEAD"], capture_output=True,
                              text=True, timeout=5).stdout.strip() or None
    except Exception:
        return None


def cmd_run(args) -> int:
    from .cache.pages import PAGE, pages_for
    from .config import load_model_config
    from .engine import Engine
    from .sampling import SamplingParams
    _, config = load_model_config(args.model)
    check_token_ids(args.prompt_ids, config.vocab_size)
    # the cache holds prompt + new tokens of every prompt (src/cli/command.rs:91-101)
    need = sum(pages_for(len(p) + args.max_new_tokens) * PAGE for p in args.prompt_ids)
    engine = Engine.from_folder(args.model, dtype=args.dtype, max_tokens=need,
                                max_slots=len(args.prompt_ids))
    out = engine.generate(args.prompt_ids, args.max_new_tokens,
                          sampling=SamplingParams(args.temperature, args.seed),
                          ignore_eos=args.ignore_eos)
    log.info("Generated tokens. prompt_tokens=%s generated_tokens=%s prefill_ms=%.1f "
             "decode_steps=%d decode_ms_total=%.1f", [len(p) for p in args.prompt_ids],
             [len(r) for r in out.token_ids], out.prefill * 1e3, len(out.decode_steps),
             sum(out.decode_steps) * 1e3)
    for row in out.token_ids:
        write_token_ids(sys.stdout, row)
    return 0


def cmd_bench(args) -> int:
    import torch
    from .bench import BenchConfig, run_bench
    from .cache.pages import PAGE, pages_for
    from .engine import Engine
    from .weights import WeightFiles
    cfg = BenchConfig(args.prompt_tokens, args.new_tokens, args.timing_scope, args.depth,
                      args.warmup_runs, args.warmup_ms, args.runs, args.batch_size, args.seed,
                      args.profile)
    per_seq = cfg.depth + cfg.prompt_tokens + cfg.decode_step_count()  # command.rs:152-169
    engine = Engine.from_folder(args.model, dtype=args.dtype,
                                max_tokens=max(PAGE, pages_for(per_seq) * PAGE * cfg.batch_size),
                                max_slots=cfg.batch_size)
    files = WeightFiles.open(args.model)
    report = run_bench(engine, cfg)
    record = {
        "metadata": {
            "git_commit": _git_commit(),
            "test_time": datetime.datetime.now(datetime.timezone.utc).isoformat(),
            "device": "cuda", "device_name": torch.cuda.get_device_name(engine.device),
            "model_id": os.path.abspath(args.model), "model_bytes": files.nbytes(),
            "model_parameter_count": files.numel(),
        },
        **report,
    }
    os.makedirs(args.out, exist_ok=True)
    path = os.path.join(args.out, "report.json")
    with open(path, "w") as handle:
        json.dump(record, handle, indent=2)
        handle.write("\n")
    m = report["metrics"]
    log.info("Benchmarked the model. prompt_tokens_per_s=%s decode_tokens_per_s=%s report=%s",
             m["prompt_tokens_per_s"] and m["prompt_tokens_per_s"]["mean"],
             m["decode_tokens_per_s"] and m["decode_tokens_per_s"]["mean"], path)
    return 0


def main(argv=None) -> int:
    logging.basicConfig(stream=sys.stderr, level=logging.INFO, format="%(levelname)s %(message)s")
    args = build_parser().parse_args(argv)
    return {"run": cmd_run, "bench": cmd_bench}[args.command](args)


if __name__ == "__main__":
    sys.exit(main())
