"""The `foundry` command line: `run` and `bench`, with the reference's option
names and meanings (src/cli/mod.rs:29-136).

    foundry run   --model DIR --prompt-ids 1,2,3 --max-new-tokens N
    foundry bench --model DIR --prompt-tokens P --new-tokens N --out DIR [...]

Differences: `--model` is a folder holding config.json and model.safetensors
(the reference resolves `owner/name` in the local Hugging Face cache,
src/cli/command.rs:314-347); `--prompt-ids` may be repeated for a batch;
`--temperature`, `--seed`, `--dtype` are added, and `--config NAME
--random-weights SEED` stands in for a folder (with `--max-seq-len` / `--context`
sizing the cache); the report also holds the step's bytes and operations and
the fractions of the memory's and the tensor cores' rates they reach. The reference's `eval`
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


def _add_model_options(sub, with_context: str) -> None:
    sub.add_argument("--model", help="Folder with config.json and model.safetensors.")
    sub.add_argument("--config", help="A named configuration instead of a folder "
                                      "(llama-3.2-1b, llama-3.2-3b, llama-3.1-8b, tiny-a, tiny-b); "
                                      "needs --random-weights.")
    sub.add_argument("--random-weights", type=int, metavar="SEED", default=None,
                     help="Draw the weights of --config from this seed on the device.")
    sub.add_argument("--dtype", default="bfloat16", choices=["bfloat16", "float32"],
                     help="bfloat16 is the serving path; float32 runs everything in 32 bits.")
    sub.add_argument(with_context, type=int, default=None, metavar="TOKENS",
                     help="Cache tokens kept per sequence (default: what the request needs).")


def build_parser() -> argparse.ArgumentParser:
    parser = argparse.ArgumentParser(prog="foundry", description="Token generation with the "
                                     "foundry_b200 engine on one B200.")
    sub = parser.add_subparsers(dest="command", required=True)
    run = sub.add_parser("run", help="Continue prompts given as token ids; one JSON array of new "
                                     "ids per prompt goes to standard output.")
    _add_model_options(run, "--max-seq-len")
    run.add_argument("--prompt-ids", required=True, type=_ids, action="append",
                     help="A prompt as comma-separated token ids; give the option again for "
                          "each further prompt of the batch.")
    run.add_argument("--max-new-tokens", required=True, type=int,
                     help="Upper bound of new tokens per prompt.")
    run.add_argument("--temperature", type=float, default=0.0,
                     help="Sampling temperature; 0 always takes the most likely token.")
    run.add_argument("--seed", type=int, default=0, help="Seed of the sampling streams.")
    run.add_argument("--ignore-eos", action="store_true", help="Do not stop at stop tokens.")

    bench = sub.add_parser("bench", help="Time prompt processing and greedy decoding on seeded "
                                         "random token ids; report.json goes to --out.")
    _add_model_options(bench, "--context")
    bench.add_argument("--prompt-tokens", required=True, type=int,
                       help="Length of every prompt, processed as one step; with 0 only decoding "
                            "is timed, from random start ids.")
    bench.add_argument("--new-tokens", required=True, type=int,
                       help="New tokens per sequence, the prompt step's token being the first; "
                            "with 0 only the prompt step is timed.")
    bench.add_argument("--timing-scope", default="generation", choices=["forward", "generation"],
                       help="Where a step's clock stops: forward = the logits exist on the "
                            "device; generation = the chosen token is on the host.")
    bench.add_argument("--depth", type=int, default=0,
                       help="Tokens put into each sequence's cache, untimed, before a run.")
    bench.add_argument("--warmup-runs", type=int, default=1, help="Untimed runs first, at least.")
    bench.add_argument("--warmup-ms", type=int, default=0,
                       help="Keep warming up until this many milliseconds have passed.")
    bench.add_argument("--runs", type=int, default=10, help="Timed runs.")
    bench.add_argument("--batch-size", type=int, default=1,
                       help="Sequences per run; each draws its own prompt of --prompt-tokens ids.")
    bench.add_argument("--seed", type=int, default=0, help="Seed of the token ids.")
    bench.add_argument("--profile", choices=["steps", "kernels"], default=None,
                       help="Add per-step kernel counts and allocations to the report (steps), "
                            "or also each kernel's GPU time, launched one at a time without "
                            "graph replay, which lengthens the wall times (kernels).")
    bench.add_argument("--peaks", default=None, metavar="FILE",
                       help="JSON with measured hbm_gbs and bf16_tflops to hold the rates "
                            "against (default: $FOUNDRY_B200_PEAKS, else built-in figures).")
    bench.add_argument("--out", required=True, help="Folder for report.json (made if absent).")
    return parser


def check_model_options(args) -> None:
    """Exactly one of `--model DIR` and `--config NAME --random-weights SEED`."""
    if (args.model is None) == (args.config is None):
        raise SystemExit("give either --model DIR or --config NAME --random-weights SEED")
    if args.model is not None and args.random_weights is not None:
        raise SystemExit("--random-weights goes with --config, not with --model")
    if args.config is not None:
        from .bench.presets import preset
        if args.random_weights is None:
            raise SystemExit("--config needs --random-weights SEED")
        try:
            preset(args.config)
        except ValueError as exc:
            raise SystemExit(str(exc))


def open_engine(args, max_tokens: int, max_slots: int):
    """The engine `--model DIR` or `--config NAME --random-weights SEED` names,
    and what the report says about the weights (id, bytes, parameters)."""
    from .engine import Engine
    check_model_options(args)
    if args.model is not None:
        from .weights import WeightFiles
        engine = Engine.from_folder(args.model, dtype=args.dtype, max_tokens=max_tokens,
                                    max_slots=max_slots)
        files = WeightFiles.open(args.model)
        return engine, {"model_id": os.path.abspath(args.model), "model_bytes": files.nbytes(),
                        "model_parameter_count": files.numel()}
    from .bench.presets import preset
    engine = Engine.from_random(preset(args.config), args.random_weights, dtype=args.dtype, max_tokens=max_tokens,
                                max_slots=max_slots)
    expected = engine.model.expected_tensors()
    count = sum(_numel(e.shape) for e in expected.values())
    size = 2 if args.dtype == "bfloat16" else 4
    return engine, {"model_id": f"{args.config} (random weights, seed {args.random_weights})",
                    "model_bytes": count * size, "model_parameter_count": count}


def _numel(shape) -> int:
    n = 1
    for d in shape:
        n *= int(d)
    return n


def _vocab_size(args) -> int:
    check_model_options(args)
    if args.model is not None:
        from .config import load_model_config
        return load_model_config(args.model)[1].vocab_size
    from .bench.presets import preset
    return int(preset(args.config)["vocab_size"])


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
    from .sampling import SamplingParams
    check_token_ids(args.prompt_ids, _vocab_size(args))
    # the cache holds prompt + new tokens of every prompt (src/cli/command.rs:91-101)
    per_seq = [len(p) + args.max_new_tokens for p in args.prompt_ids]
    if args.max_seq_len is not None:
        if args.max_seq_len < max(per_seq):
            raise SystemExit(f"--max-seq-len {args.max_seq_len} is less than the {max(per_seq)} "
                             f"tokens a prompt and its new tokens take")
        per_seq = [args.max_seq_len] * len(per_seq)
    need = sum(pages_for(n) * PAGE for n in per_seq)
    engine, _ = open_engine(args, need, len(args.prompt_ids))
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
    from .bench.costs import load_peaks
    from .cache.pages import PAGE, pages_for
    cfg = BenchConfig(args.prompt_tokens, args.new_tokens, args.timing_scope, args.depth,
                      args.warmup_runs, args.warmup_ms, args.runs, args.batch_size, args.seed,
                      args.profile)
    per_seq = cfg.depth + cfg.prompt_tokens + cfg.decode_step_count()  # command.rs:152-169
    if args.context is not None:
        if args.context < per_seq:
            raise SystemExit(f"--context {args.context} is less than the {per_seq} tokens a "
                             f"sequence of this run comes to hold")
        per_seq = args.context
    engine, weights = open_engine(args, max(PAGE, pages_for(per_seq) * PAGE * cfg.batch_size),
                                  cfg.batch_size)
    report = run_bench(engine, cfg, load_peaks(args.peaks))
    record = {
        "metadata": {
            "git_commit": _git_commit(),
            "test_time": datetime.datetime.now(datetime.timezone.utc).isoformat(),
            "device": "cuda", "device_name": torch.cuda.get_device_name(engine.device),
            "dtype": args.dtype, **weights,
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
