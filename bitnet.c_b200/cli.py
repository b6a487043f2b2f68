"""Command line in the manner of the reference's ``./bitnet <model.gguf> [options]`` (src/main.c:110-168).

Option names and meanings are the reference's where it has them: ``-p``, ``--prompt-token-ids``,
``-n``, ``--temp``, ``--topp``, ``--seed``, ``--maxseq``, ``--repeat-penalty``, ``--no-prefill``,
``--quiet``, ``--token-ids``, ``--benchmark-runs``, ``--benchmark-warmup-runs``, with the same defaults
(256 tokens, temperature 0 = greedy, top-p 0.9, seed 42, repeat penalty 1.1 over 64 tokens).  The model
is a folder with ``config.json`` and ``model.safetensors`` instead of a GGUF file.  New here:
``--random-weights`` writes such a folder from ``--config`` and ``--weight-seed``; ``--dtype`` picks
bfloat16 or true float32; ``--prompt-token-ids`` may be given several times for a batch.  Options of
the reference that select CPU threads, other backends, quantized caches, speculative decoding, chat
mode or diagnostics of its GPU backends have no counterpart.  Its tensor dumps (``--dump-binary``,
``--dump-tag``, ``--dump-layer``, ``--dump-pos``) are here, with ``--dump-stats`` for its text line of
statistics, ``--top-logits`` for its BN_TOP_LOGITS and ``--profile`` for its per-category timers.
"""
from __future__ import annotations

import argparse
import json
import sys
import time
from typing import List


def parse_ids(text: str, vocab: int) -> List[int]:
    """Comma-separated token ids, each checked against the vocabulary (src/main.c:190-222)."""
    out = []
    for part in text.replace(" ", "").split(","):
        if part == "":
            continue
        try:
            v = int(part)
        except ValueError:
            raise SystemExit(f"--prompt-token-ids: '{part}' is not an integer") from None
        if not 0 <= v < vocab:
            raise SystemExit(f"--prompt-token-ids: id {v} is outside the vocabulary of {vocab}")
        out.append(v)
    if not out:
        raise SystemExit("--prompt-token-ids: no ids given")
    return out


def build_parser() -> argparse.ArgumentParser:
    ap = argparse.ArgumentParser(prog="bitnet", description="Generate with a Llama-style model on one B200.")
    ap.add_argument("model", help="model folder (config.json + model.safetensors); with --random-weights it is written first")
    ap.add_argument("-p", dest="prompt", default=None, help="input prompt as text (needs a tokenizer; none ships, use --prompt-token-ids)")
    ap.add_argument("--prompt-token-ids", action="append", default=[], metavar="IDS",
                    help="comma-separated prompt token ids; repeat the option for a batch")
    ap.add_argument("-n", dest="n_tokens", type=int, default=256, help="number of tokens to generate (default 256; 0 = prompt only)")
    ap.add_argument("--temp", type=float, default=0.0, help="temperature (default 0.0 = greedy)")
    ap.add_argument("--topp", type=float, default=0.9, help="top-p sampling, used when temperature > 0 (default 0.9)")
    ap.add_argument("--seed", type=int, default=42, help="random seed (default 42)")
    ap.add_argument("--maxseq", type=int, default=0, help="max sequence length (default: model max)")
    ap.add_argument("--repeat-penalty", type=float, default=1.1, help="repetition penalty over the last 64 tokens (default 1.1)")
    ap.add_argument("--no-prefill", action="store_true", help="feed the prompt one token per step instead of in one step")
    ap.add_argument("--quiet", action="store_true", help="suppress generated token output")
    ap.add_argument("--token-ids", action="store_true", help="print generated token ids to stderr as token_id=N")
    ap.add_argument("--benchmark-runs", type=int, default=1, help="measured runs sharing one loaded model")
    ap.add_argument("--benchmark-warmup-runs", type=int, default=0, help="full warm-up runs before the measured runs")
    ap.add_argument("--dtype", choices=["bfloat16", "float32"], default="bfloat16", help="compute type (default bfloat16)")
    ap.add_argument("--random-weights", action="store_true", help="write a random model into the model folder first (needs --config)")
    ap.add_argument("--config", default=None, help="config.json for --random-weights")
    ap.add_argument("--weight-seed", type=int, default=None, help="seed of --random-weights (default: --seed)")
    ap.add_argument("--stop-ids", default=None, help="comma-separated stop token ids (default: the model's eos_token_id)")
    ap.add_argument("--loop-abort", action="store_true",
                    help="end a request when its last four tokens repeat the four before (the reference does unless BN_DISABLE_LOOP_ABORT is set)")
    from .engine import diagnostics
    ap.add_argument("--plugin", action="append", default=[], metavar="MODULE",
                    help="a Python module to import before the model is read: it may register parts or a whole "
                         "architecture of its own (may be repeated)")
    diagnostics.add_arguments(ap)
    return ap


def main(argv=None) -> int:
    args = build_parser().parse_args(argv)
    import bitnet_c_b200 as bn
    from .engine.batch import SeqStep

    bn.load_plugins(args.plugin)
    if args.random_weights:
        if not args.config:
            raise SystemExit("--random-weights needs --config <config.json>")
        with open(args.config, "r", encoding="utf-8") as f:
            cfg = json.load(f)
        bn.write_random_model(args.model, cfg, args.weight_seed if args.weight_seed is not None else args.seed,
                              dtype=args.dtype)
    if args.prompt is not None and not args.prompt_token_ids:
        raise SystemExit("-p needs a tokenizer and none ships with this library; give --prompt-token-ids a,b,c")
    if not args.prompt_token_ids:
        raise SystemExit("give a prompt with --prompt-token-ids a,b,c")

    t0 = time.time()
    model = bn.load_model(args.model, dtype=args.dtype, max_seq=args.maxseq)
    load_ms = (time.time() - t0) * 1e3
    from .engine import diagnostics
    model.diagnostics = diagnostics.from_args(args)
    if model.diagnostics is not None:
        model.diagnostics.start_profile()
    vocab = model.spec.vocab_size
    prompts = [parse_ids(t, vocab) for t in args.prompt_token_ids]
    stop_ids = None if args.stop_ids is None else parse_ids(args.stop_ids, vocab)
    S = model.spec.max_positions
    for p in prompts:
        if len(p) >= S:
            raise SystemExit(f"prompt of {len(p)} tokens does not fit the context of {S}")
    # the reference caps generation to the room left in the context (src/main.c:1503-1506)
    max_new = [max(0, min(args.n_tokens, S - len(p))) for p in prompts]

    def emit(request: int, token: int) -> bool:
        if args.token_ids:
            print(f"token_id={token}", file=sys.stderr, flush=True)
        return False

    import torch
    results = None
    for run in range(args.benchmark_warmup_runs + args.benchmark_runs):
        measured = run >= args.benchmark_warmup_runs
        torch.cuda.synchronize()
        t1 = time.time()
        prompt_ms = 0.0
        if args.no_prefill:
            # token by token through the same step function (src/generate.c:405-416)
            results = _generate_no_prefill(bn, model, prompts, max_new, args, stop_ids, emit)
        else:
            results = bn.generate(model, prompts, max_new, temperature=args.temp, top_p=args.topp, seed=args.seed,
                                  repeat_penalty=args.repeat_penalty, stop_ids=stop_ids,
                                  callback=emit if args.token_ids and measured else None, loop_abort=args.loop_abort)
        torch.cuda.synchronize()
        total_ms = (time.time() - t1) * 1e3
        n_out = sum(len(r.tokens) for r in results)
        if measured:
            print(f"Generation complete tokens={n_out} tok/s={n_out / max(total_ms, 1e-9) * 1e3:.2f} "
                  f"prompt_tokens={sum(len(p) for p in prompts)} total_ms={total_ms:.1f} load_ms={load_ms:.1f} "
                  f"requests={len(prompts)} dtype={args.dtype}", file=sys.stderr, flush=True)
    if model.diagnostics is not None:
        for line in model.diagnostics.profile_lines():
            print(line, file=sys.stderr)
    if not args.quiet:
        for r in results:
            print(",".join(str(t) for t in r.tokens))
    return 0


def _generate_no_prefill(bn, model, prompts, max_new, args, stop_ids, emit):
    """--no-prefill: every prompt token is its own step; then the usual loop continues."""
    from .engine.runner import ModelEngine
    from .engine.generate import generate
    from .engine.batch import SeqStep
    from .sampling import SamplingParams
    from .cache.pages import PAGE, pages_for

    class OneByOne(ModelEngine):
        def step_and_sample(self, seqs, rows):
            longest = max(len(s.tokens) for s in seqs)
            if longest == 1:
                return super().step_and_sample(seqs, rows)
            for j in range(longest - 1):
                part = [SeqStep(s.slot, [s.tokens[j]], []) for s in seqs if j < len(s.tokens) - 1]
                self.model.step(self.cache, part)
            return super().step_and_sample([SeqStep(s.slot, [s.tokens[-1]], [0]) for s in seqs], rows)

    S = model.spec.max_positions
    need = sum(pages_for(min(len(p) + m, S)) * PAGE for p, m in zip(prompts, max_new))
    cache = model.new_cache(max_tokens=max(need, PAGE), max_seqs=len(prompts))
    params = SamplingParams(temperature=args.temp, top_p=args.topp, seed=args.seed, repeat_penalty=args.repeat_penalty)
    stops = tuple(model.spec.stop_ids) if stop_ids is None else tuple(stop_ids)
    return generate(OneByOne(model, cache, params), prompts, max_new, stop_ids=stops,
                    callback=emit if args.token_ids else None, loop_abort=args.loop_abort)


if __name__ == "__main__":
    sys.exit(main())
