"""Command line in the manner of the reference's ``llmgen``
(cmd/llmgen/main.go:15-28): single-dash options, ``-model`` a model folder,
``-prompt`` a text, ``-tokens`` how many tokens to generate (default 50),
``-gpu`` the GPU path.  Beyond those: token ids in place of a text, a batch of
prompts, temperature sampling with a seed, stop tokens, the numeric path and
random weights.

    llmgen -model DIR [-prompt TEXT | -ids 1,2,3 [-ids ...] | -ids-file F] [-tokens N]
           [-temp T] [-seed S] [-stop 2,7] [-dtype bfloat16|float32] [-random-weights]
           [-max-len N] [-slots N]

``-slots`` is how many sequences run together (the cache's slots; more prompts
than that run batch after batch) and ``-max-len`` the longest sequence, prompt
and new tokens together, a slot holds: the cache is sized for ``slots`` sequences
of ``max-len`` tokens, and a sequence that reaches it ends there.

This library runs on the GPU only: ``-gpu`` is accepted and changes nothing,
``-gpu-layers`` must be 0 (all layers).  The reference's ``-turbo-quant``,
``-speculative*`` and ``-eager-load`` options belong to features outside this
library and are refused with a message.
"""
from __future__ import annotations

import argparse
import os
import sys
import time
from typing import List, Optional


def _ids(text: str) -> List[int]:
    try:
        return [int(t) for t in text.replace(",", " ").split()]
    except ValueError:
        raise argparse.ArgumentTypeError(f"token ids must be integers: {text!r}") from None


def parser() -> argparse.ArgumentParser:
    ap = argparse.ArgumentParser(prog="llmgen", description=__doc__,
                                 formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("-model", "--model", default="", help="model directory (config.json + model.safetensors)")
    ap.add_argument("-prompt", "--prompt", default=None, help="input prompt (needs tokenizer.json in the model directory)")
    ap.add_argument("-ids", "--ids", action="append", type=_ids, default=None,
                    help="prompt as token ids, comma or space separated; repeat for a batch")
    ap.add_argument("-ids-file", "--ids-file", default=None, help="file with one prompt of token ids per line")
    ap.add_argument("-tokens", "--tokens", type=int, default=50, help="tokens to generate")
    ap.add_argument("-gpu", "--gpu", action="store_true", help="use the GPU (always on: there is no CPU path)")
    ap.add_argument("-gpu-layers", "--gpu-layers", type=int, default=0, help="number of layers on GPU (0=all; only 0 is supported)")
    ap.add_argument("-temp", "--temp", type=float, default=0.0, help="sampling temperature; 0 is greedy")
    ap.add_argument("-seed", "--seed", type=int, default=0, help="seed of temperature sampling and of -random-weights")
    ap.add_argument("-stop", "--stop", type=_ids, default=None, help="stop token ids (default: config.json's eos_token_id)")
    ap.add_argument("-dtype", "--dtype", default="bfloat16", choices=["bfloat16", "float32"], help="numeric path")
    ap.add_argument("-random-weights", "--random-weights", action="store_true",
                    help="write seeded random weights into the model directory if it has none")
    ap.add_argument("-slots", "--slots", "-max-batch", "--max-batch", dest="slots", type=int, default=64,
                    help="sequences that run together: the cache's slots")
    ap.add_argument("-max-len", "--max-len", type=int, default=0,
                    help="longest sequence (prompt + new tokens) a slot holds; 0: what the prompts need")
    for flag in ("turbo-quant", "speculative", "eager-load"):
        ap.add_argument(f"-{flag}", f"--{flag}", action="store_true", help=argparse.SUPPRESS)
    return ap


def main(argv: Optional[List[str]] = None) -> int:
    args = parser().parse_args(argv)
    if not args.model:
        print("usage: llmgen -model <dir> [-prompt text | -ids 1,2,3] [-tokens N]", file=sys.stderr)
        return 1
    if args.tokens < 0:
        print("tokens must be non-negative", file=sys.stderr)
        return 1
    for flag in ("turbo_quant", "speculative", "eager_load"):
        if getattr(args, flag):
            print(f"-{flag.replace('_', '-')} is not part of this library", file=sys.stderr)
            return 1
    if args.slots <= 0 or args.max_len < 0:
        print("-slots must be positive and -max-len non-negative", file=sys.stderr)
        return 1
    if args.gpu_layers != 0:
        print("-gpu-layers: all layers run on the GPU; only 0 is supported", file=sys.stderr)
        return 1

    import torch
    from .. import Model, write_random_model
    from ..config import ConfigError, read_config_json
    from ..engine.generate import generate
    from ..weights import WeightError

    if not torch.cuda.is_available():
        print("llmgen: no CUDA device; this library has no CPU path", file=sys.stderr)
        return 1
    try:
        has_weights = any(os.path.exists(os.path.join(args.model, f))
                          for f in ("model.safetensors", "model.safetensors.index.json"))
        if args.random_weights and not has_weights:
            print(f"Writing random weights (seed {args.seed}) to {args.model}...")
            write_random_model(args.model, read_config_json(args.model), seed=args.seed, dtype=args.dtype)
        print(f"Loading model from {args.model}...")
        t0 = time.time()
        model = Model.load(args.model, dtype=args.dtype, device="cuda")
    except (ConfigError, WeightError, FileNotFoundError, ValueError) as e:
        print(f"load: {e}", file=sys.stderr)
        return 1
    cfg = model.config
    print(f"Loaded in {time.time() - t0:.2f}s ({len(model.plan.layers)} layers, h={model.plan.hidden_size})")

    tok = None
    tok_path = os.path.join(args.model, "tokenizer.json")
    if os.path.exists(tok_path):
        from .tokenizer import Tokenizer
        tok = Tokenizer(tok_path)
    prompts: List[List[int]] = []
    if args.ids:
        prompts += args.ids
    if args.ids_file:
        with open(args.ids_file) as f:
            prompts += [_ids(line) for line in f if line.strip()]
    if args.prompt is not None or not prompts:
        text = args.prompt if args.prompt is not None else "The meaning of life is"
        if tok is None:
            print(f"tokenizer: {tok_path} not found; give the prompt as token ids with -ids", file=sys.stderr)
            return 1
        prompts.append(tok.encode(text))
        print(f"Prompt: '{text}' ({len(prompts[-1])} tokens)")
    if any(len(p) == 0 for p in prompts):
        print("a prompt is empty", file=sys.stderr)
        return 1
    print(f"Generating {args.tokens} tokens for {len(prompts)} prompt(s)...\n")

    torch.cuda.synchronize()
    start = time.time()
    try:
        cache = None
        if args.max_len:
            slots = min(args.slots, len(prompts))
            cache = model.new_cache(max_tokens=slots * ((args.max_len + 63) // 64 * 64), max_slots=slots)
        results = generate(model, prompts, args.tokens, temperature=args.temp, seed=args.seed,
                           stop=args.stop, max_batch=args.slots, cache=cache,
                           max_sequence=args.max_len or None)
    except ValueError as e:
        print(f"generate: {e}", file=sys.stderr)
        return 1
    torch.cuda.synchronize()
    elapsed = time.time() - start

    print("--- Output ---")
    for i, (p, r) in enumerate(zip(prompts, results)):
        if tok is not None:
            print(f"[{i}] {tok.decode(list(p) + r.tokens)}")
        print(f"[{i}] ids: {' '.join(str(t) for t in r.tokens)}  ({r.finish_reason})")
    print("--- End ---\n")
    n_prompt = sum(len(p) for p in prompts)
    n_new = sum(len(r.tokens) for r in results)
    print(f"Prompt tokens:    {n_prompt}")
    print(f"Generated tokens: {n_new}")
    print(f"Total time:       {elapsed:.2f}s")
    if n_new and elapsed > 0:
        print(f"Tokens/sec:       {n_new / elapsed:.1f}")
        print(f"ms/token:         {elapsed / n_new * 1000:.1f}")
    return 0


if __name__ == "__main__":
    sys.exit(main())
