"""The command line, in the manner of the reference's `wpc-runtime` binary
(wpc-runtime/src/main.rs:30-63): `--model DIR` and `--max-tokens N` (default 40) mean what
they mean there.  The reference tokenizes `--prompt TEXT`; this library takes token ids, so
the prompt is `--prompt-ids "1,2,3;4,5"` (`;` separates the requests of a batch).  Added:
`--temperature`, `--seed`, `--stop-ids`, `--dtype`, `--random-weights` (with `--config FILE`,
writes a model folder into `--model` first), `--max-seq-len`, `--print-logits K`, `--max-batch`,
`--cache-tokens`.  `--arch` names the architecture or `auto`
(config.json decides, main.rs:69-82).  Standard output carries one JSON line per request;
diagnostics go to standard error in the reference's wording (main.rs:100-104, 294, 309, 424,
429).
"""
from __future__ import annotations

import argparse
import json
import os
import sys
import time


def parse_prompt_ids(text: str):
    prompts = []
    for part in text.split(";"):
        ids = [int(x) for x in part.replace(",", " ").split()]
        if not ids:
            raise ValueError("an empty prompt among --prompt-ids")
        prompts.append(ids)
    return prompts


def build_parser() -> argparse.ArgumentParser:
    ap = argparse.ArgumentParser(prog="wpc-runtime", description="Qwen2 generation on one B200")
    ap.add_argument("--model", required=True, help="directory containing model.safetensors and config.json")
    ap.add_argument("--arch", default="auto", help="auto (from config.json) or an architecture name / model_type")
    ap.add_argument("--prompt-ids", help='token ids of the prompt(s): "1,2,3" or "1,2,3;4,5"')
    ap.add_argument("--prompt-ids-file", help="file with one prompt per line")
    ap.add_argument("--max-tokens", type=int, default=40, help="number of tokens to generate")
    ap.add_argument("--temperature", type=float, default=0.0, help="0: greedy")
    ap.add_argument("--seed", type=int, default=0)
    ap.add_argument("--stop-ids", default=None, help="stop token ids; default: eos_token_id of the model folder")
    ap.add_argument("--dtype", default="bfloat16", choices=["bfloat16", "float32", "bf16", "fp32"])
    ap.add_argument("--random-weights", action="store_true",
                    help="write random weights for --config into --model before loading")
    ap.add_argument("--config", help="config.json for --random-weights")
    ap.add_argument("--max-batch", type=int, default=None)
    ap.add_argument("--cache-tokens", type=int, default=None, help="positions the cache holds (default: what fits the prompts)")
    ap.add_argument("--max-seq-len", type=int, default=None,
                    help="longest sequence (prompt plus generated tokens) that is accepted; default: the model's "
                         "max_position_embeddings")
    ap.add_argument("--print-logits", type=int, default=0, metavar="K",
                    help="also print the K greatest next-token logits after each prompt, one JSON line per request")
    return ap


def main(argv=None) -> int:
    args = build_parser().parse_args(argv)
    import torch
    from . import Engine, GenerationOptions, generate, write_random_model
    from .cache import PAGE
    from .config import read_config_json
    from .registry import resolve
    from .sampling import banned_from_env, stop_ids_of_folder

    if args.prompt_ids_file:
        with open(args.prompt_ids_file) as f:
            prompts = [p for line in f if line.strip() for p in parse_prompt_ids(line.strip())]
    elif args.prompt_ids:
        prompts = parse_prompt_ids(args.prompt_ids)
    else:
        print("error: --prompt-ids or --prompt-ids-file is required", file=sys.stderr)
        return 2

    dtype = {"bf16": "bfloat16", "fp32": "float32"}.get(args.dtype, args.dtype)
    if args.random_weights:
        if not args.config:
            print("error: --random-weights needs --config FILE", file=sys.stderr)
            return 2
        raw = read_config_json(args.config)
        cfg = resolve(raw).config_class.from_dict(raw)
        write_random_model(args.model, cfg, args.seed, torch.bfloat16 if dtype == "bfloat16" else torch.float32)
        print(f"wrote random weights (seed {args.seed}) to {args.model}", file=sys.stderr)

    if args.max_seq_len is not None:
        for i, p in enumerate(prompts):
            if len(p) + args.max_tokens > args.max_seq_len:
                print(f"error: request {i} needs {len(p)} + {args.max_tokens} positions, --max-seq-len is {args.max_seq_len}",
                      file=sys.stderr)
                return 2

    raw = read_config_json(args.model)
    if args.arch != "auto":
        raw = dict(raw, architectures=[args.arch]) if args.arch[:1].isupper() else dict(raw, architectures=[], model_type=args.arch)
    arch = resolve(raw)
    print(f"architecture: {arch.name}", file=sys.stderr)
    t0 = time.time()
    need = sum((len(p) + args.max_tokens + PAGE - 1) // PAGE * PAGE for p in prompts)
    if args.max_batch:
        need = max((len(p) + args.max_tokens + PAGE - 1) // PAGE * PAGE for p in prompts) * args.max_batch
    engine = Engine.from_folder(args.model, dtype=dtype, device="cuda", max_tokens=args.cache_tokens or need)
    c = engine.config
    print(f"config: hidden={c.hidden_size} layers={c.num_hidden_layers} heads={c.num_attention_heads} "
          f"kv_heads={c.num_key_value_heads} vocab={c.vocab_size}", file=sys.stderr)
    print(f"model loaded in {time.time() - t0:.3f}s", file=sys.stderr)
    for p in prompts:
        print(f"prompt tokens ({len(p)}): {p}", file=sys.stderr)
    stop = [int(x) for x in args.stop_ids.replace(",", " ").split()] if args.stop_ids is not None \
        else stop_ids_of_folder(args.model)
    if stop:
        print(f"stop tokens: {stop}", file=sys.stderr)
    if args.print_logits > 0:
        from . import SequenceStep
        for i, p in enumerate(prompts):
            slot = engine.open_sequence()
            try:
                row = engine.step([SequenceStep(slot, p, want=[len(p) - 1])])[0].float()
            finally:
                engine.close_sequence(slot)
            vals, ids = torch.topk(row, min(args.print_logits, row.numel()))
            print(json.dumps({"request": i, "top_logits": [[int(t), float(v)] for t, v in zip(ids.tolist(), vals.tolist())]}))
    opts = GenerationOptions(max_tokens=args.max_tokens, temperature=args.temperature, seed=args.seed,
                             stop_token_ids=stop, banned_token_ids=banned_from_env(), max_batch=args.max_batch)
    t1 = time.time()
    outputs = generate(engine, prompts, opts)
    torch.cuda.synchronize()
    n = sum(len(o) for o in outputs)
    print(f"generated {n} tokens in {time.time() - t1:.3f}s", file=sys.stderr)
    for i, out in enumerate(outputs):
        print(f"generated token ids: {out}", file=sys.stderr)
        print(json.dumps({"request": i, "prompt_tokens": len(prompts[i]), "generated": out}))
    return 0


if __name__ == "__main__":
    sys.exit(main())
