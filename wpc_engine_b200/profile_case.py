"""A small, self-contained workload for profilers: a few decode steps or prefills at the
layer sizes of a large model but with few layers, so that a capture ends quickly while every
kernel sees its real shapes.

    python -m wpc_engine_b200.profile_case --mode decode --layers 4 --batch 8 --context 4000 --steps 3
    python -m wpc_engine_b200.profile_case --mode prefill --layers 4 --tokens 2048 --steps 2

Random weights are drawn on the device; the cache is filled with random keys and values up to
`--context`.  Steps run directly (no CUDA graph), so that a profiler sees each kernel launch.
"""
from __future__ import annotations

import argparse
import json
import sys


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--mode", choices=["decode", "prefill"], default="decode")
    ap.add_argument("--layers", type=int, default=4)
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--context", type=int, default=4000, help="cached positions per sequence before the steps")
    ap.add_argument("--tokens", type=int, default=2048, help="prompt length in prefill mode")
    ap.add_argument("--steps", type=int, default=3)
    ap.add_argument("--config", help="a config.json; default: the Qwen2.5-7B layer sizes")
    ap.add_argument("--dtype", default="bfloat16", choices=["bfloat16", "float32"])
    args = ap.parse_args(argv)

    import torch
    from . import Engine, SequenceStep, ops
    from .config import read_config_json
    from .registry import resolve

    if args.config:
        raw = read_config_json(args.config)
    else:
        raw = dict(architectures=["Qwen2ForCausalLM"], hidden_size=3584, num_attention_heads=28,
                   num_key_value_heads=4, intermediate_size=18944, vocab_size=152064, rope_theta=1000000.0,
                   rms_norm_eps=1e-6, tie_word_embeddings=False)
    raw = dict(raw, num_hidden_layers=args.layers)
    cfg = resolve(raw).config_class.from_dict(raw)
    per_seq = (args.context + args.steps if args.mode == "decode" else args.tokens) + 64
    batch = args.batch if args.mode == "decode" else 1
    eng = Engine.from_random(cfg, 0, args.dtype, "cuda:0", max_tokens=batch * (per_seq + 64),
                             max_sequences=batch + 1, use_graphs=False)
    for g in eng.cache.groups:
        if hasattr(g, "k"):
            ops.fill_normal(g.k, 11, 0.0, 1.0)
            ops.fill_normal(g.v, 12, 0.0, 1.0)
    gen = torch.Generator().manual_seed(0)
    vocab = cfg.vocab_size
    if args.mode == "decode":
        slots = [eng.open_sequence() for _ in range(batch)]
        for s in slots:
            eng.cache.reserve(s, args.context)
            eng.cache.commit(s, args.context)
        eng.set_sampler_state(slots, 0, list(range(batch)))
        for _ in range(args.steps):
            toks = torch.randint(0, vocab, (batch,), generator=gen).tolist()
            logits = eng.step([SequenceStep(s, [t], want=[0]) for s, t in zip(slots, toks)])
            eng.sample(logits, slots, 0.0)
    else:
        for _ in range(args.steps):
            slot = eng.open_sequence()
            toks = torch.randint(0, vocab, (args.tokens,), generator=gen).tolist()
            eng.step([SequenceStep(slot, toks, want=[args.tokens - 1])])
            torch.cuda.synchronize()
            eng.close_sequence(slot)
    torch.cuda.synchronize()
    print(json.dumps({"mode": args.mode, "layers": args.layers, "batch": batch, "steps": args.steps,
                      "kernel_launches": ops.launch_count, "device_status": ops.device_status()}))
    return 0


if __name__ == "__main__":
    sys.exit(main())
