#!/usr/bin/env python3
"""The headline measurement: decode tokens a second at batch 8 (and 1, 64) and prefill tokens
a second at 2,048 tokens, at the Qwen2.5-7B shape with random bfloat16 weights on one B200.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--impl ours|reference] [--layers L]
    python bench.py --shape 0.5b|32b        # the two other measured shapes, each with its own workload

Prints one JSON line.  `value` is device-timed decode tokens a second (CUDA events around K
single-token steps of the engine, sampling included); `e2e` is the same through the Python
entry point `generate`, token ids from the host in and out every step: its prompts are real
prompts, prefilled by the same call, and its last K single-token steps are timed (the first
32 or so after the prefill run with the SM clock still held down by the power cap and count
as warm-up; `all_steps_value` includes them).  `prefill` runs one
2,048-token prompt; `roofline` divides the bytes a decode step has to read (every weight once,
and the cache of the live requests) by its time; `points` holds decode at batch 1 and 64.
Peaks come from MEASURED_PEAKS.json beside this file when it exists, else the fallback
6.65 TB/s and 1.59 PFLOP/s.  Weights are far larger than L2, so nothing is flushed between
steps.  A decode step runs at the end of a 4,096-token context: the cache is filled with
random keys and values up to the starting length, which costs a decode step exactly what a
real prompt would.
"""
import argparse
import json
import os
import statistics
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

SHAPE_7B = dict(architectures=["Qwen2ForCausalLM"], model_type="qwen2", num_hidden_layers=28, hidden_size=3584,
                num_attention_heads=28, num_key_value_heads=4, intermediate_size=18944, vocab_size=152064,
                rope_theta=1000000.0, rms_norm_eps=1e-6, max_position_embeddings=32768,
                use_sliding_window=False, tie_word_embeddings=False)
FULL_LAYERS = 28
# The other shapes that are measured, each with the workload it is quoted on: a batch of
# prompts through generate(), then a fixed number of single-token steps.
OTHER_SHAPES = {
    "0.5b": dict(name="Qwen2.5-0.5B shape", batch=16, prompt_lens=(64, 1024), decode_steps=256,
                 raw=dict(architectures=["Qwen2ForCausalLM"], model_type="qwen2", num_hidden_layers=24, hidden_size=896,
                          num_attention_heads=14, num_key_value_heads=2, intermediate_size=4864, vocab_size=151936,
                          rope_theta=1000000.0, rms_norm_eps=1e-6, max_position_embeddings=32768,
                          use_sliding_window=False, tie_word_embeddings=True)),
    "32b": dict(name="Qwen2.5-32B shape", batch=8, prompt_lens=(1024, 1024), decode_steps=512,
                raw=dict(architectures=["Qwen2ForCausalLM"], model_type="qwen2", num_hidden_layers=64, hidden_size=5120,
                         num_attention_heads=40, num_key_value_heads=8, intermediate_size=27648, vocab_size=152064,
                         rope_theta=1000000.0, rms_norm_eps=1e-6, max_position_embeddings=32768,
                         use_sliding_window=False, tie_word_embeddings=False)),
}
CONTEXT = 4096
PREFILL_TOKENS = 2048
BATCH = 8


def peaks():
    hbm, tf, src = 6650.0, 1590.0, "fallback"
    try:
        with open(os.path.join(ROOT, "MEASURED_PEAKS.json")) as f:
            m = json.load(f)
        got = [k for k in ("hbm_gbs", "bf16_tflops") if isinstance(m.get(k), (int, float)) and m[k] > 0]
        hbm = float(m["hbm_gbs"]) if "hbm_gbs" in got else hbm
        tf = float(m["bf16_tflops"]) if "bf16_tflops" in got else tf       # the burst figure: the larger denominator
        src = "measured" if len(got) == 2 else ("fallback" if not got else "measured " + got[0] + ", fallback for the other")
    except (OSError, ValueError, TypeError, AttributeError):
        pass
    return hbm, tf, src


class ClockSampler:
    """Samples SM clock and throttle reasons through NVML while the timed region runs."""

    def __init__(self, period=0.05):
        self.period, self.samples, self.reasons, self.max_mhz = period, [], set(), None
        self._stop = threading.Event()
        self._thread = None
        try:
            import pynvml
            pynvml.nvmlInit()
            self.nv = pynvml
            self.h = pynvml.nvmlDeviceGetHandleByIndex(0)
            self.max_mhz = pynvml.nvmlDeviceGetMaxClockInfo(self.h, pynvml.NVML_CLOCK_SM)
        except Exception:
            self.nv = None

    _NAMES = {0x2: "applications_clocks_setting", 0x4: "sw_power_cap", 0x8: "hw_slowdown", 0x10: "sync_boost",
              0x20: "sw_thermal_slowdown", 0x40: "hw_thermal_slowdown", 0x80: "hw_power_brake_slowdown",
              0x100: "display_clock_setting"}

    def _run(self):
        while not self._stop.is_set():
            try:
                self.samples.append(self.nv.nvmlDeviceGetClockInfo(self.h, self.nv.NVML_CLOCK_SM))
                bits = self.nv.nvmlDeviceGetCurrentClocksEventReasons(self.h)
                for bit, name in self._NAMES.items():
                    if bits & bit:
                        self.reasons.add(name)
            except Exception:
                pass
            self._stop.wait(self.period)

    def __enter__(self):
        if self.nv is not None:
            self._thread = threading.Thread(target=self._run, daemon=True)
            self._thread.start()
        return self

    def __exit__(self, *a):
        self._stop.set()
        if self._thread is not None:
            self._thread.join()

    def summary(self):
        return {"sm_mhz": statistics.median(self.samples) if self.samples else None,
                "sm_max_mhz": self.max_mhz, "reasons": sorted(self.reasons)}


def weight_bytes(cfg, layers):
    h, i = cfg.hidden_size, cfg.intermediate_size
    per_layer = (cfg.q_size + 2 * cfg.kv_size) * h + h * cfg.q_size + 3 * i * h
    vectors = (cfg.q_size + 2 * cfg.kv_size) * 4 + 2 * h * 4
    head = cfg.vocab_size * h
    return layers * (per_layer * 2 + vectors) + head * 2 + h * 4


def kv_bytes_per_token(cfg, layers):
    return layers * 2 * cfg.kv_size * 2


def prefill_flops(cfg, layers, T):
    h, i = cfg.hidden_size, cfg.intermediate_size
    linear = 2 * T * layers * ((cfg.q_size + 2 * cfg.kv_size) * h + h * cfg.q_size + 3 * i * h)
    attn = layers * 4 * cfg.head_dim * cfg.num_attention_heads * T * (T + 1) // 2
    return linear + attn + 2 * cfg.vocab_size * h


def other_shape(args):
    """One of OTHER_SHAPES through generate(): unequal prompts prefilled in one step, then the
    workload's number of single-token steps, host token ids in and out.  The first call warms up
    (kernels compile, graphs are captured); the second is timed by generate()'s own clocks."""
    import torch
    import wpc_engine_b200 as wpc
    from wpc_engine_b200 import ops
    from wpc_engine_b200.cache import PAGE

    torch.cuda.set_device(0)
    hbm_peak, tf_peak, peak_src = peaks()
    w = OTHER_SHAPES[args.shape]
    full = w["raw"]["num_hidden_layers"]
    layers = args.layers if args.layers is not None else full
    cfg = wpc.Qwen2Config.from_dict(dict(w["raw"], num_hidden_layers=layers))
    batch, steps = w["batch"], w["decode_steps"]
    gen = torch.Generator().manual_seed(0)
    lo, hi = w["prompt_lens"]
    lens = [lo] * batch if lo == hi else torch.randint(lo, hi + 1, (batch,), generator=gen).tolist()
    prompts = [torch.randint(0, cfg.vocab_size, (n,), generator=gen).tolist() for n in lens]
    need = sum((n + steps + PAGE) // PAGE * PAGE for n in lens)
    engine = wpc.Engine.from_random(cfg, seed=0, dtype="bfloat16", device="cuda:0", max_tokens=need + PAGE,
                                    max_sequences=batch + 1)
    opts = wpc.GenerationOptions(max_tokens=steps + 1)       # the first token comes from the prefill step
    wpc.generate(engine, prompts, opts, stats={})
    stats = {}
    l0 = ops.launch_count + engine.graph_launches
    with ClockSampler() as clocks:
        wpc.generate(engine, prompts, opts, stats=stats)
    launches = ops.launch_count + engine.graph_launches - l0
    n_steps = len(stats["decode_step_s"])
    secs = stats["decode_s"]
    value = stats["decode_tokens"] / secs
    tail = min(args.steps, n_steps)
    mean_ctx = sum(lens) / batch + (n_steps + 1) / 2
    step_bytes = weight_bytes(cfg, layers) + batch * mean_ctx * kv_bytes_per_token(cfg, layers)
    achieved = step_bytes / (secs / n_steps) / 1e9
    T = stats["prefill_tokens"]
    pre_flops = sum(prefill_flops(cfg, layers, n) for n in lens)
    from wpc_engine_b200.engine.batch import StepLayout
    lay = StepLayout(batch, batch, batch, (max(lens) + steps + PAGE) // PAGE, 1)
    line = {
        "metric": f"decode tokens/s at batch {batch} ({w['name']}, bf16), through generate()",
        "value": value, "unit": "tokens/s", "n_gpus": 1, "steps": n_steps, "warmup": n_steps + 1,
        "ms_per_step": secs / n_steps * 1e3, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "bf16", "data": "synthetic: random N(0, 0.02) weights, uniform random token ids",
        "config": {"model": w["name"], "global_batch": batch, "seq_len": max(lens) + steps,
                   "parallelism": "single GPU", "layers": layers, "layers_of_shape": full,
                   "hidden": cfg.hidden_size, "heads": cfg.num_attention_heads, "kv_heads": cfg.num_key_value_heads,
                   "head_dim": cfg.head_dim, "intermediate": cfg.intermediate_size, "vocab": cfg.vocab_size,
                   "prompt_len_min": min(lens), "prompt_len_max": max(lens), "prefill_tokens": T,
                   "decode_steps": n_steps, "l2": "inputs larger than L2 (weights), no flush",
                   "cuda_graphs": engine.use_graphs},
        "e2e": {"value": value, "unit": "tokens/s", "h2d_bytes_per_step": lay.total * 4 + batch * 4,
                "d2h_bytes_per_step": batch * 4,
                "last_steps_value": sum(stats["decode_step_tokens"][-tail:]) / sum(stats["decode_step_s"][-tail:]),
                "last_steps": tail},
        "gpu_launches": launches,
        "prefill": {"value": T / stats["prefill_s"], "tokens": T, "ms": stats["prefill_s"] * 1e3,
                    "frac": pre_flops / stats["prefill_s"] / (tf_peak * 1e12)},
        "roofline": {"bound": "hbm", "achieved": achieved, "peak": hbm_peak, "unit": "GB/s", "frac": achieved / hbm_peak,
                     "peaks": peak_src},
        "clocks": clocks.summary(), "impl": "ours",
    }
    print(json.dumps(line))
    return 0


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=64)
    ap.add_argument("--warmup", type=int, default=4)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--layers", type=int, default=None, help="fewer layers than the shape has (named in config)")
    ap.add_argument("--shape", default="7b", choices=["7b"] + sorted(OTHER_SHAPES),
                    help="7b: the headline; the others run their own workload through generate()")
    ap.add_argument("--skip-points", action="store_true", help="leave out batch 1 and 64")
    args = ap.parse_args()

    if args.impl == "reference":
        print(json.dumps({"impl": "reference", "unavailable":
                          "the reference is a Rust workspace: pip cannot install it (no setup.py or pyproject.toml) "
                          "and no Rust toolchain exists offline"}))
        return 0
    if args.gpus != 1:
        print(f"bench.py measures one GPU only (asked for {args.gpus}): this library has no multi-GPU path")
        return 2
    if args.warmup < 3:
        args.warmup = 3
    if args.shape != "7b":
        return other_shape(args)
    if args.layers is None:
        args.layers = FULL_LAYERS

    import torch
    import wpc_engine_b200 as wpc
    from wpc_engine_b200 import ops
    from wpc_engine_b200.cache import PAGE

    torch.cuda.set_device(0)
    hbm_peak, tf_peak, peak_src = peaks()
    raw = dict(SHAPE_7B, num_hidden_layers=args.layers)
    cfg = wpc.Qwen2Config.from_dict(raw)
    K, W = args.steps, args.warmup
    start_ctx = CONTEXT - (K + W) - 1
    max_b = BATCH if args.skip_points else 64
    engine = wpc.Engine.from_random(cfg, seed=0, dtype="bfloat16", device="cuda:0",
                                    max_tokens=max_b * CONTEXT + 2 * PAGE, max_sequences=max_b + 1)
    for g in engine.cache.groups:           # random keys and values stand for the prompts' cache
        ops.fill_normal(g.k, 11, 0.0, 1.0)
        ops.fill_normal(g.v, 12, 0.0, 1.0)
    gen = torch.Generator().manual_seed(0)
    vocab = cfg.vocab_size

    def decode_run(batch, steps, warmup):
        """Device-timed single-token steps at the end of the context; returns (seconds, launches)."""
        slots = [engine.open_sequence() for _ in range(batch)]
        try:
            for s in slots:
                engine.cache.reserve(s, start_ctx)
                engine.cache.commit(s, start_ctx)
            engine.set_sampler_state(slots, 0, list(range(batch)))
            toks = torch.randint(0, vocab, (warmup + steps, batch), generator=gen).tolist()
            ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            for i in range(warmup):
                logits = engine.step([wpc.SequenceStep(s, [t], want=[0]) for s, t in zip(slots, toks[i])],
                                     borrow=True, check=False)
                engine.sample(logits, slots, 0.0)
            torch.cuda.synchronize()
            l0 = ops.launch_count + engine.graph_launches
            ev0.record()
            for i in range(warmup, warmup + steps):
                logits = engine.step([wpc.SequenceStep(s, [t], want=[0]) for s, t in zip(slots, toks[i])],
                                     borrow=True, check=False)
                engine.sample(logits, slots, 0.0)
            ev1.record()
            torch.cuda.synchronize()
            ops.check_device_status()
            return ev0.elapsed_time(ev1) / 1e3, ops.launch_count + engine.graph_launches - l0
        finally:
            for s in slots:
                engine.close_sequence(s)

    # ---- prefill of 2,048 tokens (one sequence, logits of the last place) -----------------------
    prompt = torch.randint(0, vocab, (PREFILL_TOKENS,), generator=gen).tolist()
    pre_ms = []
    for i in range(2 + 3):
        slot = engine.open_sequence()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        e0.record()
        engine.step([wpc.SequenceStep(slot, prompt, want=[PREFILL_TOKENS - 1])], check=False)
        e1.record()
        torch.cuda.synchronize()
        ops.check_device_status()
        engine.close_sequence(slot)
        if i >= 2:
            pre_ms.append(e0.elapsed_time(e1))
    pre = statistics.median(pre_ms)
    prefill = {"value": PREFILL_TOKENS / (pre / 1e3), "tokens": PREFILL_TOKENS, "ms": pre,
               "frac": prefill_flops(cfg, args.layers, PREFILL_TOKENS) / (pre / 1e3) / (tf_peak * 1e12)}

    # ---- decode at batch 8: the headline, with clocks sampled meanwhile ---------------------------
    with ClockSampler() as clocks:
        secs, launches = decode_run(BATCH, K, W)
    value = BATCH * K / secs
    mean_ctx = start_ctx + W + (K + 1) / 2
    step_bytes = weight_bytes(cfg, args.layers) + BATCH * mean_ctx * kv_bytes_per_token(cfg, args.layers)
    achieved = step_bytes / (secs / K) / 1e9
    roofline = {"bound": "hbm", "achieved": achieved, "peak": hbm_peak, "unit": "GB/s", "frac": achieved / hbm_peak,
                "peaks": peak_src}

    # ---- end to end through generate(): host token ids in, host token ids out, every step ------------
    # The prompts' own prefill (half a second at the power cap) leaves the SM clock low for about
    # 25 single-token steps; those count as warm-up, the last K steps are timed.
    e2e_warm = max(W, 32)
    e2e_prompt_len = CONTEXT - (e2e_warm + K) - 1
    prompts = [torch.randint(0, vocab, (e2e_prompt_len,), generator=gen).tolist() for _ in range(BATCH)]
    stats = {}
    wpc.generate(engine, prompts, wpc.GenerationOptions(max_tokens=e2e_warm + K + 1), stats=stats)
    stats = {}
    wpc.generate(engine, prompts, wpc.GenerationOptions(max_tokens=e2e_warm + K + 1), stats=stats)
    from wpc_engine_b200.engine.batch import StepLayout
    lay = StepLayout(BATCH, BATCH, BATCH, 64, 1)
    e2e = {"value": sum(stats["decode_step_tokens"][-K:]) / sum(stats["decode_step_s"][-K:]), "unit": "tokens/s",
           "steps": K, "warmup": len(stats["decode_step_s"]) - K,
           "all_steps_value": stats["decode_tokens"] / stats["decode_s"],
           "h2d_bytes_per_step": lay.total * 4 + BATCH * 4, "d2h_bytes_per_step": BATCH * 4,
           "prefill_tokens_per_s": stats["prefill_tokens"] / stats["prefill_s"]}

    points = {}
    if not args.skip_points:
        for b in (1, 64):
            s, _ = decode_run(b, max(K // 2, 8), W)
            points[f"decode_b{b}"] = b * max(K // 2, 8) / s

    line = {
        "metric": "decode tokens/s at batch 8 (Qwen2.5-7B shape, bf16, context 4096)",
        "value": value, "unit": "tokens/s", "n_gpus": 1, "steps": K, "warmup": W,
        "ms_per_step": secs / K * 1e3, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "bf16", "data": "synthetic: random N(0, 0.02) weights, uniform random token ids",
        "config": {"model": "Qwen2.5-7B shape", "global_batch": BATCH, "seq_len": CONTEXT,
                   "parallelism": "single GPU", "layers": args.layers, "layers_of_shape": FULL_LAYERS,
                   "hidden": cfg.hidden_size, "heads": cfg.num_attention_heads, "kv_heads": cfg.num_key_value_heads,
                   "head_dim": cfg.head_dim, "intermediate": cfg.intermediate_size, "vocab": cfg.vocab_size,
                   "context_len": CONTEXT, "decode_start_ctx": start_ctx + W, "prefill_tokens": PREFILL_TOKENS,
                   "l2": "inputs larger than L2 (weights), no flush", "cuda_graphs": engine.use_graphs},
        "e2e": e2e, "gpu_launches": launches, "prefill": prefill, "roofline": roofline, "points": points,
        "clocks": clocks.summary(), "impl": "ours",
    }
    print(json.dumps(line))
    return 0


if __name__ == "__main__":
    sys.exit(main())
