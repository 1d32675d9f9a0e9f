#!/usr/bin/env python3
"""The headline measurement: decode tokens a second at batch 8 (and 1, 64) and prefill tokens
a second at 2,048 tokens, at the Qwen2.5-7B shape with random bfloat16 weights on one B200.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--impl ours|reference] [--layers L]
    python bench.py --shape 0.5b|32b        # the two other measured shapes, each with its own workload
    python bench.py --case decode|prefill   # a small workload for a profiler (see profile_case)

Prints one JSON line.  `value` is device-timed decode tokens a second (CUDA events around K
single-token steps of the engine, sampling included); `e2e` is the same through the Python
entry point `generate`, token ids from the host in and out every step: its prompts are real
prompts, prefilled by the same call, and its last K single-token steps are timed (the first
32 or so after the prefill run with the SM clock still held down by the power cap and count
as warm-up; `all_steps_value` includes them).  `prefill` runs one 2,048-token prompt;
`roofline` divides the bytes a decode step has to read (every weight once, and the cache of
the live requests) by its time.  Beside these:

  points     decode at batch 1 and 64 (context 4,096), the same three batches at context 2,048,
             batch 128 and 256, contexts of 16,384 and 32,768 at batch 1 and 8, prefill of 512,
             8,192 and 32,768 tokens and of 16 unequal prompts, and 32-bit decode at batch 1:
             tokens a second each
  whole_run  batch 8 through `generate`: 2,048-token prompts, then 2,048 single-token steps,
             tokens a second over all of them (the reference times its whole loop,
             wpc-runtime/src/main.rs:299-309)
  kernels    the products and the attention of a decode step (GB/s of what each must read) and
             of a 2,048-token prefill (TFLOP/s), each launched alone on every layer's weights
             in turn between CUDA events, beside its peak

Peaks come from MEASURED_PEAKS.json beside this file when it exists, else the fallback
6.65 TB/s and 1.59 PFLOP/s.  Weights are far larger than L2, so nothing is flushed between
steps.  A decode step runs at the end of its context: the cache is filled with random keys
and values up to the starting length, which costs a decode step exactly what a real prompt
would.
"""
import argparse
import json
import os
import statistics
import sys
import threading

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


def weight_bytes(cfg, layers, elem=2):
    h, i = cfg.hidden_size, cfg.intermediate_size
    per_layer = (cfg.q_size + 2 * cfg.kv_size) * h + h * cfg.q_size + 3 * i * h
    vectors = (cfg.q_size + 2 * cfg.kv_size) * 4 + 2 * h * 4
    head = cfg.vocab_size * h
    return layers * (per_layer * elem + vectors) + head * elem + h * 4


def kv_bytes_per_token(cfg, layers, elem=2):
    return layers * 2 * cfg.kv_size * elem


def prefill_flops(cfg, layers, T):
    h, i = cfg.hidden_size, cfg.intermediate_size
    linear = 2 * T * layers * ((cfg.q_size + 2 * cfg.kv_size) * h + h * cfg.q_size + 3 * i * h)
    attn = layers * 4 * cfg.head_dim * cfg.num_attention_heads * T * (T + 1) // 2
    return linear + attn + 2 * cfg.vocab_size * h


def fill_cache(engine):
    """Random keys and values stand for the prompts' cache."""
    from wpc_engine_b200 import ops
    for g in engine.cache.groups:
        if hasattr(g, "k"):
            ops.fill_normal(g.k, 11, 0.0, 1.0)
            ops.fill_normal(g.v, 12, 0.0, 1.0)


def decode_run(engine, gen, batch, start_ctx, steps, warmup):
    """Device-timed single-token steps of `batch` sequences that hold start_ctx positions each
    before the first of them; returns (seconds of the timed steps, kernels launched in them)."""
    import torch
    import wpc_engine_b200 as wpc
    from wpc_engine_b200 import ops
    vocab = engine.vocab_size
    slots = [engine.open_sequence() for _ in range(batch)]
    try:
        for s in slots:
            engine.cache.reserve(s, start_ctx)
            engine.cache.commit(s, start_ctx)
        engine.set_sampler_state(slots, 0, list(range(batch)))
        toks = torch.randint(0, vocab, (warmup + steps, batch), generator=gen).tolist()
        ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)

        def one(i):
            logits = engine.step([wpc.SequenceStep(s, [t], want=[0]) for s, t in zip(slots, toks[i])],
                                 borrow=True, check=False)
            engine.sample(logits, slots, 0.0)
        for i in range(warmup):
            one(i)
        torch.cuda.synchronize()
        l0 = ops.launch_count + engine.graph_launches
        ev0.record()
        for i in range(warmup, warmup + steps):
            one(i)
        ev1.record()
        torch.cuda.synchronize()
        ops.check_device_status(engine.device, "a kernel of the timed steps")
        return ev0.elapsed_time(ev1) / 1e3, ops.launch_count + engine.graph_launches - l0
    finally:
        for s in slots:
            engine.close_sequence(s)


def prefill_run(engine, gen, lens, repeats=3, warm=2):
    """Median device time in ms of one step that brings prompts of `lens` tokens (the logits
    of each prompt's last place wanted)."""
    import torch
    import wpc_engine_b200 as wpc
    from wpc_engine_b200 import ops
    prompts = [torch.randint(0, engine.vocab_size, (n,), generator=gen).tolist() for n in lens]
    ms = []
    for i in range(warm + repeats):
        slots = [engine.open_sequence() for _ in prompts]
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        e0.record()
        engine.step([wpc.SequenceStep(s, p, want=[len(p) - 1]) for s, p in zip(slots, prompts)], check=False)
        e1.record()
        torch.cuda.synchronize()
        ops.check_device_status(engine.device, "a kernel of the prefill")
        for s in slots:
            engine.close_sequence(s)
        if i >= warm:
            ms.append(e0.elapsed_time(e1))
    return statistics.median(ms)


def kernel_rates(engine, cfg, layers, batch, ctx, prefill_tokens, hbm_peak, tf_peak):
    """Each product and the attention of a decode step and of a prefill, alone: one launch on
    every layer's weights in turn (together far larger than L2), replayed from a CUDA graph
    between two CUDA events, three passes, the median per launch.  Decode figures are GB/s of what the kernel must read,
    prefill figures TFLOP/s; `frac` is the share of the measured peak."""
    import torch
    from wpc_engine_b200 import ops
    dev = engine.device
    blocks = engine.model.blocks[:layers]
    h, inner = cfg.hidden_size, cfg.intermediate_size
    nh, nkv, hd = cfg.num_attention_heads, cfg.num_key_value_heads, cfg.head_dim
    g = torch.Generator(device="cpu").manual_seed(3)

    def rnd(*shape):
        return torch.randn(shape, generator=g).to(torch.bfloat16).to(dev)

    def timed(launch, n):
        """Median microseconds per launch of `launch(layer)`: the n launches are captured into a
        CUDA graph (so that the host's part of a call, tens of microseconds, is not in the
        figure) and the graph is replayed three times between events."""
        for layer in range(n):
            launch(layer)
        torch.cuda.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            for layer in range(n):
                launch(layer)
        graph.replay()
        us = []
        for _ in range(3):
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            torch.cuda.synchronize()
            e0.record()
            graph.replay()
            e1.record()
            torch.cuda.synchronize()
            us.append(e0.elapsed_time(e1) * 1e3 / n)
        return statistics.median(us)

    out = {}
    n = len(blocks)
    products = {"qkv": lambda b: (b.mixer.qkv.weight, b.mixer.qkv.bias, None),
                "o_proj": lambda b: (b.mixer.o_proj.weight, None, h),
                "down": lambda b: (b.ffn.down_proj.weight, None, h)}
    for tokens, tag in ((batch, f"decode_b{batch}"), (prefill_tokens, f"prefill_{prefill_tokens}")):
        x_h, x_q, x_i = rnd(tokens, h), rnd(tokens, nh * hd), rnd(tokens, inner)
        resid = torch.zeros((tokens, h), dtype=torch.float32, device=dev)
        for name, pick in products.items():
            x = {"qkv": x_h, "o_proj": x_q, "down": x_i}[name]

            def launch(layer, pick=pick, x=x):
                w, bias, add = pick(blocks[layer])
                ops.linear(x, w, bias, residual=resid if add else None, static_weight=True)
            w0 = pick(blocks[0])[0]
            us = timed(launch, n)
            if tokens == batch:
                gbs = w0.numel() * 2 / us / 1e3
                out[f"{tag}_{name}"] = {"value": gbs, "unit": "GB/s", "us": us, "frac": gbs / hbm_peak}
            else:
                tfs = 2 * tokens * w0.numel() / us / 1e6
                out[f"{tag}_{name}"] = {"value": tfs, "unit": "TFLOP/s", "us": us, "frac": tfs / tf_peak}
        us = timed(lambda layer: ops.gated_linear(x_h, blocks[layer].ffn.gate_up.weight, inner, blocks[layer].ffn.group,
                                                  static_weight=True), n)
        wn = 2 * inner * h
        if tokens == batch:
            out[f"{tag}_gate_up"] = {"value": wn * 2 / us / 1e3, "unit": "GB/s", "us": us, "frac": wn * 2 / us / 1e3 / hbm_peak}
        else:
            tfs = 2 * tokens * wn / us / 1e6
            out[f"{tag}_gate_up"] = {"value": tfs, "unit": "TFLOP/s", "us": us, "frac": tfs / tf_peak}
    # the output head on `batch` rows: one matrix, larger than L2 by itself
    head = engine.model.head
    table = head.tied_to.table if head.tied_to is not None else head.table
    x_h = rnd(batch, h)
    us = timed(lambda layer: ops.linear(x_h, table, None, out_dtype=torch.float32, static_weight=True), 3)
    gbs = table.numel() * 2 / us / 1e3
    out[f"decode_b{batch}_lm_head"] = {"value": gbs, "unit": "GB/s", "us": us, "frac": gbs / hbm_peak}
    # attention over the cache: a decode step of `batch` sequences of ctx positions, and a prompt
    group = next(gr for gr in engine.cache.groups if hasattr(gr, "k"))
    scale = 1.0 / hd ** 0.5

    def with_sequences(lens, body):
        slots = [engine.open_sequence() for _ in lens]
        try:
            for s, length in zip(slots, lens):
                engine.cache.reserve(s, length)
                engine.cache.commit(s, length)
            width = engine.cache.table_width(slots)
            table_t = torch.tensor(engine.cache.page_table_rows(engine.cache.kv_groups()[0], slots, width),
                                   dtype=torch.int32, device=dev)
            return body(table_t)
        finally:
            for s in slots:
                engine.close_sequence(s)

    def decode_attention(table_t):
        q = rnd(batch, nh * hd)
        cu = torch.arange(batch + 1, dtype=torch.int32, device=dev)
        lens = torch.full((batch,), ctx, dtype=torch.int32, device=dev)
        seq = torch.arange(batch, dtype=torch.int32, device=dev)
        pos = torch.full((batch,), ctx - 1, dtype=torch.int32, device=dev)
        return timed(lambda layer: ops.attention(q, nh, nkv, hd, group.k[layer], group.v[layer], table_t, cu, lens, seq,
                                                 pos, scale, None, 1, ctx), min(n, group.n_layers))

    us = with_sequences([ctx] * batch, decode_attention)
    gbs = batch * ctx * 2 * nkv * hd * 2 / us / 1e3
    out[f"decode_b{batch}_attention_ctx{ctx}"] = {"value": gbs, "unit": "GB/s", "us": us, "frac": gbs / hbm_peak}

    def prefill_attention(table_t):
        T = prefill_tokens
        q = rnd(T, (nh + 2 * nkv) * hd)
        cu = torch.tensor([0, T], dtype=torch.int32, device=dev)
        lens = torch.tensor([T], dtype=torch.int32, device=dev)
        seq = torch.zeros(T, dtype=torch.int32, device=dev)
        pos = torch.arange(T, dtype=torch.int32, device=dev)
        return timed(lambda layer: ops.attention(q, nh, nkv, hd, group.k[layer], group.v[layer], table_t, cu, lens, seq,
                                                 pos, scale, None, T, T), min(n, group.n_layers))

    us = with_sequences([prefill_tokens], prefill_attention)
    tfs = 4 * hd * nh * prefill_tokens * (prefill_tokens + 1) // 2 / us / 1e6
    out[f"prefill_{prefill_tokens}_attention"] = {"value": tfs, "unit": "TFLOP/s", "us": us, "frac": tfs / tf_peak}
    ops.check_device_status(dev, "a kernel measured alone")
    return out


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
                "d2h_bytes_per_step": batch * 4 + 4,
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


def profile_case(args):
    """A small, self-contained workload for profilers: a few decode steps or prefills at the
    layer sizes of the chosen shape but with few layers, so that a capture ends quickly while
    every kernel sees its real shapes.  Steps run directly (no CUDA graph), so that a profiler
    sees each kernel launch.

        python bench.py --case decode --layers 4 --batch 8 --context 4000 --steps 3
        python bench.py --case prefill --layers 4 --tokens 2048 --steps 2 [--shape 0.5b]

    With --timeline (decode only) the steps are replayed from CUDA graphs as in generation, and
    the kernels' start and end times come from torch.profiler: for every kernel name the
    launches a step, the mean duration, and the mean time from the end of the kernel before it
    to its own end, which is what it adds to the step (durations overlap: with programmatic
    dependent launch a kernel is resident while the one before it still runs).

        python bench.py --case decode --timeline --layers 28 --batch 8 --context 4000
    """
    import torch
    import wpc_engine_b200 as wpc
    from wpc_engine_b200 import ops

    raw = dict(SHAPE_7B if args.shape == "7b" else OTHER_SHAPES[args.shape]["raw"])
    layers = args.layers if args.layers is not None else 4
    cfg = wpc.Qwen2Config.from_dict(dict(raw, num_hidden_layers=layers))
    decode = args.case == "decode"
    per_seq = (args.context + args.steps if decode else args.tokens) + 64
    batch = args.batch if decode else 1
    eng = wpc.Engine.from_random(cfg, 0, args.dtype, "cuda:0", max_tokens=batch * (per_seq + 64),
                                 max_sequences=batch + 1, use_graphs=bool(args.timeline))
    fill_cache(eng)
    gen = torch.Generator().manual_seed(0)
    if decode and args.timeline:
        return timeline(eng, cfg, batch, args.context, gen)
    if decode:
        slots = [eng.open_sequence() for _ in range(batch)]
        for s in slots:
            eng.cache.reserve(s, args.context)
            eng.cache.commit(s, args.context)
        eng.set_sampler_state(slots, 0, list(range(batch)))
        for _ in range(args.steps):
            toks = torch.randint(0, cfg.vocab_size, (batch,), generator=gen).tolist()
            logits = eng.step([wpc.SequenceStep(s, [t], want=[0]) for s, t in zip(slots, toks)])
            eng.sample(logits, slots, 0.0)
    else:
        for _ in range(args.steps):
            slot = eng.open_sequence()
            toks = torch.randint(0, cfg.vocab_size, (args.tokens,), generator=gen).tolist()
            eng.step([wpc.SequenceStep(slot, toks, want=[args.tokens - 1])])
            eng.close_sequence(slot)
    torch.cuda.synchronize()
    print(json.dumps({"case": args.case, "layers": layers, "batch": batch, "steps": args.steps,
                      "kernel_launches": ops.launch_count, "device_status": ops.device_status()}))
    return 0


def timeline(eng, cfg, batch, context, gen, steps=4):
    import collections
    import torch
    import wpc_engine_b200 as wpc
    from torch.profiler import ProfilerActivity, profile
    slots = [eng.open_sequence() for _ in range(batch)]
    for s in slots:
        eng.cache.reserve(s, context)
        eng.cache.commit(s, context)
    eng.set_sampler_state(slots, 0, list(range(batch)))

    def one():
        toks = torch.randint(0, cfg.vocab_size, (batch,), generator=gen).tolist()
        logits = eng.step([wpc.SequenceStep(s, [t], want=[0]) for s, t in zip(slots, toks)], borrow=True, check=False)
        eng.sample(logits, slots, 0.0)
    for _ in range(6):
        one()
    torch.cuda.synchronize()
    with profile(activities=[ProfilerActivity.CUDA]) as prof:
        for _ in range(steps):
            one()
        torch.cuda.synchronize()
    events = [e for e in prof.events() if e.device_type.name == "CUDA" and "emcpy" not in e.name and "emset" not in e.name]
    events.sort(key=lambda e: e.time_range.start)
    stat, last_end = collections.OrderedDict(), None
    for e in events:
        start, end = e.time_range.start, e.time_range.end
        d = stat.setdefault(e.name.split("(")[0][-64:], [0, 0.0, 0.0])
        d[0] += 1
        d[1] += end - start
        d[2] += max(end - last_end, 0) if last_end is not None else end - start
        last_end = end if last_end is None else max(end, last_end)
    total = sum(d[2] for d in stat.values())
    print(f"batch {batch}, context {context}, {len(eng.model.blocks)} layers: {total / steps:.1f} us a step")
    print("launches a step | mean duration us | adds us each | adds us a step | kernel")
    for name, (n, dur, add) in stat.items():
        print(f"{n / steps:8.1f} | {dur / n:8.2f} | {add / n:8.2f} | {add / steps:9.1f} | {name}")
    return 0


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--warmup", type=int, default=4)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--layers", type=int, default=None, help="fewer layers than the shape has (named in config)")
    ap.add_argument("--shape", default="7b", choices=["7b"] + sorted(OTHER_SHAPES),
                    help="7b: the headline; the others run their own workload through generate()")
    ap.add_argument("--skip-points", action="store_true", help="only the headline, its end-to-end twin and the prefill")
    ap.add_argument("--case", choices=["decode", "prefill"], help="run a small profiler workload instead (see profile_case)")
    ap.add_argument("--batch", type=int, default=8, help="--case decode: sequences")
    ap.add_argument("--context", type=int, default=4000, help="--case decode: cached positions per sequence")
    ap.add_argument("--tokens", type=int, default=2048, help="--case prefill: prompt length")
    ap.add_argument("--dtype", default="bfloat16", choices=["bfloat16", "float32"], help="--case: the path to run")
    ap.add_argument("--timeline", action="store_true", help="--case decode: kernel timeline of graph-replayed steps")
    args = ap.parse_args()

    if args.impl == "reference":
        print(json.dumps({"impl": "reference", "unavailable":
                          "the reference is a Rust workspace: pip cannot install it (no setup.py or pyproject.toml) "
                          "and no Rust toolchain exists offline"}))
        return 0
    if args.gpus != 1:
        print(f"bench.py measures one GPU only (asked for {args.gpus}): this library has no multi-GPU path")
        return 2
    if args.case:
        if args.steps == 200:
            args.steps = 3
        return profile_case(args)
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
    L = args.layers
    K, W = args.steps, args.warmup
    start_ctx = CONTEXT - (K + W) - 1
    if start_ctx < 64:
        print(f"--steps {K} and --warmup {W} do not fit a context of {CONTEXT}")
        return 2
    points_on = not args.skip_points
    # the cache holds the largest point: 256 sequences of 4,096 positions (60 GB at 28 layers)
    max_b = 256 if points_on else BATCH
    engine = wpc.Engine.from_random(cfg, seed=0, dtype="bfloat16", device="cuda:0",
                                    max_tokens=max_b * CONTEXT + 2 * PAGE, max_sequences=max_b + 1)
    fill_cache(engine)
    gen = torch.Generator().manual_seed(0)
    vocab = cfg.vocab_size

    def step_bytes(batch, mean_ctx):
        return weight_bytes(cfg, L) + batch * mean_ctx * kv_bytes_per_token(cfg, L)

    # ---- prefill of 2,048 tokens (one sequence, logits of the last place) -----------------------
    pre = prefill_run(engine, gen, [PREFILL_TOKENS])
    prefill = {"value": PREFILL_TOKENS / (pre / 1e3), "tokens": PREFILL_TOKENS, "ms": pre,
               "frac": prefill_flops(cfg, L, PREFILL_TOKENS) / (pre / 1e3) / (tf_peak * 1e12)}

    # ---- decode at batch 8: the headline, with clocks sampled meanwhile ---------------------------
    with ClockSampler() as clocks:
        secs, launches = decode_run(engine, gen, BATCH, start_ctx, K, W)
    value = BATCH * K / secs
    achieved = step_bytes(BATCH, start_ctx + W + (K + 1) / 2) / (secs / K) / 1e9
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
           "h2d_bytes_per_step": lay.total * 4 + BATCH * 4, "d2h_bytes_per_step": BATCH * 4 + 4,
           "prefill_tokens_per_s": stats["prefill_tokens"] / stats["prefill_s"]}

    points, whole_run, kernels = {}, None, None
    if points_on:
        k2 = max(K // 2, 8)
        for b in (1, 64):
            s, _ = decode_run(engine, gen, b, CONTEXT - (k2 + W) - 1, k2, W)
            points[f"decode_b{b}"] = b * k2 / s
        for b in (1, 8, 64):                     # the same at the start of the generated half of the context
            s, _ = decode_run(engine, gen, b, 2048 - (k2 + W) - 1, k2, W)
            points[f"decode_b{b}_ctx2048"] = b * k2 / s
        k4 = max(K // 4, 8)
        for b in (128, 256):
            s, _ = decode_run(engine, gen, b, CONTEXT - (k4 + W) - 1, k4, W)
            points[f"decode_b{b}"] = b * k4 / s
        for ctx in (16384, 32768):
            for b in (1, 8):
                s, _ = decode_run(engine, gen, b, ctx - (k4 + W) - 1, k4, W)
                points[f"decode_b{b}_ctx{ctx}"] = b * k4 / s
        for T in (512, 8192, 32768):
            ms = prefill_run(engine, gen, [T], repeats=2, warm=1)
            points[f"prefill_{T}"] = T / (ms / 1e3)
            points[f"prefill_{T}_frac"] = prefill_flops(cfg, L, T) / (ms / 1e3) / (tf_peak * 1e12)
        lens = torch.randint(64, 1025, (16,), generator=gen).tolist()
        ms = prefill_run(engine, gen, lens, repeats=2, warm=1)
        points["prefill_16_unequal"] = sum(lens) / (ms / 1e3)
        points["prefill_16_unequal_tokens"] = sum(lens)

        # ---- the whole workload of the shape at batch 8: 2,048-token prompts, 2,048 single-token steps ----
        prompts = [torch.randint(0, vocab, (2048,), generator=gen).tolist() for _ in range(BATCH)]
        stats = {}
        wpc.generate(engine, prompts, wpc.GenerationOptions(max_tokens=2049), stats=stats)
        n = len(stats["decode_step_s"])
        whole_run = {"value": stats["decode_tokens"] / stats["decode_s"], "unit": "tokens/s", "batch": BATCH,
                     "prompt_tokens": 2048, "steps": n, "seconds": stats["decode_s"],
                     "first_100_steps_value": sum(stats["decode_step_tokens"][:100]) / sum(stats["decode_step_s"][:100]),
                     "last_100_steps_value": sum(stats["decode_step_tokens"][-100:]) / sum(stats["decode_step_s"][-100:]),
                     "roofline_frac": step_bytes(BATCH, 2048 + (n + 1) / 2) / (stats["decode_s"] / n) / 1e9 / hbm_peak,
                     "prefill_tokens_per_s": stats["prefill_tokens"] / stats["prefill_s"]}
        kernels = kernel_rates(engine, cfg, L, BATCH, CONTEXT, PREFILL_TOKENS, hbm_peak, tf_peak)

        # ---- the 32-bit path: single-token steps of one sequence at the same shape ---------------------
        del engine
        torch.cuda.empty_cache()
        full = wpc.Engine.from_random(cfg, seed=0, dtype="float32", device="cuda:0", max_tokens=CONTEXT + 2 * PAGE,
                                      max_sequences=2)
        fill_cache(full)
        k8 = max(K // 8, 8)
        s, _ = decode_run(full, gen, 1, CONTEXT - (k8 + W) - 1, k8, W)
        points["decode_b1_float32"] = k8 / s
        points["decode_b1_float32_hbm_frac"] = (weight_bytes(cfg, L, 4) + CONTEXT * kv_bytes_per_token(cfg, L, 4)) / (s / k8) / 1e9 / hbm_peak
        use_graphs = full.use_graphs
        del full
    else:
        use_graphs = engine.use_graphs

    line = {
        "metric": "decode tokens/s at batch 8 (Qwen2.5-7B shape, bf16, context 4096)",
        "value": value, "unit": "tokens/s", "n_gpus": 1, "steps": K, "warmup": W,
        "ms_per_step": secs / K * 1e3, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "bf16", "data": "synthetic: random N(0, 0.02) weights, uniform random token ids",
        "config": {"model": "Qwen2.5-7B shape", "global_batch": BATCH, "seq_len": CONTEXT,
                   "parallelism": "single GPU", "layers": L, "layers_of_shape": FULL_LAYERS,
                   "hidden": cfg.hidden_size, "heads": cfg.num_attention_heads, "kv_heads": cfg.num_key_value_heads,
                   "head_dim": cfg.head_dim, "intermediate": cfg.intermediate_size, "vocab": cfg.vocab_size,
                   "context_len": CONTEXT, "decode_start_ctx": start_ctx + W, "prefill_tokens": PREFILL_TOKENS,
                   "l2": "inputs larger than L2 (weights), no flush", "cuda_graphs": use_graphs},
        "e2e": e2e, "gpu_launches": launches, "prefill": prefill, "roofline": roofline, "points": points,
        "clocks": clocks.summary(), "impl": "ours",
    }
    if whole_run is not None:
        line["whole_run"] = whole_run
    if kernels is not None:
        line["kernels"] = kernels
    print(json.dumps(line))
    return 0


if __name__ == "__main__":
    sys.exit(main())
