"""bin/trace_run as a user runs it: a subprocess fed JSON steps on standard input, its logits
files compared with the plain implementation.  The same requests are replayed whole, with the
last 32 tokens one by one, and in batches of unequal lengths, in 32-bit and in bfloat16."""
import json
import os
import subprocess
import sys

import numpy as np
import pytest

from conftest import ROOT
from helpers import bfloat16_bound, plain_logits, random_tokens

pytestmark = pytest.mark.gpu
TRACE_RUN = os.path.join(ROOT, "bin", "trace_run")


def replay(folder, dtype, steps, out_dir, max_tokens):
    text = "".join(json.dumps(s) + "\n" for s in steps)
    r = subprocess.run([sys.executable, TRACE_RUN, "--model", folder, "--dtype", dtype, "--out", out_dir,
                        "--max-tokens", str(max_tokens)], input=text, capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stderr[-2000:]
    done = [line for line in r.stdout.splitlines() if line.startswith("done ")]
    assert done == [f"done {s['step']}" for s in steps]
    return r


def read(out_dir, step, vocab):
    return np.fromfile(os.path.join(out_dir, f"{step}.f32"), dtype="<f4").reshape(-1, vocab)


def bound(want64, dtype, folder, tokens):
    if dtype == "float32":
        want32 = plain_logits(folder, tokens, np.float32)
        return 4 * np.abs(want32 - want64).max() + 1e-6
    return bfloat16_bound(want64)


@pytest.mark.parametrize("name", ["A", "B", "C"])
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_replay_three_ways(folders, tmp_path, name, dtype):
    folder = folders[(name, dtype)]
    with open(os.path.join(folder, "config.json")) as f:
        vocab = json.load(f)["vocab_size"]
    # (Tiny-A takes at most 128 positions)
    reqs = {rid: random_tokens(vocab, n, 600 + i) for i, (rid, n) in enumerate([("a", 90), ("b", 40), ("c", 7)])}
    want = {rid: plain_logits(folder, t, np.float64) for rid, t in reqs.items()}

    # (1) each request alone and whole; (2) the last 32 one by one
    steps, expect = [], []
    n = 0
    for rid, toks in reqs.items():
        steps.append({"step": n, "entries": [{"id": rid + "w", "tokens": toks, "want": list(range(len(toks)))}],
                      "end": [rid + "w"]})
        expect.append((n, rid, 0, len(toks)))
        n += 1
        head = max(len(toks) - 32, 0)
        if head:
            steps.append({"step": n, "entries": [{"id": rid + "t", "tokens": toks[:head], "want": []}], "end": []})
            n += 1
        for i in range(head, len(toks)):
            steps.append({"step": n, "entries": [{"id": rid + "t", "tokens": [toks[i]], "want": [0]}],
                          "end": [rid + "t"] if i == len(toks) - 1 else []})
            expect.append((n, rid, i, i + 1))
            n += 1
    # (3) a batch of unequal lengths, twice, so that the second reuses what the first gave back
    for round_ in range(2):
        prompts = {"a": 50, "b": 40, "c": 3}
        fed = dict(prompts)
        live = list(reqs)
        entries = [{"id": f"{rid}{round_}", "tokens": reqs[rid][:prompts[rid]], "want": [prompts[rid] - 1]}
                   for rid in live]
        rows = [(rid, prompts[rid] - 1) for rid in live]
        while live:
            ended = [rid for rid in live if fed[rid] == len(reqs[rid])]
            steps.append({"step": n, "entries": entries, "end": [f"{rid}{round_}" for rid in ended]})
            expect.append((n, rows))
            n += 1
            live = [rid for rid in live if rid not in ended]
            entries = [{"id": f"{rid}{round_}", "tokens": [reqs[rid][fed[rid]]], "want": [0]} for rid in live]
            rows = [(rid, fed[rid]) for rid in live]
            for rid in live:
                fed[rid] += 1

    out_dir = str(tmp_path / "out")
    replay(folder, dtype, steps, out_dir, max_tokens=64 * 6)
    with open(os.path.join(out_dir, "index.jsonl")) as f:
        index = {rec["step"]: rec for rec in map(json.loads, f)}
    assert sorted(index) == sorted(s["step"] for s in steps if any(e["want"] for e in s["entries"]))
    for s in steps:
        if s["step"] in index:
            rec = index[s["step"]]
            assert rec["file"] == f"{s['step']}.f32" and rec["vocab"] == vocab
            assert rec["rows"] == [{"id": e["id"], "place": p} for e in s["entries"] for p in e["want"]]
    for item in expect:
        if len(item) == 4:
            step, rid, lo, hi = item
            got = read(out_dir, step, vocab)
            err = np.abs(got - want[rid][lo:hi]).max()
            assert err <= bound(want[rid], dtype, folder, reqs[rid]), (step, rid, lo, hi, err)
        else:
            step, rows = item
            got = read(out_dir, step, vocab)
            assert got.shape[0] == len(rows)
            for g, (rid, place) in zip(got, rows):
                err = np.abs(g - want[rid][place]).max()
                assert err <= bound(want[rid], dtype, folder, reqs[rid]), (step, rid, place, err)
