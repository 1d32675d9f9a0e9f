"""bin/wpc-runtime as a user runs it: options in the reference's manner (wpc-runtime/src/main.rs:30-63
for --model and --max-tokens), token ids in, one JSON line per request out."""
import json
import os
import subprocess
import sys

import numpy as np
import pytest

from helpers import plain_logits
from plain import qwen2_plain as P

pytestmark = pytest.mark.gpu
CLI = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "bin", "wpc-runtime")


def run_cli(*args):
    return subprocess.run([sys.executable, CLI, *args], capture_output=True, text=True, timeout=600)


def test_cli_generates_greedily_and_prints_logits(folders):
    folder = folders[("A", "float32")]
    prompts = [[5, 17, 3, 9], [7, 1]]
    r = run_cli("--model", folder, "--dtype", "fp32", "--prompt-ids", "5,17,3,9;7,1", "--max-tokens", "4",
                "--stop-ids", "", "--print-logits", "3")
    assert r.returncode == 0, r.stderr
    lines = [json.loads(line) for line in r.stdout.splitlines() if line.strip()]
    tops = [x for x in lines if "top_logits" in x]
    outs = [x for x in lines if "generated" in x]
    assert [x["request"] for x in outs] == [0, 1] and [x["prompt_tokens"] for x in outs] == [4, 2]
    for i, p in enumerate(prompts):
        want = P.generate_greedy(*P.read_model_folder(folder), p, 4)
        assert outs[i]["generated"] == want
        logits = plain_logits(folder, p)[-1]
        best = np.argsort(-logits)[:3]
        assert [t for t, _ in tops[i]["top_logits"]] == best.tolist()
        assert np.allclose([v for _, v in tops[i]["top_logits"]], logits[best], atol=2e-4)
    # the diagnostics keep the reference's wording (main.rs:294, 309, 424)
    assert "prompt tokens (4): [5, 17, 3, 9]" in r.stderr and "generated 8 tokens in" in r.stderr


def test_cli_refuses_what_does_not_fit(folders):
    folder = folders[("A", "float32")]
    r = run_cli("--model", folder, "--prompt-ids", "1,2,3", "--max-tokens", "10", "--max-seq-len", "12")
    assert r.returncode == 2 and "--max-seq-len is 12" in r.stderr
    r = run_cli("--model", folder, "--max-tokens", "3")
    assert r.returncode == 2 and "--prompt-ids" in r.stderr
