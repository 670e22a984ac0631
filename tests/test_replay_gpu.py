"""Replay on the GPU against the plain implementation: each request whole; most of it in one
step and the last 32 tokens one by one; portions of changing size; and mixed batches with so
few pages that they are used again; in float32 and in bfloat16, for both tiny configurations."""
import json
import os
import subprocess
import sys

import pytest
import torch

import replay_util as ru
from tiny_configs import CONFIGS, make_model_folder

pytestmark = pytest.mark.gpu

# Largest allowed difference of a logit from the plain float64 implementation. fp32: rounding
# of fp32 sums over at most a few hundred terms on logits of size ~1. bf16: activations are
# rounded to 8 bits of mantissa at each stored tensor; the plain implementation with the same
# roundings differs from the exact one by 3e-3 on these models.
ATOL = {torch.float32: 1e-5, torch.bfloat16: 1e-2}
LENGTHS = {"A": [1, 7, 33, 64, 150], "B": [3, 17, 50, 100, 129, 200]}


@pytest.fixture(scope="module")
def folders(tmp_path_factory):
    root = tmp_path_factory.mktemp("models")
    return {n: make_model_folder(root, n) for n in CONFIGS}


@pytest.fixture(scope="module")
def plains(folders):
    return {n: ru.PlainLogits(d) for n, d in folders.items()}


def requests_of(name):
    cfg, seed, _ = CONFIGS[name]
    return {f"r{i}": ru.random_tokens(cfg["vocab_size"], n, 100 * seed + i) for i, n in enumerate(LENGTHS[name])}


def replayer(folder, name, dtype, max_tokens):
    from llm_steadyinfer_b200.engine.replay import Replayer
    return Replayer(folder, dtype, max_tokens, page_size=CONFIGS[name][2])


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16], ids=["fp32", "bf16"])
@pytest.mark.parametrize("name", ["A", "B"])
@pytest.mark.parametrize("mode", ["whole", "tail", "portions", "mixed"])
def test_replay_modes(folders, plains, name, dtype, mode):
    reqs = requests_of(name)
    longest = ru.round64(max(len(t) for t in reqs.values()))
    if mode == "whole":
        steps, max_tokens = ru.trace_whole(reqs), longest
    elif mode == "tail":
        steps, max_tokens = ru.trace_tail(reqs), longest
    elif mode == "portions":
        steps, max_tokens = ru.trace_portions(reqs), longest
    else:
        max_tokens = longest + 128            # two or three requests at a time: pages are used again
        steps = ru.trace_mixed(reqs, max_tokens, seed=7)
    rp = replayer(folders[name], name, dtype, max_tokens)
    worst = ru.compare(rp, steps, reqs, plains[name], ATOL[dtype], f"{name}/{mode}/{dtype}")
    rp.runner.manager.check_invariant()
    assert not rp.runner.manager.requests, "every request of the trace was ended"
    assert rp.runner.manager.free_pages(0) == rp.runner.manager.groups[0].pool.num_pages
    print(f"{name} {mode} {dtype}: worst difference {worst:.2e}")


def test_trace_run_program(folders, plains, tmp_path):
    """The program itself, as a user runs it: JSON lines in, .f32 files and 'done' lines out."""
    name = "B"
    reqs = requests_of(name)
    max_tokens = 256 + 128
    steps = ru.trace_mixed(reqs, max_tokens, seed=3)
    out = tmp_path / "out"
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    proc = subprocess.run(
        [sys.executable, os.path.join(root, "bin", "trace_run"), "--model", folders[name], "--dtype", "float32",
         "--out", str(out), "--max-tokens", str(max_tokens), "--page-size", str(CONFIGS[name][2])],
        input="".join(json.dumps(s) + "\n" for s in steps), capture_output=True, text=True, timeout=600)
    assert proc.returncode == 0, proc.stderr[-2000:]
    done = [l for l in proc.stdout.splitlines() if l.startswith("done ")]
    assert done == [f"done {s['step']}" for s in steps]
    import numpy as np
    V = CONFIGS[name][0]["vocab_size"]
    pos = {}
    for s in steps:
        n_want = sum(len(e["want"]) for e in s["entries"])
        path = out / f"{s['step']}.f32"
        if n_want == 0:
            assert not path.exists()
            continue
        got = torch.from_numpy(np.fromfile(path, dtype="<f4").reshape(n_want, V))
        r = 0
        for e in s["entries"]:
            base = pos.get(e["id"], 0)
            for w in e["want"]:
                ref = plains[name].of(reqs[e["id"]])[base + w]
                assert (got[r].double() - ref).abs().max().item() <= ATOL[torch.float32]
                r += 1
            pos[e["id"]] = base + len(e["tokens"])
