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
LENGTHS = {"A": [1, 7, 33, 64, 150], "B": [3, 17, 50, 100, 129, 200], "C": [2, 40, 129, 200, 330]}


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
@pytest.mark.parametrize("name", ["A", "B", "C"])
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


# One block of the Llama-3.1-8B shape (widths, head layout, frequency scaling) with a small vocabulary: the sizes
# at which serving runs its kernels (TMA and tcgen05 attention, the few-row and the tcgen05 matrix products).
LAYER_8B = {
    "architectures": ["LlamaForCausalLM"], "model_type": "llama",
    "hidden_size": 4096, "intermediate_size": 14336, "num_hidden_layers": 1,
    "num_attention_heads": 32, "num_key_value_heads": 8, "head_dim": 128,
    "vocab_size": 2000, "max_position_embeddings": 8192, "rms_norm_eps": 1e-5,
    "rope_theta": 500000.0,
    "rope_scaling": {"rope_type": "llama3", "factor": 8.0, "low_freq_factor": 1.0,
                     "high_freq_factor": 4.0, "original_max_position_embeddings": 8192},
    "tie_word_embeddings": False, "hidden_act": "silu", "attention_bias": False,
    "mlp_bias": False, "torch_dtype": "bfloat16", "bos_token_id": 0, "eos_token_id": 1,
}


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16], ids=["fp32", "bf16"])
def test_replay_at_8b_layer_shape(tmp_path_factory, dtype):
    """Mixed replay (portions beside decoded tokens, pages used again) of one block at the Llama-3.1-8B shape.
    Allowed difference: fp32 sums run over up to 14,336 terms here, so 5e-5; bf16 three times the error that
    the plain implementation predicts when it rounds activations to bf16 where serving stores them."""
    from llm_steadyinfer_b200.engine.replay import Replayer
    from llm_steadyinfer_b200.weights import write_random_model
    import plain_llama
    folder = str(tmp_path_factory.mktemp("layer8b") / "m")
    write_random_model(folder, LAYER_8B, 5, torch.bfloat16)
    plain = ru.PlainLogits(folder)
    reqs = {f"q{i}": ru.random_tokens(LAYER_8B["vocab_size"], n, 900 + i) for i, n in enumerate([5, 70, 190])}
    if dtype == torch.float32:
        atol = 5e-5
    else:
        toks = reqs["q2"]
        predicted = (plain_llama.forward(plain.cfg, plain.w, toks, round_to=torch.bfloat16) - plain.of(toks)).abs().max().item()
        atol = 3 * predicted
    max_tokens = 256 + 128
    steps = ru.trace_mixed(reqs, max_tokens, seed=11)
    rp = Replayer(folder, dtype, max_tokens, page_size=16)
    worst = ru.compare(rp, steps, reqs, plain, atol, f"8B layer shape/{dtype}")
    rp.runner.manager.check_invariant()
    print(f"8B layer shape {dtype}: worst difference {worst:.2e} (allowed {atol:.2e})")


@pytest.mark.parametrize("seed", [101, 102, 103])
def test_mixed_replay_more_orders(folders, plains, seed):
    """More random orders of the mixed replay at the layout of the TMA and tcgen05 kernels, bf16: steps with
    one request follow steps with several, so that scratch shared between steps changes its layout."""
    name = "C"
    cfg, cseed, _ = CONFIGS[name]
    reqs = {f"r{i}": ru.random_tokens(cfg["vocab_size"], n, 1000 * cseed + i)
            for i, n in enumerate([2, 40, 129, 200, 330, 65, 64, 128])}
    max_tokens = 384 + 64 * (seed % 3)
    steps = ru.trace_mixed(reqs, max_tokens, seed=seed)
    rp = replayer(folders[name], name, torch.bfloat16, max_tokens)
    ru.compare(rp, steps, reqs, plains[name], ATOL[torch.bfloat16], f"{name}/mixed/seed {seed}")
    rp.runner.manager.check_invariant()


@pytest.mark.parametrize("name", ["B", "C"])
def test_graph_decode_logits(folders, plains, name):
    """The CUDA-graph decode step (fixed shapes, padding rows, splits chosen for the bucket) against the plain
    implementation, row by row, while the set of decoding requests changes between steps, so that graphs of
    different batch buckets follow each other on the same scratch; bf16."""
    import random
    from llm_steadyinfer_b200.engine.step import ModelRunner, StepEntry
    from llm_steadyinfer_b200.weights import load_model
    cfg, cseed, page = CONFIGS[name]
    lengths = [70, 33, 150, 5, 129, 90, 64, 17, 200]
    reqs = {f"g{i}": ru.random_tokens(cfg["vocab_size"], n + 40, 7000 + 10 * cseed + i) for i, n in enumerate(lengths)}
    model = load_model(folders[name], torch.bfloat16, "cuda:0")
    rn = ModelRunner(model, page_size=page, num_pages=256, max_requests=16, max_step_tokens=512)
    assert rn.graphs_available()
    pos = {}
    for (rid, toks), n in zip(reqs.items(), lengths):          # prompts, directly
        rn.step([StepEntry(rid, toks[:n], [])])
        pos[rid] = n
    rng = random.Random(5)
    worst, buckets = 0.0, set()
    for step in range(60):
        live = [r for r in reqs if pos[r] < len(reqs[r])]
        if not live:
            break
        chosen = rng.sample(live, rng.choice([1, 1, 2, 3, 5, 8, 9][:max(1, min(7, len(live)))]) if len(live) > 1 else 1)
        chosen = chosen[:len(live)]
        logits = rn.step_decode_graph([StepEntry(r, [reqs[r][pos[r]]], [0]) for r in chosen])
        buckets.add(len(chosen))
        for i, r in enumerate(chosen):
            ref = plains[name].of(reqs[r])[pos[r]]
            d = (logits[i].double().cpu() - ref).abs().max().item()
            assert d <= ATOL[torch.bfloat16], f"{name}: step {step}, request {r} at position {pos[r]} beside {chosen}: {d:.3e}"
            worst = max(worst, d)
            pos[r] += 1
    rn.check_status()
    assert len(rn._graphs) >= 3, "several batch buckets were captured"
    print(f"{name} graph decode: worst difference {worst:.2e}, batch sizes {sorted(buckets)}")


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16], ids=["fp32", "bf16"])
@pytest.mark.parametrize("name,seed", [("B", 1), ("C", 2), ("C", 3)])
def test_random_serving_through_the_runner(folders, plains, name, seed, dtype):
    """The step function driven as the entry point drives it, with given tokens: steps that mix prompt
    portions with decode rows run directly, steps of decode rows alone run from CUDA graphs, in random turn;
    requests join while others decode and leave when done, in a pool that makes them wait for pages. Every
    wanted row against the plain implementation."""
    import random
    from llm_steadyinfer_b200.engine.step import ModelRunner, StepEntry
    from llm_steadyinfer_b200.weights import load_model
    cfg, _, page = CONFIGS[name]
    rng = random.Random(seed)
    num_pages = 640 // page
    rn = ModelRunner(load_model(folders[name], dtype, "cuda:0"), page_size=page, num_pages=num_pages, max_requests=8,
                     max_step_tokens=256)
    pool = [ru.random_tokens(cfg["vocab_size"], rng.choice([3, 17, 40, 64, 65, 100, 129, 180]) + rng.choice([5, 20, 33]),
                             seed * 100 + i) for i in range(12)]
    waiting, live = list(range(len(pool))), {}                 # live: request -> [tokens done, tokens of its "prompt"]
    steps = graph_steps = 0
    worst = 0.0
    while waiting or live:
        while waiting and len(live) < 6 and rng.random() < 0.5:
            i = waiting[0]
            if sum(-(-len(pool[j]) // page) for j in list(live) + [i]) > num_pages:
                break
            waiting.pop(0)
            live[i] = [0, len(pool[i]) - rng.choice([5, 20])]
        entries, meta = [], []
        prompts = [i for i in live if live[i][0] < live[i][1]]
        for i in live:
            if live[i][0] >= live[i][1] and rng.random() < 0.85:
                entries.append(StepEntry(f"q{i}", [pool[i][live[i][0]]], [0]))
                meta.append((i, live[i][0], 1))
        from_graph = not prompts or rng.random() < 0.3
        budget = rng.choice([16, 48, 100])
        for i in ([] if from_graph else prompts):
            n = min(budget, live[i][1] - live[i][0], rng.choice([2, 7, 30, 64, 100]))
            if n <= 0:
                break
            budget -= n
            p = live[i][0]
            entries.append(StepEntry(f"q{i}", pool[i][p:p + n], [n - 1]))
            meta.append((i, p + n - 1, n))
        if not entries:
            continue
        logits = rn.step_decode_graph(entries) if from_graph else rn.step(entries)
        steps += 1
        graph_steps += from_graph
        for r, (i, p, n) in enumerate(meta):
            d = (logits[r].double().cpu() - plains[name].of(pool[i])[p]).abs().max().item()
            assert d <= ATOL[dtype], (f"{name} {dtype}: step {steps}, request q{i} position {p} ({n} tokens, "
                                      f"from a graph: {from_graph}, batch {[(m[0], m[2]) for m in meta]}): {d:.3e}")
            worst = max(worst, d)
            live[i][0] += n
        for i in [i for i in live if live[i][0] >= len(pool[i])]:
            rn.finish(f"q{i}")
            del live[i]
    rn.check_status()
    rn.manager.check_invariant()
    assert graph_steps >= 10 and steps - graph_steps >= 10
    print(f"{name} {dtype}: {steps} steps, {graph_steps} from graphs, worst difference {worst:.2e}")


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


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16], ids=["fp32", "bf16"])
def test_long_decoding(folders, plains, dtype):
    """A short prompt, then 450 tokens one by one (given tokens, every row compared): positions far
    beyond the original range of the scaled rotary frequencies, many page edges."""
    name = "B"
    cfg = CONFIGS[name][0]
    reqs = {"long": ru.random_tokens(cfg["vocab_size"], 460, 77)}
    steps = ru.trace_tail(reqs, tail=450)
    rp = replayer(folders[name], name, dtype, 512)
    worst = ru.compare(rp, steps, reqs, plains[name], ATOL[dtype], f"long decode {dtype}")
    assert len(steps) == 451
    print(f"long decoding {dtype}: worst difference {worst:.2e}")


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16], ids=["fp32", "bf16"])
@pytest.mark.parametrize("name", ["A", "B"])
def test_first_tokens_one_by_one(folders, plains, name, dtype):
    """A sequence fed from its very first token in single-token steps, beside another that starts
    two steps later: position 0, the first page, the first page edge."""
    cfg, _, page = CONFIGS[name]
    reqs = {"p": ru.random_tokens(cfg["vocab_size"], 2 * page + 3, 5), "q": ru.random_tokens(cfg["vocab_size"], page + 2, 6)}
    steps = []
    for i in range(len(reqs["p"])):
        entries = [{"id": "p", "tokens": [reqs["p"][i]], "want": [0]}]
        j = i - 2
        if 0 <= j < len(reqs["q"]):
            entries.append({"id": "q", "tokens": [reqs["q"][j]], "want": [0]})
        end = [r for r, k in (("p", i), ("q", j)) if k == len(reqs[r]) - 1]
        steps.append({"step": i, "entries": entries, "end": end})
    rp = replayer(folders[name], name, dtype, 256)
    ru.compare(rp, steps, reqs, plains[name], ATOL[dtype], f"first tokens {name} {dtype}")
    assert not rp.runner.manager.requests


def test_step_rejects_what_it_cannot_hold(folders):
    """Too many tokens for the pool: one clear error, nothing taken, and the engine goes on."""
    from llm_steadyinfer_b200.cache import OutOfPages
    from llm_steadyinfer_b200.engine.step import StepError
    rp = replayer(folders["A"], "A", torch.float32, 64)
    toks = ru.random_tokens(512, 60, 1)
    rp.run_step([{"id": "a", "tokens": toks[:40], "want": []}], [])
    with pytest.raises(OutOfPages):
        rp.run_step([{"id": "b", "tokens": toks[:40], "want": []}], [])
    assert rp.runner.manager.free_pages(0) == 1 and rp.runner.manager.table(0, "b") == []
    with pytest.raises(StepError):
        rp.run_step([{"id": "a", "tokens": [1], "want": [3]}], [])
    with pytest.raises(StepError):
        rp.run_step([{"id": "a", "tokens": [999999], "want": [0]}], [])      # outside the vocabulary: flagged
    rp.run_step([], ["a", "b"])
    rp.runner.manager.check_invariant()
    assert rp.runner.manager.free_pages(0) == 4


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16], ids=["fp32", "bf16"])
def test_a_name_used_again(folders, plains, dtype):
    """A request ends and a new one comes under the same name, with other tokens, after its pages have gone
    to someone else, and with a table that has changed as often as the first one's: nothing kept from the first
    (its block table) may serve the second, or it writes into the other request's pages."""
    name = "B"
    cfg, _, page = CONFIGS[name]
    rp = replayer(folders[name], name, dtype, 256)
    first = ru.random_tokens(cfg["vocab_size"], 20, 31)
    other = ru.random_tokens(cfg["vocab_size"], 12, 32)
    second = ru.random_tokens(cfg["vocab_size"], 20, 33)
    steps = [
        ("x", first, 0, 20, ["x"]),          # whole, in one step, and gone
        ("z", other, 0, 9, []),              # takes the pages that x gave back
        ("x", second, 0, 20, []),            # the name again, again in one step
        ("z", other, 9, 3, ["x", "z"]),      # z goes on: its first pages must still hold its keys
    ]
    for rid, toks, start, n, end in steps:
        out = rp.run_step([{"id": rid, "tokens": toks[start:start + n], "want": list(range(n))}], end)
        for w in range(n):
            ref = plains[name].of(toks)[start + w]
            assert (out[w].double().cpu() - ref).abs().max().item() <= ATOL[dtype], (rid, start + w)
    rp.runner.manager.check_invariant()


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16], ids=["fp32", "bf16"])
@pytest.mark.parametrize("name", ["A", "B", "C"])
def test_mixed_replay_with_requests_cut_back(folders, plains, name, dtype):
    """The mixed replay with a "truncate" record every few steps: a live request is cut back to a random
    length as a preemption cuts it (whole pages stay, the rest goes back to the pool and is used by others),
    and its cut tokens are computed again in portions beside the other requests. Every row that is computed
    again, and every row after it, against the plain implementation."""
    reqs = requests_of(name)
    page = CONFIGS[name][2]
    max_tokens = ru.round64(max(len(t) for t in reqs.values())) + 128
    kept = lambda held, keep: min(keep // page * page, held // page * page)
    steps = ru.trace_mixed(reqs, max_tokens, seed=13, cut_every=3, kept=kept)
    cuts = [t for s in steps for t in s.get("truncate", ())]
    assert len(cuts) >= 4
    rp = replayer(folders[name], name, dtype, max_tokens)
    assert all(rp.kept_after_truncate(h, k) == kept(h, k) for h, k in ((37, 20), (64, 64), (5, 100), (200, 17)))
    worst = ru.compare(rp, steps, reqs, plains[name], ATOL[dtype], f"{name}/cut back/{dtype}")
    rp.runner.manager.check_invariant()
    assert not rp.runner.manager.requests
    assert rp.runner.manager.free_pages(0) == rp.runner.manager.groups[0].pool.num_pages
    print(f"{name} cut back {dtype}: {len(cuts)} cuts, worst difference {worst:.2e}")


def test_trace_run_program_with_truncate_records(folders, plains, tmp_path):
    """The "truncate" record through the program itself, in bfloat16."""
    name = "C"
    reqs = requests_of(name)
    page = CONFIGS[name][2]
    max_tokens = 384 + 128
    kept = lambda held, keep: min(keep // page * page, held // page * page)
    steps = ru.trace_mixed(reqs, max_tokens, seed=5, cut_every=4, kept=kept)
    out = tmp_path / "out"
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    proc = subprocess.run(
        [sys.executable, os.path.join(root, "bin", "trace_run"), "--model", folders[name], "--dtype", "bfloat16",
         "--out", str(out), "--max-tokens", str(max_tokens), "--page-size", str(page)],
        input="".join(json.dumps(s) + "\n" for s in steps), capture_output=True, text=True, timeout=600)
    assert proc.returncode == 0, proc.stderr[-2000:]
    assert [l for l in proc.stdout.splitlines() if l.startswith("done ")] == [f"done {s['step']}" for s in steps]
    import numpy as np
    V = CONFIGS[name][0]["vocab_size"]
    pos, checked = {}, 0
    for s in steps:
        for t in s.get("truncate", ()):
            pos[t["id"]] = kept(pos[t["id"]], t["keep"])
        n_want = sum(len(e["want"]) for e in s["entries"])
        if n_want == 0:
            continue
        got = torch.from_numpy(np.fromfile(out / f"{s['step']}.f32", dtype="<f4").reshape(n_want, V))
        r = 0
        for e in s["entries"]:
            base = pos.get(e["id"], 0)
            for w in e["want"]:
                ref = plains[name].of(reqs[e["id"]])[base + w]
                assert (got[r].double() - ref).abs().max().item() <= ATOL[torch.bfloat16], (s["step"], e["id"], base + w)
                r += 1
                checked += 1
            pos[e["id"]] = base + len(e["tokens"])
    assert checked > 100


@pytest.mark.parametrize("own_rows", [False, True], ids=["library", "gemm_rows"])
@pytest.mark.parametrize("name", ["C"])
def test_graph_decode_logits_at_17_to_64_rows(folders, plains, name, own_rows, monkeypatch):
    """Decode steps of 17 to 64 live requests, bfloat16, through the recorded step: above 16 rows every
    projection leaves the few-row product (for the library product, or for the package's tcgen05 kernel for up
    to 128 rows when that is turned on), decode attention gets more items than one wave of shares, and the
    buckets 24, 32, 48 and 64 are recorded. Every row of every step against the plain implementation."""
    import random
    from llm_steadyinfer_b200.parts import linear as linear_mod
    monkeypatch.setattr(linear_mod, "USE_ROWS", own_rows)
    from llm_steadyinfer_b200.engine.step import ModelRunner, StepEntry
    from llm_steadyinfer_b200.weights import load_model
    cfg, cseed, page = CONFIGS[name]
    rng = random.Random(3)
    lengths = [rng.choice([3, 17, 33, 64, 65, 90, 129, 150]) for _ in range(64)]
    extra = 14
    reqs = {f"g{i}": ru.random_tokens(cfg["vocab_size"], n + extra, 8000 + i) for i, n in enumerate(lengths)}
    model = load_model(folders[name], torch.bfloat16, "cuda:0")
    pages = sum(-(-(n + extra) // page) for n in lengths) + 8
    rn = ModelRunner(model, page_size=page, num_pages=pages, max_requests=64, max_step_tokens=1024)
    pos = {}
    ids = list(reqs)
    for a in range(0, 64, 8):                                   # prompts, eight requests a step
        rn.step([StepEntry(r, reqs[r][:lengths[int(r[1:])]], []) for r in ids[a:a + 8]])
    for r in ids:
        pos[r] = lengths[int(r[1:])]
    worst, sizes = 0.0, []
    for step, size in enumerate([64, 17, 33, 24, 48, 64, 17, 40, 64, 20, 33, 64, 25, 57]):
        chosen = rng.sample([r for r in ids if pos[r] < len(reqs[r])], size)
        logits = rn.step_decode_graph([StepEntry(r, [reqs[r][pos[r]]], [0]) for r in chosen])
        sizes.append(size)
        got = logits.double().cpu()
        for i, r in enumerate(chosen):
            d = (got[i] - plains[name].of(reqs[r])[pos[r]]).abs().max().item()
            assert d <= ATOL[torch.bfloat16], f"step {step} of {size} rows, request {r} at position {pos[r]}: {d:.3e}"
            worst = max(worst, d)
            pos[r] += 1
    rn.check_status()
    assert {b for b, _ in rn._graphs} >= {24, 32, 48, 64} and not rn.capture_failed
    print(f"{name} graph decode at {sorted(set(sizes))} rows: worst difference {worst:.2e}")


def test_graph_decode_logits_at_33_rows_8b_layer_shape(tmp_path_factory):
    """The same at the widths of one Llama-3.1-8B block (small vocabulary): 33 and 20 live requests, bfloat16,
    recorded steps; the projections run as library products here and decode attention on the TMA kernel.
    Allowed: three times the error that the plain implementation predicts with bf16 roundings."""
    import plain_llama
    from llm_steadyinfer_b200.engine.step import ModelRunner, StepEntry
    from llm_steadyinfer_b200.weights import load_model, write_random_model
    folder = str(tmp_path_factory.mktemp("layer8b_rows") / "m")
    write_random_model(folder, LAYER_8B, 6, torch.bfloat16)
    plain = ru.PlainLogits(folder)
    lengths = [5 + (7 * i) % 40 for i in range(33)]
    extra = 4
    reqs = {f"h{i}": ru.random_tokens(LAYER_8B["vocab_size"], n + extra, 8100 + i) for i, n in enumerate(lengths)}
    toks = reqs["h32"]
    atol = 3 * (plain_llama.forward(plain.cfg, plain.w, toks, round_to=torch.bfloat16) - plain.of(toks)).abs().max().item()
    model = load_model(folder, torch.bfloat16, "cuda:0")
    rn = ModelRunner(model, page_size=16, num_pages=33 * 4, max_requests=48, max_step_tokens=1024)
    ids = list(reqs)
    rn.step([StepEntry(r, reqs[r][:lengths[i]], []) for i, r in enumerate(ids)])
    pos = {r: lengths[i] for i, r in enumerate(ids)}
    worst = 0.0
    for step, chosen in enumerate([ids, ids[:20], ids[5:], ids]):
        chosen = [r for r in chosen if pos[r] < len(reqs[r])]
        logits = rn.step_decode_graph([StepEntry(r, [reqs[r][pos[r]]], [0]) for r in chosen]).double().cpu()
        for i, r in enumerate(chosen):
            d = (logits[i] - plain.of(reqs[r])[pos[r]]).abs().max().item()
            assert d <= atol, f"step {step} of {len(chosen)} rows, request {r} at position {pos[r]}: {d:.3e} (allowed {atol:.2e})"
            worst = max(worst, d)
            pos[r] += 1
    rn.check_status()
    print(f"8B layer shape, 20 to 33 decode rows: worst difference {worst:.2e} (allowed {atol:.2e})")


LONG = {
    "architectures": ["LlamaForCausalLM"], "model_type": "llama",
    "hidden_size": 512, "intermediate_size": 1024, "num_hidden_layers": 2,
    "num_attention_heads": 4, "num_key_value_heads": 1, "head_dim": 128,
    "vocab_size": 500, "max_position_embeddings": 16384, "rms_norm_eps": 1e-5,
    "rope_theta": 500000.0,
    "rope_scaling": {"rope_type": "llama3", "factor": 8.0, "low_freq_factor": 1.0,
                     "high_freq_factor": 4.0, "original_max_position_embeddings": 8192},
    "tie_word_embeddings": True, "hidden_act": "silu", "attention_bias": False,
    "mlp_bias": False, "torch_dtype": "bfloat16", "bos_token_id": 0, "eos_token_id": 1,
}


@pytest.fixture(scope="module")
def long_model(tmp_path_factory):
    """The folder of the long-context model and its plain logits (half a minute on the host: made once)."""
    from safetensors.torch import load_file
    from llm_steadyinfer_b200.weights import write_random_model, write_safetensors
    folder = str(tmp_path_factory.mktemp("long") / "m")
    write_random_model(folder, LONG, 7, torch.bfloat16)
    path = os.path.join(folder, "model.safetensors")
    t = load_file(path)
    for k in t:
        if k.endswith("q_proj.weight") or k.endswith("k_proj.weight"):
            t[k] = (t[k].float() * 3.0).to(torch.bfloat16)
    write_safetensors(path, t)
    plain = ru.PlainLogits(folder)
    toks = ru.random_tokens(LONG["vocab_size"], 9016, 1)
    plain.of(toks)
    return folder, plain, toks


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16], ids=["fp32", "bf16"])
def test_long_context_replay(long_model, dtype):
    """A narrow model with the Llama-3.1-8B head size and frequency scaling taken to 9,016 tokens: the prompt in
    portions of 2,048 up to 8,152, 80 tokens one by one across position 8,192, a further portion up to 9,000 and
    16 more tokens, with a short request decoding beside it (so that the long one is cut into many more shares
    than the short one). Block tables of 564 pages, decode attention in up to 32 splits, positions beyond the
    original range of the scaled frequencies. The query and key projections are scaled up so that the softmax
    picks out few keys at whatever distance they lie, and a fault in one far tile shows in the logits."""
    import plain_llama
    from llm_steadyinfer_b200.engine.replay import Replayer
    folder, plain, long_toks = long_model
    V = LONG["vocab_size"]
    short_toks = ru.random_tokens(V, 40 + 95, 2)
    ref = plain.of(long_toks)
    steps, p = [], 0

    def portion(n, beside=None):
        nonlocal p
        want = sorted(set(range(0, n, 97)) | {n - 1})
        e = [{"id": "L", "tokens": long_toks[p:p + n], "want": want}]
        if beside is not None:
            e.append(beside)
        steps.append({"step": len(steps), "entries": e, "end": []})
        p += n

    sp = 0

    def short_row():
        nonlocal sp
        if sp == 0:
            e, sp = {"id": "S", "tokens": short_toks[:40], "want": [39]}, 40
        else:
            e, sp = {"id": "S", "tokens": [short_toks[sp]], "want": [0]}, sp + 1
        return e

    for n in (2048, 2048, 2048, 2008):
        portion(n)
    for _ in range(80):
        portion(1, short_row())
    portion(768)
    for _ in range(16):
        portion(1, short_row())
    steps[-1]["end"] = ["L", "S"]
    assert p == 9016 and sp == 135
    reqs = {"L": long_toks, "S": short_toks}
    if dtype == torch.float32:
        atol = 5e-5
    else:
        probe = long_toks[:600]
        atol = 3 * (plain_llama.forward(plain.cfg, plain.w, probe, round_to=torch.bfloat16) - plain.of(probe)).abs().max().item()
    rp = Replayer(folder, dtype, max_tokens=9088 + 192, page_size=16)
    worst = ru.compare(rp, steps, reqs, plain, atol, f"long context/{dtype}")
    assert not rp.runner.manager.requests
    rp.runner.manager.check_invariant()
    print(f"long context {dtype}: worst difference {worst:.2e} (allowed {atol:.2e}); logits up to {ref.abs().max().item():.1f}")


def test_random_weights_drawn_on_the_gpu_equal_a_written_folder(tmp_path):
    """``init_random`` on the device and ``write_random_model`` on the host give the same tensors, bit for bit."""
    from llm_steadyinfer_b200.config import config_from_dict
    from llm_steadyinfer_b200.models import Model
    from llm_steadyinfer_b200.weights import init_random, load_model, write_random_model
    cfg = CONFIGS["B"][0]
    folder = str(tmp_path / "m")
    write_random_model(folder, cfg, 4, torch.bfloat16)
    a = load_model(folder, torch.bfloat16, "cuda:0")
    b = Model(config_from_dict(cfg), torch.bfloat16, "cuda:0")
    init_random(b, seed=4)
    assert torch.equal(a.embed, b.embed) and torch.equal(a.lm_head, b.lm_head)
    assert torch.equal(a.final_norm.weight, b.final_norm.weight)
    for x, y in zip(a.blocks, b.blocks):
        assert torch.equal(x.mixer.qkv, y.mixer.qkv) and torch.equal(x.mixer.o, y.mixer.o)
        assert torch.equal(x.feed_forward.gate_up, y.feed_forward.gate_up) and torch.equal(x.feed_forward.down, y.feed_forward.down)
        assert torch.equal(x.mixer_norm.weight, y.mixer_norm.weight)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16], ids=["fp32", "bf16"])
def test_8b_shape_drawn_on_the_gpu_against_plain_on_the_same_draw(dtype):
    """One block of the Llama-3.1-8B shape with its weights drawn on the device, as the benchmark draws its 32
    blocks, against the plain implementation on the same draw made on the host: the counter-based draw is what
    lets a model that was never written to disk be checked."""
    import plain_llama
    from llm_steadyinfer_b200.config import config_from_dict
    from llm_steadyinfer_b200.engine.step import ModelRunner, StepEntry
    from llm_steadyinfer_b200.models import Model
    from llm_steadyinfer_b200.weights import init_random
    from llm_steadyinfer_b200.weights.random_init import random_tensors
    cfg = config_from_dict(LAYER_8B)
    model = Model(cfg, dtype, "cuda:0")
    init_random(model, seed=12)
    w = {k: v.double() for k, v in random_tensors(Model(cfg, torch.float32, "cpu"), 12, torch.bfloat16).items()}
    toks = ru.random_tokens(LAYER_8B["vocab_size"], 150, 5)
    want = plain_llama.forward(LAYER_8B, w, toks)
    rn = ModelRunner(model, page_size=16, num_pages=16, max_requests=2, max_step_tokens=256)
    rows = [0, 1, 63, 127, 128]
    got = rn.step([StepEntry("r", toks[:129], rows)]).double().cpu()
    tail = [rn.step([StepEntry("r", [toks[p]], [0])]).double().cpu()[0] for p in range(129, 150)]
    rn.check_status()
    if dtype == torch.float32:
        atol = 5e-5
    else:
        atol = 3 * (plain_llama.forward(LAYER_8B, w, toks, round_to=torch.bfloat16) - want).abs().max().item()
    for r, g in list(zip(rows, got)) + list(zip(range(129, 150), tail)):
        d = (g - want[r]).abs().max().item()
        assert d <= atol, f"position {r}: {d:.3e} (allowed {atol:.2e})"


@pytest.mark.parametrize("first", [0, 6, 12])
def test_random_configurations_replay(tmp_path, first):
    """A random search over configurations (head sizes in steps of 16 up to 256 and some that are no multiple of
    16, any numbers of heads and groups, widths and vocabularies that are no power of two, some odd, with and
    without frequency scaling, tied and untied head,
    pages of 4 to 64 tokens, pools from one request's size up) and mixed traces with cuts, in both precisions:
    whatever the configuration allows runs through some kernel and gives the plain implementation's logits."""
    import random
    from llm_steadyinfer_b200.engine.replay import Replayer
    from llm_steadyinfer_b200.weights import write_random_model
    for seed in range(first, first + 6):
        rng = random.Random(seed)
        hs = rng.choice([8, 16, 24, 32, 48, 64, 64, 80, 96, 112, 128, 128, 136, 192, 256])
        KV, G = rng.choice([1, 2, 3, 5]), rng.choice([1, 2, 3, 4, 7, 8])
        while KV * G > 16:
            G = rng.choice([1, 2, 3, 4])
        scaling = {"rope_type": "llama3", "factor": rng.choice([2.0, 8.0, 32.0]), "low_freq_factor": 1.0,
                   "high_freq_factor": rng.choice([2.0, 4.0]), "original_max_position_embeddings": rng.choice([32, 64, 128])}
        cfg = {"architectures": ["LlamaForCausalLM"], "model_type": "llama",
               "hidden_size": rng.choice([64, 67, 96, 100, 136, 200, 256, 328]),
               "intermediate_size": rng.choice([72, 75, 100, 192, 328, 520]),
               "num_hidden_layers": rng.choice([1, 2, 3]), "num_attention_heads": KV * G, "num_key_value_heads": KV,
               "head_dim": hs, "vocab_size": rng.choice([130, 512, 777, 1000, 2003]), "max_position_embeddings": 1024,
               "rms_norm_eps": rng.choice([1e-5, 1e-6, 3e-6]), "rope_theta": rng.choice([1e4, 5e5]),
               "rope_scaling": rng.choice([None, scaling]), "tie_word_embeddings": rng.random() < 0.5,
               "hidden_act": "silu", "attention_bias": False, "mlp_bias": False, "torch_dtype": "bfloat16",
               "bos_token_id": 0, "eos_token_id": 1}
        page = rng.choice([4, 8, 16, 32, 64])
        folder = str(tmp_path / f"m{seed}")
        write_random_model(folder, cfg, seed, torch.bfloat16)
        reqs = {f"r{i}": ru.random_tokens(cfg["vocab_size"], rng.choice([3, 20, 45, 64, 65, 100, 129, 200, 300]), 100 * seed + i)
                for i in range(5)}
        max_tokens = max(ru.round64(len(t)) for t in reqs.values()) + rng.choice([0, 64, 192, 512])
        plain = ru.PlainLogits(folder)
        cut_every = rng.choice([0, 4, 7])
        for dtype in (torch.float32, torch.bfloat16):
            rp = Replayer(folder, dtype, max_tokens, page_size=page)
            steps = ru.trace_mixed(reqs, max_tokens, seed=seed, cut_every=cut_every, kept=rp.kept_after_truncate)
            ru.compare(rp, steps, reqs, plain, ATOL[dtype],
                       f"seed {seed}: head size {hs}, {KV * G} heads, {KV} groups, page {page}, {dtype}")
            rp.runner.manager.check_invariant()
