"""The plain implementation: against the stored outputs of the reference's own CPU model code,
and its parts against their definitions."""
import ast
import math
import os

import numpy as np
import pytest
import torch

import plain_llama as pl

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")


def load_golden(name):
    z = np.load(os.path.join(GOLDEN, f"golden_{name}.npz"))
    cfg = ast.literal_eval(str(z["config"]))
    w = {k[2:]: torch.from_numpy(z[k]).to(pl.DT) for k in z.files if k.startswith("w:")}
    return cfg, w, z


@pytest.mark.parametrize("name", ["g1", "g2"])
def test_plain_equals_reference_cpu_code(name):
    cfg, w, z = load_golden(name)
    prompt = z["prompt"].tolist()
    got = pl.forward(cfg, w, prompt)
    ref = torch.from_numpy(z["logits"]).double()
    assert (got - ref).abs().max().item() < 5e-6        # the reference computes in fp32
    assert pl.generate(cfg, w, prompt, 8) == z["gen_full"].tolist()
    assert pl.generate(cfg, w, prompt[:3], 8) == z["gen_short"].tolist()


@pytest.mark.parametrize("hs", [16, 32, 64])
def test_rope_angles_equal_the_reference_tables_at_other_thetas(hs):
    """The reference's own sine / cosine table function takes theta as an argument
    (src/source/op/kernels/cpu/rope_kernel.cpp:3-16; entry 2i of a row is the pair's angle, :76-77): its tables
    at theta 1e4, 5e5 and 1e6 against the frequencies and the rotation of the plain implementation."""
    z = np.load(os.path.join(GOLDEN, "golden_rope.npz"))
    theta = float(z[f"theta_{hs}"])
    sin_t, cos_t = torch.from_numpy(z[f"sin_{hs}"]), torch.from_numpy(z[f"cos_{hs}"])        # [positions, hs]
    n = sin_t.shape[0]
    freqs = pl.rope_frequencies(hs, theta, None)
    ang = torch.arange(n, dtype=torch.float32)[:, None] * freqs[None, :]
    # the reference forms theta^(-j/hs) with a float pow: a frequency may differ by an ulp, an angle by 95 ulps of it
    assert (torch.sin(ang) - sin_t[:, 0::2]).abs().max().item() < 2e-5
    assert (torch.cos(ang) - cos_t[:, 0::2]).abs().max().item() < 2e-5
    g = torch.Generator().manual_seed(hs)
    x = torch.randn(n, 3, hs, generator=g, dtype=pl.DT)
    got = pl.rope(x, torch.arange(n), freqs)
    c, s = cos_t[:, 0::2].double()[:, None, :], sin_t[:, 0::2].double()[:, None, :]
    x0, x1 = x[..., :hs // 2], x[..., hs // 2:]
    want = torch.cat([c * x0 - s * x1, c * x1 + s * x0], dim=-1)      # the reference's rotation with its own tables
    assert (got - want).abs().max().item() < 1e-4


def test_rmsnorm_definition():
    x = torch.tensor([[3.0, 4.0]], dtype=pl.DT)
    y = pl.rmsnorm(x, torch.tensor([2.0, 0.5], dtype=pl.DT), 0.0)
    assert torch.allclose(y, torch.tensor([[2 * 3 / math.sqrt(12.5), 0.5 * 4 / math.sqrt(12.5)]], dtype=pl.DT))


def test_rope_is_a_rotation_and_relative():
    f = pl.rope_frequencies(8, 10000.0, None)
    assert torch.allclose(f.double(), torch.tensor([1.0, 0.1, 0.01, 0.001], dtype=pl.DT), rtol=1e-6)
    g = torch.Generator().manual_seed(0)
    q = torch.randn(1, 1, 8, generator=g, dtype=pl.DT)
    k = torch.randn(1, 1, 8, generator=g, dtype=pl.DT)
    assert torch.equal(pl.rope(q, torch.tensor([0]), f), q)
    dots = []
    for p in (0, 5, 40):
        rq = pl.rope(q, torch.tensor([p + 3]), f)
        rk = pl.rope(k, torch.tensor([p]), f)
        assert abs(rq.norm().item() - q.norm().item()) < 1e-6
        dots.append((rq * rk).sum().item())
    assert max(dots) - min(dots) < 1e-5, "the score depends on the distance only"


def test_llama3_frequency_scaling_bands():
    sc = {"rope_type": "llama3", "factor": 8.0, "low_freq_factor": 1.0, "high_freq_factor": 4.0,
          "original_max_position_embeddings": 64}
    base = pl.rope_frequencies(32, 500000.0, None).double()
    f = pl.rope_frequencies(32, 500000.0, sc).double()
    wl = 2 * math.pi / base
    hi, lo = wl < 64 / 4, wl > 64 / 1
    assert hi.any() and lo.any() and (~hi & ~lo).any()
    assert torch.allclose(f[hi], base[hi]) and torch.allclose(f[lo], base[lo] / 8, rtol=1e-6)
    mid = ~hi & ~lo
    assert ((f[mid] < base[mid]) & (f[mid] > base[mid] / 8)).all()


def test_attention_is_causal_grouped_and_windowed():
    g = torch.Generator().manual_seed(1)
    T, H, KV, hs = 9, 4, 2, 8
    q, k, v = (torch.randn(T, n, hs, generator=g, dtype=pl.DT) for n in (H, KV, KV))
    out = pl.attention(q, k, v, 0.3)
    k2, v2 = k.clone(), v.clone()
    k2[5:] += 1.0; v2[5:] -= 2.0
    out2 = pl.attention(q, k2, v2, 0.3)
    assert torch.equal(out[:5], out2[:5]) and not torch.allclose(out[5:], out2[5:])
    assert torch.allclose(out[0], v[0].repeat_interleave(2, 0)), "position 0 sees itself only; heads 0,1 -> kv 0"
    w1 = pl.attention(q, k, v, 0.3, window=1)
    assert torch.allclose(w1, v.repeat_interleave(2, 1))
    w3 = pl.attention(q, k, v, 0.3, window=3)
    assert torch.allclose(w3[:3], out[:3]) and not torch.allclose(w3[3:], out[3:])


def test_swiglu_definition():
    a = torch.tensor([0.0, 1.0, -2.0], dtype=pl.DT)
    b = torch.tensor([5.0, 2.0, 3.0], dtype=pl.DT)
    want = torch.tensor([0.0, 2.0 / (1 + math.exp(-1.0)), -6.0 / (1 + math.exp(2.0))], dtype=pl.DT)
    assert torch.allclose(pl.swiglu(a, b), want)


def test_sampling_rules():
    x = torch.tensor([1.0, 3.0, 3.0, 0.0, 2.0])
    assert pl.sample(x) == 1                                   # tie: lowest index
    assert pl.sample(x, temperature=1.0, top_k=1, seed=3, counter=9) in (1, 2)   # ties of the k-th are kept
    seen = {pl.sample(x, 1.0, top_k=3, seed=5, counter=c) for c in range(200)}
    assert seen == {1, 2, 4}
    p = torch.softmax(x.double(), 0)
    seen = {pl.sample(x, 1.0, top_p=float(p[1] + p[2]) - 1e-6, seed=5, counter=c) for c in range(200)}
    assert seen == {1, 2}
    a = [pl.sample(x, 0.9, seed=7, counter=c) for c in range(20)]
    assert a == [pl.sample(x, 0.9, seed=7, counter=c) for c in range(20)] and len(set(a)) > 1
    u = [pl.uniform01(1, c) for c in range(2000)]
    assert 0 <= min(u) and max(u) < 1 and abs(sum(u) / 2000 - 0.5) < 0.03
