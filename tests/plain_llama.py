"""Plain, slow Llama 3 on the CPU: whole sequences, no cache, one function per part, float64
arithmetic by default. It shares no code with the package; every function is written from the
formulas of the reference (paths are relative to the reference project's root).

It was compared once with the reference's own CPU model code on a tiny random model; the
script and its small outputs are under tests/golden/ (see tests/golden/README.md). Of the options that
the reference's model code fixes, theta is covered at three values through its table function, which
takes theta as an argument; eps (1e-6), frequency scaling (none), head size (hidden/heads) and sampling
(greedy) are covered at the reference's values only, and their other values rest on the formulas cited
at each function.
"""
from __future__ import annotations

import json
import math
import os
from typing import Dict, List, Optional, Sequence

import torch

DT = torch.float64


def read_model_folder(model_dir: str):
    """config.json as a dict and the tensors of model.safetensors widened to float64."""
    from safetensors.torch import load_file
    with open(os.path.join(model_dir, "config.json")) as f:
        cfg = json.load(f)
    w = {k: v.to(DT) for k, v in load_file(os.path.join(model_dir, "model.safetensors")).items()}
    return cfg, w


def embedding(tokens: torch.Tensor, table: torch.Tensor) -> torch.Tensor:
    """h[t, :] = E[tok[t], :]  (src/source/op/kernels/cpu/emb_kernel.cpp:4-29)."""
    return table[tokens.long()]


def rmsnorm(x: torch.Tensor, g: torch.Tensor, eps: float) -> torch.Tensor:
    """y = g * (x * 1/sqrt(mean(x^2) + eps))  (src/source/op/kernels/cpu/rmsnorm_kernel.cpp:59-71;
    the reference fixes eps = 1e-6 at :56, here it is an argument)."""
    ms = (x * x).sum(-1, keepdim=True) / x.shape[-1]
    return g * (x * (1.0 / torch.sqrt(ms + eps)))


def rope_frequencies(head_dim: int, theta: float, scaling: Optional[dict]) -> torch.Tensor:
    """freq of pair i = theta^(-2i/head_dim): the reference fills table entry j with
    theta^(-j/head_size) and reads entry 2i (src/source/op/kernels/cpu/rope_kernel.cpp:3-16, 76-77).
    The reference has no frequency scaling; the "llama3" rule is the published one: by
    wavelength L = 2*pi/f, L < orig/high keeps f, L > orig/low gives f/factor, else
    s = (orig/L - low)/(high - low) and f' = (1-s) f/factor + s f."""
    out = []
    for i in range(head_dim // 2):
        f = float(theta) ** (-(2.0 * i) / head_dim)
        if scaling is not None and scaling.get("rope_type", scaling.get("type")) == "llama3":
            factor, low, high = scaling["factor"], scaling["low_freq_factor"], scaling["high_freq_factor"]
            orig = scaling["original_max_position_embeddings"]
            wl = 2.0 * math.pi / f
            if wl < orig / high:
                pass
            elif wl > orig / low:
                f = f / factor
            else:
                s = (orig / wl - low) / (high - low)
                f = (1.0 - s) * f / factor + s * f
        out.append(f)
    # the engine keeps frequencies, angles, sines and cosines in fp32
    return torch.tensor(out, dtype=torch.float64).to(torch.float32)


def rope(x: torch.Tensor, positions: torch.Tensor, freqs: torch.Tensor) -> torch.Tensor:
    """x: [T, heads, hs]. Rotate-half pairs (x[i], x[i+hs/2]):
    x[i] <- c x[i] - s x[i+hs/2];  x[i+hs/2] <- c x[i+hs/2] + s x[i]
    (src/source/op/kernels/cpu/rope_kernel.cpp:66-88). The angle pos*freq and its sine and
    cosine are formed in fp32 as the reference does (rope_kernel.cpp:7-11)."""
    half = x.shape[-1] // 2
    ang = positions.to(torch.float32)[:, None] * freqs[None, :]          # fp32 product
    c = torch.cos(ang).to(x.dtype)[:, None, :]
    s = torch.sin(ang).to(x.dtype)[:, None, :]
    x0, x1 = x[..., :half], x[..., half:]
    return torch.cat([c * x0 - s * x1, c * x1 + s * x0], dim=-1)


def attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, scale: float,
              window: Optional[int] = None) -> torch.Tensor:
    """q: [T, H, hs], k, v: [T, KV, hs], one whole sequence. For head h, kv head
    g = h * KV // H; scores s_j = (q_h . k_j) * scale over j <= t, softmax with the maximum
    subtracted, out = sum_j p_j v_j / sum_j p_j
    (src/source/op/kernels/cpu/mha_kernel.cpp:112-171). A window keeps j > t - window."""
    T, H, hs = q.shape
    KV = k.shape[1]
    out = torch.zeros_like(q)
    for h in range(H):
        g = h * KV // H
        s = (q[:, h, :] @ k[:, g, :].T) * scale                          # [T, T]
        j = torch.arange(T)
        mask = j[None, :] > j[:, None]
        if window is not None:
            mask = mask | (j[None, :] <= j[:, None] - window)
        s = s.masked_fill(mask, float("-inf"))
        p = torch.exp(s - s.max(-1, keepdim=True).values)
        out[:, h, :] = (p @ v[:, g, :]) / p.sum(-1, keepdim=True)
    return out


def swiglu(a: torch.Tensor, b: torch.Tensor) -> torch.Tensor:
    """(a * 1/(1+exp(-a))) * b  (src/source/op/kernels/cpu/swiglu_kernel.cpp:21-22)."""
    return (a * (1.0 / (1.0 + torch.exp(-a)))) * b


def forward(cfg: dict, w: Dict[str, torch.Tensor], tokens: Sequence[int],
            round_to=None, window: Optional[int] = None) -> torch.Tensor:
    """Logits [T, V] of one whole sequence; order of operations of the reference's
    ``forward_batch`` (src/source/model/llama3.cpp:996-1194). ``round_to`` (a torch dtype)
    rounds activations where the serving precision stores them, to predict its error."""
    d = cfg["hidden_size"]
    H = cfg["num_attention_heads"]
    KV = cfg.get("num_key_value_heads") or H
    hs = cfg.get("head_dim") or d // H
    eps = cfg["rms_norm_eps"]
    rnd = (lambda t: t.to(round_to).to(DT)) if round_to is not None else (lambda t: t)
    tok = torch.as_tensor(list(tokens))
    pos = torch.arange(len(tokens))
    freqs = rope_frequencies(hs, cfg["rope_theta"], cfg.get("rope_scaling"))
    h = embedding(tok, w["model.embed_tokens.weight"])
    for l in range(cfg["num_hidden_layers"]):
        p = f"model.layers.{l}."
        x = rnd(rmsnorm(h, w[p + "input_layernorm.weight"], eps))
        q = rnd(x @ w[p + "self_attn.q_proj.weight"].T).view(-1, H, hs)
        k = rnd(x @ w[p + "self_attn.k_proj.weight"].T).view(-1, KV, hs)
        v = rnd(x @ w[p + "self_attn.v_proj.weight"].T).view(-1, KV, hs)
        q, k = rnd(rope(q, pos, freqs)), rnd(rope(k, pos, freqs))
        a = rnd(attention(q, k, v, 1.0 / math.sqrt(hs), window)).reshape(-1, H * hs)
        h = h + rnd(a @ w[p + "self_attn.o_proj.weight"].T)
        x = rnd(rmsnorm(h, w[p + "post_attention_layernorm.weight"], eps))
        m = rnd(swiglu(rnd(x @ w[p + "mlp.gate_proj.weight"].T), rnd(x @ w[p + "mlp.up_proj.weight"].T)))
        h = h + rnd(m @ w[p + "mlp.down_proj.weight"].T)
    x = rnd(rmsnorm(h, w["model.norm.weight"], eps))
    head = w["model.embed_tokens.weight"] if cfg.get("tie_word_embeddings") else w["lm_head.weight"]
    return x @ head.T


# ---- sampling -------------------------------------------------------------------------------

_M64 = (1 << 64) - 1


def uniform01(seed: int, counter: int) -> float:
    """splitmix64 finaliser over seed ^ (counter * golden) -> 24-bit uniform in [0, 1)."""
    z = (seed ^ ((counter * 0x9E3779B97F4A7C15) & _M64)) & _M64
    z = (z + 0x9E3779B97F4A7C15) & _M64
    z = ((z ^ (z >> 30)) * 0xBF58476D1CE4E5B9) & _M64
    z = ((z ^ (z >> 27)) * 0x94D049BB133111EB) & _M64
    z ^= z >> 31
    return (z >> 40) / 16777216.0


def sample(logits: torch.Tensor, temperature: float = 0.0, top_k: int = 0, top_p: float = 1.0,
           seed: int = 0, counter: int = 0) -> int:
    """One token from one row of logits. Greedy is argmax with ties to the lowest index
    (src/source/op/kernels/cuda/argmax_kernel.cu:14-19). Otherwise p = softmax(x / T); keep the
    top_k largest logits (all ties of the k-th); among them keep the largest logits, all ties
    included, down to the threshold at which their mass first reaches top_p of the kept mass;
    draw by inverse CDF in index order with u = uniform01(seed, counter)."""
    x = logits.to(torch.float32)
    if not temperature > 0:
        return int(torch.argmax(x))          # torch returns the first maximum
    V = x.numel()
    keep = torch.ones(V, dtype=torch.bool)
    if 0 < top_k < V:
        kth = torch.sort(x, descending=True).values[top_k - 1]
        keep &= x >= kth
    p = torch.exp(((x - x.max()) / temperature).to(torch.float64))
    if top_p < 1.0:
        z = p[keep].sum()
        vals = torch.unique(x[keep])          # ascending
        thr = vals[0]
        for t in reversed(vals.tolist()):     # from the largest down
            if p[keep & (x >= t)].sum() >= top_p * z:
                thr = t
                break
        keep &= x >= thr
    pk = torch.where(keep, p, torch.zeros_like(p))
    target = uniform01(seed, counter) * float(pk.sum())
    c = torch.cumsum(pk, 0)
    idx = torch.nonzero((c > target) & keep)
    return int(idx[0]) if idx.numel() else int(torch.nonzero(keep)[-1])


def generate(cfg, w, prompt: Sequence[int], n_new: int, temperature=0.0, top_k=0, top_p=1.0,
             seed=0, stop: Sequence[int] = ()) -> List[int]:
    """Whole-sequence recomputation per new token; output token i uses counter i."""
    toks = list(prompt)
    out: List[int] = []
    for i in range(n_new):
        lg = forward(cfg, w, toks)[-1]
        t = sample(lg, temperature, top_k, top_p, seed, i)
        out.append(t)
        toks.append(t)
        if t in stop:
            break
    return out
