"""Parts of a layer, each alone against the plain implementation, and the generality of the
composition: a toy architecture defined here (a mixer with per-request state of its own, a
routed feed-forward, another position encoding, a windowed attention layer, a layer that reads
another layer's cache, a layer that runs twice) is registered, built, loaded and stepped without
any change to the package, and agrees with a whole-sequence computation written here."""
import math
import os
from dataclasses import dataclass

import pytest
import torch

import plain_llama as pl
import replay_util as ru
from tiny_configs import CONFIGS, make_model_folder

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


@pytest.fixture(scope="module")
def folders(tmp_path_factory):
    root = tmp_path_factory.mktemp("models")
    return {n: make_model_folder(root, n) for n in CONFIGS}


def _runner(folder, dtype, page_size, num_pages=64, max_requests=4):
    from llm_steadyinfer_b200.engine.step import ModelRunner
    from llm_steadyinfer_b200.weights import load_model
    model = load_model(folder, dtype, DEV)
    return ModelRunner(model, page_size=page_size, num_pages=num_pages, max_requests=max_requests, max_step_tokens=512)


# ---- each built-in part alone ------------------------------------------------------------------

def test_rotary_part_frequencies():
    from llm_steadyinfer_b200.parts.rotary import Rotary
    for name in CONFIGS:
        cfg = CONFIGS[name][0]
        part = Rotary({"head_dim": cfg["head_dim"], "theta": cfg["rope_theta"], "scaling": cfg["rope_scaling"]},
                      torch.float32, DEV)
        inv_freq, rot = part.rotary()
        assert rot == cfg["head_dim"]
        want = pl.rope_frequencies(cfg["head_dim"], cfg["rope_theta"], cfg["rope_scaling"])
        assert torch.equal(inv_freq.cpu(), want)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_norm_and_mlp_parts(folders, dtype):
    from llm_steadyinfer_b200.weights import load_model
    cfg, w = pl.read_model_folder(folders["B"])
    model = load_model(folders["B"], dtype, DEV)
    blk = model.blocks[1]
    g = torch.Generator().manual_seed(0)
    T, d = 9, cfg["hidden_size"]
    resid = torch.randn(T, d, generator=g)
    delta = (0.3 * torch.randn(T, d, generator=g)).to(dtype)
    x = torch.empty(T, d, dtype=dtype, device=DEV)
    r = resid.clone().to(DEV)
    blk.feed_forward_norm.forward(r, delta.to(DEV), x)
    h = resid.double() + delta.double()
    want = pl.rmsnorm(h, w["model.layers.1.post_attention_layernorm.weight"], cfg["rms_norm_eps"])
    tol = 1e-5 if dtype == torch.float32 else 2 ** -8 * want.abs().max().item()
    assert (x.double().cpu() - want).abs().max().item() <= tol
    assert (r.double().cpu() - h).abs().max().item() <= 1e-6
    # the norm alone, off the residual stream (what a mixer with a norm of its own would call)
    y3 = (0.5 * torch.randn(T, 3, d, generator=g)).to(dtype).to(DEV)
    want3 = pl.rmsnorm(y3.double().cpu(), w["model.layers.1.post_attention_layernorm.weight"], cfg["rms_norm_eps"])
    blk.feed_forward_norm.normalize(y3)
    assert (y3.double().cpu() - want3).abs().max().item() <= (1e-5 if dtype == torch.float32 else 2 ** -7 * want3.abs().max().item())

    class Ctx:                                   # the feed-forward needs scratch and the status word only
        status = None

        def buf(self, key, shape, dt):
            return torch.empty(shape, dtype=dt, device=DEV)
    y = blk.feed_forward.forward(x, Ctx())
    xin = x.double().cpu()
    p = "model.layers.1.mlp."
    wm = pl.swiglu(xin @ w[p + "gate_proj.weight"].T, xin @ w[p + "up_proj.weight"].T) @ w[p + "down_proj.weight"].T
    tol = 1e-5 if dtype == torch.float32 else 2 ** -7 * max(1e-2, wm.abs().max().item())
    assert (y.double().cpu() - wm).abs().max().item() <= tol


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("name", ["A", "B"])
def test_attention_part_and_block_alone(folders, name, dtype):
    """The attention mixer and the whole block on rows of our choosing: a portion of 19 tokens after
    a prefix of 21 that an earlier step stored, beside a single row of another sequence."""
    from llm_steadyinfer_b200.engine.step import StepEntry
    cfg, w = pl.read_model_folder(folders[name])
    rn = _runner(folders[name], dtype, CONFIGS[name][2])
    V, d = cfg["vocab_size"], cfg["hidden_size"]
    H, KV, hs = cfg["num_attention_heads"], cfg["num_key_value_heads"], cfg["head_dim"]
    toks = {"a": ru.random_tokens(V, 40, 1), "b": ru.random_tokens(V, 6, 2)}
    rn.step([StepEntry("a", toks["a"][:21]), StepEntry("b", toks["b"][:5])])
    # the next step's context, without running the model: feed the first layer our own rows
    entries = [StepEntry("a", toks["a"][21:]), StepEntry("b", toks["b"][5:])]
    ctx = rn._prepare(entries)
    caches = rn.storage.layer_views(rn._tables)
    rn.model.prepare(ctx, caches)
    blk = rn.model.blocks[0]
    # plain: hidden states of layer 0 for the whole sequences are the embeddings
    freqs = pl.rope_frequencies(hs, cfg["rope_theta"], cfg.get("rope_scaling"))
    p = "model.layers.0."
    outs, blocks_out = {}, {}
    for rid, t in toks.items():
        h = pl.embedding(torch.tensor(t), w["model.embed_tokens.weight"])
        x = pl.rmsnorm(h, w[p + "input_layernorm.weight"], cfg["rms_norm_eps"])
        pos = torch.arange(len(t))
        q = pl.rope((x @ w[p + "self_attn.q_proj.weight"].T).view(-1, H, hs), pos, freqs)
        k = pl.rope((x @ w[p + "self_attn.k_proj.weight"].T).view(-1, KV, hs), pos, freqs)
        v = (x @ w[p + "self_attn.v_proj.weight"].T).view(-1, KV, hs)
        a = pl.attention(q, k, v, hs ** -0.5).reshape(-1, H * hs) @ w[p + "self_attn.o_proj.weight"].T
        outs[rid] = (x, a)
        h2 = h + a
        x2 = pl.rmsnorm(h2, w[p + "post_attention_layernorm.weight"], cfg["rms_norm_eps"])
        m = pl.swiglu(x2 @ w[p + "mlp.gate_proj.weight"].T, x2 @ w[p + "mlp.up_proj.weight"].T) @ w[p + "mlp.down_proj.weight"].T
        blocks_out[rid] = (h, h2, m)
    x_rows = torch.cat([outs["a"][0][21:], outs["b"][0][5:]]).to(dtype).to(DEV)
    got = blk.mixer.forward(x_rows, ctx, caches[0])
    want = torch.cat([outs["a"][1][21:], outs["b"][1][5:]])
    tol = 2e-6 if dtype == torch.float32 else 4e-3
    assert (got.double().cpu() - want).abs().max().item() <= tol
    # the whole block: stream in, pending delta and updated stream out
    resid = torch.cat([blocks_out["a"][0][21:], blocks_out["b"][0][5:]]).float().to(DEV)
    delta = blk.forward(resid, None, ctx, caches[0])
    want_h2 = torch.cat([blocks_out["a"][1][21:], blocks_out["b"][1][5:]])
    want_m = torch.cat([blocks_out["a"][2][21:], blocks_out["b"][2][5:]])
    assert (resid.double().cpu() - want_h2).abs().max().item() <= (2e-6 if dtype == torch.float32 else 4e-3)
    assert (delta.double().cpu() - want_m).abs().max().item() <= (2e-6 if dtype == torch.float32 else 4e-3)
    rn.check_status()


# ---- a toy architecture, defined in this test only -------------------------------------------------

TOY = {
    "architectures": ["ToyForCausalLM"], "hidden_size": 48, "vocab_size": 300, "num_heads": 6, "num_kv_heads": 2,
    "head_dim": 16, "intermediate_size": 80, "num_experts": 3, "window": 11, "eps": 1e-5, "decay": 0.8,
    "max_position": 256, "rope_theta": 10000.0,
}


def _toy_register():
    """Registers the toy parts and the toy architecture (idempotent)."""
    from llm_steadyinfer_b200.config.base import (FeedForwardSpec, LayerSpec, MixerSpec, ModelConfig, ModelSpec,
                                                  NormSpec, PositionSpec, register_architecture)
    from llm_steadyinfer_b200.parts import (FeedForward, Mixer, PositionEncoding, StateNeed, register_feed_forward,
                                            register_mixer, register_position)

    class Recurrence(Mixer):
        """s <- decay * s + W_in x_t; y_t = W_out s: state of fixed size per request, carried
        from step to step in the request's state slot."""

        def __init__(self, params, dtype, device, position=None):
            super().__init__(params, dtype, device, position)
            self.d, self.decay = params["hidden_size"], params["decay"]

        def weight_shapes(self):
            return {"in_proj.weight": (self.d, self.d), "out_proj.weight": (self.d, self.d)}

        def load_weights(self, t):
            self.w_in, self.w_out = t["in_proj.weight"].float(), t["out_proj.weight"].float()

        def state_need(self):
            return StateNeed((self.d,), torch.float32)

        def forward(self, x, ctx, cache):
            u = x.float() @ self.w_in.T
            y = torch.empty_like(u)
            for s in range(ctx.num_seqs):
                a, b = int(ctx.h_q_start[s]), int(ctx.h_q_start[s + 1])
                st = cache.state[int(ctx.h_slots[s])]
                for r in range(a, b):
                    st.mul_(self.decay).add_(u[r])
                    y[r] = st
            return (y @ self.w_out.T).to(self.dtype)

    class RoutedMLP(FeedForward):
        """Top-1 routing over small gated experts; router logits in fp32."""

        def __init__(self, params, dtype, device):
            super().__init__(params, dtype, device)
            self.d, self.f, self.e = params["hidden_size"], params["intermediate_size"], params["num_experts"]

        def weight_shapes(self):
            s = {"router.weight": (self.e, self.d)}
            for i in range(self.e):
                s[f"experts.{i}.gate.weight"] = (self.f, self.d)
                s[f"experts.{i}.up.weight"] = (self.f, self.d)
                s[f"experts.{i}.down.weight"] = (self.d, self.f)
            return s

        def load_weights(self, t):
            self.w = {k: v.float() for k, v in t.items()}

        def forward(self, x, ctx):
            xf = x.float()
            choice = torch.argmax(xf @ self.w["router.weight"].T, dim=-1)
            out = torch.zeros_like(xf)
            for i in range(self.e):
                rows = choice == i
                if rows.any():
                    xi = xf[rows]
                    g, u = xi @ self.w[f"experts.{i}.gate.weight"].T, xi @ self.w[f"experts.{i}.up.weight"].T
                    out[rows] = (torch.nn.functional.silu(g) * u) @ self.w[f"experts.{i}.down.weight"].T
            return out.to(self.dtype)

    class Sway(PositionEncoding):
        """Not a rotation: scales q and k by 1 + 0.3 sin(0.37 pos), through the unfused hook."""

        def apply(self, q, k, ctx):
            f = (1.0 + 0.3 * torch.sin(0.37 * ctx.positions.float()))[:, None, None]
            q.copy_((q.float() * f).to(q.dtype))
            k.copy_((k.float() * f).to(k.dtype))

    @dataclass(frozen=True)
    class ToyConfig(ModelConfig):
        d: dict
        architecture = "ToyForCausalLM"

        @classmethod
        def from_dict(cls, d):
            return cls(dict(d))

        def to_dict(self):
            return dict(self.d)

        def model_spec(self):
            c = self.d
            norm = NormSpec("rmsnorm", {"size": c["hidden_size"], "eps": c["eps"]})
            attn = lambda window, pos: MixerSpec("attention", {
                "hidden_size": c["hidden_size"], "num_heads": c["num_heads"], "num_kv_heads": c["num_kv_heads"],
                "head_dim": c["head_dim"], "scale": c["head_dim"] ** -0.5, "window": window}, position=pos)
            rotary = PositionSpec("rotary", {"head_dim": c["head_dim"], "theta": c["rope_theta"], "scaling": None})
            mlp = FeedForwardSpec("gated_mlp", {"hidden_size": c["hidden_size"], "intermediate_size": c["intermediate_size"]})
            routed = FeedForwardSpec("toy_routed", {"hidden_size": c["hidden_size"], "intermediate_size": c["intermediate_size"] // 2,
                                                    "num_experts": c["num_experts"]})
            rec = MixerSpec("toy_recurrence", {"hidden_size": c["hidden_size"], "decay": c["decay"]})
            L = lambda i, mixer, ffn, **kw: LayerSpec(mixer=mixer, feed_forward=ffn, mixer_norm=norm, feed_forward_norm=norm,
                                                      weight_prefix=f"toy.layers.{i}.", mixer_prefix="mixer.",
                                                      feed_forward_prefix="ffn.", mixer_norm_name="norm1.",
                                                      feed_forward_norm_name="norm2.", **kw)
            layers = [L(0, rec, mlp),
                      L(1, attn(c["window"], PositionSpec("toy_sway", {})), routed),
                      L(2, attn(None, rotary), mlp),
                      L(3, attn(None, rotary), routed, cache_from=2)]
            return ModelSpec(hidden_size=c["hidden_size"], vocab_size=c["vocab_size"], layers=layers,
                             order=[0, 1, 2, 3, 1], final_norm=norm, tie_word_embeddings=True,
                             embed_name="toy.embed.weight", final_norm_name="toy.norm.", max_position=c["max_position"])

    register_mixer("toy_recurrence", Recurrence)
    register_feed_forward("toy_routed", RoutedMLP)
    register_position("toy_sway", Sway)
    register_architecture("ToyForCausalLM", ToyConfig)


def _toy_plain(cfg, w, tokens):
    """Whole sequence, float64, written from the definitions of the toy parts above."""
    c = cfg
    d, H, KV, hs = c["hidden_size"], c["num_heads"], c["num_kv_heads"], c["head_dim"]
    T = len(tokens)
    pos = torch.arange(T)
    freqs = pl.rope_frequencies(hs, c["rope_theta"], None)
    h = w["toy.embed.weight"][torch.tensor(tokens)]
    kv_of = {}

    def attn(i, x, window, rotary, source=None):
        p = f"toy.layers.{i}.mixer."
        q = (x @ w[p + "q_proj.weight"].T).view(T, H, hs)
        k = (x @ w[p + "k_proj.weight"].T).view(T, KV, hs)
        v = (x @ w[p + "v_proj.weight"].T).view(T, KV, hs)
        if rotary:
            q, k = pl.rope(q, pos, freqs), pl.rope(k, pos, freqs)
        else:
            f = (1.0 + 0.3 * torch.sin(0.37 * pos.float())).double()[:, None, None]
            q, k = q * f, k * f
        if source is not None:
            k, v = kv_of[source]
        kv_of[i] = (k, v)
        return pl.attention(q, k, v, hs ** -0.5, window).reshape(T, H * hs) @ w[p + "o_proj.weight"].T

    def recurrence(i, x):
        p = f"toy.layers.{i}.mixer."
        u = x @ w[p + "in_proj.weight"].T
        s = torch.zeros(d, dtype=pl.DT)
        ys = []
        for t in range(T):
            s = c["decay"] * s + u[t]
            ys.append(s)
        return torch.stack(ys) @ w[p + "out_proj.weight"].T

    def mlp(i, x):
        p = f"toy.layers.{i}.ffn."
        return pl.swiglu(x @ w[p + "gate_proj.weight"].T, x @ w[p + "up_proj.weight"].T) @ w[p + "down_proj.weight"].T

    def routed(i, x):
        p = f"toy.layers.{i}.ffn."
        choice = torch.argmax(x @ w[p + "router.weight"].T, dim=-1)
        out = torch.zeros_like(x)
        for t in range(T):
            e = int(choice[t])
            out[t] = pl.swiglu(x[t] @ w[p + f"experts.{e}.gate.weight"].T, x[t] @ w[p + f"experts.{e}.up.weight"].T) \
                @ w[p + f"experts.{e}.down.weight"].T
        return out

    mixers = {0: lambda x: recurrence(0, x), 1: lambda x: attn(1, x, c["window"], False),
              2: lambda x: attn(2, x, None, True), 3: lambda x: attn(3, x, None, True, source=2)}
    ffns = {0: lambda x: mlp(0, x), 1: lambda x: routed(1, x), 2: lambda x: mlp(2, x), 3: lambda x: routed(3, x)}
    for i in [0, 1, 2, 3, 1]:
        p = f"toy.layers.{i}."
        h = h + mixers[i](pl.rmsnorm(h, w[p + "norm1.weight"], c["eps"]))
        h = h + ffns[i](pl.rmsnorm(h, w[p + "norm2.weight"], c["eps"]))
    return pl.rmsnorm(h, w["toy.norm.weight"], c["eps"]) @ w["toy.embed.weight"].T


def test_toy_architecture_is_registered_built_and_stepped(tmp_path):
    _toy_register()
    from llm_steadyinfer_b200.engine.replay import Replayer
    from llm_steadyinfer_b200.weights import write_random_model
    folder = os.path.join(str(tmp_path), "toy")
    write_random_model(folder, TOY, seed=5, store_dtype=torch.float32)
    from safetensors.torch import load_file
    w = {k: v.double() for k, v in load_file(os.path.join(folder, "model.safetensors")).items()}
    reqs = {"x": ru.random_tokens(TOY["vocab_size"], 70, 41), "y": ru.random_tokens(TOY["vocab_size"], 33, 42),
            "z": ru.random_tokens(TOY["vocab_size"], 90, 43)}
    want = {r: _toy_plain(TOY, w, t) for r, t in reqs.items()}
    for mode in ("whole", "portions", "mixed"):
        rp = Replayer(folder, torch.float32, max_tokens=256, page_size=8)
        mgr = rp.runner.manager
        assert len(mgr.groups) == 2, "windowed and full attention have pools of their own"
        assert sum(s is not None for s in rp.runner.layout.states) == 1
        steps = {"whole": ru.trace_whole, "portions": ru.trace_portions}.get(mode, lambda r: ru.trace_mixed(r, 256, seed=1))(reqs)
        worst = 0.0
        for rid, p, row in ru.replay_in_process(rp, steps):
            diff = (row.double() - want[rid][p]).abs().max().item()
            assert diff <= 2e-5, f"toy model, {mode}: request {rid} position {p} differs by {diff:.2e}"
            worst = max(worst, diff)
        mgr.check_invariant()
        assert not mgr.requests and all(mgr.free_pages(g) == mgr.groups[g].pool.num_pages for g in range(2))
        print(f"toy {mode}: worst {worst:.2e}")


def test_window_gives_pages_back_while_stepping(tmp_path):
    """The windowed group's pages fall behind the window and are used again while a request grows."""
    _toy_register()
    from llm_steadyinfer_b200.engine.replay import Replayer
    from llm_steadyinfer_b200.weights import write_random_model
    folder = os.path.join(str(tmp_path), "toy")
    write_random_model(folder, TOY, seed=5, store_dtype=torch.float32)
    rp = Replayer(folder, torch.float32, max_tokens=128, page_size=8)
    toks = ru.random_tokens(TOY["vocab_size"], 100, 7)
    mgr = rp.runner.manager
    win = [g for g in range(2) if mgr.groups[g].window is not None][0]
    for a in range(0, 100, 10):
        rp.run_step([{"id": "r", "tokens": toks[a:a + 10], "want": []}], [])
        held = sum(1 for p in mgr.table(win, "r") if p >= 0)
        assert held <= -(-(TOY["window"] + 10) // 8) + 1
    assert sum(1 for p in mgr.table(1 - win, "r") if p >= 0) == 13
    rp.run_step([], ["r"])
    mgr.check_invariant()


def _windowed_llama_register():
    """An architecture of this test: the Llama arrangement with a window on every attention layer."""
    from dataclasses import replace
    from llm_steadyinfer_b200.config.base import ModelConfig, register_architecture
    from llm_steadyinfer_b200.models.llama import LlamaConfig

    @dataclass(frozen=True)
    class WindowedConfig(ModelConfig):
        d: dict
        architecture = "WindowedToyForCausalLM"

        @classmethod
        def from_dict(cls, d):
            return cls(dict(d))

        def to_dict(self):
            return dict(self.d)

        def model_spec(self):
            d = {k: v for k, v in self.d.items() if k != "window"}
            base = LlamaConfig.from_dict({**d, "architectures": ["LlamaForCausalLM"]}).model_spec()
            layers = [replace(l, mixer=replace(l.mixer, params={**l.mixer.params, "window": self.d["window"]}))
                      for l in base.layers]
            return replace(base, layers=layers)

    register_architecture("WindowedToyForCausalLM", WindowedConfig)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16], ids=["fp32", "bf16"])
@pytest.mark.parametrize("head_dim,heads,kv_heads,window,page_size", [(64, 4, 2, 40, 16), (128, 3, 1, 100, 16), (64, 6, 3, 11, 8),
                                                                      (96, 2, 2, 70, 32)])
def test_windowed_layers_with_pages_given_back(tmp_path, dtype, head_dim, heads, kv_heads, window, page_size):
    """Windowed attention at head sizes that the tensor-core kernels take, cut every way. Those kernels
    round the first key down to a tile of 64 keys, and pages inside that tile have been given back
    (table entries of -1) once the window has passed them: they are neither looked up nor reported.
    Compared with the plain implementation and its own window, within what the other replay tests allow."""
    _windowed_llama_register()
    from llm_steadyinfer_b200.engine.replay import Replayer
    from llm_steadyinfer_b200.weights import write_random_model
    cfg = {
        "architectures": ["WindowedToyForCausalLM"], "hidden_size": 136, "intermediate_size": 200,
        "num_hidden_layers": 3, "num_attention_heads": heads, "num_key_value_heads": kv_heads, "head_dim": head_dim,
        "vocab_size": 411, "max_position_embeddings": 512, "rms_norm_eps": 1e-5, "rope_theta": 10000.0,
        "rope_scaling": None, "tie_word_embeddings": False, "hidden_act": "silu", "window": window,
    }
    folder = os.path.join(str(tmp_path), "windowed")
    write_random_model(folder, cfg, seed=6, store_dtype=torch.bfloat16)
    _, w = pl.read_model_folder(folder)
    reqs = {"x": ru.random_tokens(cfg["vocab_size"], 300, 41), "y": ru.random_tokens(cfg["vocab_size"], 133, 42),
            "z": ru.random_tokens(cfg["vocab_size"], 190, 43)}
    want = {r: pl.forward(cfg, w, t, window=window) for r, t in reqs.items()}
    atol = 1e-5 if dtype == torch.float32 else 1e-2
    for mode in ("whole", "tail", "portions", "mixed"):
        rp = Replayer(folder, dtype, max_tokens=704, page_size=page_size)
        steps = {"whole": ru.trace_whole, "tail": ru.trace_tail,
                 "portions": ru.trace_portions}.get(mode, lambda r: ru.trace_mixed(r, 704, seed=1))(reqs)
        worst = 0.0
        for rid, p, row in ru.replay_in_process(rp, steps):
            diff = (row.double() - want[rid][p]).abs().max().item()
            assert diff <= atol, f"windowed layers, {mode}: request {rid} position {p} differs by {diff:.2e}"
            worst = max(worst, diff)
        mgr = rp.runner.manager
        mgr.check_invariant()
        assert not mgr.requests and mgr.free_pages(0) == mgr.groups[0].pool.num_pages
        print(f"windowed head_dim {head_dim} window {window} {dtype} {mode}: worst {worst:.2e}")


def _greedy(logits_of, prompt, n_new):
    toks, out = list(prompt), []
    for _ in range(n_new):
        t = int(torch.argmax(logits_of(toks)[-1]))
        out.append(t)
        toks.append(t)
    return out


def test_toy_architecture_generates_through_the_entry_point(tmp_path):
    """The toy parts read host values in ``forward`` and leave ``capturable`` at its default, so no
    decode step of theirs is captured into a graph; requests come and go with so few pages that
    some are put back, and the state slots are zeroed for each admission."""
    _toy_register()
    from llm_steadyinfer_b200 import LLM, SamplingParams
    from llm_steadyinfer_b200.weights import write_random_model
    from safetensors.torch import load_file
    folder = os.path.join(str(tmp_path), "toy")
    write_random_model(folder, TOY, seed=5, store_dtype=torch.float32)
    w = {k: v.double() for k, v in load_file(os.path.join(folder, "model.safetensors")).items()}
    prompts = [ru.random_tokens(TOY["vocab_size"], n, 60 + i) for i, n in enumerate([3, 41, 18, 70, 9])]
    want = [_greedy(lambda t: _toy_plain(TOY, w, t), p, 20) for p in prompts]
    llm = LLM(folder, dtype="float32", max_batch=3, max_seq_len=96, max_gen_len=20, block_size=8,
              max_num_batched_tokens=32, num_blocks=20)
    got = llm.generate(prompts, SamplingParams(ignore_eos=True))
    assert [g.token_ids for g in got] == want
    assert llm.stats["graph_steps"] == 0 and llm.stats["ahead_steps"] == 0
    llm.runner.manager.check_invariant()
    assert not llm.runner.manager.requests


@pytest.mark.parametrize("ahead", [False, True])
def test_windowed_layers_generate_through_the_entry_point(tmp_path, ahead):
    """Windowed layers through the scheduler, captured decode steps and steps launched ahead: the
    windowed group gives pages back while requests decode, and its pool is smaller than the
    requests' lengths would need without a window."""
    _windowed_llama_register()
    from llm_steadyinfer_b200 import LLM, SamplingParams
    from llm_steadyinfer_b200.weights import write_random_model
    cfg = {
        "architectures": ["WindowedToyForCausalLM"], "hidden_size": 72, "intermediate_size": 100,
        "num_hidden_layers": 2, "num_attention_heads": 4, "num_key_value_heads": 2, "head_dim": 32,
        "vocab_size": 211, "max_position_embeddings": 256, "rms_norm_eps": 1e-5, "rope_theta": 10000.0,
        "rope_scaling": None, "tie_word_embeddings": True, "hidden_act": "silu", "window": 24,
    }
    folder = os.path.join(str(tmp_path), "windowed")
    write_random_model(folder, cfg, seed=8, store_dtype=torch.float32)
    _, w = pl.read_model_folder(folder)
    prompts = [ru.random_tokens(cfg["vocab_size"], n, 80 + i) for i, n in enumerate([5, 90, 33, 120])]
    want = [_greedy(lambda t: pl.forward(cfg, w, t, window=24), p, 40) for p in prompts]
    # 4 requests of up to 160 tokens would hold 80 pages of 8 without a window; with it, 4 + 1 + the step's growth each
    llm = LLM(folder, dtype="float32", max_batch=4, max_seq_len=160, max_gen_len=40, block_size=8,
              max_num_batched_tokens=32, num_blocks=40, async_decode=ahead)
    got = llm.generate(prompts, SamplingParams(ignore_eos=True))
    assert [g.token_ids for g in got] == want
    assert llm.stats["graph_steps"] > 0
    assert (llm.stats["ahead_steps"] > 0) == ahead
    llm.runner.manager.check_invariant()
    assert not llm.runner.manager.requests


# ---- another arrangement of a block, registered from this test ------------------------------------

PARALLEL = {
    "architectures": ["ParallelToyForCausalLM"], "hidden_size": 80, "intermediate_size": 136,
    "num_hidden_layers": 3, "num_attention_heads": 5, "num_key_value_heads": 5, "head_dim": 16,
    "vocab_size": 333, "max_position_embeddings": 256, "rms_norm_eps": 1e-5, "rope_theta": 10000.0,
    "rope_scaling": None, "tie_word_embeddings": False, "hidden_act": "silu",
}


def _parallel_register():
    """A block whose mixer and feed-forward both read the one normalised stream and whose results are added
    together: ``h += delta_in; x = norm1(h); return mixer(x) + ffn(x)``. The second norm of the spec is not run.
    Middle layer only; the layers around it keep the built-in arrangement."""
    from dataclasses import replace
    from llm_steadyinfer_b200.config.base import ModelConfig, register_architecture
    from llm_steadyinfer_b200.models.llama import LlamaConfig
    from llm_steadyinfer_b200.parts import register_arrangement

    def parallel(block, resid, delta, ctx, cache):
        T, d = resid.shape
        x = ctx.buf("block_x", (T, d), block.mixer.dtype)
        block.norm(block.mixer_norm, resid, delta, x)
        a = block.mixer.forward(x, ctx, cache)
        kept = ctx.buf("toy_parallel_a", (T, d), a.dtype)         # the feed-forward writes where the mixer wrote
        kept.copy_(a)
        m = block.feed_forward.forward(x, ctx)
        m.add_(kept)
        return m

    @dataclass(frozen=True)
    class ParallelConfig(ModelConfig):
        d: dict
        architecture = "ParallelToyForCausalLM"

        @classmethod
        def from_dict(cls, d):
            return cls(dict(d))

        def to_dict(self):
            return dict(self.d)

        def model_spec(self):
            base = LlamaConfig.from_dict({**self.d, "architectures": ["LlamaForCausalLM"]}).model_spec()
            layers = [replace(l, arrangement="toy_parallel") if i == 1 else l for i, l in enumerate(base.layers)]
            return replace(base, layers=layers)

    register_arrangement("toy_parallel", parallel, capturable=True)
    register_architecture("ParallelToyForCausalLM", ParallelConfig)


def _parallel_plain(cfg, w, tokens):
    d, H, hs, eps = cfg["hidden_size"], cfg["num_attention_heads"], cfg["head_dim"], cfg["rms_norm_eps"]
    KV = cfg["num_key_value_heads"]
    pos = torch.arange(len(tokens))
    freqs = pl.rope_frequencies(hs, cfg["rope_theta"], None)
    h = pl.embedding(torch.tensor(tokens), w["model.embed_tokens.weight"])
    for l in range(cfg["num_hidden_layers"]):
        p = f"model.layers.{l}."
        x = pl.rmsnorm(h, w[p + "input_layernorm.weight"], eps)
        q = pl.rope((x @ w[p + "self_attn.q_proj.weight"].T).view(-1, H, hs), pos, freqs)
        k = pl.rope((x @ w[p + "self_attn.k_proj.weight"].T).view(-1, KV, hs), pos, freqs)
        v = (x @ w[p + "self_attn.v_proj.weight"].T).view(-1, KV, hs)
        a = pl.attention(q, k, v, hs ** -0.5).reshape(-1, H * hs) @ w[p + "self_attn.o_proj.weight"].T
        if l != 1:
            h = h + a
            x = pl.rmsnorm(h, w[p + "post_attention_layernorm.weight"], eps)
        m = pl.swiglu(x @ w[p + "mlp.gate_proj.weight"].T, x @ w[p + "mlp.up_proj.weight"].T) @ w[p + "mlp.down_proj.weight"].T
        h = h + a + m if l == 1 else h + m
    return pl.rmsnorm(h, w["model.norm.weight"], eps) @ w["lm_head.weight"].T


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16], ids=["fp32", "bf16"])
def test_another_block_arrangement_is_registered_and_replayed(tmp_path, dtype):
    _parallel_register()
    from llm_steadyinfer_b200 import LLM, SamplingParams
    from llm_steadyinfer_b200.engine.replay import Replayer
    from llm_steadyinfer_b200.weights import write_random_model
    folder = os.path.join(str(tmp_path), "parallel")
    write_random_model(folder, PARALLEL, seed=9, store_dtype=torch.bfloat16)
    _, w = pl.read_model_folder(folder)
    reqs = {"x": ru.random_tokens(PARALLEL["vocab_size"], 90, 1), "y": ru.random_tokens(PARALLEL["vocab_size"], 47, 2),
            "z": ru.random_tokens(PARALLEL["vocab_size"], 130, 3)}
    want = {r: _parallel_plain(PARALLEL, w, t) for r, t in reqs.items()}
    # the arrangement matters: the built-in one gives other logits
    assert (pl.forward({**PARALLEL, "num_key_value_heads": 5}, w, reqs["y"]) - want["y"]).abs().max().item() > 1e-3
    atol = 1e-5 if dtype == torch.float32 else 1e-2
    for mode in ("whole", "tail", "portions", "mixed"):
        rp = Replayer(folder, dtype, max_tokens=320, page_size=16)
        steps = {"whole": ru.trace_whole, "tail": ru.trace_tail,
                 "portions": ru.trace_portions}.get(mode, lambda r: ru.trace_mixed(r, 320, seed=2))(reqs)
        for rid, p, row in ru.replay_in_process(rp, steps):
            diff = (row.double() - want[rid][p]).abs().max().item()
            assert diff <= atol, f"parallel block, {mode}: request {rid} position {p} differs by {diff:.2e}"
    if dtype == torch.float32:
        # through the entry point with recorded decode steps: the arrangement says that it can be captured
        prompts = [reqs["y"][:9], reqs["x"][:30]]
        greedy = [_greedy(lambda t: _parallel_plain(PARALLEL, w, t), p, 12) for p in prompts]
        llm = LLM(folder, dtype="float32", max_batch=2, max_seq_len=64, max_gen_len=12)
        assert [g.token_ids for g in llm.generate(prompts, SamplingParams(ignore_eos=True))] == greedy
        assert llm.stats["graph_steps"] > 0
