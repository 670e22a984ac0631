"""The allocation-free decode attention entry point, called through its exported C symbol,
against the ordinary entry point (which takes its scratch from the caller). It serves callers
that cannot allocate device memory at call time (a runtime that forbids cudaMalloc after
start-up, a plug-in inside another process's context, a real-time loop): the scratch of the
split kernel lives in a fixed array inside the library. Two calls in a row share that array,
so the second must not be disturbed by what the first left behind. Collected last on purpose:
a run that stops at the first failure has then already run every other test."""
import ctypes
import math

import pytest
import torch

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def _lib():
    from llm_steadyinfer_b200.csrc import build
    lib = build.load("attention_noalloc")
    c_int, c_ll, c_f, c_p = ctypes.c_int, ctypes.c_longlong, ctypes.c_float, ctypes.c_void_p
    lib.si_attn_decode_noalloc.restype = c_int
    lib.si_attn_decode_noalloc.argtypes = [c_p, c_ll, c_p, c_p, c_p, c_int, c_p, c_int, c_p, c_ll, c_int, c_int, c_int,
                                           c_int, c_int, c_int, c_f, c_int, c_int, c_p, c_p]
    lib.si_attn_decode_noalloc_words.restype = c_ll
    lib.si_attn_decode_noalloc_words.argtypes = [c_int] * 5
    lib.si_noalloc_last_error.restype = ctypes.c_char_p
    lib.si_noalloc_init.restype = c_int
    lib.si_noalloc_init.argtypes = []
    lib.si_noalloc_poison_tickets.restype = c_int
    lib.si_noalloc_poison_tickets.argtypes = [c_int, c_p]
    return lib


def _case(batch, ctx, H, KV, hs, page_size, seed, tokens=1):
    """``tokens``: rows per item (the last ``tokens`` positions of each sequence attend)."""
    g = torch.Generator(device=DEV).manual_seed(seed)
    blocks = -(-ctx // page_size)
    pages = batch * blocks
    kc = torch.randn(pages, KV, page_size, hs, generator=g, device=DEV).to(torch.bfloat16)
    vc = torch.randn(pages, KV, page_size, hs, generator=g, device=DEV).to(torch.bfloat16)
    table = torch.randperm(pages, generator=g, device=DEV).to(torch.int32).view(batch, blocks)
    q = torch.randn(batch * tokens, H * hs, generator=g, device=DEV).to(torch.bfloat16)
    lens = [ctx - 5 * i for i in range(batch)]
    items = torch.tensor([(s, s * tokens, tokens, lens[s] - tokens) for s in range(batch)], dtype=torch.int32, device=DEV)
    return q, kc, vc, table, items


def _plain(case, H, KV, hs, page_size, window):
    """softmax(scale q K^T) V in float32 with torch, on the pages gathered through the table: row r of an
    item at position p reads keys first..p, first = max(0, p - window + 1) with a window."""
    q, kc, vc, table, items = case
    out = torch.zeros(q.shape, dtype=torch.float32, device=DEV)
    G = H // KV
    for s, row0, n, pos0 in items.tolist():
        k = kc[table[s].long()].float().permute(1, 0, 2, 3).reshape(KV, -1, hs)       # [KV, blocks * page, hs]
        v = vc[table[s].long()].float().permute(1, 0, 2, 3).reshape(KV, -1, hs)
        for t in range(n):
            p = pos0 + t
            first = max(0, p - window + 1) if window else 0
            qh = q[row0 + t].float().view(KV, G, hs)
            sc = torch.einsum("kgd,kjd->kgj", qh, k[:, first:p + 1]) / math.sqrt(hs)
            out[row0 + t] = torch.einsum("kgj,kjd->kgd", torch.softmax(sc, -1), v[:, first:p + 1]).reshape(-1)
    return out


def _both(lib, case, H, KV, hs, page_size, nsplit, window=0):
    from llm_steadyinfer_b200.csrc import ops
    q, kc, vc, table, items = case
    batch = items.shape[0]
    scale = 1.0 / math.sqrt(hs)
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    want = torch.empty_like(q)
    scratch = torch.zeros(max(1, ops.attn_decode_scratch_floats(batch, H, KV, hs, nsplit)), device=DEV)
    ops.attn_decode(q, kc, vc, table, items, want, page_size, batch, H, KV, hs, scale, window,
                    nsplit=nsplit, scratch=scratch if nsplit > 1 else None, status=status)
    got = torch.full_like(q, float("nan"))
    p = lambda t: ctypes.c_void_p(t.data_ptr())
    rc = lib.si_attn_decode_noalloc(p(q), q.stride(0), p(kc), p(vc), p(table), table.shape[1], p(items), batch,
                                    p(got), got.stride(0), kc.shape[0], page_size, batch, H, KV, hs, scale, window, nsplit,
                                    p(status), ctypes.c_void_p(torch.cuda.current_stream().cuda_stream))
    assert rc == 0, lib.si_noalloc_last_error().decode()
    torch.cuda.synchronize()
    assert status.item() == 0
    return got, want


def test_no_alloc_entry_point_twice_in_a_row():
    lib = _lib()
    assert lib.si_noalloc_init() == 0, lib.si_noalloc_last_error().decode()
    assert lib.si_noalloc_init() == 0                       # set up already: nothing more to do
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    # first call: many splits of long contexts; second: another layout and size, a window and items of two
    # tokens, on the same array; third: the first again
    first = dict(batch=6, ctx=1500, H=32, KV=8, hs=128, page_size=16, nsplit=5)
    second = dict(batch=3, ctx=700, H=12, KV=4, hs=64, page_size=8, nsplit=3, window=300, tokens=2)
    for i, c in enumerate((first, second, first)):
        window, tokens = c.get("window", 0), c.get("tokens", 1)
        case = _case(c["batch"], c["ctx"], c["H"], c["KV"], c["hs"], c["page_size"], seed=20 + i, tokens=tokens)
        assert 0 < lib.si_attn_decode_noalloc_words(c["batch"], c["H"], c["KV"], c["hs"], c["nsplit"]) <= 4 * 1024 * 1024
        if i > 0:
            # what a call that was cut short might leave: the tickets of this call are not at zero
            assert lib.si_noalloc_poison_tickets(c["batch"] * c["KV"] + 7, stream) == 0
        got, want = _both(lib, case, c["H"], c["KV"], c["hs"], c["page_size"], c["nsplit"], window)
        assert not torch.isnan(got.float()).any()
        # the same kernel, the same splits and the same order of the merge as the entry point that is
        # given its scratch: equal bit for bit
        assert torch.equal(got, want), f"call {i}: differs from attn_decode by {(got.float() - want.float()).abs().max().item():.3e}"
        # and both right: float32 attention by torch on the gathered pages (outputs below 4 in size, bf16 rounding
        # of the probabilities and of the result)
        ref = _plain(case, c["H"], c["KV"], c["hs"], c["page_size"], window)
        assert (got.float() - ref).abs().max().item() <= 2 ** -8 * 4


def test_no_alloc_entry_point_refuses_what_does_not_fit():
    lib = _lib()
    H, KV, hs, page_size = 32, 8, 128, 16
    batch, nsplit = 64, 64                      # 64*8*64*16*130 words: far beyond the fixed array
    assert lib.si_attn_decode_noalloc_words(batch, H, KV, hs, nsplit) > 4 * 1024 * 1024
    case = _case(batch, 64, H, KV, hs, page_size, seed=30)
    q, kc, vc, table, items = case
    out = torch.zeros_like(q)
    p = lambda t: ctypes.c_void_p(t.data_ptr())
    rc = lib.si_attn_decode_noalloc(p(q), q.stride(0), p(kc), p(vc), p(table), table.shape[1], p(items), batch,
                                    p(out), out.stride(0), kc.shape[0], page_size, batch, H, KV, hs, 0.1, 0, nsplit,
                                    None, ctypes.c_void_p(torch.cuda.current_stream().cuda_stream))
    assert rc == -4
    msg = lib.si_noalloc_last_error().decode()
    assert "words" in msg and "4194304" in msg
    torch.cuda.synchronize()
    assert out.abs().max().item() == 0, "nothing was launched"
    assert lib.si_noalloc_poison_tickets(1 << 20, None) == -2
