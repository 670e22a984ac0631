"""Each kernel alone against a plain fp32 reference of the same op, at sizes other than the
engine tests': widths and vocabularies that are no power of two, odd head counts, head sizes in
steps of 16, pages of several sizes."""
import math

import pytest
import torch

import plain_llama

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def ops():
    from llm_steadyinfer_b200.csrc import ops as o
    return o


def graph_time_us(fn, n=20):
    """Device time of one call of ``fn(i)`` in microseconds: calls i = 0 .. n-1 recorded into a CUDA graph and
    replayed, so that the host's part of a call (tens of microseconds from Python) is not in the figure."""
    fn(0)
    torch.cuda.synchronize()
    graph, side = torch.cuda.CUDAGraph(), torch.cuda.Stream()
    with torch.cuda.stream(side):
        fn(0)
        torch.cuda.synchronize()
        with torch.cuda.graph(graph, stream=side):
            for i in range(n):
                fn(i)
    for _ in range(2):
        graph.replay()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    torch.cuda.synchronize()
    e0.record()
    graph.replay()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) * 1000 / n


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("V,d,T", [(1000, 96, 7), (4099, 1336, 33)])
def test_embedding(dtype, V, d, T):
    g = torch.Generator().manual_seed(0)
    table = torch.randn(V, d, generator=g).to(dtype).to(DEV)
    tok = torch.randint(0, V, (T,), generator=g, dtype=torch.int32).to(DEV)
    out = torch.empty(T, d, dtype=torch.float32, device=DEV)
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    ops().embedding_gather(tok, table, out, status)
    assert torch.equal(out, table[tok.long()].float())
    assert status.item() == 0
    tok[T // 2] = V                                  # outside the vocabulary: flagged, row zeroed
    ops().embedding_gather(tok, table, out, status)
    assert status.item() == 1 and out[T // 2].abs().max().item() == 0


@pytest.mark.parametrize("xdtype,wdtype", [(torch.float32, torch.float32), (torch.bfloat16, torch.bfloat16),
                                           (torch.bfloat16, torch.float32)])
@pytest.mark.parametrize("d,T,eps", [(96, 5, 1e-6), (1336, 19, 1e-5), (5120, 3, 1e-5)])
def test_add_rmsnorm(xdtype, wdtype, d, T, eps):
    g = torch.Generator().manual_seed(1)
    resid = torch.randn(T, d, generator=g).to(DEV)
    delta = torch.randn(T, d, generator=g).to(xdtype).to(DEV)
    w = (1 + 0.1 * torch.randn(d, generator=g)).to(wdtype).to(DEV)
    h = resid.double() + delta.double()
    want = plain_llama.rmsnorm(h.cpu(), w.double().cpu(), eps)
    r2 = resid.clone()
    out = torch.empty(T, d, dtype=xdtype, device=DEV)
    ops().add_rmsnorm(r2, delta, w, eps, out)
    assert torch.allclose(r2.double(), h, atol=1e-6)
    tol = 1e-5 if xdtype == torch.float32 else 2 ** -8 * want.abs().max().item()
    assert (out.double().cpu() - want).abs().max().item() <= tol
    # rows: only the listed rows, stream untouched
    rows = torch.tensor([T - 1, 0, T - 1], dtype=torch.int32, device=DEV)
    r3 = resid.clone()
    out2 = torch.empty(3, d, dtype=xdtype, device=DEV)
    ops().add_rmsnorm(r3, delta, w, eps, out2, rows=rows)
    assert torch.equal(r3, resid)
    assert torch.equal(out2, out[rows.long()])
    # without delta
    out3 = torch.empty(T, d, dtype=xdtype, device=DEV)
    ops().add_rmsnorm(r3, None, w, eps, out3)
    want3 = plain_llama.rmsnorm(resid.double().cpu(), w.double().cpu(), eps)
    assert (out3.double().cpu() - want3).abs().max().item() <= tol
    # with something to fetch ahead into L2 (a hint for the launch after this one): the same numbers,
    # for tensors below one chunk, of an odd size, and larger than the most that is fetched
    for n in (100, 4096 * 3 + 72, 20 << 20):
        nxt = torch.zeros(n, dtype=torch.uint8, device=DEV)
        r4 = resid.clone()
        out4 = torch.empty(T, d, dtype=xdtype, device=DEV)
        ops().add_rmsnorm(r4, delta, w, eps, out4, ahead=nxt)
        assert torch.equal(out4, out) and torch.equal(r4, r2)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("T,F", [(3, 320), (17, 1336)])
def test_swiglu(dtype, T, F):
    g = torch.Generator().manual_seed(2)
    gu = (3 * torch.randn(T, 2 * F, generator=g)).to(dtype).to(DEV)
    out = torch.empty(T, F, dtype=dtype, device=DEV)
    ops().swiglu(gu, out)
    want = plain_llama.swiglu(gu[:, :F].double().cpu(), gu[:, F:].double().cpu())
    tol = 1e-5 if dtype == torch.float32 else 2 ** -8 * want.abs().max().item()
    assert (out.double().cpu() - want).abs().max().item() <= tol


def _interleave(gate, up, group):
    """Columns of gate and up interleaved in groups of `group`, as the stacked projection lays them out."""
    T, F = gate.shape
    return torch.stack([gate.view(T, F // group, group), up.view(T, F // group, group)], 2).reshape(T, 2 * F)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("T,F,group", [(3, 320, 8), (5, 1336, 8), (4, 36, 4), (2, 30, 3)])
def test_swiglu_interleaved(dtype, T, F, group):
    g = torch.Generator().manual_seed(22)
    gate = (3 * torch.randn(T, F, generator=g)).to(dtype)
    up = (3 * torch.randn(T, F, generator=g)).to(dtype)
    gu = _interleave(gate, up, group).contiguous().to(DEV)
    out = torch.empty(T, F, dtype=dtype, device=DEV)
    ops().swiglu(gu, out, group)
    want = plain_llama.swiglu(gate.double(), up.double())
    tol = 1e-5 if dtype == torch.float32 else 2 ** -8 * want.abs().max().item()
    assert (out.double().cpu() - want).abs().max().item() <= tol


@pytest.mark.parametrize("M,F,K", [(1, 64, 96), (8, 1336, 320), (11, 40, 1000), (16, 256, 72)])
def test_gemm_skinny_swiglu(M, F, K):
    """The few-row gate/up product with the activation in its epilogue equals the product stored in bf16
    followed by the activation kernel."""
    g = torch.Generator().manual_seed(23)
    a = torch.randn(M, K, generator=g).to(torch.bfloat16).to(DEV)
    wg = (torch.randn(F, K, generator=g) / math.sqrt(K)).to(torch.bfloat16)
    wu = (torch.randn(F, K, generator=g) / math.sqrt(K)).to(torch.bfloat16)
    w = _interleave(wg.t().contiguous(), wu.t().contiguous(), 8).t().contiguous().to(DEV)     # rows interleaved
    out = torch.full((M, F), float("nan"), dtype=torch.bfloat16, device=DEV)
    ops().gemm_skinny_swiglu(a, w, out)
    gu = torch.empty(M, 2 * F, dtype=torch.bfloat16, device=DEV)
    ops().gemm_skinny(a, w, gu)
    two = torch.empty(M, F, dtype=torch.bfloat16, device=DEV)
    ops().swiglu(gu, two, 8)
    assert torch.equal(out, two)
    want = plain_llama.swiglu(a.double().cpu() @ wg.double().T, a.double().cpu() @ wu.double().T)
    assert (out.double().cpu() - want).abs().max().item() <= 2 ** -7 * max(1.0, want.abs().max().item())


@pytest.mark.parametrize("M,N,K", [(1, 1000, 96), (7, 513, 320), (130, 200, 1336), (64, 64, 16), (3, 5, 7)])
def test_gemm_f32(M, N, K):
    g = torch.Generator().manual_seed(3)
    a = torch.randn(M, K, generator=g).to(DEV)
    w = torch.randn(N, K, generator=g).to(DEV)
    out = torch.empty(M, N, device=DEV)
    ops().gemm_f32(a, w, out)
    want = a.double() @ w.double().T
    assert (out.double() - want).abs().max().item() <= 1e-6 * K * 4
    # a row's result does not depend on the other rows of the call
    one = torch.empty(1, N, device=DEV)
    ops().gemm_f32(a[M - 1:M], w, one)
    assert torch.equal(one[0], out[M - 1])


def build_cache(dtype, lengths, H, KV, hs, page_size, seed, shuffle=True):
    """Random q/k/v of several whole sequences laid into a paged cache with shuffled pages."""
    g = torch.Generator().manual_seed(seed)
    S = len(lengths)
    blocks = [-(-n // page_size) for n in lengths]
    num_pages = sum(blocks) + 3
    perm = torch.randperm(num_pages, generator=g).tolist() if shuffle else list(range(num_pages))
    W = max(blocks)
    table = torch.full((S, W), -1, dtype=torch.int32)
    kc = torch.zeros(num_pages, KV, page_size, hs)
    vc = torch.zeros(num_pages, KV, page_size, hs)
    seqs = []
    p = 0
    for s, n in enumerate(lengths):
        q = torch.randn(n, H, hs, generator=g).to(dtype).float()
        k = torch.randn(n, KV, hs, generator=g).to(dtype).float()
        v = torch.randn(n, KV, hs, generator=g).to(dtype).float()
        for b in range(blocks[s]):
            page = perm[p]; p += 1
            table[s, b] = page
            m = min(page_size, n - b * page_size)
            kc[page, :, :m] = k[b * page_size:b * page_size + m].transpose(0, 1)
            vc[page, :, :m] = v[b * page_size:b * page_size + m].transpose(0, 1)
        seqs.append((q, k, v))
    return seqs, table, kc.to(dtype), vc.to(dtype)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("H,KV,hs,page_size,window", [(4, 2, 16, 16, None), (3, 1, 32, 8, None), (6, 3, 48, 4, None),
                                                     (8, 2, 128, 16, None), (5, 5, 80, 32, 7), (2, 1, 256, 16, 40)])
def test_paged_attention_ref(dtype, H, KV, hs, page_size, window):
    lengths = [1, 37, 130]
    seqs, table, kc, vc = build_cache(dtype, lengths, H, KV, hs, page_size, seed=4)
    scale = 1.0 / math.sqrt(hs)
    # rows: the last 5 positions of each sequence (a portion that continues from the cache)
    qrows, pos, rseq, want = [], [], [], []
    for s, (q, k, v) in enumerate(seqs):
        full = plain_llama.attention(q.double(), k.double(), v.double(), scale, window)
        for t in range(max(0, lengths[s] - 5), lengths[s]):
            qrows.append(q[t].reshape(-1)); pos.append(t); rseq.append(s); want.append(full[t].reshape(-1))
    q = torch.stack(qrows).to(dtype).to(DEV)
    out = torch.empty_like(q)
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    ops().paged_attention_ref(q, kc.to(DEV), vc.to(DEV), table.to(DEV), torch.tensor(rseq, dtype=torch.int32, device=DEV),
                              torch.tensor(pos, dtype=torch.int32, device=DEV), out, page_size, len(lengths),
                              H, KV, hs, scale, window or 0, status)
    assert status.item() == 0
    tol = 2e-6 if dtype == torch.float32 else 2 ** -8
    assert (out.double().cpu() - torch.stack(want)).abs().max().item() <= tol * 4


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("H,KV,hs,rot,page_size", [(4, 2, 16, 16, 16), (3, 1, 32, 32, 8), (5, 5, 80, 40, 4), (8, 2, 128, 128, 16)])
def test_rope_kv_write(dtype, H, KV, hs, rot, page_size):
    g = torch.Generator().manual_seed(5)
    lengths = [9, 40]
    T = sum(lengths)
    qkv = torch.randn(T, (H + 2 * KV) * hs, generator=g).to(dtype)
    pos = torch.cat([torch.arange(100, 100 + n) for n in lengths]).to(torch.int32)     # far positions
    rseq = torch.cat([torch.full((n,), s) for s, n in enumerate(lengths)]).to(torch.int32)
    W = (100 + max(lengths)) // page_size + 1
    num_pages = 2 * W
    table = torch.randperm(num_pages, generator=g).to(torch.int32).view(2, W)
    freqs = plain_llama.rope_frequencies(rot, 500000.0, {"rope_type": "llama3", "factor": 8.0, "low_freq_factor": 1.0,
                                                         "high_freq_factor": 4.0, "original_max_position_embeddings": 64})
    kc = torch.zeros(num_pages, KV, page_size, hs, dtype=dtype, device=DEV)
    vc = torch.zeros_like(kc)
    dq = qkv.clone().to(DEV)
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    ops().rope_kv_write(dq, pos.to(DEV), rseq.to(DEV), freqs.to(DEV), rot, table.to(DEV), kc, vc, page_size, 2,
                        H, KV, hs, status)
    assert status.item() == 0
    x = qkv.double()
    q3 = x[:, :H * hs].view(T, H, hs); k3 = x[:, H * hs:(H + KV) * hs].view(T, KV, hs); v3 = x[:, (H + KV) * hs:].view(T, KV, hs)
    def rot_part(t3):
        r = plain_llama.rope(t3[..., :rot], pos, freqs)
        return torch.cat([r, t3[..., rot:]], -1)
    tol = 1e-5 if dtype == torch.float32 else 2 ** -8 * 5
    wq, wk = rot_part(q3), rot_part(k3)
    assert (dq[:, :H * hs].double().cpu().view(T, H, hs) - wq).abs().max().item() <= tol
    kc, vc = kc.double().cpu(), vc.double().cpu()
    for t in range(T):
        page = table[rseq[t], pos[t] // page_size].item()
        off = pos[t].item() % page_size
        assert (kc[page, :, off] - wk[t]).abs().max().item() <= tol
        assert torch.equal(vc[page, :, off], v3[t])


@pytest.mark.parametrize("R,V", [(1, 31), (5, 1000), (24, 50257), (3, 128256)])
def test_argmax_split(R, V):
    """The greedy pick with a row split over many blocks: ties to the lowest index, also across blocks;
    repeated calls with different numbers of rows share one scratch buffer."""
    g = torch.Generator().manual_seed(60 + R)
    o = ops()
    scratch = torch.zeros(o.argmax_scratch_words(32), dtype=torch.int32, device=DEV)
    for rows in (R, max(1, R // 2), R):
        logits = (2.5 * torch.randn(rows, V, generator=g)).float()
        top = logits.max().item() + 1
        logits[0, V // 3] = logits[0, V - 1] = top                 # a tie in different blocks
        dl = logits.to(DEV)
        out = torch.full((rows,), -1, dtype=torch.int32, device=DEV)
        o.argmax(dl, out, scratch)
        assert out.tolist() == [plain_llama.sample(logits[r]) for r in range(rows)]
        assert out[0].item() == V // 3
        one = torch.full((rows,), -1, dtype=torch.int32, device=DEV)
        o.sample(dl, one)
        assert torch.equal(one, out)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_rmsnorm_rows_off_the_residual_stream(dtype):
    """The norm alone over rows, and over the heads of a token inside a stacked projection (a 3-D view with two
    strides), in place and into another buffer, against torch; what lies beside the rows is not touched."""
    g = torch.Generator().manual_seed(29)
    T, H, KV, hs, eps = 37, 5, 2, 48, 3e-6
    w = (1 + 0.1 * torch.randn(hs, generator=g)).to(dtype).to(DEV)
    qkv = torch.randn(T, (H + 2 * KV) * hs, generator=g).to(dtype).to(DEV)
    before = qkv.clone()
    q = qkv[:, :H * hs].view(T, H, hs)
    want = plain_llama.rmsnorm(before[:, :H * hs].double().cpu().view(T, H, hs), w.double().cpu(), eps)
    ops().rmsnorm_rows(q, w, eps)
    tol = 1e-5 if dtype == torch.float32 else 2 ** -7 * want.abs().max().item()
    assert (qkv[:, :H * hs].double().cpu().view(T, H, hs) - want).abs().max().item() <= tol
    assert torch.equal(qkv[:, H * hs:], before[:, H * hs:]), "keys and values beside the queries are as they were"
    x = torch.randn(9, 1336, generator=g).to(dtype).to(DEV)
    w2 = (1 + 0.1 * torch.randn(1336, generator=g)).to(DEV)                      # a weight kept in 32-bit
    out = torch.full_like(x, float("nan"))
    ops().rmsnorm_rows(x, w2, 1e-5, out)
    want = plain_llama.rmsnorm(x.double().cpu(), w2.double().cpu(), 1e-5)
    assert (out.double().cpu() - want).abs().max().item() <= (1e-5 if dtype == torch.float32 else 2 ** -7 * want.abs().max().item())
    with pytest.raises(ops().KernelError):
        ops().rmsnorm_rows(x.t(), w2, 1e-5)


def test_sampling_kernel_matches_plain():
    g = torch.Generator().manual_seed(6)
    V, R = 1000, 24
    logits = (2.5 * torch.randn(R, V, generator=g)).float()
    logits[3, 17] = logits[3, 400] = logits[3].max() + 1          # a tie: the lowest index wins
    dl = logits.to(DEV)
    out = torch.empty(R, dtype=torch.int32, device=DEV)
    ops().sample(dl, out)
    assert out.tolist() == [plain_llama.sample(logits[r]) for r in range(R)]
    assert out[3].item() == 17
    cases = [(0.7, 0, 0.9), (1.0, 5, 1.0), (1.3, 50, 0.5), (0.5, 0, 1.0), (1.0, 1, 1.0), (2.0, 0, 0.1)]
    for temp, k, p in cases:
        t = torch.full((R,), temp, device=DEV)
        tk = torch.full((R,), k, dtype=torch.int32, device=DEV)
        tp = torch.full((R,), p, device=DEV)
        seed = torch.arange(R, dtype=torch.int64, device=DEV) * 7919 + 1
        ctr = torch.arange(R, dtype=torch.int64, device=DEV) % 5
        ops().sample(dl, out, temperature=t, top_k=tk, top_p=tp, seed=seed, counter=ctr)
        want = [plain_llama.sample(logits[r], temp, k, p, seed=int(seed[r]), counter=int(ctr[r])) for r in range(R)]
        assert out.tolist() == want, (temp, k, p)


def test_sampling_treats_both_zeros_as_equal():
    """-0.0 and +0.0 are equal logits: top-k keeps all ties of the k-th, whichever zero they are, and the draw
    goes over all of them in index order, as the plain sampler's (a random search with rounded logits found the
    kernel's integer image of the logits telling the two zeros apart)."""
    V, R = 40, 16
    logits = torch.full((R, V), -3.0)
    zeros = [3, 7, 8, 21, 39]
    for r in range(R):
        for j, i in enumerate(zeros):
            logits[r, i] = -0.0 if (r + j) % 2 else 0.0
    dl = logits.to(DEV)
    out = torch.empty(R, dtype=torch.int32, device=DEV)
    seed = torch.arange(R, dtype=torch.int64, device=DEV) * 31 + 5
    ctr = torch.arange(R, dtype=torch.int64, device=DEV)
    for temp, k, p in [(1.0, 1, 1.0), (0.7, 2, 0.5), (1.5, 0, 0.0001)]:
        ops().sample(dl, out, temperature=torch.full((R,), temp, device=DEV),
                     top_k=torch.full((R,), k, dtype=torch.int32, device=DEV), top_p=torch.full((R,), p, device=DEV),
                     seed=seed, counter=ctr)
        want = [plain_llama.sample(logits[r], temp, k, p, seed=int(seed[r]), counter=int(ctr[r])) for r in range(R)]
        assert out.tolist() == want, (temp, k, p)
        assert len(set(want)) > 1 and set(want) <= set(zeros), "the draws spread over all five zeros"


def test_sampling_distribution():
    """Draws over many counters follow softmax(x / T) restricted by top-p."""
    V = 37
    g = torch.Generator().manual_seed(7)
    x = torch.randn(V, generator=g).float()
    R = 4096
    dl = x.to(DEV).repeat(R, 1)
    out = torch.empty(R, dtype=torch.int32, device=DEV)
    t = torch.full((R,), 0.8, device=DEV)
    tp = torch.full((R,), 0.9, device=DEV)
    seed = torch.full((R,), 1234, dtype=torch.int64, device=DEV)
    ctr = torch.arange(R, dtype=torch.int64, device=DEV)
    ops().sample(dl, out, temperature=t, top_p=tp, seed=seed, counter=ctr)
    p = torch.softmax(x.double() / 0.8, 0)
    order = torch.argsort(p, descending=True)
    csum = torch.cumsum(p[order], 0)
    kept = order[: int((csum < 0.9).sum()) + 1]
    pk = torch.zeros(V, dtype=torch.double); pk[kept] = p[kept] / p[kept].sum()
    freq = torch.bincount(out.cpu().long(), minlength=V).double() / R
    assert freq[pk == 0].sum().item() == 0
    assert (freq - pk).abs().max().item() < 4 * math.sqrt(0.25 / R)


# ---- tensor-core attention -----------------------------------------------------------------

def _torch_attention(q_row, kc, vc, table_row, pos, H, KV, hs, scale, window=0):
    """One query row [H * hs] at position ``pos`` against the pages of its sequence, in float32 with torch
    alone (no kernel of the package): softmax(scale q K^T) V over keys first..pos."""
    G = H // KV
    n_blocks = pos // kc.shape[2] + 1
    k = kc[table_row[:n_blocks].long()].float().permute(1, 0, 2, 3).reshape(KV, -1, hs)[:, :pos + 1]
    v = vc[table_row[:n_blocks].long()].float().permute(1, 0, 2, 3).reshape(KV, -1, hs)[:, :pos + 1]
    first = max(0, pos - window + 1) if window else 0
    sc = torch.einsum("kgd,kjd->kgj", q_row.float().view(KV, G, hs), k[:, first:]) * scale
    return torch.einsum("kgj,kjd->kgd", torch.softmax(sc, -1), v[:, first:]).reshape(-1)


def _items_for(lengths, tails, dec_tokens, por_tokens):
    """Rows = the last ``tails[s]`` tokens of each sequence, cut into kernel items."""
    dec, por, rows = [], [], []
    row = 0
    for s, (n, tl) in enumerate(zip(lengths, tails)):
        tl = min(tl, n)
        pos0 = n - tl
        if tl <= dec_tokens:
            dec.append((s, row, tl, pos0))
        else:
            for b in range(0, tl, por_tokens):
                por.append((s, row + b, min(por_tokens, tl - b), pos0 + b))
        rows += [(s, pos0 + i) for i in range(tl)]
        row += tl
    return dec, por, rows


def _run_tc_attention(seqs, table, kc, vc, lengths, tails, H, KV, hs, page_size, window, nsplit, tma=False, tc05=False):
    o = ops()
    G = H // KV
    if tc05 and not o.attn_portion_tc05_ok(H, KV, hs, page_size):
        pytest.skip("the tcgen05 portion kernel does not take this layout")
    if tma and not o.attn_decode_tma_ok(H, KV, hs, page_size):
        pytest.skip("the TMA decode kernel does not take this layout")
    dec_tokens = (o.attn_decode_tma_rows(H, KV) if tma else o.attn_decode_rows(H, KV, hs)) // G
    por_tokens = o.attn_portion_tc05_tokens(H, KV) if tc05 else o.attn_portion_tokens(H, KV, hs)
    dec, por, rows = _items_for(lengths, tails, dec_tokens, por_tokens)
    q = torch.stack([seqs[s][0][p].reshape(-1) for s, p in rows]).to(torch.bfloat16).to(DEV)
    out = torch.full_like(q, float("nan"))
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    scale = 1.0 / math.sqrt(hs)
    kcd, vcd, tb = kc.to(DEV), vc.to(DEV), table.to(DEV)
    if dec:
        items = torch.tensor(dec, dtype=torch.int32, device=DEV)
        scratch = None
        floats = o.attn_decode_tma_scratch_floats if tma else o.attn_decode_scratch_floats
        if nsplit > 1:
            scratch = torch.zeros(floats(len(dec), H, KV, hs, nsplit), device=DEV)
        more = {"max_rows": max(d[2] for d in dec) * G} if tma else {}      # few rows: the swapped products
        (o.attn_decode_tma if tma else o.attn_decode)(
            q, kcd, vcd, tb, items, out, page_size, len(lengths), H, KV, hs, scale, window or 0,
            nsplit=nsplit, scratch=scratch, status=status, **more)
    if por:
        items = torch.tensor(por, dtype=torch.int32, device=DEV)
        (o.attn_portion_tc05 if tc05 else o.attn_portion)(
            q, kcd, vcd, tb, items, out, page_size, len(lengths), H, KV, hs, scale, window or 0, status=status)
    assert status.item() == 0
    return out.double().cpu(), rows, bool(dec), bool(por)


@pytest.mark.parametrize("H,KV,hs,page_size,window", [
    (4, 2, 16, 16, None), (3, 1, 32, 8, None), (6, 3, 48, 4, None), (8, 2, 128, 16, None), (32, 8, 128, 16, None),
    (5, 5, 80, 32, 7), (2, 1, 256, 16, 40), (32, 1, 64, 16, None), (40, 1, 128, 16, None), (24, 8, 128, 16, 100),
    (14, 2, 64, 64, None), (9, 3, 96, 16, 65), (8, 8, 64, 8, None), (20, 1, 128, 32, 200), (16, 2, 64, 16, 70)])
@pytest.mark.parametrize("nsplit", [1, 3])
@pytest.mark.parametrize("tma", [False, True, "tc05"], ids=["cp_async", "tma", "tcgen05"])
def test_attention_tensor_cores(H, KV, hs, page_size, window, nsplit, tma):
    tc05 = tma == "tc05"
    tma = bool(tma)
    if tc05 and nsplit != 1:
        pytest.skip("splits concern the decode kernel only")
    lengths = [1, 37, 130, 700, 64, 129]
    tails = [1, 1, 3, 700, 64, 2]           # decode rows, short runs, a whole long prompt, an exact tile
    seqs, table, kc, vc = build_cache(torch.bfloat16, lengths, H, KV, hs, page_size, seed=8)
    out, rows, used_dec, used_por = _run_tc_attention(seqs, table, kc, vc, lengths, tails, H, KV, hs, page_size, window,
                                                      nsplit, tma, tc05)
    assert used_por
    scale = 1.0 / math.sqrt(hs)
    full = [plain_llama.attention(q.double(), k.double(), v.double(), scale, window) for q, k, v in seqs]
    want = torch.stack([full[s][p].reshape(-1) for s, p in rows])
    assert not torch.isnan(out).any(), "every row was written"
    # probabilities and outputs are rounded to bf16 (2^-9 relative each): 2^-8 of the largest value
    vmax = max(v.abs().max().item() for _, _, v in seqs)
    assert (out - want).abs().max().item() <= 2 ** -8 * vmax


@pytest.mark.parametrize("hs,page_size", [(128, 16), (64, 8), (32, 4)])
def test_attention_finds_one_far_key(hs, page_size):
    """One key among hundreds matches the query strongly: the output is that key's value row,
    wherever the key lies (first and last slot of a page, edges of the 64-key tiles, the row's
    own position), for a decode row, with and without splits, and for a row inside a portion."""
    H, KV = 4, 2
    n = 333
    g = torch.Generator().manual_seed(9)
    for target in [0, page_size - 1, page_size, 63, 64, 65, 127, 128, 200, n - 2, n - 1]:
        q = 0.1 * torch.randn(n, H, hs, generator=g)
        k = 0.1 * torch.randn(n, KV, hs, generator=g)
        v = torch.randn(n, KV, hs, generator=g)
        direction = torch.randn(hs, generator=g)
        direction /= direction.norm()
        k[target, :, :] = 6.0 * direction
        q[n - 1, :, :] = 6.0 * math.sqrt(hs) * direction        # score 36 against ~0 elsewhere
        q[n - 5, :, :] = 6.0 * math.sqrt(hs) * direction
        seqs = [(q.to(torch.bfloat16).float(), k.to(torch.bfloat16).float(), v.to(torch.bfloat16).float())]
        blocks = -(-n // page_size)
        perm = torch.randperm(blocks + 2, generator=g)
        table = perm[:blocks].to(torch.int32).view(1, -1)
        kc = torch.zeros(blocks + 2, KV, page_size, hs); vc = torch.zeros_like(kc)
        for b in range(blocks):
            m = min(page_size, n - b * page_size)
            kc[table[0, b], :, :m] = seqs[0][1][b * page_size:b * page_size + m].transpose(0, 1)
            vc[table[0, b], :, :m] = seqs[0][2][b * page_size:b * page_size + m].transpose(0, 1)
        kc, vc = kc.to(torch.bfloat16), vc.to(torch.bfloat16)
        for tails, nsplit, tma, tc05 in (([1], 1, False, False), ([1], 4, False, False), ([n], 1, False, False),
                                         ([1], 1, True, False), ([1], 4, True, False), ([n], 1, True, True)):
            if tma and not ops().attn_decode_tma_ok(H, KV, hs, page_size):
                continue
            if tc05 and not ops().attn_portion_tc05_ok(H, KV, hs, page_size):
                continue
            out, rows, _, _ = _run_tc_attention(seqs, table, kc, vc, [n], tails, H, KV, hs, page_size, None, nsplit, tma, tc05)
            for r, (s, p) in enumerate(rows):
                if p not in (n - 1, n - 5) or target > p:
                    continue
                got = out[r].view(H, hs)
                want = seqs[0][2][target].double().repeat_interleave(H // KV, 0)
                assert (got - want).abs().max().item() < 0.02, (target, tails, nsplit, p)


def test_attention_window_edge():
    """The key just inside the window counts, the one just outside does not."""
    H, KV, hs, page_size, window, n = 2, 1, 64, 16, 50, 180
    g = torch.Generator().manual_seed(10)
    direction = torch.randn(hs, generator=g); direction /= direction.norm()
    for target, visible in ((n - 1 - window, False), (n - window, True)):
        q = 0.1 * torch.randn(n, H, hs, generator=g)
        k = 0.1 * torch.randn(n, KV, hs, generator=g)
        v = torch.randn(n, KV, hs, generator=g)
        k[target] = 6.0 * direction
        q[n - 1] = 6.0 * math.sqrt(hs) * direction
        seqs = [(q.to(torch.bfloat16).float(), k.to(torch.bfloat16).float(), v.to(torch.bfloat16).float())]
        blocks = -(-n // page_size)
        table = torch.arange(blocks, dtype=torch.int32).view(1, -1)
        kc = torch.zeros(blocks, KV, page_size, hs); vc = torch.zeros_like(kc)
        for b in range(blocks):
            m = min(page_size, n - b * page_size)
            kc[b, :, :m] = seqs[0][1][b * page_size:b * page_size + m].transpose(0, 1)
            vc[b, :, :m] = seqs[0][2][b * page_size:b * page_size + m].transpose(0, 1)
        for tails, tma, tc05 in (([1], False, False), ([n], False, False), ([1], True, False), ([n], True, True)):
            out, rows, _, _ = _run_tc_attention(seqs, table, kc.to(torch.bfloat16), vc.to(torch.bfloat16), [n], tails,
                                                H, KV, hs, page_size, window, 1, tma, tc05)
            got = out[-1].view(H, hs)
            hit = (got - seqs[0][2][target].double()).abs().max().item() < 0.02
            assert hit == visible, (target, tails)


@pytest.mark.parametrize("H,KV,hs,page_size,window", [
    (4, 2, 64, 16, 40), (8, 2, 128, 16, 100), (2, 1, 64, 8, 11), (6, 3, 64, 16, 70), (5, 5, 80, 32, 7),
    (16, 2, 128, 32, 200), (3, 1, 32, 4, 5), (2, 1, 256, 16, 129)])
@pytest.mark.parametrize("nsplit", [1, 3])
@pytest.mark.parametrize("tma", [False, True, "tc05"], ids=["cp_async", "tma", "tcgen05"])
def test_attention_window_with_pages_given_back(H, KV, hs, page_size, window, nsplit, tma):
    """Pages that lie wholly before the window of a step's first token have been given back: their table
    entries are -1 and the pages hold someone else's data (NaN here). The kernels round the first key
    down to a tile of 64, so such pages fall inside their first tile; they are neither looked up
    nor read, and no status is raised."""
    tc05 = tma == "tc05"
    tma = bool(tma)
    if tc05 and nsplit != 1:
        pytest.skip("splits concern the decode kernel only")
    lengths = [1, 37, 130, 700, 64, 129, 650, 333]
    tails = [1, 1, 3, 45, 64, 2, 300, 1]
    seqs, table, kc, vc = build_cache(torch.bfloat16, lengths, H, KV, hs, page_size, seed=12)
    gone = 0
    for s, (n, tl) in enumerate(zip(lengths, tails)):
        first_needed = (n - min(tl, n)) - window + 1          # what the step's first token reads from
        for b in range(max(0, first_needed) // page_size):
            kc[table[s, b]] = float("nan"); vc[table[s, b]] = float("nan")
            table[s, b] = -1
            gone += 1
    assert gone > 20
    out, rows, used_dec, used_por = _run_tc_attention(seqs, table, kc, vc, lengths, tails, H, KV, hs, page_size, window,
                                                      nsplit, tma, tc05)
    assert used_dec and used_por
    scale = 1.0 / math.sqrt(hs)
    full = [plain_llama.attention(q.double(), k.double(), v.double(), scale, window) for q, k, v in seqs]
    want = torch.stack([full[s][p].reshape(-1) for s, p in rows])
    assert not torch.isnan(out).any(), "every row was written, and nothing of a page given back was read"
    vmax = max(v.abs().max().item() for _, _, v in seqs)
    assert (out - want).abs().max().item() <= 2 ** -8 * vmax


@pytest.mark.parametrize("H,KV,hs,page_size,window", [(32, 8, 128, 16, None), (4, 2, 64, 8, None), (16, 2, 128, 32, 300),
                                                     (8, 8, 64, 16, None), (40, 1, 128, 16, None)])
@pytest.mark.parametrize("budget", [1, 7, 37, 200])
def test_decode_with_shares_of_equal_length(H, KV, hs, page_size, window, budget):
    """Decode items of very different lengths, each cut into its own number of shares by ``split_work``:
    the same outputs as whole sequences give, whatever the budget of shares, with empty items and unused
    work entries in between, twice over the same scratch."""
    o = ops()
    if not o.attn_decode_tma_ok(H, KV, hs, page_size):
        pytest.skip("the TMA decode kernel does not take this layout")
    G = H // KV
    lengths = [2000, 3, 64, 700, 129, 1, 65, 1200]
    seqs, table, kc, vc = build_cache(torch.bfloat16, lengths, H, KV, hs, page_size, seed=21)
    dec = [(s, s, 1, n - 1) for s, n in enumerate(lengths)]
    dec.insert(3, (0, 0, 0, 0))                                  # an empty item, as fixed shapes are padded with
    tiles = []
    for (_, _, n, pos0) in dec:
        first = max(0, pos0 - window + 1) // 64 * 64 if window else 0
        tiles.append(-(-(pos0 + n - first) // 64) if n else 0)
    entries = budget + len(dec)
    work_h = o.split_work(tiles, budget, entries, 32, 2)
    live = work_h[work_h[:, 0] >= 0]
    assert len(live) <= budget + len(lengths) and set(live[:, 0].tolist()) == {i for i, t in enumerate(tiles) if t}
    for i in set(live[:, 0].tolist()):
        mine = live[live[:, 0] == i]
        assert sorted(mine[:, 1].tolist()) == list(range(mine[0, 2])) and len(set(mine[:, 3].tolist())) == 1
    if budget >= 37 and not window:
        shares = {i: (live[:, 0] == i).sum() for i in range(len(dec))}
        assert shares[0] > 4 * shares[1 + 1], "the longest item is cut into the most shares"
    q = torch.stack([seqs[s][0][n - 1].reshape(-1) for s, n in enumerate(lengths)]).to(torch.bfloat16).to(DEV)
    items = torch.tensor(dec, dtype=torch.int32, device=DEV)
    work = torch.tensor(work_h, dtype=torch.int32, device=DEV)
    scratch = torch.zeros(o.attn_decode_tma_work_floats(entries, H, KV, hs), device=DEV)
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    scale = 1.0 / math.sqrt(hs)
    full = [plain_llama.attention(qq.double(), k.double(), v.double(), scale, window) for qq, k, v in seqs]
    want = torch.stack([full[s][n - 1].reshape(-1) for s, n in enumerate(lengths)])
    vmax = max(v.abs().max().item() for _, _, v in seqs)
    for turn in range(2):
        out = torch.full_like(q, float("nan"))
        o.attn_decode_tma(q, kc.to(DEV), vc.to(DEV), table.to(DEV), items, out, page_size, len(lengths), H, KV, hs, scale,
                          window or 0, work=work, scratch=scratch, status=status, max_rows=G)
        assert status.item() == 0
        assert not torch.isnan(out).any(), "every row was written"
        assert (out.double().cpu() - want).abs().max().item() <= 2 ** -8 * vmax, turn


@pytest.mark.parametrize("tma", [False, True], ids=["cp_async", "tma"])
def test_split_decode_shares_its_scratch_between_shapes(tma):
    """One scratch buffer serves launches with different numbers of items and splits, as the engine's does
    from step to step: a launch with many items and splits fills it with partial results, a launch with few
    follows and must find its tickets at zero all the same (they have a region of their own)."""
    o = ops()
    H, KV, hs, page_size = 16, 1, 64, 16                # 16 query heads per KV head: every row of a partial tile is written
    lengths = [300, 290, 280, 270, 260, 250]
    seqs, table, kc, vc = build_cache(torch.bfloat16, lengths, H, KV, hs, page_size, seed=31)
    kcd, vcd, tb = kc.to(DEV), vc.to(DEV), table.to(DEV)
    floats = o.attn_decode_tma_scratch_floats if tma else o.attn_decode_scratch_floats
    decode = o.attn_decode_tma if tma else o.attn_decode
    scratch = torch.zeros(floats(len(lengths), H, KV, hs, 4), device=DEV)
    scale = 1.0 / math.sqrt(hs)
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    full = [plain_llama.attention(q.double(), k.double(), v.double(), scale, None) for q, k, v in seqs]
    vmax = max(v.abs().max().item() for _, _, v in seqs)
    for which, nsplit in (([0, 1, 2, 3, 4, 5], 4), ([1], 2), ([0, 2, 4], 3), ([5], 4), ([0, 1, 2, 3, 4, 5], 2)):
        items = torch.tensor([(s, i, 1, lengths[s] - 1) for i, s in enumerate(which)], dtype=torch.int32, device=DEV)
        q = torch.stack([seqs[s][0][lengths[s] - 1].reshape(-1) for s in which]).to(torch.bfloat16).to(DEV)
        out = torch.full_like(q, float("nan"))
        decode(q, kcd, vcd, tb, items, out, page_size, len(lengths), H, KV, hs, scale, 0, nsplit=nsplit,
               scratch=scratch, status=status)
        want = torch.stack([full[s][lengths[s] - 1].reshape(-1) for s in which])
        assert status.item() == 0
        assert not torch.isnan(out).any(), (which, nsplit)
        assert (out.double().cpu() - want).abs().max().item() <= 2 ** -8 * vmax, (which, nsplit)


@pytest.mark.parametrize("batch,ctx,nsplit", [(8, 8192, 4), (64, 2048, 1), (1, 8192, 32)])
@pytest.mark.parametrize("tma", [False, True], ids=["cp_async", "tma"])
def test_attention_decode_at_serving_size(batch, ctx, nsplit, tma):
    """Decode rows at the Llama-3.1-8B head layout over long contexts (a cache larger than L2):
    the tensor-core kernel against the plain kernel, and its achieved bandwidth (printed)."""
    o = ops()
    H, KV, hs, page_size = 32, 8, 128, 16
    g = torch.Generator(device=DEV).manual_seed(11)
    blocks = -(-ctx // page_size)
    num_pages = batch * blocks
    kc = torch.randn(num_pages, KV, page_size, hs, generator=g, device=DEV, dtype=torch.float32).to(torch.bfloat16)
    vc = torch.randn(num_pages, KV, page_size, hs, generator=g, device=DEV, dtype=torch.float32).to(torch.bfloat16)
    table = torch.randperm(num_pages, generator=g, device=DEV).to(torch.int32).view(batch, blocks)
    q = torch.randn(batch, H * hs, generator=g, device=DEV, dtype=torch.float32).to(torch.bfloat16)
    lens = [ctx - 3 * i for i in range(batch)]
    items = torch.tensor([(s, s, 1, lens[s] - 1) for s in range(batch)], dtype=torch.int32, device=DEV)
    pos = torch.tensor([n - 1 for n in lens], dtype=torch.int32, device=DEV)
    rseq = torch.arange(batch, dtype=torch.int32, device=DEV)
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    scale = 1.0 / math.sqrt(hs)
    want = torch.empty_like(q)
    o.paged_attention_ref(q, kc, vc, table, rseq, pos, want, page_size, batch, H, KV, hs, scale, 0, status)
    out = torch.empty_like(q)
    floats = o.attn_decode_tma_scratch_floats if tma else o.attn_decode_scratch_floats
    scratch = torch.zeros(max(1, floats(batch, H, KV, hs, nsplit)), device=DEV)
    decode = o.attn_decode_tma if tma else o.attn_decode
    more = {"max_rows": H // KV} if tma else {}
    run = lambda: decode(q, kc, vc, table, items, out, page_size, batch, H, KV, hs, scale, 0,
                         nsplit=nsplit, scratch=scratch if nsplit > 1 else None, status=status, **more)
    run()
    assert status.item() == 0
    assert (out.float() - want.float()).abs().max().item() <= 2 ** -8 * 4       # outputs of size up to ~4 in bf16
    # and against torch alone, so that the yardstick is not a kernel of the package: the first, a middle and the last row
    for s_ in sorted({0, batch // 2, batch - 1}):
        ref = _torch_attention(q[s_], kc, vc, table[s_], lens[s_] - 1, H, KV, hs, scale)
        assert (out[s_].float() - ref).abs().max().item() <= 2 ** -8 * 4, f"sequence {s_} against torch"
    for _ in range(3):
        run()
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    torch.cuda.synchronize()
    a.record()
    for _ in range(10):
        run()
    b.record()
    torch.cuda.synchronize()
    us = a.elapsed_time(b) * 100
    gbs = sum(lens) * KV * hs * 2 * 2 / (us * 1e-6) / 1e9
    print(f"attn_decode {'tma' if tma else 'cp.async'} batch {batch} ctx {ctx} nsplit {nsplit}: {us:.1f} us, "
          f"{gbs:.0f} GB/s of cache read")


@pytest.mark.parametrize("lens", [[8192] * 8, [8192] + [512] * 7, [8192, 4096, 2048, 1024, 512, 256, 128, 64],
                                  [8192] + [256] * 63, [8192] * 40], ids=["even", "one_long", "halving", "one_long_of_64", "forty"])
def test_attention_decode_shares_at_serving_size(lens):
    """Sequences of unequal length at the Llama-3.1-8B head layout: shares of equal length (``split_work``)
    against the same number of splits for every sequence; the same outputs, and the time of both (printed)."""
    o = ops()
    H, KV, hs, page_size = 32, 8, 128, 16
    batch = len(lens)
    g = torch.Generator(device=DEV).manual_seed(11)
    blocks = [-(-n // page_size) for n in lens]
    num_pages = sum(blocks)
    kc = torch.randn(num_pages, KV, page_size, hs, generator=g, device=DEV, dtype=torch.float32).to(torch.bfloat16)
    vc = torch.randn(num_pages, KV, page_size, hs, generator=g, device=DEV, dtype=torch.float32).to(torch.bfloat16)
    perm = torch.randperm(num_pages, generator=g, device=DEV).to(torch.int32)
    table = torch.full((batch, max(blocks)), -1, dtype=torch.int32, device=DEV)
    at = 0
    for s_, nb in enumerate(blocks):
        table[s_, :nb] = perm[at:at + nb]
        at += nb
    q = torch.randn(batch, H * hs, generator=g, device=DEV, dtype=torch.float32).to(torch.bfloat16)
    items = torch.tensor([(s_, s_, 1, n - 1) for s_, n in enumerate(lens)], dtype=torch.int32, device=DEV)
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    scale = 1.0 / math.sqrt(hs)
    nsplit = max(1, min(32, 296 // (batch * KV)))
    scratch = torch.zeros(max(1, o.attn_decode_tma_scratch_floats(batch, H, KV, hs, nsplit)), device=DEV)
    entries = 296 // KV + 4 * batch
    work = torch.tensor(o.split_work([-(-n // 64) for n in lens], 296 // KV, entries, 32, 2), dtype=torch.int32, device=DEV)
    scratch2 = torch.zeros(o.attn_decode_tma_work_floats(entries, H, KV, hs), device=DEV)
    outs, times = [], []
    for kw in ({"nsplit": nsplit, "scratch": scratch if nsplit > 1 else None}, {"work": work, "scratch": scratch2}):
        out = torch.empty_like(q)
        run = lambda: o.attn_decode_tma(q, kc, vc, table, items, out, page_size, batch, H, KV, hs, scale, 0,
                                        status=status, max_rows=H // KV, **kw)
        for _ in range(3):
            run()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        a.record()
        for _ in range(10):
            run()
        b.record()
        torch.cuda.synchronize()
        outs.append(out)
        times.append(a.elapsed_time(b) * 100)
    assert status.item() == 0
    assert (outs[0].float() - outs[1].float()).abs().max().item() <= 2 ** -8 * 4
    mb = sum(lens) * KV * hs * 2 * 2 / 1e6
    print(f"attn_decode tma {batch} sequences, {sum(lens)} tokens ({mb:.0f} MB): {nsplit} splits each {times[0]:.1f} us, "
          f"shares of equal length {times[1]:.1f} us ({mb / times[1]:.2f} TB/s)")


@pytest.mark.parametrize("out_dtype", [torch.bfloat16, torch.float32])
@pytest.mark.parametrize("M,N,K", [(1, 1000, 96), (3, 513, 320), (8, 200, 1336), (16, 64, 16), (9, 37, 8), (5, 4096, 4096)])
def test_gemm_skinny(M, N, K, out_dtype):
    g = torch.Generator().manual_seed(12)
    a = torch.randn(M, K, generator=g).to(torch.bfloat16).to(DEV)
    w = torch.randn(N, K, generator=g).to(torch.bfloat16).to(DEV)
    out = torch.full((M, N), float("nan"), dtype=out_dtype, device=DEV)
    ops().gemm_skinny(a, w, out)
    want = a.double() @ w.double().T
    tol = 1e-4 * math.sqrt(K) if out_dtype == torch.float32 else 2 ** -8 * want.abs().max().item()
    assert (out.double() - want).abs().max().item() <= tol
    # a row does not depend on the rows beside it; a strided view of x works
    wide = torch.zeros(M, K + 24, dtype=torch.bfloat16, device=DEV)
    wide[:, :K] = a
    one = torch.empty(1, N, dtype=out_dtype, device=DEV)
    ops().gemm_skinny(wide[M - 1:M, :K], w, one)
    assert torch.equal(one[0], out[M - 1])


@pytest.mark.parametrize("M,H,KV,hs,K,page_size", [(1, 4, 2, 64, 256, 16), (8, 32, 8, 128, 4096, 16), (16, 3, 1, 32, 96, 8),
                                                   (11, 6, 3, 16, 136, 4), (5, 2, 2, 96, 320, 32)])
def test_gemm_skinny_qkv_rope(M, H, KV, hs, K, page_size):
    """The q/k/v product with the rotation and the cache store in its epilogue against the three kernels it
    stands for (product, then rotation and store): rotated q, and the pages of k and v, a padding row included."""
    g = torch.Generator(device=DEV).manual_seed(31)
    o = ops()
    x = torch.randn(M, K, generator=g, device=DEV).to(torch.bfloat16)
    w = (torch.randn((H + 2 * KV) * hs, K, generator=g, device=DEV) / K ** 0.5).to(torch.bfloat16)
    inv_freq = (1.0 / (10000.0 ** (torch.arange(0, hs, 2, dtype=torch.float64) / hs))).float().to(DEV)
    num_seqs, width = M, 6
    num_pages = num_seqs * width + 3
    table = torch.randperm(num_pages, generator=g, device=DEV)[:num_seqs * width].to(torch.int32).view(num_seqs, width)
    positions = torch.randint(0, width * page_size, (M,), generator=g, device=DEV).to(torch.int32)
    row_seq = torch.arange(M, dtype=torch.int32, device=DEV)
    if M > 2:
        row_seq[M - 2] = -1                       # a padding row of a fixed-shape step: nothing stored for it
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    caches = []
    outs = []
    for fused in (False, True):
        kc = torch.zeros(num_pages, KV, page_size, hs, dtype=torch.bfloat16, device=DEV)
        vc = torch.zeros_like(kc)
        qkv = torch.zeros(M, (H + 2 * KV) * hs, dtype=torch.bfloat16, device=DEV)
        if fused:
            o.gemm_skinny_qkv_rope(x, w, qkv, positions, row_seq, inv_freq, table, kc, vc, page_size, num_seqs, H, KV, hs, status)
        else:
            o.gemm_skinny(x, w, qkv)
            o.rope_kv_write(qkv, positions, row_seq, inv_freq, hs, table, kc, vc, page_size, num_seqs, H, KV, hs, status)
        assert status.item() == 0
        outs.append(qkv[:, :H * hs].float())
        caches.append((kc.float(), vc.float()))
    # the same roundings in the same places; a product and a sum may be contracted differently: one bf16 step
    step = 2 ** -7
    assert (outs[0] - outs[1]).abs().max().item() <= step * max(1.0, outs[0].abs().max().item())
    assert (caches[0][0] - caches[1][0]).abs().max().item() <= step * max(1.0, caches[0][0].abs().max().item())
    assert torch.equal(caches[0][1], caches[1][1]), "v is stored as the product gave it"
    assert caches[1][0].abs().sum().item() > 0 and caches[1][1].abs().sum().item() > 0
    # against torch alone: one row's rotated first q head
    m = 0
    q0 = (x[m].double() @ w[:hs].double().T).to(torch.bfloat16).double()
    ang = positions[m].item() * inv_freq.double().cpu()
    c, sn = torch.cos(ang).to(DEV), torch.sin(ang).to(DEV)
    want = torch.cat([q0[:hs // 2] * c - q0[hs // 2:] * sn, q0[hs // 2:] * c + q0[:hs // 2] * sn])
    assert (outs[1][m, :hs].double() - want).abs().max().item() <= 2 ** -7 * max(1.0, want.abs().max().item())
    # a table entry outside the pool is reported, nothing is written for that row
    bad = table.clone()
    bad[0] = num_pages + 5
    kc = torch.zeros(num_pages, KV, page_size, hs, dtype=torch.bfloat16, device=DEV)
    o.gemm_skinny_qkv_rope(x[:1], w, torch.zeros(1, (H + 2 * KV) * hs, dtype=torch.bfloat16, device=DEV), positions[:1],
                           row_seq[:1], inv_freq, bad, kc, torch.zeros_like(kc), page_size, num_seqs, H, KV, hs, status)
    assert status.item() == 2 and kc.abs().sum().item() == 0


def test_gemm_skinny_at_serving_size():
    """The four projections of the Llama-3.1-8B block at 8 rows: achieved weight bandwidth (printed)
    beside the library product."""
    g = torch.Generator(device=DEV).manual_seed(13)
    for name, N, K in (("qkv", 6144, 4096), ("o", 4096, 4096), ("gate_up", 28672, 4096), ("down", 4096, 14336)):
        a = torch.randn(8, K, generator=g, device=DEV).to(torch.bfloat16)
        # several copies of the weight so that consecutive runs do not find it in L2
        ws = [(0.02 * torch.randn(N, K, generator=g, device=DEV)).to(torch.bfloat16) for _ in range(4)]
        out = torch.empty(8, N, dtype=torch.bfloat16, device=DEV)
        res = {}
        for label, fn in (("skinny", lambda w: ops().gemm_skinny(a, w, out)), ("library", lambda w: torch.mm(a, w.t(), out=out))):
            for w in ws:
                fn(w)
            torch.cuda.synchronize()
            graph = torch.cuda.CUDAGraph()           # replayed from a graph: the host's launch cost stays out
            with torch.cuda.graph(graph):
                for _ in range(5):
                    for w in ws:
                        fn(w)
            graph.replay()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            torch.cuda.synchronize()
            e0.record()
            graph.replay()
            e1.record()
            torch.cuda.synchronize()
            res[label] = e0.elapsed_time(e1) * 1e3 / 20
        want = a.double() @ ws[-1].double().T
        ops().gemm_skinny(a, ws[-1], out)
        assert (out.double() - want).abs().max().item() <= 2 ** -8 * want.abs().max().item()
        mb = N * K * 2 / 1e6
        print(f"{name}: skinny {res['skinny']:.1f} us ({mb / res['skinny']:.2f} TB/s), "
              f"library {res['library']:.1f} us ({mb / res['library']:.2f} TB/s)")


@pytest.mark.parametrize("out_dtype", [torch.bfloat16, torch.float32])
@pytest.mark.parametrize("M,N,K", [(128, 128, 64), (128, 128, 256), (256, 384, 512), (200, 1000, 320), (33, 96, 1336),
                                   (1, 128, 64), (2048, 512, 4096)])
def test_gemm_tc05(M, N, K, out_dtype):
    g = torch.Generator().manual_seed(14)
    a = torch.randn(M, K, generator=g).to(torch.bfloat16).to(DEV)
    w = torch.randn(N, K, generator=g).to(torch.bfloat16).to(DEV)
    out = torch.full((M, N), float("nan"), dtype=out_dtype, device=DEV)
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    ops().gemm_tc05(a, w, out, status)
    torch.cuda.synchronize()
    assert status.item() == 0
    want = a.double() @ w.double().T
    tol = 1e-4 * math.sqrt(K) if out_dtype == torch.float32 else 2 ** -8 * want.abs().max().item()
    assert not torch.isnan(out).any()
    assert (out.double() - want).abs().max().item() <= tol


@pytest.mark.parametrize("M,F,K", [(128, 128, 64), (200, 1336, 320), (2048, 512, 4096), (77, 40, 72)])
def test_gemm_tc05_swiglu(M, F, K):
    """The many-row gate/up product with the activation in its epilogue equals the product stored in bf16
    followed by the activation kernel."""
    g = torch.Generator().manual_seed(24)
    a = torch.randn(M, K, generator=g).to(torch.bfloat16).to(DEV)
    w = (torch.randn(2 * F, K, generator=g) / math.sqrt(K)).to(torch.bfloat16).to(DEV)
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    out = torch.full((M, F), float("nan"), dtype=torch.bfloat16, device=DEV)
    ops().gemm_tc05_swiglu(a, w, out, status)
    gu = torch.empty(M, 2 * F, dtype=torch.bfloat16, device=DEV)
    ops().gemm_tc05(a, w, gu, status)
    two = torch.empty(M, F, dtype=torch.bfloat16, device=DEV)
    ops().swiglu(gu, two, 8)
    assert status.item() == 0
    assert torch.equal(out, two)
    ref = (a.double() @ w.double().T).view(M, F // 8, 2, 8)
    want = plain_llama.swiglu(ref[:, :, 0].reshape(M, F).cpu(), ref[:, :, 1].reshape(M, F).cpu())
    assert (out.double().cpu() - want).abs().max().item() <= 2 ** -7 * max(1.0, want.abs().max().item())


@pytest.mark.parametrize("out_dtype", [torch.bfloat16, torch.float32])
@pytest.mark.parametrize("M,N,K", [(17, 128, 64), (1, 1000, 96), (33, 513, 320), (64, 200, 1336), (128, 384, 4096), (100, 6144, 512),
                                   (16, 64, 16), (127, 37, 8), (48, 4096, 4096), (5, 128256, 256)])
def test_gemm_rows(M, N, K, out_dtype):
    """The product for up to 128 rows: tiles shared between blocks (their partial sums added by the tile's
    owner), tails in every dimension, and the same call twice (the flags are back at zero)."""
    g = torch.Generator(device=DEV).manual_seed(21)
    a = torch.randn(M, K, generator=g, device=DEV).to(torch.bfloat16)
    w = torch.randn(N, K, generator=g, device=DEV).to(torch.bfloat16)
    want = a.double() @ w.double().T
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    tol = (2 ** -8 if out_dtype == torch.bfloat16 else 2e-6) * max(1.0, want.abs().max().item()) + 1e-5 * K ** 0.5
    for _ in range(2):
        out = torch.full((M, N), float("nan"), dtype=out_dtype, device=DEV)
        ops().gemm_rows(a, w, out, status)
        assert status.item() == 0
        assert not torch.isnan(out).any()
        assert (out.double() - want).abs().max().item() <= tol
    # a row's result does not depend on the other rows of the call
    if M > 1:
        alone = torch.empty(1, N, dtype=out_dtype, device=DEV)
        ops().gemm_rows(a[M // 2:M // 2 + 1], w, alone, status)
        assert torch.equal(alone[0], out[M // 2])


@pytest.mark.parametrize("M,F,K", [(17, 64, 96), (64, 1336, 320), (128, 520, 4096), (30, 40, 72), (100, 14336, 256)])
def test_gemm_rows_swiglu(M, F, K):
    g = torch.Generator(device=DEV).manual_seed(22)
    a = torch.randn(M, K, generator=g, device=DEV).to(torch.bfloat16)
    gate = (0.3 * torch.randn(F, K, generator=g, device=DEV)).to(torch.bfloat16)
    up = (0.3 * torch.randn(F, K, generator=g, device=DEV)).to(torch.bfloat16)
    w = torch.stack([gate.view(F // 8, 8, K), up.view(F // 8, 8, K)], 1).reshape(2 * F, K).contiguous()
    gd = (a.double() @ gate.double().T).to(torch.bfloat16).double()
    ud = (a.double() @ up.double().T).to(torch.bfloat16).double()
    want = gd / (1 + torch.exp(-gd)) * ud
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    out = torch.full((M, F), float("nan"), dtype=torch.bfloat16, device=DEV)
    ops().gemm_rows_swiglu(a, w, out, status)
    assert status.item() == 0 and not torch.isnan(out).any()
    # gate and up are rounded to bf16 before the activation: a rounding that falls the other way moves the result by
    # one bf16 step of gate or up
    scale = max(1.0, want.abs().max().item())
    assert (out.double() - want).abs().max().item() <= 2 ** -6 * scale


def test_gemm_rows_at_serving_size():
    """The projections of the Llama-3.1-8B block and the output head at 8 to 128 rows: time from a CUDA graph and
    bandwidth of the weight stream (printed) beside the few-row kernel (up to 16 rows) and the library; the calls
    of a graph go round several copies of the weight, so that none finds its weight in L2."""
    g = torch.Generator(device=DEV).manual_seed(23)
    shapes = (("qkv", 6144, 4096), ("o", 4096, 4096), ("gate_up", 28672, 4096), ("down", 4096, 14336), ("head", 128256, 4096))
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    for M in (8, 16, 32, 64, 128):
        for name, N, K in shapes:
            a = torch.randn(M, K, generator=g, device=DEV).to(torch.bfloat16)
            # copies of the weight, 300 MB of them: a call does not find its weight in L2 (126 MB) from the call before
            ws = [(0.02 * torch.randn(N, K, generator=g, device=DEV)).to(torch.bfloat16)
                  for _ in range(max(1, -(-300_000_000 // (N * K * 2))))]
            w = ws[-1]
            out = torch.empty(M, N, dtype=torch.bfloat16, device=DEV)
            runs = {"rows": lambda i: ops().gemm_rows(a, ws[i % len(ws)], out, status),
                    "library": lambda i: torch.mm(a, ws[i % len(ws)].t(), out=out)}
            if M <= 16:
                runs["few-row"] = lambda i: ops().gemm_skinny(a, ws[i % len(ws)], out)
            res = {label: graph_time_us(fn) for label, fn in runs.items()}
            assert status.item() == 0
            out.fill_(float("nan"))
            ops().gemm_rows(a, w, out, status)
            want = a.double() @ w[:4096].double().T
            assert (out[:, :4096].double() - want).abs().max().item() <= 2 ** -8 * want.abs().max().item()
            assert not torch.isnan(out).any()
            gb = N * K * 2 / 1e3
            print(f"{M:4d} rows {name:8s}: " + ", ".join(f"{k} {v:.1f} us ({gb / v:.0f} GB/s)" for k, v in res.items()))


@pytest.mark.parametrize("M,N,K", [(128, 128, 64), (200, 1000, 320), (300, 4096, 512), (129, 96, 1336), (2048, 520, 256)])
def test_gemm_tc05_add_into_the_residual_stream(M, N, K):
    """The product that adds itself into an fp32 tensor: equal, bit for bit, to storing the product in bf16 and
    adding that (what the norm kernel after it would do), with one CTA a tile and with pairs."""
    g = torch.Generator(device=DEV).manual_seed(41)
    a = torch.randn(M, K, generator=g, device=DEV).to(torch.bfloat16)
    w = (torch.randn(N, K, generator=g, device=DEV) / K ** 0.5).to(torch.bfloat16)
    resid0 = torch.randn(M, N, generator=g, device=DEV)
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    stored = torch.empty(M, N, dtype=torch.bfloat16, device=DEV)
    ops().gemm_tc05(a, w, stored, status)
    want = resid0 + stored.float()
    got = resid0.clone()
    ops().gemm_tc05_add(a, w, got, status)
    assert status.item() == 0
    assert torch.equal(got, want)
    ref = resid0.double() + (a.double() @ w.double().T)
    assert (got.double() - ref).abs().max().item() <= 2 ** -8 * max(1.0, (a.double() @ w.double().T).abs().max().item())


def test_gemm_tc05_at_prefill_size():
    """The projections of the Llama-3.1-8B block at 2,048 rows: achieved TFLOP/s (printed) beside the library."""
    g = torch.Generator(device=DEV).manual_seed(15)
    M = 2048
    for name, N, K in (("qkv", 6144, 4096), ("o", 4096, 4096), ("gate_up", 28672, 4096), ("down", 4096, 14336)):
        a = torch.randn(M, K, generator=g, device=DEV).to(torch.bfloat16)
        w = (0.02 * torch.randn(N, K, generator=g, device=DEV)).to(torch.bfloat16)
        out = torch.empty(M, N, dtype=torch.bfloat16, device=DEV)
        status = torch.zeros(1, dtype=torch.int32, device=DEV)
        res = {}
        for label, fn in (("tcgen05", lambda: ops().gemm_tc05(a, w, out, status)), ("library", lambda: torch.mm(a, w.t(), out=out))):
            for _ in range(3):
                fn()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            torch.cuda.synchronize()
            e0.record()
            for _ in range(10):
                fn()
            e1.record()
            torch.cuda.synchronize()
            res[label] = e0.elapsed_time(e1) * 100
        assert status.item() == 0
        out.fill_(float("nan"))
        ops().gemm_tc05(a, w, out, status)
        want = a.double() @ w.double().T                     # every element of every tile
        assert not torch.isnan(out).any()
        assert (out.double() - want).abs().max().item() <= 2 ** -8 * want.abs().max().item()
        del want
        tf = 2.0 * M * N * K / 1e6
        print(f"{name}: tcgen05 {res['tcgen05']:.1f} us ({tf / res['tcgen05']:.0f} TFLOP/s), "
              f"library {res['library']:.1f} us ({tf / res['library']:.0f} TFLOP/s)")


def test_attention_portion_at_prefill_size():
    """A 2,048-token prompt at the Llama-3.1-8B head layout: both portion kernels against the plain
    kernel on sampled rows, and their times (printed)."""
    o = ops()
    H, KV, hs, page_size, T = 32, 8, 128, 16, 2048
    g = torch.Generator(device=DEV).manual_seed(16)
    blocks = T // page_size
    kc = torch.randn(blocks + 5, KV, page_size, hs, generator=g, device=DEV).to(torch.bfloat16)
    vc = torch.randn(blocks + 5, KV, page_size, hs, generator=g, device=DEV).to(torch.bfloat16)
    table = torch.randperm(blocks + 5, generator=g, device=DEV)[:blocks].to(torch.int32).view(1, blocks)
    q = torch.randn(T, H * hs, generator=g, device=DEV).to(torch.bfloat16)
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    scale = 1.0 / math.sqrt(hs)
    rows = torch.tensor([0, 1, 15, 16, 127, 128, 129, 1000, 2046, 2047], device=DEV)
    want = torch.empty(len(rows), H * hs, dtype=torch.bfloat16, device=DEV)
    o.paged_attention_ref(q[rows], kc, vc, table, torch.zeros(len(rows), dtype=torch.int32, device=DEV),
                          rows.to(torch.int32), want, page_size, 1, H, KV, hs, scale, 0, status)
    for label, fn, tok in (("mma.sync", o.attn_portion, o.attn_portion_tokens(H, KV, hs)),
                           ("tcgen05", o.attn_portion_tc05, o.attn_portion_tc05_tokens(H, KV))):
        items = torch.tensor([(0, b, min(tok, T - b), b) for b in range(0, T, tok)], dtype=torch.int32, device=DEV)
        out = torch.full_like(q, float("nan"))
        run = lambda: fn(q, kc, vc, table, items, out, page_size, 1, H, KV, hs, scale, 0, status=status)
        run()
        assert status.item() == 0 and not torch.isnan(out).any()
        assert (out[rows].float() - want.float()).abs().max().item() <= 2 ** -8 * 4
        for r in rows.tolist():                            # and against torch alone
            ref = _torch_attention(q[r], kc, vc, table[0], r, H, KV, hs, scale)
            assert (out[r].float() - ref).abs().max().item() <= 2 ** -8 * 4, f"{label}: row {r} against torch"
        for _ in range(2):
            run()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        e0.record()
        for _ in range(10):
            run()
        e1.record()
        torch.cuda.synchronize()
        us = e0.elapsed_time(e1) * 100
        flops = 4.0 * H * hs * T * (T + 1) / 2
        print(f"attn_portion {label}: {us:.1f} us, {flops / us / 1e6:.0f} TFLOP/s (causal)")


def test_attention_portion_at_the_end_of_a_long_context():
    """The last 2,048 tokens of a 16,384-token prompt at the Llama-3.1-8B head layout (what a prompt cut into
    portions asks of the kernel): sampled rows against torch, and the time (printed). Nearly every key tile lies
    before the diagonal here, so the figure is the kernel's steady rate, without the causal edge."""
    o = ops()
    H, KV, hs, page_size, T, C = 32, 8, 128, 16, 2048, 16384
    if not o.attn_portion_tc05_ok(H, KV, hs, page_size):
        pytest.skip("the tcgen05 kernel does not take this layout")
    g = torch.Generator(device=DEV).manual_seed(61)
    blocks = C // page_size
    kc = torch.randn(blocks + 7, KV, page_size, hs, generator=g, device=DEV).to(torch.bfloat16)
    vc = torch.randn(blocks + 7, KV, page_size, hs, generator=g, device=DEV).to(torch.bfloat16)
    table = torch.randperm(blocks + 7, generator=g, device=DEV)[:blocks].to(torch.int32).view(1, blocks)
    q = torch.randn(T, H * hs, generator=g, device=DEV).to(torch.bfloat16)
    q[777] *= 6.0                                           # one row whose softmax is sharp: a far key must be found
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    scale = 1.0 / math.sqrt(hs)
    tok = o.attn_portion_tc05_tokens(H, KV)
    items = torch.tensor([(0, b, min(tok, T - b), C - T + b) for b in range(0, T, tok)], dtype=torch.int32, device=DEV)
    out = torch.full_like(q, float("nan"))
    run = lambda: o.attn_portion_tc05(q, kc, vc, table, items, out, page_size, 1, H, KV, hs, scale, 0, status=status)
    run()
    assert status.item() == 0 and not torch.isnan(out).any()
    for r in (0, 1, 63, 64, 777, 1024, 2046, 2047):
        ref = _torch_attention(q[r], kc, vc, table[0], C - T + r, H, KV, hs, scale)
        assert (out[r].float() - ref).abs().max().item() <= 2 ** -8 * 4, f"row {r} against torch"
    us = graph_time_us(lambda i: run(), n=5)
    flops = 4.0 * H * hs * sum(C - T + r + 1 for r in range(T))
    print(f"attn_portion tcgen05, 2,048 tokens ending at {C}: {us:.1f} us, {flops / us / 1e6:.0f} TFLOP/s")


# ---- random searches over sizes ---------------------------------------------------------------------------------

def _swiglu_of_interleaved(y, F):
    """silu(gate) * up of a product whose columns hold 8 gates, their 8 ups, 8 gates, ... (both rounded to bf16)."""
    y = y.to(torch.bfloat16).double().view(y.shape[0], F // 8, 2, 8)
    gate, up = y[:, :, 0], y[:, :, 1]
    return (gate / (1 + torch.exp(-gate)) * up).reshape(y.shape[0], F)


def test_matrix_products_at_random_sizes():
    """Every matrix-product kernel of the package (few rows, up to 128 rows, many rows; plain, with the gated
    activation, into the residual stream) at 400 random sizes and row strides against a float64 product."""
    import random
    o = ops()
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    for seed in range(400):
        rng = random.Random(seed)
        g = torch.Generator(device=DEV).manual_seed(seed)
        kind = rng.choice(["skinny", "skinny_swiglu", "tc05", "tc05", "tc05_swiglu", "tc05_add", "rows", "rows_swiglu"])
        K = 8 * rng.choice([1, 2, 5, 8, 12, 33, 64, 100, 167, 512, 1792])
        M = (rng.randint(1, 16) if kind.startswith("skinny") else rng.randint(1, 128) if kind.startswith("rows")
             else rng.choice([1, 17, 100, 127, 128, 129, 200, 255, 256, 257, 300, 511, 513, 700, 1025]))
        N = rng.choice([8, 16, 40, 96, 128, 136, 256, 264, 520, 1000, 1024, 2056, 4096 + 8 * rng.randint(0, 40)])
        if "swiglu" in kind:
            N = 2 * (N // 2 // 8 * 8 or 8)
        ldx, ldw = K + 8 * rng.choice([0, 0, 1, 3]), K + 8 * rng.choice([0, 0, 2])
        x = torch.randn(M, ldx, generator=g, device=DEV).to(torch.bfloat16)[:, :K]
        w = (torch.randn(N, ldw, generator=g, device=DEV) / K ** 0.5).to(torch.bfloat16)[:, :K]
        want = x.double() @ w.double().T
        what = f"seed {seed}: {kind}, {M} x {N} x {K}, row strides {ldx} and {ldw}"
        if kind in ("skinny", "tc05", "rows"):
            odt = rng.choice([torch.bfloat16, torch.float32])
            out = torch.full((M, N), float("nan"), dtype=odt, device=DEV)
            {"skinny": lambda: o.gemm_skinny(x, w, out), "tc05": lambda: o.gemm_tc05(x, w, out, status),
             "rows": lambda: o.gemm_rows(x, w, out, status)}[kind]()
            tol = 2 ** -8 * max(1.0, want.abs().max().item()) if odt == torch.bfloat16 else 1e-3
            err = (out.double() - want).abs().max().item()
        elif kind == "tc05_add":
            resid = torch.randn(M, N, generator=g, device=DEV)
            before = resid.clone()
            o.gemm_tc05_add(x, w, resid, status)
            err = (resid.double() - (before.double() + want.to(torch.bfloat16).double())).abs().max().item()
            tol = 2 ** -7 * max(1.0, want.abs().max().item())
        else:
            F = N // 2
            out = torch.full((M, F), float("nan"), dtype=torch.bfloat16, device=DEV)
            {"skinny_swiglu": lambda: o.gemm_skinny_swiglu(x, w, out), "tc05_swiglu": lambda: o.gemm_tc05_swiglu(x, w, out, status),
             "rows_swiglu": lambda: o.gemm_rows_swiglu(x, w, out, status)}[kind]()
            ref = _swiglu_of_interleaved(want, F)
            err = (out.double() - ref).abs().max().item()
            tol = 2 ** -6 * max(1.0, ref.abs().max().item())
        assert err <= tol and status.item() == 0, f"{what}: off by {err:.3e} (allowed {tol:.3e}), status {status.item()}"


def test_attention_kernels_at_random_layouts():
    """The tensor-core attention kernels at 250 random layouts (head sizes, heads, groups, page sizes, windows),
    lengths around the edges of pages and tiles, tails from one decode row to whole prompts, and numbers of
    splits, against the plain attention. Layouts that a kernel declines by contract are passed over."""
    import random
    ran = 0
    for seed in range(250):
        rng = random.Random(seed)
        hs = rng.choice([16, 32, 48, 64, 64, 64, 80, 96, 128, 128, 128, 256])
        KV, G = rng.choice([1, 2, 3, 8]), rng.choice([1, 2, 3, 4, 5, 8, 16, 32])
        if KV * G > 40:
            G = rng.choice([1, 2, 4])
        H, page = KV * G, rng.choice([4, 8, 16, 32, 64])
        window = rng.choice([None, None, 5, 64, 65, 130])
        S = rng.randint(1, 6)
        lengths = [rng.choice([1, 2, 15, 16, 17, 63, 64, 65, 127, 128, 129, 200, 333, 512, 640]) for _ in range(S)]
        tails = [rng.choice([1, 1, 1, 2, 3, 8, 40, 64, 128, 10 ** 6]) for _ in range(S)]
        mode = rng.choice(["cp_async", "tma", "tcgen05"])
        nsplit = 1 if mode == "tcgen05" else rng.choice([1, 1, 2, 3, 5, 8])
        what = (f"seed {seed}: {mode}, {H} heads, {KV} groups, head size {hs}, page {page}, window {window}, "
                f"lengths {lengths}, tails {tails}, {nsplit} splits")
        seqs, table, kc, vc = build_cache(torch.bfloat16, lengths, H, KV, hs, page, seed=seed)
        try:
            out, rows, _, _ = _run_tc_attention(seqs, table, kc, vc, lengths, tails, H, KV, hs, page, window, nsplit,
                                                mode != "cp_async", mode == "tcgen05")
        except pytest.skip.Exception:
            continue
        except ops().KernelError as e:
            assert "do not fit" in str(e) or "outside what the kernel supports" in str(e), f"{what}: {e}"
            continue
        ran += 1
        scale = 1.0 / math.sqrt(hs)
        full = [plain_llama.attention(q.double(), k.double(), v.double(), scale, window) for q, k, v in seqs]
        want = torch.stack([full[s][p].reshape(-1) for s, p in rows])
        vmax = max(v.abs().max().item() for _, _, v in seqs)
        assert not torch.isnan(out).any(), f"{what}: a row was not written"
        err = (out - want).abs().max().item()
        assert err <= 2 ** -8 * vmax, f"{what}: off by {err:.3e}"
    assert ran >= 100


def test_sampling_at_random_rows():
    """The sampling kernel against the plain sampler over 300 random batches: vocabularies from 2 to 4,099,
    temperatures, top-k from 1 to beyond the vocabulary, top-p down to 0.0001, ties, many equal logits (both
    zeros among them), rows half masked with -inf, flat rows."""
    import random
    for seed in range(300):
        rng = random.Random(seed)
        g = torch.Generator().manual_seed(seed)
        V, R = rng.choice([2, 3, 31, 32, 33, 130, 1000, 1024, 4099]), rng.randint(1, 9)
        scale = rng.choice([0.01, 1.0, 2.5, 30.0])
        logits = (scale * torch.randn(R, V, generator=g)).float()
        kind = rng.choice(["plain", "ties", "rounded", "masked", "flat"])
        if kind == "ties":
            for r in range(R):
                logits[r, torch.randint(0, V, (min(V, 5),), generator=g)] = logits[r].max() + rng.choice([0.0, 1.0])
        elif kind == "rounded":
            logits = (logits * 2).round() / 2
        elif kind == "masked":
            mask = torch.rand(R, V, generator=g) < 0.5
            mask[:, 0] = False
            logits[mask] = float("-inf")
        elif kind == "flat":
            logits[:] = 1.25
        temps = [rng.choice([0.0, 0.3, 0.7, 1.0, 1.5]) for _ in range(R)]
        ks = [rng.choice([0, 1, 2, 5, 50, V, V + 5]) for _ in range(R)]
        ps = [rng.choice([1.0, 0.99, 0.9, 0.5, 0.1, 0.0001]) for _ in range(R)]
        seeds, ctrs = [rng.randrange(2 ** 31) for _ in range(R)], [rng.randrange(1000) for _ in range(R)]
        out = torch.empty(R, dtype=torch.int32, device=DEV)
        ops().sample(logits.to(DEV), out, temperature=torch.tensor(temps, device=DEV),
                     top_k=torch.tensor(ks, dtype=torch.int32, device=DEV), top_p=torch.tensor(ps, device=DEV),
                     seed=torch.tensor(seeds, dtype=torch.int64, device=DEV), counter=torch.tensor(ctrs, dtype=torch.int64, device=DEV))
        want = [plain_llama.sample(logits[r], temps[r], ks[r], ps[r], seed=seeds[r], counter=ctrs[r]) for r in range(R)]
        got = out.tolist()
        for r in range(R):
            if got[r] == want[r]:
                continue
            # a draw that lands within rounding of a boundary between two kept tokens may fall either way (the
            # kernel sums in float32, the plain sampler in float64): both must then be kept tokens of equal
            # or neighbouring cumulative mass; anything else is a fault
            assert temps[r] > 0 and logits[r, got[r]] > float("-inf"), (
                f"seed {seed}, {kind}, row {r}: kernel {got[r]}, plain {want[r]} (T {temps[r]}, k {ks[r]}, p {ps[r]})")
            p = torch.softmax(logits[r].double() / temps[r], 0)
            lo, hi = sorted((got[r], want[r]))
            between = p[lo:hi + 1].sum().item() - max(p[lo].item(), p[hi].item())
            assert between <= 1e-5, (
                f"seed {seed}, {kind}, row {r}: kernel {got[r]}, plain {want[r]} with mass {between:.2e} between them")
