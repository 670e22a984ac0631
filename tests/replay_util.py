"""Builders of replay traces (the JSON records bin/trace_run reads) and the comparison of
replayed logits with the plain implementation."""
import random
from typing import Dict, List, Sequence

import torch

import plain_llama


def random_tokens(vocab: int, n: int, seed: int) -> List[int]:
    g = torch.Generator().manual_seed(seed)
    return torch.randint(0, vocab, (n,), generator=g).tolist()


def round64(n: int) -> int:
    return -(-n // 64) * 64


def trace_whole(reqs: Dict[str, List[int]]) -> List[dict]:
    """Each request alone and whole, every row wanted."""
    steps = []
    for i, (rid, toks) in enumerate(reqs.items()):
        steps.append({"step": i, "entries": [{"id": rid, "tokens": toks, "want": list(range(len(toks)))}],
                      "end": [rid]})
    return steps


def trace_tail(reqs: Dict[str, List[int]], tail: int = 32) -> List[dict]:
    """Most of a request in one step, its last ``tail`` tokens one by one."""
    steps = []
    for rid, toks in reqs.items():
        head = max(1, len(toks) - tail)
        steps.append({"step": len(steps), "entries": [{"id": rid, "tokens": toks[:head], "want": [head - 1]}], "end": []})
        for p in range(head, len(toks)):
            steps.append({"step": len(steps), "entries": [{"id": rid, "tokens": [toks[p]], "want": [0]}],
                          "end": [rid] if p == len(toks) - 1 else []})
        if head == len(toks):
            steps[-1]["end"] = [rid]
    return steps


def trace_portions(reqs: Dict[str, List[int]], sizes: Sequence[int] = (17, 5, 2, 31, 3, 64, 2, 9, 1, 40)) -> List[dict]:
    """Portions of changing size, down to two tokens (and one), every row wanted."""
    steps = []
    for rid, toks in reqs.items():
        p, i = 0, 0
        while p < len(toks):
            n = min(sizes[i % len(sizes)], len(toks) - p)
            i += 1
            steps.append({"step": len(steps),
                          "entries": [{"id": rid, "tokens": toks[p:p + n], "want": list(range(n))}],
                          "end": [rid] if p + n == len(toks) else []})
            p += n
    return steps


def trace_mixed(reqs: Dict[str, List[int]], max_tokens: int, seed: int = 0, max_live: int = 4,
                prompt_frac: float = 0.6, cut_every: int = 0, kept=None, max_cuts: int = 6) -> List[dict]:
    """Up to ``max_live`` live requests: portions of some prompts beside single "decoded" tokens
    of others; a request is admitted only when its whole length (rounded up to 64) still fits
    in ``max_tokens``, so pages of ended requests are used again by later ones. Some requests
    sit a step out. With ``cut_every`` = n, every n-th step first cuts one live request back to a
    random length as a preemption does (a "truncate" record; ``kept(held, keep)`` says how many tokens
    stay) and the trace computes the cut tokens again, in portions, beside the others; at most ``max_cuts`` cuts in
    all, so that the trace ends."""
    rng = random.Random(seed)
    waiting = list(reqs.items())
    live: Dict[str, dict] = {}
    steps: List[dict] = []
    held = 0
    cuts_left = max_cuts
    while waiting or live:
        while waiting and len(live) < max_live and held + round64(len(waiting[0][1])) <= max_tokens:
            rid, toks = waiting.pop(0)
            live[rid] = {"toks": toks, "pos": 0, "prompt": max(1, int(len(toks) * prompt_frac))}
            held += round64(len(toks))
        assert live, "max_tokens is too small for the next request"
        entries, end, cuts = [], [], []
        if cut_every and cuts_left > 0 and len(steps) % cut_every == cut_every - 1:
            cand = [r for r, st in live.items() if st["pos"] > 1]
            if cand:
                cuts_left -= 1
                rid = rng.choice(cand)
                st = live[rid]
                keep = rng.randrange(0, st["pos"])
                cuts.append({"id": rid, "keep": keep})
                # what was computed behind the cut is a prompt now: it comes again in portions
                st["prompt"] = max(st["prompt"], st["pos"])
                st["pos"] = kept(st["pos"], keep)
        for rid, st in list(live.items()):
            if len(live) > 1 and rng.random() < 0.2:
                continue                                   # left out of this step
            p, toks = st["pos"], st["toks"]
            if p < st["prompt"]:
                n = min(rng.choice([2, 3, 7, 16, 29, 50]), st["prompt"] - p)
                want = [n - 1] if rng.random() < 0.5 else list(range(n))
            else:
                n, want = 1, [0]
            entries.append({"id": rid, "tokens": toks[p:p + n], "want": want})
            st["pos"] = p + n
            if st["pos"] == len(toks):
                end.append(rid)
                held -= round64(len(toks))
                del live[rid]
        if entries or cuts:
            steps.append({"step": len(steps), "entries": entries, "end": end, **({"truncate": cuts} if cuts else {})})
    return steps


def replay_in_process(replayer, steps: List[dict]):
    """Yields (request id, position, logits row) for every wanted row."""
    pos: Dict[str, int] = {}
    for rec in steps:
        out = replayer.run_step(rec["entries"], rec["end"], rec.get("truncate", ()))
        for t in rec.get("truncate", ()):
            pos[t["id"]] = replayer.kept_after_truncate(pos[t["id"]], t["keep"])
        r = 0
        for e in rec["entries"]:
            base = pos.get(e["id"], 0)
            for w in e.get("want", ()):
                yield e["id"], base + w, out[r]
                r += 1
            pos[e["id"]] = base + len(e["tokens"])
        for rid in rec["end"]:
            pos.pop(rid, None)
        assert (out is None and r == 0) or out.shape[0] == r


class PlainLogits:
    """Whole-sequence logits of the plain implementation, computed once per request."""

    def __init__(self, model_dir: str):
        self.cfg, self.w = plain_llama.read_model_folder(model_dir)
        self._cache: Dict[tuple, torch.Tensor] = {}

    def of(self, tokens: Sequence[int]) -> torch.Tensor:
        key = tuple(tokens)
        if key not in self._cache:
            self._cache[key] = plain_llama.forward(self.cfg, self.w, tokens)
        return self._cache[key]


def compare(replayer, steps, reqs, plain: PlainLogits, atol: float, what: str) -> float:
    """Every wanted row against the plain logits of its request and position; returns the
    largest difference seen. Names the first wrong place."""
    worst = 0.0
    n = 0
    for rid, p, row in replay_in_process(replayer, steps):
        ref = plain.of(reqs[rid])[p]
        diff = (row.to(torch.float64) - ref).abs().max().item()
        assert diff == diff and diff <= atol, (
            f"{what}: request {rid!r} position {p}: logits differ from the plain implementation by "
            f"{diff:.3e} (allowed {atol:.1e})")
        worst = max(worst, diff)
        n += 1
    assert n > 0
    return worst
