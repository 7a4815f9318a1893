"""CPU oracle for tree verify + accept.  TEST INFRASTRUCTURE ONLY.

A restatement, on torch CPU tensors and plain Python loops, of the reference's
verification path.  Only tests/, __graft_entry__.smoke() and bench.py's CPU
baseline may import this module; the product (subspec_b200) never does.

Pinned against the reference: tests/golden/verify_*.json hold outputs of the
reference's own `verify_tree` / `lossy_bottom_up_verify` (run unmodified from a
read-only checkout by tests/golden/make_golden.py) on seeded inputs, and
tests/test_oracle_golden.py checks this restatement against them, together with
the eight hand-built cases of the reference's tests/test_lossy_tree_verify.py.

What follows what (reference file:line):
  target_probs          GeneratorBase._sample_token      generators/base.py:109-139
                        + HF Temperature/TopP warpers    transformers logits_process.py
  exact_walk            verify_tree, exact branch        models/utils/tree_verify.py:49-106
                        + _verify_step                   generators/classic_sd.py:111-116
  lossy_verify          lossy_bottom_up_verify           models/utils/lossy_tree_verify.py:9-291
  normalised_entropy    _compute_entropy_list            models/utils/lossy_tree_verify.py:66-72

Sampling: the reference draws with torch.multinomial from the global RNG, which
cannot be reproduced from a per-node uniform.  Here (and in the CUDA path) the
draw for node u is the inverse-CDF pick for an injected uniform u01[u]: the
first vocabulary index whose cumulative probability exceeds u01[u].  That mode is
pinned too: tests/golden/sampled_cases.json holds what the reference returned with
do_sample=True when its torch.multinomial was replaced by this pick (its warpers,
softmax, walk and lossy verifier untouched).  residual_walk has no counterpart in
the reference: parity unpinned for that function alone.
"""
from __future__ import annotations

import math
from dataclasses import dataclass, field
from typing import List, Optional, Sequence, Tuple

import torch


# ---------------------------------------------------------------------------------
# probabilities
# ---------------------------------------------------------------------------------
def top_p_filter(scores: torch.Tensor, top_p: float) -> torch.Tensor:
    """Nucleus filter as HF's TopPLogitsWarper (min_tokens_to_keep=1): sort ascending,
    drop entries whose cumulative softmax mass is <= 1 - top_p, always keep the largest.

    One deliberate difference: the sort here is STABLE.  transformers calls torch.sort
    without `stable=True`, and on CPU that sort leaves tied logits in an arbitrary order, so
    which of the tokens tied at the nucleus boundary get dropped is an accident of the sort
    implementation there.  Here (and in the CUDA path) the lowest vocabulary indices go first."""
    sorted_logits, sorted_idx = torch.sort(scores, descending=False, dim=-1, stable=True)
    cum = sorted_logits.softmax(dim=-1).cumsum(dim=-1)
    remove = cum <= (1 - top_p)
    remove[..., -1:] = False
    mask = remove.scatter(-1, sorted_idx, remove)
    return scores.masked_fill(mask, -float("inf"))


def top_k_filter(scores: torch.Tensor, top_k: int) -> torch.Tensor:
    """HF's TopKLogitsWarper: everything strictly below the k-th largest score goes (ties with it stay)."""
    k = min(int(top_k), scores.shape[-1])
    kth = torch.topk(scores, k, dim=-1).values[..., -1:]
    return scores.masked_fill(scores < kth, -float("inf"))


def target_probs(logits: torch.Tensor, do_sample: bool = False, temperature: float = 1.0,
                 top_p: float = 1.0, upcast: bool = False, top_k: int = 0) -> torch.Tensor:
    """[N, V] probabilities in the logits' dtype (or fp32 when `upcast`), as _sample_token returns them
    (generators/base.py:109-139 with the warpers of :42-64: temperature, top-k, top-p in that order)."""
    x = logits.float() if upcast else logits
    x = x.reshape(-1, x.shape[-1])
    if do_sample:
        if temperature != 1.0:
            x = x / temperature
        if top_k:
            x = top_k_filter(x, top_k)
        if top_p < 1.0:
            x = top_p_filter(x, top_p)
    return torch.softmax(x, dim=-1)


def normalised_entropy(probs: torch.Tensor) -> List[float]:
    v = int(probs.shape[1])
    denom = math.log(v) if v > 1 else 1.0
    return (torch.special.entr(probs).sum(dim=-1) / denom).tolist()


def inverse_cdf_pick(row: torch.Tensor, u01: float) -> int:
    """First index whose cumulative probability (fp64, vocabulary order) exceeds u01 * total."""
    cdf = row.double().cumsum(0)
    total = float(cdf[-1])
    i = int(torch.searchsorted(cdf, torch.tensor(u01 * total, dtype=torch.float64), right=True))
    nz = torch.nonzero(row > 0).reshape(-1)
    last = int(nz[-1]) if nz.numel() else 0
    return min(i, last)


def sampling_margins(logits: torch.Tensor, temperature: float, top_p: float, uniforms: Sequence[float],
                     top_k: int = 0):
    """Per row, how far the two discrete decisions of the sampler are from flipping (fp64):
    `boundary`: distance of the nucleus threshold from the nearest cumulative probability, in
    units of that token's probability; `pick`: distance of u from the nearest CDF edge, relative
    to the total.  Rows with tiny margins are decided by rounding, not by the algorithm."""
    x = logits.double().reshape(-1, logits.shape[-1]) / temperature
    if top_k:
        x = top_k_filter(x, top_k)
    out = []
    for u in range(x.shape[0]):
        sorted_logits, sorted_idx = torch.sort(x[u], descending=False, stable=True)
        p = sorted_logits.softmax(dim=-1)
        boundary = float("inf")
        keep = torch.ones_like(p, dtype=torch.bool)
        if top_p < 1.0:
            cum = p.cumsum(0)
            thr = float(torch.tensor(1.0 - top_p, dtype=torch.float32))
            j = int(torch.argmin((cum - thr).abs()))
            boundary = float((cum[j] - thr).abs() / p[j])
            remove = cum <= thr
            remove[-1] = False
            keep = ~remove
        q = torch.zeros_like(p)
        q[sorted_idx] = torch.where(keep, p, torch.zeros_like(p))
        cdf = q.cumsum(0)
        total = float(cdf[-1])
        pick = float(((cdf - float(uniforms[u]) * total).abs()).min() / total)
        out.append((boundary, pick))
    return out


def target_tokens(probs: torch.Tensor, do_sample: bool, uniforms: Optional[Sequence[float]]) -> List[int]:
    if not do_sample:
        return probs.argmax(dim=-1).tolist()
    return [inverse_cdf_pick(probs[u], float(uniforms[u])) for u in range(probs.shape[0])]


# ---------------------------------------------------------------------------------
# walks
# ---------------------------------------------------------------------------------
@dataclass
class VerifyResult:
    tokens: List[int]
    hidden: List[int]
    total_len: int
    accept_len: int
    target: List[int] = field(default_factory=list)
    entropy: List[float] = field(default_factory=list)
    exact_after: List[int] = field(default_factory=list)
    best_len: List[int] = field(default_factory=list)
    best_next: List[int] = field(default_factory=list)
    min_gate_margin: float = float("inf")


def exact_walk(*, target: Sequence[int], token_ids: Sequence[int], children: Sequence[Sequence[int]],
               root: int, n_rows: int, eos: Optional[int]) -> VerifyResult:
    """Greedy / sample-and-match walk (tree_verify.py:61-104).  Indices are local
    (node 0 = first decoded node); `children` lists are NOT cut to the decoded rows."""
    out_t: List[int] = []
    out_h: List[int] = []
    total = acc = 0
    cur = root
    bonus = None
    go = len(children[cur]) > 0
    while go:
        total += 1
        s = int(target[cur])
        match = next((c for c in children[cur] if int(token_ids[c]) == s), None)
        if match is None:
            bonus = s
            break
        acc += 1
        out_t.append(s)
        out_h.append(cur)
        if eos is not None and s == int(eos):
            break
        cur = match
        if not children[cur]:
            break
        if min(children[cur]) >= n_rows:
            break
    if not out_t or eos is None or out_t[-1] != int(eos):
        if bonus is None:
            bonus = int(target[cur])
        out_t.append(bonus)
        out_h.append(cur)
    return VerifyResult(out_t, out_h, total, acc, target=list(target))


def lossy_verify(*, probs: torch.Tensor, token_ids: Sequence[int], children: Sequence[Sequence[int]],
                 root: int, eos: Optional[int], threshold: float, window: int, use_entropy: bool,
                 target: Optional[Sequence[int]] = None, entropy: Optional[Sequence[float]] = None) -> VerifyResult:
    """Reverse-index DP + top-down walk (lossy_tree_verify.py:107-168, 247-291)."""
    n = int(probs.shape[0])
    tgt = list(target) if target is not None else probs.argmax(dim=-1).tolist()
    ent = list(entropy) if entropy is not None else (normalised_entropy(probs) if use_entropy else [0.0] * n)
    need = max(0, int(window))
    thr = float(threshold)
    ea = [0] * n
    bl = [0] * n
    bn = [-1] * n
    margin = float("inf")
    for u in range(n - 1, -1, -1):
        ch = children[u]
        if not ch:
            continue
        exact = [c for c in ch if int(token_ids[c]) == tgt[u]]
        if exact:
            ea[u] = 1 + max(ea[c] for c in exact)
        best_c, best_total, best_exact, best_p = -1, 0, False, -1.0
        for c in ch:
            tok = int(token_ids[c])
            is_exact = tok == tgt[u]
            p = -1.0
            if not is_exact:
                if ea[c] < need:
                    continue
                if use_entropy:
                    margin = min(margin, abs(float(ent[u]) - thr))
                    if float(ent[u]) >= thr:
                        continue
                p = float(probs[u, tok].item())
                if not use_entropy:
                    margin = min(margin, abs(p - thr))
                    if p < thr:
                        continue
            tl = 1 + bl[c]
            if tl > best_total:
                best_c, best_total, best_exact, best_p = c, tl, is_exact, p
            elif tl == best_total:
                if is_exact and not best_exact:
                    best_c, best_exact, best_p = c, True, p
                elif (not is_exact) and (not best_exact) and p > best_p:
                    best_c, best_p = c, p
        if best_c >= 0 and best_total > 0:
            bn[u], bl[u] = best_c, best_total
    out_t: List[int] = []
    out_h: List[int] = []
    ctx, acc = root, 0
    while True:
        nxt = bn[ctx]
        if nxt < 0:
            break
        tok = int(token_ids[nxt])
        out_t.append(tok)
        out_h.append(ctx)
        acc += 1
        if eos is not None and tok == int(eos):
            break
        ctx = nxt
    if not out_t or eos is None or out_t[-1] != int(eos):
        out_t.append(int(tgt[ctx]))
        out_h.append(ctx)
    return VerifyResult(out_t, out_h, len(out_t), acc, target=tgt, entropy=ent, exact_after=ea, best_len=bl,
                        best_next=bn, min_gate_margin=margin)


def children_from_parents(parents: Sequence[int]) -> List[List[int]]:
    ch: List[List[int]] = [[] for _ in parents]
    for i, p in enumerate(parents):
        if p >= 0:
            ch[p].append(i)
    return ch


def verify(*, logits: torch.Tensor, token_ids: Sequence[int], children: Sequence[Sequence[int]], root: int = 0,
           eos: Optional[int] = None, method: str = "exact", do_sample: bool = False, temperature: float = 1.0,
           top_p: float = 1.0, uniforms: Optional[Sequence[float]] = None, threshold: float = 0.0,
           window: int = 1, threshold_method: str = "prob", upcast: bool = False,
           input_is_probs: bool = False, top_k: int = 0) -> VerifyResult:
    """One sequence, local indexing, every node decoded (n_rows = len(token_ids) = logits.shape[0])."""
    probs = logits if input_is_probs else target_probs(logits, do_sample, temperature, top_p, upcast, top_k)
    n = int(probs.shape[0])
    tgt = target_tokens(probs, do_sample, uniforms)
    if method == "exact":
        return exact_walk(target=tgt, token_ids=token_ids, children=children, root=root, n_rows=n, eos=eos)
    return lossy_verify(probs=probs, token_ids=token_ids, children=[[c for c in ch if c < n] for ch in children[:n]],
                        root=root, eos=eos, threshold=threshold, window=window,
                        use_entropy=threshold_method == "entropy", target=tgt)


def residual_walk(*, logits: torch.Tensor, draft_logits: torch.Tensor, token_ids: Sequence[int],
                  children: Sequence[Sequence[int]], accept_uniforms: Sequence[float], uniforms: Sequence[float],
                  root: int = 0, eos: Optional[int] = None, temperature: float = 1.0, top_p: float = 1.0,
                  top_k: int = 0, draft_temperature: float = 1.0, trace: Optional[dict] = None):
    """Residual (p - q) acceptance over the tree, fp64.  NOT in the reference (which samples and matches,
    classic_sd.py:111-116): this is the restatement of the rule the kernel's header states.  Returns
    (VerifyResult, margin) where margin is the smallest distance of an accept test's uniform from its
    threshold or of a draw's uniform from a CDF edge.  `trace`, when given, counts the branches taken:
    "accept_after_reject" (a child accepted from a distribution that already had q subtracted) and
    "residual_bonus" (a bonus token drawn from such a distribution)."""
    n = int(logits.shape[0])
    if trace is not None:
        trace.setdefault("accept_after_reject", 0)
        trace.setdefault("residual_bonus", 0)
    p_all = target_probs(logits, True, temperature, top_p, upcast=True, top_k=top_k).double()
    q_all = torch.softmax(draft_logits.double() / draft_temperature, dim=-1)
    toks, hidden = [], []
    acc = total = 0
    margin = float("inf")
    cur = root

    def draw(dist: torch.Tensor, ctx: int) -> int:
        nonlocal margin
        cdf = dist.cumsum(0)
        tot = float(cdf[-1])
        margin = min(margin, float(((cdf - float(uniforms[ctx]) * tot).abs()).min() / tot) * 1e2)
        return inverse_cdf_pick(dist, float(uniforms[ctx]))

    go = len(children[cur]) > 0
    if not go:
        toks.append(draw(p_all[cur], cur))
        hidden.append(cur)
    while go:
        ch = list(children[cur])
        total += 1
        pr, qr = p_all[cur].clone(), q_all[cur]
        live = True
        rejected = False
        got = None
        for c in ch:
            x = int(token_ids[c])
            ratio = 0.0
            if live:
                px, qx = float(pr[x]), float(qr[x])
                ratio = px / qx if qx > 0 else (float("inf") if px > 0 else 0.0)
            thr = min(1.0, ratio)
            margin = min(margin, abs(float(accept_uniforms[c]) - thr))
            if float(accept_uniforms[c]) < thr:
                got = c
                break
            rejected = True
            if live:
                pr = torch.clamp(pr - qr, min=0)
                z = float(pr.sum())
                if z > 0:
                    pr = pr / z
                else:
                    live = False
        if trace is not None:
            trace["accept_after_reject"] += int(got is not None and rejected and live)
            trace["residual_bonus"] += int(got is None and rejected and live)
        if got is None:
            toks.append(draw(pr if (rejected and live) else p_all[cur], cur))
            hidden.append(cur)
            break
        x = int(token_ids[got])
        toks.append(x)
        hidden.append(cur)
        acc += 1
        if eos is not None and x == eos:
            break
        cur = got
        if not children[cur] or min(children[cur]) >= n:  # a leaf, or an undecoded level: a fresh draw there
            toks.append(draw(p_all[cur], cur))
            hidden.append(cur)
            break
    return VerifyResult(tokens=toks, hidden=hidden, total_len=total, accept_len=acc), margin


def top2_logit_gap(logits: torch.Tensor) -> float:
    """Smallest gap between the two largest logits over all rows (argmax flip margin)."""
    top = torch.topk(logits.float(), 2, dim=-1).values
    return float((top[:, 0] - top[:, 1]).min())
