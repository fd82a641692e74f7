"""Lufatar on the GPU against the plain float64 oracle (oracle/lufatar_oracle.py): every mechanism's
kernel alone, then whole models (own small configurations, random weights) under every way the engine
can be driven: whole prompts, token-by-token decoding, portions down to two tokens, mixed batches of
unequal requests, pages and slots that are freed and reused, long decoding, greedy generation through
the scheduler, the command line and the trace runner."""
import json
import math
import os
import subprocess
import sys
from pathlib import Path

import pytest
import torch

from oracle import lufatar_oracle as O

pytestmark = pytest.mark.gpu
BF, F32, F64 = torch.bfloat16, torch.float32, torch.float64
ROOT = Path(__file__).resolve().parent.parent


def _ops():
    from vila_b200 import ops
    return ops


def rel(a, b):
    a, b = a.double().cpu(), b.double().cpu()
    return float((a - b).abs().max() / b.abs().max().clamp_min(1e-30))


def tol(dtype):
    return 2e-5 if dtype == F32 else 5e-2   # max abs error over the largest expected entry


def rnd(*shape, seed=0, scale=1.0):
    return torch.randn(*shape, generator=torch.Generator().manual_seed(seed), dtype=F64) * scale


# ------------------------------------------------------------------------------------------------
# configurations (none of them a size combination of a published or given model)
# ------------------------------------------------------------------------------------------------
def att(heads, kv_heads, dim, vdim, rot_dims, base, scale):
    return {"type": "attention", "mixer": dict(heads=heads, kv_heads=kv_heads, dim=dim, vdim=vdim,
                                               rot={"base": base, "dims": rot_dims}, scale=scale)}


def moe(experts, top, ff, limit, count=1, keep=1):
    return {"kind": "moe", "expert": {"ff": ff, "limit": limit},
            "router": {"experts": experts, "top": top, "groups": {"count": count, "keep": keep}}}


def config(width, vocab, layers, *, groups, taps, bigram, mult, side=None, loop=None, eps=1e-5):
    d = {"architecture": "Lufatar", "canon": {"taps": taps},
         "embedding": {"bigram": dict(zip(("buckets", "mul_prev", "mul_cur"), bigram))},
         "layers": [dict(l, mlp=m) for l, m in layers], "norm": {"eps": eps, "groups": groups},
         "residual_mult": mult, "vocab": vocab, "width": width}
    if side:
        d["token_side"] = {"dim": side}
    if loop:
        d["loop"] = dict(zip(("start", "stop", "times"), loop))
    return d


CONFIGS = {
    # nothing is a multiple of 8 where it need not be; three norm pieces; full multi-head, one shared
    # key/value head and a pair; rotation of a part, of the whole head and none; a layer without
    # feed-forward; groups of one expert; the middle two layers run three times
    "odd": config(72, 97, [
        (att(3, 3, 12, 20, 8, 100.0, 0.4), moe(6, 2, 20, 0.8, count=3, keep=2)),
        (att(4, 1, 10, 6, 10, 10000.0, 0.3), None),
        (att(2, 2, 16, 16, 0, 10.0, 0.25), moe(4, 1, 24, 2.0, count=4, keep=2)),
        (att(6, 2, 6, 10, 4, 50.0, 0.5), moe(5, 5, 12, 1.5)),
    ], groups=3, taps=3, bigram=(53, 31, 5), mult=0.6, side=10, loop=(1, 3, 3), eps=1e-6),
    # sizes the tensor-core GEMM takes; one norm piece; no repeated block
    "aligned": config(128, 256, [
        (att(8, 2, 32, 32, 16, 500000.0, 0.17), moe(8, 2, 64, 1.0, count=4, keep=2)),
        (att(4, 4, 32, 64, 32, 10000.0, 0.2), moe(8, 4, 32, 3.0)),
    ], groups=1, taps=4, bigram=(509, 1000003, 7919), mult=0.8, side=16),
    # the optional parts left out: one tap (no convolution state), no side input, no loop; a single
    # layer repeated twice is "plain2"
    "plain": config(40, 61, [
        (att(2, 1, 8, 8, 8, 100.0, 0.35), moe(3, 1, 16, 5.0)),
        (att(1, 1, 24, 12, 12, 1000.0, 0.2), None),
    ], groups=1, taps=1, bigram=(7, 3, 2), mult=1.0),
    # a width that is no multiple of 4 (no 16-byte rows anywhere), two taps, pieces of 14 channels
    "narrow": config(42, 35, [
        (att(3, 1, 14, 9, 6, 300.0, 0.3), moe(6, 3, 10, 0.5, count=2, keep=2)),
        (att(2, 2, 5, 7, 4, 20.0, 0.45), moe(2, 1, 6, 1.0, count=2, keep=1)),
    ], groups=3, taps=2, bigram=(19, 23, 29), mult=0.9, side=7, loop=(1, 2, 2)),
    "plain2": config(48, 50, [
        (att(2, 2, 12, 12, 6, 100.0, 0.3), moe(4, 2, 8, 1.0, count=2, keep=1)),
    ], groups=2, taps=6, bigram=(11, 13, 17), mult=0.5, side=4, loop=(0, 1, 2)),
}


def build(name, dtype, seed=0):
    """name: a key of CONFIGS or a configuration dictionary"""
    if name == "narrow" and dtype == BF:
        # heads of 5 columns and a side input of 7: when such a short vector is nearly zero, its unit norm
        # multiplies the bf16 rounding of the projection before it, and single rows leave the tolerance
        # (seen in about one row of 150 per model).  The narrow sizes run in fp32; bf16 on widths that are no
        # multiple of 8 is covered by "odd" and by the kernels' own tests.
        pytest.skip("the narrow model is compared in fp32 only")
    from vila_b200.model import LufatarConfig, LufatarForCausalLM
    cfg = CONFIGS[name] if isinstance(name, str) else name
    model = LufatarForCausalLM(LufatarConfig.from_dict(cfg), "cuda", dtype).init_random(seed, scale=1.5)
    if dtype == BF:
        # Two choice values closer than the bf16 noise of the router's input would pick another expert
        # than the float64 oracle.  The bf16 models get decisive corrections (2 apart) and a small input
        # term: the chosen set is then nearly fixed per layer while the weights still vary per token.
        # Routing that changes from token to token is covered by the fp32 models and test_moe_route_sigmoid.
        t = model.state_dict()
        g = torch.Generator().manual_seed(seed + 100)
        for n in list(t):
            if n.endswith("mlp.router"):
                t[n] = (t[n].float() * 0.25).to(BF)
            elif n.endswith("mlp.correction"):
                t[n] = (torch.randperm(t[n].numel(), generator=g).float() * 2.0).to(BF)
        model.load_weights(t)
    return cfg, model


def tokens_for(cfg, n, seed):
    g = torch.Generator().manual_seed(seed)
    return torch.randint(0, cfg["vocab"], (n,), generator=g).tolist()


def run_schedule(model, prompts, schedule, max_tokens, slots=4):
    """schedule: steps of [(name, rows)]; the logits of every row are collected per request; a request
    is released with its last row.  -> {name: [len, vocab] fp32 on the CPU}"""
    from vila_b200.serving import TokenEngine
    eng = TokenEngine(model, max_tokens=max_tokens, slots=slots)
    at = {k: 0 for k in prompts}
    got = {k: [] for k in prompts}
    for step in schedule:
        entries = []
        for name, n in step:
            entries.append((name, prompts[name][at[name]:at[name] + n], list(range(n))))
            at[name] += n
        lg = eng.step(entries).cpu()
        o = 0
        for name, n in step:
            got[name].append(lg[o:o + n])
            o += n
            if at[name] == len(prompts[name]):
                eng.release(name)
    assert not eng.seqs and eng.cache.allocator.available == eng.cache.n_pages
    return {k: torch.cat(v) for k, v in got.items()}


def rows_close(got, want, dtype, what=""):
    """every row within tolerance (relative to the largest entry of the expected tensor)"""
    got, want = got.double().cpu(), want.double().cpu()
    assert bool(torch.isfinite(got).all()), what
    err = (got - want).abs().amax(-1) / want.abs().max()
    bad = int((err >= tol(dtype)).sum())
    assert bad == 0, (what, bad, err.numel(), float(err.max()))


def check_logits(cfg, model, prompts, got, dtype):
    for name, toks in prompts.items():
        want = O.forward(cfg, model.state_dict(), toks)[0]
        assert got[name].shape == want.shape
        rows_close(got[name], want, dtype, name)


# ------------------------------------------------------------------------------------------------
# mechanisms alone
# ------------------------------------------------------------------------------------------------
@pytest.mark.parametrize("dtype", [F32, BF])
@pytest.mark.parametrize("rows,cols,groups", [(1, 7, 1), (37, 96, 3), (9, 2100, 2), (300, 1030, 1), (5, 12, 12)])
def test_group_rmsnorm_rows(cuda, dtype, rows, cols, groups):
    ops = _ops()
    x, w = rnd(rows, cols, seed=1, scale=3.0).to(dtype), (1 + rnd(cols, seed=2, scale=0.2)).to(dtype)
    got = ops.rmsnorm_rows(x.cuda(), w.cuda(), 1e-5, groups=groups, out_dtype=F32)
    want = O.group_norm(x.double(), w.double(), groups, 1e-5)
    assert rel(got, want) < 1e-5
    # a piece's root mean square is its own: scaling one piece leaves the others alone
    if groups > 1:
        x2 = x.clone()
        x2[:, :cols // groups] *= 8
        got2 = ops.rmsnorm_rows(x2.cuda(), w.cuda(), 1e-5, groups=groups, out_dtype=F32)
        assert torch.equal(got2[:, cols // groups:], got[:, cols // groups:])


def test_embed_pair_rows(cuda):
    ops = _ops()
    vocab, width, buckets = 90, 24, 37
    table, pair = rnd(vocab, width, seed=1).to(BF), rnd(buckets + 1, width, seed=2).to(BF)
    ids = torch.tensor([5, 89, 0, 17, 17, 3], dtype=torch.int32)
    prev = torch.tensor([-1, 5, 89, -1, 17, 88], dtype=torch.int32)
    for mp, mc in ((31, 5), (2 ** 31 - 1, 2 ** 20 + 7)):          # products beyond 32 bits
        got = ops.embed_pair_rows(table.cuda(), pair.cuda(), ids.cuda(), prev.cuda(), mp, mc, buckets)
        rows = [buckets if p < 0 else (int(p) * mp + int(i) * mc) % buckets for i, p in zip(ids, prev)]
        want = table.double()[ids.long()] + pair.double()[rows]
        assert rel(got, want) < 1e-6
    # the oracle on one sequence: only the first token reads the last row
    W = {"embed": table.double(), "bigram": pair.double()}
    toks = [5, 89, 0, 17]
    prev = torch.tensor([-1, 5, 89, 0], dtype=torch.int32)
    got = ops.embed_pair_rows(table.cuda(), pair.cuda(), torch.tensor(toks, dtype=torch.int32).cuda(), prev.cuda(), 31, 5, buckets)
    assert rel(got, O.token_embedding(W, toks, {"buckets": buckets, "mul_prev": 31, "mul_cur": 5})) < 1e-6


@pytest.mark.parametrize("taps", [1, 2, 4, 7])
def test_short_conv_in_portions_through_reused_slots(cuda, taps):
    """Two sequences fed in portions of 1, 2, ... rows (shorter and longer than the taps reach) next to
    each other, in slots whose state is stale from an earlier sequence, against the whole-sequence sum."""
    ops = _ops()
    C, slots = 40, 3
    w = rnd(C, taps, seed=3, scale=0.5)
    seqs = {"a": rnd(23, C, seed=4), "b": rnd(31, C, seed=5)}
    want = {k: O.short_conv_residual(v, w) for k, v in seqs.items()}
    state = torch.full((slots, max(taps - 1, 1), C), 77.0, device="cuda")[:, :taps - 1].contiguous()  # stale garbage
    slot = {"a": 2, "b": 0}
    cuts = {"a": [1, 2, 1, 5, 1, 1, 3, 9], "b": [2, 2, 7, 1, 1, 1, 17]}
    at = {"a": 0, "b": 0}
    got = {"a": [], "b": []}
    for step in range(8):
        rows, sq, rseq, names = [], [], [], []
        for name in ("b", "a"):
            if step < len(cuts[name]):
                n = cuts[name][step]
                sq.append((sum(r.shape[0] for r in rows), n, at[name], slot[name]))
                rseq += [len(sq) - 1] * n
                rows.append(seqs[name][at[name]:at[name] + n])
                names.append((name, n))
                at[name] += n
        h = torch.cat(rows).float().cuda()
        out = ops.short_conv_rows(h, w.float().cuda(), state if taps > 1 else None,
                                  torch.tensor(sq, dtype=torch.int32).cuda(), torch.tensor(rseq, dtype=torch.int32).cuda())
        o = 0
        for name, n in names:
            got[name].append(out[o:o + n].cpu())
            o += n
    for name in seqs:
        assert rel(torch.cat(got[name]), want[name]) < 1e-5, name


@pytest.mark.parametrize("dtype", [F32, BF])
@pytest.mark.parametrize("taps,groups,nsub", [(1, 1, 2), (3, 3, 1), (4, 2, 2), (6, 1, 2)])
def test_fused_norm_and_short_conv_in_portions(cuda, dtype, taps, groups, nsub):
    """group norm + convolution of one or two sublayers in one pass, two sequences in portions of 1, 2, ...
    rows through stale slots, against norm-then-convolution over the whole sequence"""
    ops = _ops()
    C, slots = 48, 3
    nw = [1 + rnd(C, seed=10 + k, scale=0.2) for k in range(nsub)]
    cw = [rnd(C, taps, seed=20 + k, scale=0.5).to(dtype) for k in range(nsub)]
    seqs = {"a": rnd(23, C, seed=4, scale=3.0).float(), "b": rnd(31, C, seed=5, scale=0.2).float()}
    want = {n: [O.short_conv_residual(O.group_norm(v.double(), nw[k], groups, 1e-5), cw[k].double()) for k in range(nsub)]
            for n, v in seqs.items()}
    state = [torch.full((slots, max(taps - 1, 1), C), 55.0, device="cuda")[:, :taps - 1].contiguous() for _ in range(nsub)]
    slot = {"a": 1, "b": 2}
    cuts = {"a": [1, 2, 1, 5, 1, 1, 3, 9], "b": [2, 2, 7, 1, 1, 1, 17]}
    at = {"a": 0, "b": 0}
    got = {n: [[] for _ in range(nsub)] for n in seqs}
    for step in range(8):
        rows, sq, rseq, names = [], [], [], []
        for name in ("a", "b"):
            if step < len(cuts[name]):
                n = cuts[name][step]
                sq.append((sum(r.shape[0] for r in rows), n, at[name], slot[name]))
                rseq += [len(sq) - 1] * n
                rows.append(seqs[name][at[name]:at[name] + n])
                names.append((name, n))
                at[name] += n
        outs = ops.norm_conv_rows(torch.cat(rows).cuda(), [w.float().cuda() for w in nw], [w.cuda() for w in cw],
                                  state if taps > 1 else [None] * nsub, torch.tensor(sq, dtype=torch.int32).cuda(),
                                  torch.tensor(rseq, dtype=torch.int32).cuda(), groups=groups, eps=1e-5, out_dtype=F32)
        o = 0
        for name, n in names:
            for k in range(nsub):
                got[name][k].append(outs[k][o:o + n].cpu())
            o += n
    for name in seqs:
        for k in range(nsub):
            assert rel(torch.cat(got[name][k]), want[name][k]) < 1e-5, (name, k)


def test_fused_norm_conv_many_rows(cuda):
    """steps of more than 256 rows take the streaming form (statistics kernel + channel-slice CTAs): two
    sequences whose portions start inside the other's row blocks, states carried from step to step"""
    ops = _ops()
    C, taps, groups = 1040, 4, 2            # two channel slices, the second one partly empty
    nw = [1 + rnd(C, seed=10 + k, scale=0.2) for k in range(2)]
    cw = [rnd(C, taps, seed=20 + k, scale=0.5).float() for k in range(2)]
    seqs = {"a": rnd(300, C, seed=4, scale=3.0).float(), "b": rnd(295, C, seed=5, scale=0.2).float()}
    want = {n: [O.short_conv_residual(O.group_norm(v.double(), nw[k], groups, 1e-5), cw[k].double()) for k in range(2)]
            for n, v in seqs.items()}
    state = [torch.full((2, taps - 1, C), 55.0, device="cuda") for _ in range(2)]
    got = {n: [[], []] for n in seqs}
    at = {"a": 0, "b": 0}
    for step in ([("a", 270), ("b", 5)], [("b", 290), ("a", 30)]):
        rows, sq, rseq = [], [], []
        for name, n in step:
            sq.append((sum(r.shape[0] for r in rows), n, at[name], 0 if name == "a" else 1))
            rseq += [len(sq) - 1] * n
            rows.append(seqs[name][at[name]:at[name] + n])
            at[name] += n
        outs = ops.norm_conv_rows(torch.cat(rows).cuda(), [w.float().cuda() for w in nw], [w.cuda() for w in cw], state,
                                  torch.tensor(sq, dtype=torch.int32).cuda(), torch.tensor(rseq, dtype=torch.int32).cuda(),
                                  groups=groups, eps=1e-5, out_dtype=F32)
        o = 0
        for name, n in step:
            for k in range(2):
                got[name][k].append(outs[k][o:o + n].cpu())
            o += n
    for name in seqs:
        for k in range(2):
            assert rel(torch.cat(got[name][k]), want[name][k]) < 1e-5, (name, k)


@pytest.mark.parametrize("dtype", [F32, BF])
@pytest.mark.parametrize("H,G,dim,vdim,rot", [(3, 3, 12, 20, 8), (4, 1, 10, 6, 10), (2, 2, 16, 16, 0), (10, 2, 64, 32, 32)])
def test_rope_append(cuda, dtype, H, G, dim, vdim, rot):
    """positions near 0, at a page border and very far (the phase of a far position needs more than fp32
    for position x frequency); q comes back rotated and unit-normed, k | v land in the named pool rows"""
    ops = _ops()
    pos = [0, 1, 63, 64, 65, 1000, 123457]
    T = len(pos)
    qkv = rnd(T, H * dim + G * (dim + vdim), seed=6, scale=2.0).to(dtype)
    rows = torch.tensor([9, 3, 70, 0, 33, 12, 5], dtype=torch.int32)
    pool = torch.zeros(80, G * (dim + vdim), dtype=dtype, device="cuda")
    inv = (torch.tensor(1000.0, dtype=F64) ** (-2.0 * torch.arange(rot // 2, dtype=F64) / rot)).cuda() if rot else None
    q = ops.rope_append(qkv.cuda(), torch.tensor(pos, dtype=torch.int32).cuda(), rows.cuda(), pool, heads=H,
                        kv_heads=G, dim=dim, vdim=vdim, inv_freq=inv, unit_norm=True, eps=1e-6)

    def turned(v, heads):
        """token t is rotated by its own position, then every head is unit-normed"""
        v = v.view(T, heads, dim).clone()
        if rot:
            i = torch.arange(rot // 2, dtype=F64)
            ang = torch.tensor(pos, dtype=F64)[:, None, None] * (1000.0 ** (-2.0 * i / rot))[None, None, :]
            a_, b_ = v[..., 0:rot:2].clone(), v[..., 1:rot:2].clone()
            v[..., 0:rot:2] = a_ * torch.cos(ang) - b_ * torch.sin(ang)
            v[..., 1:rot:2] = b_ * torch.cos(ang) + a_ * torch.sin(ang)
        return O.unit(v, 1e-6)

    x = qkv.double()
    want_q = turned(x[:, :H * dim], H).reshape(T, H * dim)
    want_k = turned(x[:, H * dim:(H + G) * dim], G).reshape(T, G * dim)
    t = 1e-5 if dtype == F32 else 1e-2
    assert rel(q, want_q) < 1e-5
    got = pool.cpu()[rows.long()]
    assert rel(got[:, :G * dim], want_k) < t
    assert torch.equal(got[:, G * dim:], qkv[:, (H + G) * dim:])
    untouched = torch.ones(80, dtype=torch.bool)
    untouched[rows.long()] = False
    assert float(pool.cpu()[untouched].abs().max()) == 0.0


def test_rotation_matches_the_oracle_on_a_sequence(cuda):
    ops = _ops()
    T, H, dim = 50, 2, 12
    v = rnd(T, H * dim + 1 * (dim + 4), seed=7)
    pool = torch.zeros(64, dim + 4, dtype=F32, device="cuda")
    inv = (torch.tensor(77.0, dtype=F64) ** (-2.0 * torch.arange(3, dtype=F64) / 6)).cuda()
    ar = torch.arange(T, dtype=torch.int32).cuda()
    q = ops.rope_append(v.float().cuda(), ar, ar, pool, heads=H, kv_heads=1, dim=dim, vdim=4, inv_freq=inv,
                        unit_norm=True, eps=1e-5)
    want = O.unit(O.rotate_pairs(v[:, :H * dim].view(T, H, dim), 77.0, 6), 1e-5).reshape(T, -1)
    assert rel(q, want) < 1e-5


def attend_direct(q, K, V, talk, sink, scale, pos0):
    """q [n, H, dk] at positions pos0.., K [N, G, dk], V [N, G, dv] (N >= pos0 + n) -> [n, H * dv], float64"""
    n, H, _ = q.shape
    G = K.shape[1]
    own = torch.arange(H) // (H // G)
    s = torch.einsum("ihd,jhd->hij", q, K[:, own]) * scale
    if talk is not None:
        s = torch.einsum("hg,gij->hij", talk, s)
    j = torch.arange(K.shape[0])[None, :]
    i = torch.arange(n)[:, None] + pos0
    s = s.masked_fill((j > i)[None], -math.inf)
    m = s.max(-1, keepdim=True).values
    if sink is not None:
        m = torch.maximum(m, sink[:, None, None])
    e = torch.exp(s - m)
    den = e.sum(-1, keepdim=True) + (torch.exp(sink[:, None, None] - m) if sink is not None else 0.0)
    return torch.einsum("hij,jhd->ihd", e / den, V[:, own]).reshape(n, -1)


def make_pool(seq_kv, page, n_pages, dtype, seed=0):
    """seq_kv: per slot (K [N, G, dk], V [N, G, dv]); pages are handed out in a shuffled order"""
    order = torch.randperm(n_pages, generator=torch.Generator().manual_seed(seed)).tolist()
    width = seq_kv[0][0][0].numel() + seq_kv[0][1][0].numel()
    pool = torch.full((n_pages * page, width), 9.0, dtype=dtype)          # unowned rows hold garbage
    tables = torch.zeros(len(seq_kv), n_pages, dtype=torch.int32)
    for s, (K, V) in enumerate(seq_kv):
        for j in range(K.shape[0]):
            if j % page == 0:
                tables[s, j // page] = order.pop()
            pool[int(tables[s, j // page]) * page + j % page] = torch.cat([K[j].reshape(-1), V[j].reshape(-1)]).to(dtype)
    return pool.cuda(), tables.cuda()


@pytest.mark.parametrize("dtype", [F32, BF])
@pytest.mark.parametrize("H,G,dk,dv", [(3, 3, 12, 20), (4, 1, 10, 6), (6, 2, 6, 10), (16, 4, 64, 64), (1, 1, 130, 5), (40, 8, 16, 24),
                                         (8, 2, 128, 128), (32, 8, 128, 128)])
def test_paged_attention(cuda, dtype, H, G, dk, dv):
    """Two sequences in one launch; portions that start and end inside pages; single decoded rows with the
    keys split over 1, 3 and 16 CTAs; with and without head mixing and sink."""
    ops = _ops()
    page, lens = 16, (75, 40)
    kv = [(rnd(n, G, dk, seed=10 + s).to(dtype), rnd(n, G, dv, seed=20 + s).to(dtype)) for s, n in enumerate(lens)]
    pool, tables = make_pool(kv, page, 9, dtype)
    talk = (torch.eye(H, dtype=F64) + rnd(H, H, seed=30, scale=0.3))
    sink = rnd(H, seed=31)
    # rows: seq 0 positions 30..74 (45 rows: tiles of 16, 16, 13), seq 1 positions 37..39, seq 1... no: one portion per sequence
    portions = [(0, 30, 45), (1, 37, 3)]
    qs = [rnd(n, H, dk, seed=40 + s) for s, _, n in portions]
    q = torch.cat([x.reshape(x.shape[0], -1) for x in qs]).float().cuda()
    tiles, at = [], 0
    for s, p0, n in portions:
        for o in range(0, n, 16):
            tiles.append((at + o, min(16, n - o), p0 + o, s))
        at += n
    tiles = torch.tensor(tiles, dtype=torch.int32).cuda()
    for tk, sk in ((talk, sink), (None, None), (talk, torch.zeros(H, dtype=F64))):
        got = ops.paged_attention(q, pool, tables, tiles, heads=H, kv_heads=G, dim=dk, vdim=dv, page=page, scale=0.3,
                                  talk=None if tk is None else tk.float().cuda(),
                                  sink=None if sk is None else sk.float().cuda(), out_dtype=F32)
        want = torch.cat([attend_direct(qs[k], kv[s][0].double()[:p0 + n], kv[s][1].double()[:p0 + n], tk, sk, 0.3, p0)
                          for k, (s, p0, n) in enumerate(portions)])
        assert rel(got, want) < (1e-5 if dtype == F32 else 2e-2), (tk is None, sk is None)
    # decoded rows: the last position of each sequence (and position 0 of a fresh one in slot 1's pages)
    dec = [(0, 74), (1, 39), (1, 0)]
    qd = rnd(3, H, dk, seed=50)
    dt = torch.tensor([(r, 1, p, s) for r, (s, p) in enumerate(dec)], dtype=torch.int32).cuda()
    want = torch.cat([attend_direct(qd[r:r + 1], kv[s][0].double()[:p + 1], kv[s][1].double()[:p + 1], talk, sink, 0.3, p)
                      for r, (s, p) in enumerate(dec)])
    for nsplit in (1, 3, 16):
        got = ops.paged_attention(qd.reshape(3, -1).float().cuda(), pool, tables, dt, heads=H, kv_heads=G, dim=dk,
                                  vdim=dv, page=page, scale=0.3, talk=talk.float().cuda(), sink=sink.float().cuda(),
                                  out_dtype=F32, max_rows=1, nsplit=nsplit)
        assert rel(got, want) < (1e-5 if dtype == F32 else 2e-2), nsplit


@pytest.mark.parametrize("decode", [False, True])
def test_attention_far_key_next_key_and_sink_show(cuda, decode):
    """(1) one key 700 positions back gets a score far above the rest: the output is its value; (2) the
    key right AFTER the query is made dominant instead: it must not be seen; (3) all scores very
    negative: the sink takes the mass and the output vanishes (an ordinary softmax would average)."""
    ops = _ops()
    H, G, dk, dv, page, N = 4, 2, 8, 8, 64, 900
    K, V = rnd(N, G, dk, seed=1, scale=0.1), rnd(N, G, dv, seed=2)
    qpos = 800
    q = rnd(1, H, dk, seed=3, scale=0.1)
    q[0, :, 0] = 6.0

    def run(Kx, sink, n_rows=16):
        pool, tables = make_pool([(Kx.float(), V.float())], page, 16, F32, seed=4)
        if decode:
            tiles = torch.tensor([(0, 1, qpos, 0)], dtype=torch.int32).cuda()
            qq, kw = q, dict(max_rows=1, nsplit=4)
        else:
            p0 = qpos - 5
            tiles = torch.tensor([(0, n_rows, p0, 0)], dtype=torch.int32).cuda()
            qq = torch.cat([rnd(5, H, dk, seed=5, scale=0.1), q, rnd(n_rows - 6, H, dk, seed=6, scale=0.1)])
            kw = dict(max_rows=16)
        out = ops.paged_attention(qq.reshape(qq.shape[0], -1).float().cuda(), pool, tables, tiles, heads=H, kv_heads=G,
                                  dim=dk, vdim=dv, page=page, scale=1.0, sink=sink, out_dtype=F32, **kw)
        return out[0 if decode else 5].cpu().double().view(H, dv)

    zero = torch.zeros(H, device="cuda")
    far = K.clone()
    far[qpos - 700, :, 0] = 6.0            # score 36 against ~0
    own = torch.arange(H) // (H // G)
    assert float((run(far, zero) - V[qpos - 700][own]).abs().max()) < 1e-4
    nxt = K.clone()
    nxt[qpos + 1, :, 0] = 6.0              # would win if the row could see one position ahead
    base = run(K, zero)
    assert float((run(nxt, zero) - base).abs().max()) == 0.0
    low = K.clone()
    low[:, :, 0] = -6.0                    # every score about -36: exp(0) of the sink dominates
    assert float(run(low, zero).abs().max()) < 1e-9
    assert float(run(low, None).abs().max()) > 1e-3


def test_moe_route_sigmoid(cuda):
    ops = _ops()
    cases = [(6, 2, 3, 2), (4, 1, 4, 2), (5, 5, 1, 1), (8, 3, 2, 1), (16, 4, 8, 3), (12, 6, 3, 2), (64, 8, 8, 4)]
    for E, top, count, keep in cases:
        for rows, seed in ((3, 1), (1500, 2)):      # a CTA per token and a warp per token
            x = rnd(rows, 48, seed=seed)
            W = {"r.router": rnd(E, 48, seed=3, scale=0.4), "r.correction": rnd(E, seed=4, scale=0.3) - 0.2}
            r = {"experts": E, "top": top, "groups": {"count": count, "keep": keep}}
            idx, wt = O.route(x, W, "r.", r)
            gi, gw = ops.moe_route_sigmoid(x.float().cuda(), W["r.router"].float().cuda(), W["r.correction"].float().cuda(),
                                           top, count, keep)
            same = (gi.cpu().long() == idx).all(-1)
            assert float(same.float().mean()) > 0.995, (E, top, count, keep)      # fp32 against float64 near ties
            assert rel(gw.cpu()[same], wt[same]) < 1e-5


def test_router_masks_with_minus_infinity_and_weights_skip_the_correction(cuda):
    """All choice values negative (correction -5): an expert of a dropped group must still lose against
    the kept groups' negative values; the weights are the plain sigmoid scores."""
    ops = _ops()
    E, top, count, keep = 8, 3, 4, 2
    x = rnd(50, 32, seed=1)
    wr = rnd(E, 32, seed=2, scale=0.3)
    corr = torch.full((E,), -5.0, dtype=F64)
    corr[2:4] += 2.5      # group 1 and group 3 are the best groups, whatever the scores in (0, 1) add
    corr[6:8] += 1.5
    gi, gw = ops.moe_route_sigmoid(x.float().cuda(), wr.float().cuda(), corr.float().cuda(), top, count, keep)
    assert set(gi.cpu().flatten().tolist()) <= {2, 3, 6, 7}
    s = torch.sigmoid(x @ wr.T)
    assert rel(gw.cpu(), s.gather(1, gi.cpu().long())) < 1e-5 and float(gw.min()) > 0


@pytest.mark.parametrize("dtype", [F32, BF])
@pytest.mark.parametrize("M", [3, 40, 300])
def test_clamped_gated_experts(cuda, dtype, M):
    """route -> group -> grouped up-projection with the clamped gated unit -> grouped down-projection,
    against the oracle's expert by expert sum; inputs large enough that both clamps bind"""
    ops = _ops()
    E, top, ff, width, limit = 5, 2, 24, 32, 0.7
    W = {}
    for e in range(E):
        W[f"m.e{e}.gate"], W[f"m.e{e}.up"] = rnd(ff, width, seed=10 + e, scale=0.3).to(dtype).double(), rnd(ff, width, seed=20 + e, scale=0.3).to(dtype).double()
        W[f"m.e{e}.down"] = rnd(width, ff, seed=30 + e, scale=0.3).to(dtype).double()
    W["m.router"], W["m.correction"] = rnd(E, width, seed=40, scale=0.05), torch.arange(E, dtype=F64) * 1.5
    h = rnd(M, width, seed=41).to(dtype)
    mlp = {"expert": {"ff": ff, "limit": limit}, "router": {"experts": E, "top": top, "groups": {"count": 1, "keep": 1}}}
    want = O.routed_experts(h.double(), W, "m.", mlp)
    gu = torch.empty(E, 2 * ff, width, dtype=dtype)
    for e in range(E):
        gu[e, 0::2], gu[e, 1::2] = W[f"m.e{e}.gate"].to(dtype), W[f"m.e{e}.up"].to(dtype)
    down = torch.stack([W[f"m.e{e}.down"].to(dtype) for e in range(E)])
    hc = h.cuda()
    idx, wt = ops.moe_route_sigmoid(hc, W["m.router"].float().cuda(), W["m.correction"].float().cuda(), top)
    seg, srt = ops.moe_group(idx, E)
    act = ops.glinear(hc, gu.cuda(), groups=E, seg=seg, a_rows=srt, a_row_div=top, glu_clamp=(1.702, limit))
    parts = ops.glinear(act, down.cuda(), groups=E, seg=seg, o_rows=srt, row_scale=wt.view(-1), out_dtype=F32,
                        out_rows_total=M * top)
    x = torch.zeros(M, width, device="cuda")
    ops.residual_add_rows(x, None, parts, n_partials=top, mult=1.0)
    assert rel(x, want) < (1e-5 if dtype == F32 else 3e-2)
    # the clamps bind somewhere and leave something alone
    g = h.double() @ W["m.e4.gate"].T
    assert bool((g > limit).any()) and bool((g < limit).any())


def test_small_row_ops(cuda):
    ops = _ops()
    x0 = rnd(9, 20, seed=1)
    a, parts, vec = rnd(9, 20, seed=2).to(BF), rnd(27, 20, seed=3), rnd(20, seed=4)
    x = x0.float().cuda()
    ops.residual_add_rows(x, a.cuda(), parts.float().cuda(), n_partials=3, mult=0.7)
    assert rel(x, x0 + 0.7 * (a.double() + parts.view(9, 3, 20).sum(1))) < 1e-6
    x = x0.float().cuda()
    xc = ops.residual_add_rows(x, a.cuda(), None, mult=0.5, copy_dtype=BF)
    assert rel(x, x0 + 0.5 * a.double()) < 1e-6 and torch.equal(xc, x.to(BF))
    x = x0.float().cuda()
    ops.add_row_vector(x, vec.float().cuda())
    assert rel(x, x0 + vec) < 1e-6
    # unit-normed, weighted update with a multiplier
    y, w = rnd(9, 20, seed=5), rnd(20, seed=6)
    x = x0.float().cuda()
    ops.gated_norm_residual(x, y.float().cuda(), w=w.float().cuda(), eps=1e-5, mult=0.6)
    assert rel(x, x0 + 0.6 * O.unit(y, 1e-5) * w) < 1e-6
    # gelu(z) * slice of a per-token table
    z, table = rnd(9, 6, seed=7, scale=2.0), rnd(30, 18, seed=8).to(BF)
    ids = torch.randint(0, 30, (9,), generator=torch.Generator().manual_seed(9), dtype=torch.int32)
    got = ops.gelu_mul_gather(z.float().cuda(), table.cuda(), ids.cuda(), 12, out_dtype=F32)
    assert rel(got, O.gelu_tanh(z) * table.double()[ids.long()][:, 12:18]) < 1e-6


# ------------------------------------------------------------------------------------------------
# whole models through the engine
# ------------------------------------------------------------------------------------------------
@pytest.mark.parametrize("dtype", [F32, BF])
@pytest.mark.parametrize("name", list(CONFIGS))
def test_whole_prompt_and_layers(cuda, name, dtype):
    from vila_b200.serving import TokenEngine
    cfg, model = build(name, dtype)
    toks = tokens_for(cfg, 150, 1)
    eng = TokenEngine(model, max_tokens=192, slots=1)
    layers = []
    lg = eng.step([("a", toks, list(range(len(toks))))], layer_outputs=layers)
    want, after = O.forward(cfg, model.state_dict(), toks)
    assert len(layers) == len(after) == len(O.layer_runs(cfg))
    for i, (a, b) in enumerate(zip(layers, after)):
        rows_close(a, b, dtype, f"after layer run {i}")
    rows_close(lg, want, dtype, "logits")
    # a one-token sequence in the slot and pages the long one gave back
    eng.release("a")
    assert rel(eng.step([("b", toks[:1], [0])]), want[:1]) < 2 * tol(dtype)


@pytest.mark.parametrize("dtype", [F32, BF])
@pytest.mark.parametrize("name", ["odd", "aligned", "plain2", "narrow"])
def test_decode_and_portions_match_whole(cuda, name, dtype):
    cfg, model = build(name, dtype, seed=3)
    prompts = {"p": tokens_for(cfg, 140, 2)}
    token_by_token = [[("p", 1)] for _ in range(140)]
    head_then_decode = [[("p", 70)]] + [[("p", 1)] for _ in range(70)]
    portions = [[("p", n)] for n in (2, 3, 2, 57, 1, 16, 17, 2, 33, 5, 2)]
    assert sum(s[0][1] for s in portions) == 140
    for schedule in (token_by_token, head_then_decode, portions):
        got = run_schedule(model, prompts, schedule, max_tokens=192, slots=1)
        check_logits(cfg, model, prompts, got, dtype)


@pytest.mark.parametrize("dtype", [F32, BF])
@pytest.mark.parametrize("name", ["odd", "aligned"])
def test_mixed_batches_reuse_pages_and_slots(cuda, name, dtype):
    """Four unequal requests share 2 slots and a pool that holds two of them: c and d run in the pages
    and slots a and b gave back; portions sit next to single tokens of the other request."""
    cfg, model = build(name, dtype, seed=4)
    prompts = {"a": tokens_for(cfg, 100, 5), "b": tokens_for(cfg, 37, 6), "c": tokens_for(cfg, 128, 7),
               "d": tokens_for(cfg, 3, 8)}
    schedule = [[("a", 30), ("b", 2)], [("a", 1), ("b", 1)], [("a", 1), ("b", 1)], [("a", 1), ("b", 1)],   # two-row
                [("a", 1), ("b", 30)], [("b", 1), ("a", 47)], [("a", 19), ("b", 1)],   # decode steps: eager, captured, replayed
                [("c", 63)], [("d", 1), ("c", 2)], [("c", 1), ("d", 2)], [("c", 62)]]
    got = run_schedule(model, prompts, schedule, max_tokens=192, slots=2)
    check_logits(cfg, model, prompts, got, dtype)
    if dtype == F32:   # batching must not change a sequence beyond rounding
        alone = run_schedule(model, {"c": prompts["c"]}, [[("c", 128)]], max_tokens=128, slots=1)
        assert rel(got["c"], alone["c"]) < 1e-5


def test_engine_refuses_what_does_not_fit(cuda):
    from vila_b200.serving import TokenEngine
    cfg, model = build("plain", BF)
    eng = TokenEngine(model, max_tokens=128, slots=1)
    eng.step([("a", tokens_for(cfg, 100, 1), [])])
    with pytest.raises(MemoryError):
        eng.step([("b", [1, 2], [])])           # no slot
    with pytest.raises(MemoryError):
        eng.step([("a", tokens_for(cfg, 40, 2), [])])   # no page
    eng.release("a")
    assert eng.step([("b", [1, 2], [1])]).shape == (1, cfg["vocab"])


def test_long_decode_across_page_borders(cuda):
    """300 decoded tokens after a short prompt in fp32: K | V pages, the convolution states of every pass
    and the previous token are carried across 300 steps (graph replays) and five page borders."""
    cfg, model = build("aligned", F32, seed=5)
    prompts = {"p": tokens_for(cfg, 330, 9)}
    got = run_schedule(model, prompts, [[("p", 30)]] + [[("p", 1)] for _ in range(300)], max_tokens=384, slots=1)
    check_logits(cfg, model, prompts, got, F32)


def test_sharp_attention_over_a_long_context(cuda):
    """With a large score scale the softmax of the second layer is sharp: every row attends to the one
    best-matching token among up to 700 earlier ones, wherever it is, so a far key that is missed (or a
    neighbour that is taken instead) changes the logits.  Whole prompt, decoded tail, 64-token portions."""
    cfg = json.loads(json.dumps(CONFIGS["plain"]))
    cfg["layers"][1]["mixer"]["scale"] = 2.5
    cfg, model = build(cfg, F32, seed=6)
    toks = tokens_for(cfg, 700, 11)
    for schedule in ([[("p", 700)]], [[("p", 690)]] + [[("p", 1)]] * 10, [[("p", 64)]] * 10 + [[("p", 58)], [("p", 2)]]):
        got = run_schedule(model, {"p": toks}, schedule, max_tokens=704, slots=1)
        check_logits(cfg, model, {"p": toks}, got, F32)


def test_generate_through_scheduler_matches_oracle_greedy(cuda):
    """Greedy generation through generate_tokens (continuous batching, chunked prefill, 2 slots for 3
    prompts, small step budget) against greedy decoding with the oracle."""
    from vila_b200.serving import generate_tokens
    cfg, model = build("odd", F32, seed=6)
    prompts = [tokens_for(cfg, n, 10 + n) for n in (41, 5, 70)]
    out = generate_tokens(model, prompts, max_new_tokens=12, slots=2, max_step_tokens=24)
    for p, ids in zip(prompts, out):
        want, margins = O.greedy(cfg, model.state_dict(), p, 12)
        for k, (a, b) in enumerate(zip(ids, want)):
            if margins[k] < 1e-3:
                break       # a tie in the oracle itself
            assert a == b, (k, ids, want)
    # EOS stops a request and frees its slot; sampling with a seed is reproducible
    eos = out[1][3]
    short = generate_tokens(model, prompts[1:2], max_new_tokens=12, eos_token_ids=[eos])
    assert short[0] == out[1][:out[1].index(eos) + 1]
    s1 = generate_tokens(model, prompts[:2], max_new_tokens=6, sample=True, temperature=0.9, top_k=20, top_p=0.9, seed=1)
    s2 = generate_tokens(model, prompts[:2], max_new_tokens=6, sample=True, temperature=0.9, top_k=20, top_p=0.9, seed=1)
    assert s1 == s2 and all(len(s) == 6 for s in s1)


def test_checkpoint_round_trip_and_registry(cuda, tmp_path):
    from vila_b200.model import load_language_model
    from vila_b200.serving import TokenEngine
    cfg, model = build("plain2", BF, seed=7)
    model.save_pretrained(tmp_path / "m")
    again = load_language_model(tmp_path / "m", dtype="bfloat16")
    assert type(again) is type(model) and again.config.to_dict() == model.config.to_dict()
    toks = tokens_for(cfg, 20, 3)
    a = TokenEngine(model, 64, 1).step([("x", toks, [19])])
    b = TokenEngine(again, 64, 1).step([("x", toks, [19])])
    assert torch.equal(a, b)


def test_command_line_generates_ids(cuda, tmp_path, capsys):
    from llava.cli import infer
    cfg, model = build("plain2", F32, seed=8)
    model.save_pretrained(tmp_path / "m")
    prompt = tokens_for(cfg, 9, 4)
    text = infer.main(["--model-path", str(tmp_path / "m"), "--token-ids", ",".join(map(str, prompt)),
                       "--max-new-tokens", "5", "--dtype", "float32"])
    assert [int(t) for t in text.split(",")] == model.generate(prompt, max_new_tokens=5)[0]
    assert text in capsys.readouterr().out


def test_trace_runner_replays_steps(cuda, tmp_path):
    """bin/trace_run on a saved model: three requests over two slots' worth of pages, portions beside
    single tokens, a step that wants nothing, ids released and their pages used again."""
    cfg, model = build("odd", F32, seed=9)
    model.save_pretrained(tmp_path / "m")
    p = {"a": tokens_for(cfg, 70, 1), "b": tokens_for(cfg, 9, 2), "c": tokens_for(cfg, 66, 3)}
    steps = [
        {"step": 0, "entries": [{"id": "a", "tokens": p["a"][:50], "want": [0, 49]}, {"id": "b", "tokens": p["b"][:2], "want": [1]}], "end": []},
        {"step": 1, "entries": [{"id": "b", "tokens": p["b"][2:8], "want": []}], "end": []},
        {"step": 2, "entries": [{"id": "a", "tokens": p["a"][50:51], "want": [0]}, {"id": "b", "tokens": p["b"][8:], "want": [0]}], "end": ["b"]},
        {"step": 3, "entries": [{"id": "a", "tokens": p["a"][51:], "want": [18]}], "end": ["a"]},
        {"step": 4, "entries": [{"id": "c", "tokens": p["c"], "want": [64, 65]}], "end": ["c"]},
    ]
    out = tmp_path / "out"
    r = subprocess.run([sys.executable, str(ROOT / "bin" / "trace_run"), "--model", str(tmp_path / "m"), "--dtype", "float32",
                        "--out", str(out), "--max-tokens", "128"], input="\n".join(json.dumps(s) for s in steps) + "\n",
                       capture_output=True, text=True, timeout=600, cwd=str(ROOT))
    assert r.returncode == 0, r.stderr[-2000:]
    assert [l for l in r.stdout.splitlines() if l.startswith("done")] == ["done %d" % k for k in range(5)]
    assert not (out / "1.f32").exists()
    want = {k: O.forward(cfg, model.state_dict(), v)[0] for k, v in p.items()}
    import numpy as np
    rows = {0: [want["a"][0], want["a"][49], want["b"][1]], 2: [want["a"][50], want["b"][8]], 3: [want["a"][69]],
            4: [want["c"][64], want["c"][65]]}
    for k, exp in rows.items():
        got = torch.from_numpy(np.fromfile(out / f"{k}.f32", dtype="<f4").reshape(len(exp), cfg["vocab"]))
        assert rel(got, torch.stack(exp)) < tol(F32), k
