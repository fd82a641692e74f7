"""Moronex on the GPU against the plain float64 oracle (oracle/moronex_oracle.py): every mechanism's
kernel alone, then whole models (own small configurations, random weights) under every way the
engine can be driven: whole prompts, token-by-token decoding, portions down to two tokens, mixed
batches of unequal requests, pages and slots that are freed and reused, long decoding, and greedy
generation through the scheduler."""
import math

import pytest
import torch

from oracle import moronex_oracle as O

pytestmark = pytest.mark.gpu
BF, F32 = torch.bfloat16, torch.float32


def _ops():
    from vila_b200 import ops
    return ops


def rel(a, b):
    a, b = a.double().cpu(), b.double().cpu()
    return float((a - b).abs().max() / b.abs().max().clamp_min(1e-30))


def tol(dtype):
    return 2e-5 if dtype == F32 else 5e-2   # max abs error over the largest expected entry


# ------------------------------------------------------------------------------------------------
# configurations (none of them a size combination of a published or given model)
# ------------------------------------------------------------------------------------------------
def lat(heads, dim, vdim, kv_rank, q_rank, scale, kv_from=None):
    m = dict(heads=heads, dim=dim, vdim=vdim, kv_rank=kv_rank, q_rank=q_rank, scale=scale)
    if kv_from is not None:
        m["kv_from"] = kv_from
    return {"type": "latent_attention", "mixer": m}


def rec(heads, dim, vdim):
    return {"type": "hgrn2", "mixer": dict(heads=heads, dim=dim, vdim=vdim)}


def dense(ff):
    return {"kind": "dense", "ff": ff}


def moe(experts, top, ff):
    return {"kind": "moe", "expert": {"ff": ff}, "router": {"experts": experts, "top": top}}


def config(width, vocab, layers, eps=1e-5):
    return {"architecture": "Moronex", "layers": [dict(l, mlp=m) for l, m in layers], "norm": {"eps": eps},
            "vocab": vocab, "width": width}


CONFIGS = {
    # odd sizes everywhere: nothing is a multiple of 8 where it need not be, a recurrent layer first, a
    # layer without feed-forward, two layers reading layer 1's latent, one head, top == 1, top == 3 of 5
    "odd": config(96, 131, [
        (rec(3, 8, 24), moe(5, 3, 40)),
        (lat(3, 24, 40, 48, 56, 0.3), dense(136)),
        (lat(5, 16, 8, 48, 32, 0.25, kv_from=1), None),
        (lat(1, 32, 32, 20, 24, 0.2), moe(4, 1, 24)),
        (rec(1, 40, 72), dense(64)),
        (lat(2, 8, 16, 48, 16, 0.5, kv_from=1), moe(3, 3, 16)),
    ], eps=1e-6),
    # sizes the tensor-core GEMM takes
    "aligned": config(128, 256, [
        (lat(4, 32, 32, 64, 64, 0.17), moe(8, 2, 64)),
        (rec(2, 64, 64), dense(256)),
        (lat(4, 32, 32, 64, 64, 0.17, kv_from=0), dense(128)),
        (rec(4, 16, 32), moe(6, 2, 32)),
    ]),
    # a width that is no multiple of 8
    "narrow": config(100, 77, [
        (lat(2, 10, 12, 36, 28, 0.31), dense(50)),
        (rec(2, 12, 20), moe(4, 2, 30)),
    ]),
}


def build(name, dtype, seed=0):
    from vila_b200.model import MoronexConfig, MoronexForCausalLM
    cfg = CONFIGS[name]
    model = MoronexForCausalLM(MoronexConfig.from_dict(cfg), "cuda", dtype).init_random(seed, scale=1.5)
    if dtype == BF:
        # A router logit pair closer than the bf16 noise of its input would pick another expert than the
        # float64 oracle, and the recurrent layers carry that one row's difference into the rows after
        # it.  The bf16 models therefore get decisive routers: biases 2 apart and a small input term (the
        # chosen set is then nearly fixed per layer, the weights still vary per token).  Routing that
        # changes from token to token is covered by the fp32 models and by test_moe_route.
        t = model.state_dict()
        g = torch.Generator().manual_seed(seed + 100)
        for n in list(t):
            if n.endswith("mlp.router"):
                t[n] = (t[n].float() * 0.25).to(BF)
            elif n.endswith("mlp.router.b"):
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
        rows_close(got[name], O.forward(cfg, model.state_dict(), toks)[0], dtype, name)


# ------------------------------------------------------------------------------------------------
# kernels alone
# ------------------------------------------------------------------------------------------------
@pytest.mark.parametrize("dtype", [F32, BF])
@pytest.mark.parametrize("rows,cols", [(1, 7), (37, 96), (300, 1030)])
def test_rmsnorm_rows(cuda, dtype, rows, cols):
    ops = _ops()
    g = torch.Generator().manual_seed(1)
    x = torch.randn(rows, cols + 5, generator=g).cuda()[:, 2:2 + cols]     # strided view
    w = (torch.randn(cols, generator=g) * 0.2).cuda()
    for off in (0.0, 1.0):
        out = ops.rmsnorm_rows(x, w, 1e-5, w_offset=off, out_dtype=dtype)
        want = O.rms(x.double(), 1e-5) * (w.double() + off)
        assert rel(out, want) < (1e-6 if dtype == F32 else 5e-3)
    # scatter into a pool through a row map
    pool = torch.zeros(rows * 3, cols, device="cuda", dtype=dtype)
    where = torch.randperm(rows * 3, generator=g)[:rows].to(torch.int32).cuda()
    ops.rmsnorm_rows(x, w, 1e-5, out=pool, out_rows=where)
    assert rel(pool[where.long()], O.rms(x.double(), 1e-5) * w.double()) < (1e-6 if dtype == F32 else 5e-3)
    untouched = torch.ones(rows * 3, dtype=torch.bool)
    untouched[where.long().cpu()] = False
    assert float(pool[untouched.cuda()].abs().max() if untouched.any() else 0) == 0


@pytest.mark.parametrize("dtype", [F32, BF])
def test_gated_norm_residual(cuda, dtype):
    ops = _ops()
    g = torch.Generator().manual_seed(2)
    rows, cols, parts = 19, 100, 3
    x = torch.randn(rows, cols, generator=g).cuda()
    y = torch.randn(rows * parts, cols, generator=g).cuda().to(dtype)
    gate = torch.randn(rows, cols + 8, generator=g).cuda().to(dtype)[:, 8:]
    gb, w = torch.randn(cols, generator=g).cuda(), (torch.randn(cols, generator=g) * 0.3).cuda()
    ysum = y.double().view(rows, parts, cols).sum(1) * torch.sigmoid(gate.double() + gb.double())
    want = x.double() + O.rms(ysum, 1e-5) * (1.0 + w.double())
    ops.gated_norm_residual(x, y, n_partials=parts, gate=gate, gate_bias=gb, w=w, w_offset=1.0, eps=1e-5)
    assert rel(x, want) < 2e-6


@pytest.mark.parametrize("dtype", [F32, BF])
@pytest.mark.parametrize("M,N,K", [(1, 5, 3), (16, 64, 16), (17, 70, 33), (130, 6, 100), (3, 448, 256)])
def test_glinear_plain_and_epilogues(cuda, dtype, M, N, K):
    ops = _ops()
    g = torch.Generator().manual_seed(3)
    a = torch.randn(M, K, generator=g).cuda().to(dtype)
    w = (torch.randn(N, K, generator=g) / K ** 0.5).cuda().to(dtype)
    ref = a.double() @ w.double().T
    t = 1e-6 if dtype == F32 else 6e-3
    assert rel(ops.glinear(a, w, out_dtype=F32), ref) < 1e-6
    assert rel(ops.glinear(a, w), ref) < t
    assert rel(ops.glinear(a, w, act=ops.ACT_RELU2, out_dtype=F32), torch.relu(ref) ** 2) < 2e-6
    if N % 2 == 0:
        sw = torch.nn.functional.silu(ref[:, 0::2]) * ref[:, 1::2]
        assert rel(ops.glinear(a, w, swiglu=True, out_dtype=F32), sw) < 2e-6


def test_glinear_groups(cuda):
    ops = _ops()
    g = torch.Generator().manual_seed(4)
    T, H, K, N = 21, 3, 10, 7
    a = torch.randn(T, H * K, generator=g).cuda()
    w = torch.randn(H, N, K, generator=g).cuda()
    out = ops.glinear(a, w, groups=H, a_group_off=K, o_group_off=N)
    want = torch.einsum("thk,hnk->thn", a.double().view(T, H, K), w.double()).reshape(T, H * N)
    assert rel(out, want) < 1e-6
    # segmented: rows routed to experts through a sorted pair list, written back scaled
    E, top, ff = 5, 2, 9
    idx = torch.stack([torch.randperm(E, generator=g)[:top] for _ in range(T)]).to(torch.int32).cuda()
    seg, srt = ops.moe_group(idx, E)
    flat = idx.view(-1).cpu()
    assert seg.tolist() == [0] + torch.cumsum(torch.bincount(flat.long(), minlength=E), 0).tolist()
    for e in range(E):
        mine = srt[seg[e]:seg[e + 1]].cpu()
        assert mine.tolist() == sorted(mine.tolist()) and bool((flat[mine.long()] == e).all())
    x = torch.randn(T, K, generator=g).cuda()
    up = torch.randn(E, ff, K, generator=g).cuda()
    scale = torch.rand(T * top, generator=g).cuda()
    act = ops.glinear(x, up, groups=E, seg=seg, a_rows=srt, a_row_div=top)
    out = ops.glinear(act, torch.eye(ff).cuda().repeat(E, 1, 1), groups=E, seg=seg, o_rows=srt,
                      row_scale=scale, out_rows_total=T * top)
    want = torch.stack([(up[int(flat[p])].double() @ x[p // top].double()) * scale[p].double()
                        for p in range(T * top)])
    assert rel(out, want) < 1e-6


@pytest.mark.parametrize("M,N,K", [(1, 8, 8), (3, 24, 40), (17, 200, 72), (300, 136, 96), (1124, 456, 256)])
def test_tensor_core_linear_agrees_with_cuda_core_linear(cuda, M, N, K):
    """The bf16 projections of the model go to vila_linear whenever N and K are multiples of 8."""
    ops = _ops()
    g = torch.Generator().manual_seed(5)
    a = torch.randn(M, K, generator=g).cuda().to(BF)
    w = (torch.randn(N, K, generator=g) / K ** 0.5).cuda().to(BF)
    assert rel(ops.linear(a, w, static_w=True), ops.glinear(a, w)) < 1e-2
    assert rel(ops.linear(a, w, static_w=True), a.double() @ w.double().T) < 1e-2


def _attend_direct(q, c, sink, gate, scale, pos0):
    """q [n, H, R] at positions pos0.., c [pos0 + n, R]: per-row softmax with the sink, fp64"""
    n, H, R = q.shape
    out = torch.zeros(n, H, R, dtype=torch.float64)
    for i in range(n):
        keys = c[:pos0 + i + 1].double()
        for h in range(H):
            s = keys @ q[i, h].double() * scale
            m = max(float(s.max()), float(sink[h]) if sink is not None else -math.inf)
            e = torch.exp(s - m)
            den = e.sum() + (math.exp(float(sink[h]) - m) if sink is not None else 0.0)
            o = (e[:, None] * keys).sum(0) / den
            out[i, h] = o * (torch.sigmoid(gate[i, h].double()) if gate is not None else 1.0)
    return out


@pytest.mark.parametrize("dtype", [F32, BF])
@pytest.mark.parametrize("R,H", [(20, 3), (64, 2), (130, 1), (300, 2), (40, 6), (96, 17)])
def test_latent_attention_kernels(cuda, dtype, R, H):
    """Portions that start and end in the middle of pages, shuffled physical pages, a second sequence in
    the same launch, with and without sink / gate; the one-row kernel at page borders."""
    ops = _ops()
    g = torch.Generator().manual_seed(R)
    page, n_pages = 64, 8
    order = torch.randperm(n_pages, generator=g)
    pt = torch.zeros(2, n_pages, dtype=torch.int32)
    pt[0, :5], pt[1, :3] = order[:5].int(), order[5:8].int()
    lens = [300, 130]
    pool = torch.zeros(n_pages * page, R, dtype=dtype).cuda()
    cs = [torch.randn(n, R, generator=g).to(dtype) for n in lens]
    for s, c in enumerate(cs):
        for j in range(lens[s]):
            pool[int(pt[s, j // page]) * page + j % page] = c[j].cuda()
    sink = torch.randn(H, generator=g)
    # sequence 0 brings rows 270..299 (tiles 16 + 14), sequence 1 rows 60..129 in tiles, row 129 again alone
    rows = [(0, 270, 30), (1, 60, 70)]
    T = sum(r[2] for r in rows)
    q = torch.randn(T, H, R, generator=g)
    gate = torch.randn(T, H + 3, generator=g).to(dtype)[:, 1:1 + H]
    tiles, want, at = [], [], 0
    for s, p0, n in rows:
        for o in range(0, n, 16):
            tiles.append((at + o, min(16, n - o), p0 + o, s))
        want.append(_attend_direct(q[at:at + n], cs[s].cpu(), sink, gate[at:at + n], 0.2, p0))
        at += n
    want = torch.cat(want)
    common = dict(heads=H, page=page, scale=0.2, sink=sink.cuda(), gate=gate.cuda(), out_dtype=F32)
    tl = torch.tensor(tiles, dtype=torch.int32).cuda()
    got = ops.latent_attention(q.view(T, -1).cuda(), pool, pt.cuda(), tl, **common)
    t = 1e-5 if dtype == F32 else 1e-2
    assert rel(got.view(T, H, R), want) < t
    # every row as a one-row tile through the decode kernel (positions 63, 64, 65, 127, 128 are among them)
    single = []
    at = 0
    for s, p0, n in rows:
        single += [(at + i, 1, p0 + i, s) for i in range(n)]
        at += n
    sg = torch.tensor(single, dtype=torch.int32).cuda()
    got1 = ops.latent_attention(q.view(T, -1).cuda(), pool, pt.cuda(), sg, decode=True, **common)
    assert rel(got1.view(T, H, R), want) < t
    for ns in (2, 5, 16):   # keys of a row dealt to several CTAs and merged (more CTAs than key blocks too)
        gots = ops.latent_attention(q.view(T, -1).cuda(), pool, pt.cuda(), sg, decode=True, nsplit=ns, **common)
        assert rel(gots.view(T, H, R), want) < t, ns
    # no sink, no gate
    plain = ops.latent_attention(q.view(T, -1).cuda(), pool, pt.cuda(), tl, heads=H, page=page, scale=0.2, out_dtype=F32)
    at, w2 = 0, []
    for s, p0, n in rows:
        w2.append(_attend_direct(q[at:at + n], cs[s].cpu(), None, None, 0.2, p0))
        at += n
    assert rel(plain.view(T, H, R), torch.cat(w2)) < t


@pytest.mark.parametrize("decode", [False, True])
def test_latent_attention_far_key_and_sink_show(cuda, decode):
    """One key far back is made to dominate: the output must be that latent row.  Then a huge sink:
    the output must vanish.  Random weights would hide both among hundreds of keys."""
    ops = _ops()
    g = torch.Generator().manual_seed(7)
    R, H, page, L = 32, 2, 64, 700   # (two heads: the one-head-per-CTA decode kernel; more heads: test above)
    n_pages = (L + page - 1) // page
    pt = torch.arange(n_pages - 1, -1, -1, dtype=torch.int32)[None].contiguous()   # pages in reverse order
    c = torch.randn(L, R, generator=g) * 0.1
    far = 3   # a key in the first page, 696 tokens back
    c[far] = torch.randn(R, generator=g) * 3
    pool = torch.zeros(n_pages * page, R)
    for j in range(L):
        pool[int(pt[0, j // page]) * page + j % page] = c[j]
    q = (c[far] * 4)[None, None].repeat(1, H, 1).reshape(1, -1)
    tile = torch.tensor([[0, 1, L - 1, 0]], dtype=torch.int32).cuda()
    kw = dict(heads=H, page=page, scale=1.0, out_dtype=F32, decode=decode, nsplit=4 if decode else 1)
    out = ops.latent_attention(q.cuda(), pool.cuda(), pt.cuda(), tile, **kw).view(H, R)
    assert rel(out[0], c[far]) < 1e-4 and rel(out[1], c[far]) < 1e-4
    # one position earlier than the key's own: invisible
    tile2 = torch.tensor([[0, 1, far - 1, 0]], dtype=torch.int32).cuda()
    out2 = ops.latent_attention(q.cuda(), pool.cuda(), pt.cuda(), tile2, **kw).view(H, R)
    assert float((out2[0].cpu() - c[far]).abs().max()) > 1.0
    sink = torch.tensor([1e4, -1e4])
    out3 = ops.latent_attention(q.cuda(), pool.cuda(), pt.cuda(), tile, sink=sink.cuda(), **kw).view(H, R)
    assert float(out3[0].abs().max()) < 1e-6 and rel(out3[1], c[far]) < 1e-4


@pytest.mark.parametrize("dtype", [F32, BF])
@pytest.mark.parametrize("H,dim,vdim", [(3, 8, 24), (1, 40, 72), (2, 128, 33), (2, 200, 64)])
def test_hgrn2_scan(cuda, dtype, H, dim, vdim):
    """Whole sequence in one call, the same in portions of 1..17 rows through a state slot that was used
    before, and two sequences in one launch."""
    ops = _ops()
    g = torch.Generator().manual_seed(dim)
    T = 75
    ld = 2 * H * dim + H * vdim + 8
    proj = torch.randn(T, ld, generator=g).to(dtype)
    fb, low = torch.randn(H * dim, generator=g), torch.rand(H * dim, generator=g) * 0.9
    q = torch.nn.functional.silu(proj[:, :H * dim].double()).view(T, H, dim)
    f = (low + (1 - low) * torch.sigmoid(proj[:, H * dim:2 * H * dim].double() + fb)).view(T, H, dim)
    v = proj[:, 2 * H * dim + 8:].double().view(T, H, vdim)
    S = torch.zeros(H, dim, vdim, dtype=torch.float64)
    want = torch.zeros(T, H, vdim, dtype=torch.float64)
    for t in range(T):
        S = f[t][:, :, None] * S + (1 - f[t])[:, :, None] * v[t][:, None, :]
        want[t] = torch.einsum("hkv,hk->hv", S, q[t])
    kw = dict(heads=H, dim=dim, vdim=vdim, q_off=0, f_off=H * dim, v_off=2 * H * dim + 8, f_bias=fb.cuda(),
              lower=low.cuda())
    state = torch.full((3, H, dim, vdim), 7.0, device="cuda")    # stale contents of used slots
    seq = torch.tensor([[0, T, 0, 1]], dtype=torch.int32).cuda()
    out = ops.hgrn2_scan(proj.cuda(), state, seq, **kw)
    assert rel(out.view(T, H, vdim), want) < 1e-5
    assert rel(state[1], S) < 1e-5 and float((state[0] - 7).abs().max()) == 0
    # portions, slot 2, interleaved with another sequence (the same rows, later positions) in slot 0
    state.fill_(-3.0)
    got, at = [], 0
    for n in [1, 2, 17, 3, 16, 1, 35]:
        both = torch.cat([proj[at:at + n], proj[:5]]).cuda()
        sq = torch.tensor([[0, n, at, 2], [n, 5, 0, 0]], dtype=torch.int32).cuda()
        o = ops.hgrn2_scan(both, state, sq, **kw)
        got.append(o[:n])
        assert rel(o[n:].view(5, H, vdim), want[:5]) < 1e-5
        at += n
    assert at == T and rel(torch.cat(got).view(T, H, vdim), want) < 1e-5


def test_moe_route(cuda):
    ops = _ops()
    g = torch.Generator().manual_seed(9)
    T, K, E, top = 50, 33, 37, 4
    x = torch.randn(T, K, generator=g).to(BF)
    wr, b = torch.randn(E, K, generator=g), torch.randn(E, generator=g)
    z = x.double() @ wr.double().T + b.double()
    val, idx = torch.topk(z, top, -1)
    gi, gw = ops.moe_route(x.cuda(), wr.cuda(), b.cuda(), top)
    assert gi.cpu().tolist() == idx.tolist()
    assert rel(gw, torch.softmax(val, -1)) < 1e-5
    # top == experts and top == 1
    gi, gw = ops.moe_route(x.cuda(), wr[:3].contiguous().cuda(), None, 3)
    assert sorted(gi[0].tolist()) == [0, 1, 2] and abs(float(gw[0].sum()) - 1) < 1e-6
    gi, gw = ops.moe_route(x.cuda(), wr.cuda(), b.cuda(), 1)
    assert gi.view(-1).cpu().tolist() == z.argmax(-1).tolist() and float((gw - 1).abs().max()) == 0


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
    for i, (a, b) in enumerate(zip(layers, after)):
        rows_close(a, b, dtype, f"after layer {i}")
    rows_close(lg, want, dtype, "logits")
    # a one-token sequence
    eng.release("a")
    assert rel(eng.step([("b", toks[:1], [0])]), want[:1]) < 2 * tol(dtype)


@pytest.mark.parametrize("dtype", [F32, BF])
@pytest.mark.parametrize("name", ["odd", "aligned"])
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
    cfg, model = build("narrow", BF)
    eng = TokenEngine(model, max_tokens=128, slots=1)
    eng.step([("a", tokens_for(cfg, 100, 1), [])])
    with pytest.raises(MemoryError):
        eng.step([("b", [1, 2], [])])           # no slot
    with pytest.raises(MemoryError):
        eng.step([("a", tokens_for(cfg, 40, 2), [])])   # no page
    eng.release("a")
    assert eng.step([("b", [1, 2], [1])]).shape == (1, cfg["vocab"])


def test_long_decode_and_far_context(cuda):
    """300 decoded tokens after a short prompt in fp32: the recurrent state and the latent pages are
    carried across 300 steps and five page borders."""
    cfg, model = build("aligned", F32, seed=5)
    prompts = {"p": tokens_for(cfg, 330, 9)}
    got = run_schedule(model, prompts, [[("p", 30)]] + [[("p", 1)] for _ in range(300)], max_tokens=384, slots=1)
    check_logits(cfg, model, prompts, got, F32)


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
    cfg, model = build("narrow", BF, seed=7)
    model.save_pretrained(tmp_path / "m")
    again = load_language_model(tmp_path / "m", dtype="bfloat16")
    assert type(again) is type(model) and again.config.to_dict() == model.config.to_dict()
    toks = tokens_for(cfg, 20, 3)
    a = TokenEngine(model, 64, 1).step([("x", toks, [19])])
    b = TokenEngine(again, 64, 1).step([("x", toks, [19])])
    assert torch.equal(a, b)


def test_command_line_generates_ids(cuda, tmp_path, capsys):
    from llava.cli import infer
    cfg, model = build("narrow", F32, seed=8)
    model.save_pretrained(tmp_path / "m")
    prompt = tokens_for(cfg, 9, 4)
    text = infer.main(["--model-path", str(tmp_path / "m"), "--token-ids", ",".join(map(str, prompt)),
                       "--max-new-tokens", "5", "--dtype", "float32"])
    assert [int(t) for t in text.split(",")] == model.generate(prompt, max_new_tokens=5)[0]
    assert text in capsys.readouterr().out


@pytest.mark.parametrize("dtype", [F32, BF])
@pytest.mark.parametrize("H,dim,vdim", [(3, 24, 40), (2, 128, 128), (1, 10, 300)])
def test_sink_attention_and_gather_rows(cuda, dtype, H, dim, vdim):
    """The un-folded kernel: keys / values as strided views of one buffer, two sequences (one continuing
    at position 150, one from 0), tiles that end at ragged sizes; gather_rows feeds it in the model."""
    ops = _ops()
    g = torch.Generator().manual_seed(dim)
    src = torch.randn(50, 12, generator=g).to(dtype).cuda()
    pick = torch.randperm(50, generator=g)[:23].to(torch.int32).cuda()
    assert torch.equal(ops.gather_rows(src, pick), src[pick.long()])
    lens, news = [200, 37], [50, 37]
    kv = torch.randn(sum(lens), H * (dim + vdim) + 8, generator=g).to(dtype)
    k, v = kv[:, :H * dim], kv[:, H * dim + 8:]
    T = sum(news)
    q = torch.randn(T, H * dim, generator=g).to(dtype)
    gate, sink = torch.randn(T, H, generator=g).to(dtype), torch.randn(H, generator=g)
    tiles, want, at, kv0 = [], torch.zeros(T, H, vdim, dtype=torch.float64), 0, 0
    for L, n in zip(lens, news):
        p0 = L - n
        for o in range(0, n, 16):
            tiles.append((at + o, min(16, n - o), p0 + o, kv0))
        for i in range(n):
            for h in range(H):
                ks = k[kv0:kv0 + p0 + i + 1, h * dim:(h + 1) * dim].double()
                vs = v[kv0:kv0 + p0 + i + 1, h * vdim:(h + 1) * vdim].double()
                s = ks @ q[at + i, h * dim:(h + 1) * dim].double() * 0.3
                m = max(float(s.max()), float(sink[h]))
                e = torch.exp(s - m)
                o_ = (e[:, None] * vs).sum(0) / (e.sum() + math.exp(float(sink[h]) - m))
                want[at + i, h] = o_ * torch.sigmoid(gate[at + i, h].double())
        at += n
        kv0 += L
    kvd = kv.cuda()
    got = ops.sink_attention(q.cuda(), kvd[:, :H * dim], kvd[:, H * dim + 8:], torch.tensor(tiles, dtype=torch.int32).cuda(),
                             heads=H, scale=0.3, sink=sink.cuda(), gate=gate.cuda(), out_dtype=F32)
    assert rel(got.view(T, H, vdim), want) < (1e-5 if dtype == F32 else 1e-2)


@pytest.mark.parametrize("ratio", [0, 4])
def test_folded_and_unfolded_attention_agree(cuda, ratio):
    """The same prompt through the folded form only (ratio 0) and with the un-folded form for large
    portions, in fp32: both against the oracle."""
    from vila_b200.serving import TokenEngine
    cfg, model = build("odd", F32, seed=9)
    toks = tokens_for(cfg, 120, 11)
    eng = TokenEngine(model, max_tokens=128, slots=1)
    eng.unfold_ratio = ratio
    got = torch.cat([eng.step([("s", toks[a:b], list(range(b - a)))]).cpu() for a, b in ((0, 70), (70, 73), (73, 120))])
    rows_close(got, O.forward(cfg, model.state_dict(), toks)[0], F32, f"ratio {ratio}")
