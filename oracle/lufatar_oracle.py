"""Plain, slow restatement of the Lufatar architecture in float64 PyTorch (test infrastructure only;
the product never imports it).  One function per mechanism; whole sequences only: no cache, no
pages, no state, no batching, no fused forms, so every schedule of the engine can be compared
against it.

Notation: x residual [T, width]; W[name] checkpoint tensors (linear weights [out, in]); t a position
(0-based inside its sequence); unit(v) = v / sqrt(mean(v^2) + eps)."""
from __future__ import annotations

import math
from typing import Dict, List, Tuple

import torch

F64 = torch.float64


def unit(v: torch.Tensor, eps: float) -> torch.Tensor:
    return v / torch.sqrt(v.pow(2).mean(-1, keepdim=True) + eps)


def group_norm(v: torch.Tensor, w: torch.Tensor, groups: int, eps: float) -> torch.Tensor:
    """every one of `groups` equal consecutive pieces of a row gets its own root mean square"""
    T, C = v.shape
    return unit(v.view(T, groups, C // groups), eps).reshape(T, C) * w


def gelu_tanh(z: torch.Tensor) -> torch.Tensor:
    return 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def token_embedding(W, tokens, bg: dict) -> torch.Tensor:
    """word row + hashed (previous, current) pair row; the first token reads the table's last row"""
    ids = torch.as_tensor(tokens, dtype=torch.long)
    rows = torch.empty_like(ids)
    rows[0] = bg["buckets"]
    rows[1:] = (ids[:-1] * bg["mul_prev"] + ids[1:] * bg["mul_cur"]) % bg["buckets"]
    return W["embed"][ids] + W["bigram"][rows]


def short_conv_residual(h: torch.Tensor, w: torch.Tensor) -> torch.Tensor:
    """h_t + sum_j w[:, j] * h_{t - (taps - 1) + j}, nothing before position 0"""
    T, taps = h.shape[0], w.shape[1]
    out = h.clone()
    for t in range(T):
        for j in range(taps):
            s = t - (taps - 1) + j
            if s >= 0:
                out[t] += w[:, j] * h[s]
    return out


def rotate_pairs(v: torch.Tensor, base: float, dims: int) -> torch.Tensor:
    """v [T, heads, dim]: columns (2i, 2i+1), i < dims / 2, turn by t * base^(-2i / dims)"""
    T = v.shape[0]
    out = v.clone()
    if dims == 0:
        return out
    i = torch.arange(dims // 2, dtype=F64)
    ang = torch.arange(T, dtype=F64)[:, None] * base ** (-2.0 * i / dims)[None, :]
    c, s = torch.cos(ang)[:, None, :], torch.sin(ang)[:, None, :]
    a, b = v[..., 0:dims:2], v[..., 1:dims:2]
    out[..., 0:dims:2] = a * c - b * s
    out[..., 1:dims:2] = b * c + a * s
    return out


def softmax_plus_one(scores: torch.Tensor) -> torch.Tensor:
    """scores [..., T] masked with -inf -> exp(s) / (1 + sum exp(s))"""
    m = torch.clamp_min(scores.max(-1, keepdim=True).values, 0.0)
    e = torch.exp(scores - m)
    return e / (e.sum(-1, keepdim=True) + torch.exp(-m))


def attention(h, W, p, m, eps) -> torch.Tensor:
    T, H, G, dk, dv = h.shape[0], m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = (h @ W[p + "q"].T).view(T, H, dk)
    k = (h @ W[p + "k"].T).view(T, G, dk)
    v = (h @ W[p + "v"].T).view(T, G, dv)
    q = unit(rotate_pairs(q, m["rot"]["base"], m["rot"]["dims"]), eps)
    k = unit(rotate_pairs(k, m["rot"]["base"], m["rot"]["dims"]), eps)
    owner = torch.arange(H) // (H // G)
    s = torch.einsum("ihd,jhd->hij", q, k[:, owner]) * m["scale"]
    s = torch.einsum("hg,gij->hij", W[p + "talk"], s)
    s = s.masked_fill(torch.triu(torch.ones(T, T, dtype=torch.bool), diagonal=1), -math.inf)
    o = torch.einsum("hij,jhd->ihd", softmax_plus_one(s), v[:, owner])
    return o.reshape(T, H * dv) @ W[p + "o"].T


def route(h, W, p, r) -> Tuple[torch.Tensor, torch.Tensor]:
    """-> (chosen experts [T, top], their weights [T, top])"""
    E, top = r["experts"], r["top"]
    count, keep = r["groups"]["count"], r["groups"]["keep"]
    s = torch.sigmoid(h @ W[p + "router"].T)
    choice = s + W[p + "correction"]
    per = choice.view(-1, count, E // count)
    gscore = per.topk(min(2, E // count), dim=-1).values.sum(-1)
    kept = torch.zeros_like(gscore, dtype=torch.bool)
    kept.scatter_(1, gscore.topk(keep, dim=-1).indices, True)
    masked = per.masked_fill(~kept[:, :, None], -math.inf).reshape(-1, E)
    idx = masked.topk(top, dim=-1).indices
    return idx, s.gather(1, idx)


def expert(h_row, W, p, limit: float) -> torch.Tensor:
    g = torch.clamp_max(W[p + "gate"] @ h_row, limit)
    u = torch.clamp(W[p + "up"] @ h_row, -limit, limit)
    return W[p + "down"] @ (g * torch.sigmoid(1.702 * g) * (u + 1.0))


def routed_experts(h, W, p, mlp) -> torch.Tensor:
    idx, wt = route(h, W, p, mlp["router"])
    y = torch.zeros(h.shape[0], W[p + "e0.down"].shape[0], dtype=h.dtype)
    for t in range(h.shape[0]):
        for j in range(idx.shape[1]):
            y[t] += wt[t, j] * expert(h[t], W, p + f"e{int(idx[t, j])}.", mlp["expert"]["limit"])
    return y


def token_side(x, W, p, tokens, layer: int, dim: int, eps: float) -> torch.Tensor:
    """the unit-normed, weighted projection of gelu(gate x) * (this layer's slice of the token's side row)"""
    e = W["side.embed"][torch.as_tensor(tokens, dtype=torch.long)][:, layer * dim:(layer + 1) * dim]
    y = (gelu_tanh(x @ W[p + "gate"].T) * e) @ W[p + "proj"].T
    return unit(y, eps) * W[p + "norm"]


def layer(x, W, i, spec, config, tokens) -> torch.Tensor:
    eps, groups, mult = config["norm"]["eps"], config["norm"]["groups"], config["residual_mult"]
    p = f"l{i}."
    h = short_conv_residual(group_norm(x, W[p + "norm1"], groups, eps), W[p + "canon1"])
    y = attention(h, W, p + "mix.", spec["mixer"], eps)
    if spec.get("mlp") is not None:
        h2 = short_conv_residual(group_norm(x, W[p + "norm2"], groups, eps), W[p + "canon2"])
        y = y + routed_experts(h2, W, p + "mlp.", spec["mlp"])
    x = x + mult * y
    if config.get("token_side") is not None:
        x = x + mult * token_side(x, W, p + "side.", tokens, i, config["token_side"]["dim"], eps)
    return x


def layer_runs(config: dict) -> List[Tuple[int, int]]:
    """(layer, pass) in execution order; pass -1: outside the repeated block"""
    n = len(config["layers"])
    lp = config.get("loop") or {"start": 0, "stop": 0, "times": 1}
    a, b, times = lp["start"], lp["stop"], lp["times"]
    if b <= a:
        return [(i, -1) for i in range(n)]
    return [(i, -1) for i in range(a)] + [(i, t) for t in range(times) for i in range(a, b)] + \
           [(i, -1) for i in range(b, n)]


def forward(config: dict, weights: Dict[str, torch.Tensor], tokens) -> Tuple[torch.Tensor, List[torch.Tensor]]:
    """config: the config.json dictionary -> (logits [T, vocab], residual after every layer run)"""
    W = {k: (v.to(F64) if v.is_floating_point() else v) for k, v in weights.items()}
    x = token_embedding(W, tokens, config["embedding"]["bigram"])
    after = []
    lp = config.get("loop") or {}
    for i, t in layer_runs(config):
        if t >= 0 and i == lp["start"]:
            x = x + W["loop.step"][t]
        x = layer(x, W, i, config["layers"][i], config, tokens)
        after.append(x.clone())
    h = group_norm(x, W["final.norm"], config["norm"]["groups"], config["norm"]["eps"])
    return h @ W["head"].T, after


def greedy(config: dict, weights, prompt, n_new: int) -> Tuple[List[int], List[float]]:
    """-> (new ids, top-2 margin of every choice): greedy decoding by re-running the whole sequence"""
    toks, ids, margins = list(prompt), [], []
    for _ in range(n_new):
        lg = forward(config, weights, toks)[0][-1]
        top2 = torch.topk(lg, 2).values
        margins.append(float(top2[0] - top2[1]))
        ids.append(int(torch.argmax(lg)))
        toks.append(ids[-1])
    return ids, margins
