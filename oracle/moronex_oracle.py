"""Plain, slow restatement of the Moronex architecture in float64 PyTorch (test infrastructure only;
the product never imports it).  One function per mechanism; whole sequences only: no cache, no
pages, no batching, no fused or absorbed forms, so every schedule of the engine can be compared
against it.

Notation: x residual [T, width]; W[name] checkpoint tensors (linear weights [out, in]);
rms(v) = v / sqrt(mean(v^2) + eps)."""
from __future__ import annotations

import math
from typing import Dict, List, Tuple

import torch

F64 = torch.float64


def rms(v: torch.Tensor, eps: float) -> torch.Tensor:
    return v / torch.sqrt(v.pow(2).mean(-1, keepdim=True) + eps)


def norm_centred(v, w, eps):
    """layer / final norms: weights are stored around zero"""
    return rms(v, eps) * (1.0 + w)


def norm_plain(v, w, eps):
    return rms(v, eps) * w


def softmax_with_sink(scores: torch.Tensor, sink: torch.Tensor) -> torch.Tensor:
    """scores [H, T, T] already masked with -inf; sink [H].  The sink adds exp(sink_h) to the
    denominator of every row and nothing else."""
    m = torch.maximum(scores.max(-1).values, sink[:, None])
    e = torch.exp(scores - m[..., None])
    return e / (e.sum(-1) + torch.exp(sink[:, None] - m))[..., None]


def latent_attention(h, W, p, m, eps, latent=None) -> Tuple[torch.Tensor, torch.Tensor]:
    """h [T, width] -> (mixer output [T, width], latent c [T, kv_rank]).  latent: another layer's c."""
    T, H, dk, dv = h.shape[0], m["heads"], m["dim"], m["vdim"]
    cq = norm_plain(h @ W[p + "dq"].T, W[p + "dq.norm"], eps)
    q = (cq @ W[p + "uq"].T).view(T, H, dk)
    c = latent if latent is not None else norm_plain(h @ W[p + "dkv"].T, W[p + "dkv.norm"], eps)
    k = (c @ W[p + "uk"].T).view(T, H, dk)
    v = (c @ W[p + "uv"].T).view(T, H, dv)
    s = torch.einsum("ihd,jhd->hij", q, k) * m["scale"]
    future = torch.triu(torch.ones(T, T, dtype=torch.bool), diagonal=1)
    s = s.masked_fill(future, -math.inf)
    pr = softmax_with_sink(s, W[p + "sink"])
    o = torch.einsum("hij,jhd->ihd", pr, v)
    o = o * torch.sigmoid(h @ W[p + "g"].T)[:, :, None]
    return o.reshape(T, H * dv) @ W[p + "o"].T, c


def hgrn2(h, W, p, m, eps) -> torch.Tensor:
    T, H, dk, dv = h.shape[0], m["heads"], m["dim"], m["vdim"]
    q = torch.nn.functional.silu(h @ W[p + "q"].T).view(T, H, dk)
    v = (h @ W[p + "v"].T).view(T, H, dv)
    low = W[p + "lower"]
    f = (low + (1.0 - low) * torch.sigmoid(h @ W[p + "f"].T + W[p + "f.b"])).view(T, H, dk)
    S = torch.zeros(H, dk, dv, dtype=h.dtype)
    o = torch.zeros(T, H, dv, dtype=h.dtype)
    for t in range(T):
        S = f[t][:, :, None] * S + (1.0 - f[t])[:, :, None] * v[t][:, None, :]
        o[t] = torch.einsum("hkv,hk->hv", S, q[t])
    o = norm_plain(o, W[p + "norm"], eps)
    return o.reshape(T, H * dv) @ W[p + "o"].T


def dense_ff(h, W, p) -> torch.Tensor:
    return (torch.nn.functional.silu(h @ W[p + "gate"].T) * (h @ W[p + "up"].T)) @ W[p + "down"].T


def routed_experts(h, W, p, experts: int, top: int) -> torch.Tensor:
    z = h @ W[p + "router"].T + W[p + "router.b"]
    val, idx = torch.topk(z, top, dim=-1)
    wt = torch.softmax(val, -1)
    y = torch.zeros(h.shape[0], W[p + "e0.down"].shape[0], dtype=h.dtype)
    for t in range(h.shape[0]):
        for j in range(top):
            e = int(idx[t, j])
            a = torch.relu(W[p + f"e{e}.up"] @ h[t]) ** 2
            y[t] += wt[t, j] * (W[p + f"e{e}.down"] @ a)
    return y


def forward(config: dict, weights: Dict[str, torch.Tensor], tokens) -> Tuple[torch.Tensor, List[torch.Tensor]]:
    """config: the config.json dictionary; -> (logits [T, vocab], residual after every layer)"""
    W = {k: v.to(F64) for k, v in weights.items()}
    eps = config["norm"]["eps"]
    x = W["embed"][torch.as_tensor(tokens, dtype=torch.long)]
    latents, after = {}, []
    for i, spec in enumerate(config["layers"]):
        p, m = f"l{i}.", spec["mixer"]
        h = norm_centred(x, W[p + "norm1"], eps)
        if spec["type"] == "latent_attention":
            src = m.get("kv_from")
            y, c = latent_attention(h, W, p + "mix.", m, eps, None if src is None else latents[src])
            if src is None:
                latents[i] = c
        else:
            y = hgrn2(h, W, p + "mix.", m, eps)
        y = y * torch.sigmoid(h @ W[p + "rg1"].T + W[p + "rg1.b"])
        x = x + norm_centred(y, W[p + "norm1b"], eps)
        mlp = spec.get("mlp")
        if mlp is not None:
            h = norm_centred(x, W[p + "norm2"], eps)
            if mlp["kind"] == "dense":
                y = dense_ff(h, W, p + "mlp.")
            else:
                y = routed_experts(h, W, p + "mlp.", mlp["router"]["experts"], mlp["router"]["top"])
            y = y * torch.sigmoid(h @ W[p + "rg2"].T + W[p + "rg2.b"])
            x = x + norm_centred(y, W[p + "norm2b"], eps)
        after.append(x.clone())
    return norm_centred(x, W["final.norm"], eps) @ W["head"].T, after


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
