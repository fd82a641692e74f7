"""Moronex: a decoder-only hybrid language model on the ragged-batch kernels.

Layer i is  x += norm1b(gate1 * mixer(norm1 x)),  x += norm2b(gate2 * ff(norm2 x))  with an fp32
residual stream x, zero-centred RMS-norm weights (1 + w) and element-wise sigmoid gates
gate = sigmoid(W_rg h + b) computed from the sublayer's own input h.  Mixers (config `layers[i].type`):

  latent_attention  queries through a normed low-rank latent, keys / values expanded per head from
                    ONE cached, normed latent c per token (optionally another layer's: `kv_from`),
                    no positional signal, causal softmax with a learned per-head sink in the
                    denominator, sigmoid output gate per head.  Run in the absorbed form: the key
                    expansion is folded into the queries and the value expansion applied after the
                    attention, so the kernels read the paged latent cache directly.
  hgrn2             gated linear recurrence S_t = diag(f_t) S_{t-1} + (1 - f_t) v_t^T, o_t = S_t^T q_t
                    with a lower-bounded forget gate, fp32 state carried per sequence slot.

Feed-forwards (`layers[i].mlp`): dense SwiGLU, routed experts (squared-ReLU experts, softmax over the
chosen logits), or none.

One step takes a RaggedBatch (rows of several sequences: prompt portions next to decoded tokens) and a
HybridCache (paged latents + recurrent state slots), both owned by the serving engine
(vila_b200/serving.py).  dtype bfloat16: projections on the tcgen05 GEMM (any shape it does not take
goes to the CUDA-core grouped kernel), everything the architecture wants in 32-bit in fp32 kernels.
dtype float32: the same kernels with fp32 tensors and the CUDA-core linear layer throughout.
"""
from __future__ import annotations

import json
import struct
from dataclasses import dataclass, field
from pathlib import Path
from typing import Dict, List, Optional

import torch

from .. import ops

ARCHITECTURE = "Moronex"


def _pad8(n: int) -> int:
    return (n + 7) // 8 * 8


@dataclass
class MoronexLayerConfig:
    type: str                       # "latent_attention" | "hgrn2"
    heads: int
    dim: int
    vdim: int
    q_rank: int = 0                 # latent_attention
    kv_rank: int = 0
    scale: float = 1.0
    kv_from: Optional[int] = None
    mlp_kind: Optional[str] = None  # "dense" | "moe" | None
    ff: int = 0                     # dense: hidden size; moe: hidden size of one expert
    experts: int = 0
    top: int = 0


@dataclass
class MoronexConfig:
    vocab: int
    width: int
    norm_eps: float
    layers: List[MoronexLayerConfig] = field(default_factory=list)
    architecture: str = ARCHITECTURE

    @staticmethod
    def from_dict(d: dict) -> "MoronexConfig":
        layers = []
        for spec in d["layers"]:
            m = spec["mixer"]
            lc = MoronexLayerConfig(type=spec["type"], heads=int(m["heads"]), dim=int(m["dim"]),
                                    vdim=int(m["vdim"]))
            if lc.type == "latent_attention":
                lc.q_rank, lc.kv_rank = int(m["q_rank"]), int(m["kv_rank"])
                lc.scale = float(m["scale"])
                lc.kv_from = None if m.get("kv_from") is None else int(m["kv_from"])
            elif lc.type != "hgrn2":
                raise ValueError(f"unknown mixer type {lc.type!r}")
            mlp = spec.get("mlp")
            if mlp is not None:
                lc.mlp_kind = mlp["kind"]
                if lc.mlp_kind == "dense":
                    lc.ff = int(mlp["ff"])
                elif lc.mlp_kind == "moe":
                    lc.ff = int(mlp["expert"]["ff"])
                    lc.experts, lc.top = int(mlp["router"]["experts"]), int(mlp["router"]["top"])
                else:
                    raise ValueError(f"unknown feed-forward kind {lc.mlp_kind!r}")
            layers.append(lc)
        return MoronexConfig(vocab=int(d["vocab"]), width=int(d["width"]), norm_eps=float(d["norm"]["eps"]),
                             layers=layers)

    def to_dict(self) -> dict:
        out = []
        for lc in self.layers:
            m = {"heads": lc.heads, "dim": lc.dim, "vdim": lc.vdim}
            if lc.type == "latent_attention":
                m.update(q_rank=lc.q_rank, kv_rank=lc.kv_rank, scale=lc.scale)
                if lc.kv_from is not None:
                    m["kv_from"] = lc.kv_from
            mlp = None
            if lc.mlp_kind == "dense":
                mlp = {"kind": "dense", "ff": lc.ff}
            elif lc.mlp_kind == "moe":
                mlp = {"kind": "moe", "expert": {"ff": lc.ff}, "router": {"experts": lc.experts, "top": lc.top}}
            out.append({"type": lc.type, "mixer": m, "mlp": mlp})
        return {"architecture": self.architecture, "layers": out, "norm": {"eps": self.norm_eps},
                "vocab": self.vocab, "width": self.width}

    def tensor_shapes(self) -> Dict[str, tuple]:
        """name -> shape of every checkpoint tensor (the layout `load_weights` expects)."""
        W, s = self.width, {}
        s["embed"] = (self.vocab, W)
        for i, lc in enumerate(self.layers):
            p = f"l{i}."
            for n in ("norm1", "norm1b"):
                s[p + n] = (W,)
            s[p + "rg1"], s[p + "rg1.b"] = (W, W), (W,)
            if lc.type == "latent_attention":
                s[p + "mix.dq"], s[p + "mix.dq.norm"] = (lc.q_rank, W), (lc.q_rank,)
                s[p + "mix.uq"] = (lc.heads * lc.dim, lc.q_rank)
                if lc.kv_from is None:
                    s[p + "mix.dkv"], s[p + "mix.dkv.norm"] = (lc.kv_rank, W), (lc.kv_rank,)
                s[p + "mix.uk"] = (lc.heads * lc.dim, lc.kv_rank)
                s[p + "mix.uv"] = (lc.heads * lc.vdim, lc.kv_rank)
                s[p + "mix.sink"], s[p + "mix.g"] = (lc.heads,), (lc.heads, W)
                s[p + "mix.o"] = (W, lc.heads * lc.vdim)
            else:
                hd = lc.heads * lc.dim
                s[p + "mix.q"], s[p + "mix.f"], s[p + "mix.f.b"], s[p + "mix.lower"] = (hd, W), (hd, W), (hd,), (hd,)
                s[p + "mix.v"], s[p + "mix.norm"] = (lc.heads * lc.vdim, W), (lc.vdim,)
                s[p + "mix.o"] = (W, lc.heads * lc.vdim)
            if lc.mlp_kind is not None:
                for n in ("norm2", "norm2b"):
                    s[p + n] = (W,)
                s[p + "rg2"], s[p + "rg2.b"] = (W, W), (W,)
            if lc.mlp_kind == "dense":
                s[p + "mlp.gate"], s[p + "mlp.up"], s[p + "mlp.down"] = (lc.ff, W), (lc.ff, W), (W, lc.ff)
            elif lc.mlp_kind == "moe":
                for e in range(lc.experts):
                    s[p + f"mlp.e{e}.up"], s[p + f"mlp.e{e}.down"] = (lc.ff, W), (W, lc.ff)
                s[p + "mlp.router"], s[p + "mlp.router.b"] = (lc.experts, W), (lc.experts,)
        s["final.norm"], s["head"] = (W,), (self.vocab, W)
        return s


_ST_DTYPES = {"BF16": torch.bfloat16, "F32": torch.float32, "F16": torch.float16, "I32": torch.int32,
              "I64": torch.int64}


def read_safetensors(path) -> Dict[str, torch.Tensor]:
    """Minimal safetensors reader: 8-byte little-endian header length, JSON header
    (name -> dtype, shape, data_offsets), then the raw little-endian data."""
    raw = Path(path).read_bytes()
    (n,) = struct.unpack("<Q", raw[:8])
    meta = json.loads(raw[8:8 + n])
    data = memoryview(raw)[8 + n:]
    out = {}
    for name, info in meta.items():
        if name == "__metadata__":
            continue
        a, b = info["data_offsets"]
        t = torch.frombuffer(bytearray(data[a:b]), dtype=_ST_DTYPES[info["dtype"]]) if b > a else \
            torch.empty(0, dtype=_ST_DTYPES[info["dtype"]])
        out[name] = t.reshape(info["shape"])
    return out


class _Layer:
    """Device tensors of one layer in the layout the kernels want."""


class MoronexForCausalLM:
    """Weights + the per-step compute of the architecture.  Sequences, pages, state slots, batching and
    sampling belong to `vila_b200.serving.TokenEngine`, which calls `forward_step` / `logits`."""

    unfolds_attention = True   # the engine may hand large prompt portions over as kv_tiles / ctx_rows

    def __init__(self, cfg: MoronexConfig, device="cuda", dtype=torch.bfloat16):
        assert dtype in (torch.bfloat16, torch.float32)
        self.config, self.device, self.dtype = cfg, torch.device(device), dtype
        self.vocab_size = cfg.vocab
        self.weights: Dict[str, torch.Tensor] = {}
        self.layers: List[_Layer] = []
        for i, lc in enumerate(cfg.layers):
            if lc.type == "latent_attention" and lc.kv_from is not None:
                src = cfg.layers[lc.kv_from]
                if not (0 <= lc.kv_from < i and src.type == "latent_attention" and src.kv_from is None
                        and src.kv_rank == lc.kv_rank):
                    raise ValueError(f"layer {i}: kv_from={lc.kv_from} must name an earlier latent-attention "
                                     "layer with its own latent of the same width")

    # ---- weights ----------------------------------------------------------------------------------
    @classmethod
    def from_pretrained(cls, model_dir, device="cuda", dtype=torch.bfloat16) -> "MoronexForCausalLM":
        d = Path(model_dir)
        cfg = MoronexConfig.from_dict(json.loads((d / "config.json").read_text()))
        files = sorted(d.glob("*.safetensors"))
        if not files:
            raise FileNotFoundError(f"no *.safetensors under {d}")
        tensors: Dict[str, torch.Tensor] = {}
        for f in files:
            tensors.update(read_safetensors(f))
        return cls(cfg, device, dtype).load_weights(tensors)

    def init_random(self, seed: int = 0, scale: float = 1.0, on_device: bool = False) -> "MoronexForCausalLM":
        """Random bf16-representable weights.  on_device: draw them on the model's device (large models)."""
        dev = self.device if on_device else torch.device("cpu")
        g = torch.Generator(device=dev).manual_seed(seed)
        t = {}
        for name, shape in self.config.tensor_shapes().items():
            if len(shape) == 2:
                v = torch.randn(shape, generator=g, device=dev) * (scale / shape[1] ** 0.5)
            elif name.endswith(".lower"):
                v = torch.rand(shape, generator=g, device=dev) * 0.9
            else:
                v = torch.randn(shape, generator=g, device=dev) * 0.1
            t[name] = v.to(torch.bfloat16)
        return self.load_weights(t)

    def load_weights(self, tensors: Dict[str, torch.Tensor]) -> "MoronexForCausalLM":
        """tensors: checkpoint name -> tensor ([out, in] linear weights).  Sizes are checked against the
        config; the fused / transposed device layouts are built here."""
        cfg, dev, dt = self.config, self.device, self.dtype
        want = cfg.tensor_shapes()
        missing = [n for n in want if n not in tensors]
        if missing:
            raise KeyError(f"checkpoint lacks {missing[:4]}{'...' if len(missing) > 4 else ''}")
        for n, shape in want.items():
            if tuple(tensors[n].shape) != tuple(shape):
                raise ValueError(f"{n}: checkpoint shape {tuple(tensors[n].shape)} != config shape {shape}")

        def w(name):  # compute-dtype copy
            return tensors[name].to(device=dev, dtype=dt).contiguous()

        def f32(name):
            return tensors[name].to(device=dev, dtype=torch.float32).contiguous()

        def cat_rows(names):
            """Stack projections that read the same input; every part starts at a multiple of 8 rows so
            its output columns are 16-byte aligned views.  -> (weight, {name: (offset, rows)})"""
            parts, offs, at = [], {}, 0
            for nm in names:
                t = w(nm)
                offs[nm] = (at, t.shape[0])
                pad = _pad8(t.shape[0]) - t.shape[0]
                parts.append(t)
                if pad:
                    parts.append(torch.zeros(pad, t.shape[1], device=dev, dtype=dt))
                at += t.shape[0] + pad
            return torch.cat(parts, 0).contiguous(), offs

        self.weights = {n: tensors[n] for n in want}
        self.embed, self.head, self.final_norm = w("embed"), w("head"), f32("final.norm")
        self.layers = []
        for i, lc in enumerate(cfg.layers):
            p, L = f"l{i}.", _Layer()
            L.cfg, L.index = lc, i
            L.norm1, L.norm1b, L.rg1_b = f32(p + "norm1"), f32(p + "norm1b"), f32(p + "rg1.b")
            if lc.type == "latent_attention":
                names = [p + "mix.dq"] + ([p + "mix.dkv"] if lc.kv_from is None else []) + [p + "mix.g", p + "rg1"]
                L.in_w, L.in_off = cat_rows(names)
                L.dq_norm = f32(p + "mix.dq.norm")
                L.dkv_norm = f32(p + "mix.dkv.norm") if lc.kv_from is None else None
                L.uq = w(p + "mix.uq")
                # key expansion per head, transposed: q'_h = uk_t[h] q_h, uk_t [H, R, dim]
                L.uk_t = w(p + "mix.uk").view(lc.heads, lc.dim, lc.kv_rank).transpose(1, 2).contiguous()
                L.uv = w(p + "mix.uv").view(lc.heads, lc.vdim, lc.kv_rank).contiguous()
                L.ukv, L.ukv_off = cat_rows([p + "mix.uk", p + "mix.uv"])   # un-folded form: one expansion GEMM
                L.sink = f32(p + "mix.sink")
                L.latent_layer = i if lc.kv_from is None else lc.kv_from
            else:
                L.in_w, L.in_off = cat_rows([p + "mix.q", p + "mix.f", p + "mix.v", p + "rg1"])
                L.f_bias, L.lower = f32(p + "mix.f.b"), f32(p + "mix.lower")
                L.out_norm = f32(p + "mix.norm")
            L.o = w(p + "mix.o")
            if lc.mlp_kind is not None:
                L.norm2, L.norm2b, L.rg2_b = f32(p + "norm2"), f32(p + "norm2b"), f32(p + "rg2.b")
                L.rg2 = w(p + "rg2")
            if lc.mlp_kind == "dense":
                gu = torch.empty(2 * lc.ff, cfg.width, device=dev, dtype=dt)  # rows gate_0, up_0, gate_1, ...
                gu[0::2], gu[1::2] = w(p + "mlp.gate"), w(p + "mlp.up")
                L.gu, L.down = gu, w(p + "mlp.down")
            elif lc.mlp_kind == "moe":
                L.up = torch.stack([w(p + f"mlp.e{e}.up") for e in range(lc.experts)]).contiguous()
                L.down = torch.stack([w(p + f"mlp.e{e}.down") for e in range(lc.experts)]).contiguous()
                L.router, L.router_b = f32(p + "mlp.router"), f32(p + "mlp.router.b")
            self.layers.append(L)
        return self

    def state_dict(self) -> Dict[str, torch.Tensor]:
        return dict(self.weights)

    def save_pretrained(self, model_dir) -> None:
        from safetensors.torch import save_file
        d = Path(model_dir)
        d.mkdir(parents=True, exist_ok=True)
        (d / "config.json").write_text(json.dumps(self.config.to_dict(), indent=1))
        save_file({k: v.detach().cpu().contiguous() for k, v in self.weights.items()}, str(d / "model.safetensors"))

    # ---- cache geometry (read by serving.HybridCache) ----------------------------------------------
    def latent_widths(self) -> Dict[int, int]:
        """layer index -> latent width, for the layers that own a paged latent cache"""
        return {i: lc.kv_rank for i, lc in enumerate(self.config.layers)
                if lc.type == "latent_attention" and lc.kv_from is None}

    def state_shapes(self) -> Dict[int, tuple]:
        """layer index -> (heads, dim, vdim) of the recurrent state a sequence keeps in its slot"""
        return {i: (lc.heads, lc.dim, lc.vdim) for i, lc in enumerate(self.config.layers) if lc.type == "hgrn2"}

    # ---- compute --------------------------------------------------------------------------------------
    def _lin(self, x: torch.Tensor, w: torch.Tensor, *, swiglu: bool = False, out_dtype=None) -> torch.Tensor:
        """x [M, K] · w[N, K]^T.  bf16 operands on the tcgen05 GEMM when it takes the shape."""
        N, K = w.shape
        if (x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and out_dtype in (None, torch.bfloat16)
                and K % 8 == 0 and N % 8 == 0 and x.stride(0) % 8 == 0 and x.data_ptr() % 16 == 0
                and (not swiglu or N % 32 == 0)):
            return ops.linear(x, w, swiglu=swiglu, static_w=True)
        return ops.glinear(x, w, swiglu=swiglu, out_dtype=out_dtype)

    def _latent_mixer(self, L: _Layer, h, batch, cache):
        lc, eps = L.cfg, self.config.norm_eps
        P = self._lin(h, L.in_w)
        a, n = L.in_off[f"l{L.index}.mix.dq"]
        cq = ops.rmsnorm_rows(P[:, a:a + n], L.dq_norm, eps)
        pool = cache.latent[L.latent_layer]
        if lc.kv_from is None:
            a, n = L.in_off[f"l{L.index}.mix.dkv"]
            ops.rmsnorm_rows(P[:, a:a + n], L.dkv_norm, eps, out=pool, out_rows=batch.cache_rows)
        q = self._lin(cq, L.uq)
        R, T = lc.kv_rank, h.shape[0]
        a, _ = L.in_off[f"l{L.index}.mix.g"]
        gate = P[:, a:a + lc.heads]
        o = None
        if batch.tiles is not None or batch.decode_tiles is not None:
            # folded form: attend over the cached latents themselves
            qa = ops.glinear(q, L.uk_t, groups=lc.heads, a_group_off=lc.dim, o_group_off=R, out_dtype=torch.float32)
            alloc = torch.zeros if batch.kv_tiles is not None else torch.empty   # rows of the other form stay finite
            ol = alloc(qa.shape, dtype=self.dtype, device=self.device)
            kw = dict(heads=lc.heads, page=cache.page, scale=lc.scale, sink=L.sink, gate=gate, out=ol)
            if batch.tiles is not None:
                ops.latent_attention(qa, pool, cache.page_tables, batch.tiles, **kw)
            if batch.decode_tiles is not None:
                ops.latent_attention(qa, pool, cache.page_tables, batch.decode_tiles, decode=True,
                                     nsplit=cache.decode_splits, **kw)
            o = ops.glinear(ol, L.uv, groups=lc.heads, a_group_off=R, o_group_off=lc.vdim)
        if batch.kv_tiles is not None:
            # un-folded form: expand keys and values of the whole context of these sequences once
            kv = self._lin(ops.gather_rows(pool, batch.ctx_rows), L.ukv)
            ka, kn = L.ukv_off[f"l{L.index}.mix.uk"]
            va, vn = L.ukv_off[f"l{L.index}.mix.uv"]
            if o is None:
                o = torch.empty(T, lc.heads * lc.vdim, dtype=self.dtype, device=self.device)
            ops.sink_attention(q, kv[:, ka:ka + kn], kv[:, va:va + vn], batch.kv_tiles, heads=lc.heads,
                               scale=lc.scale, sink=L.sink, gate=gate, out=o)
        a, n = L.in_off[f"l{L.index}.rg1"]
        return self._lin(o, L.o), P[:, a:a + n]

    def _hgrn2_mixer(self, L: _Layer, h, batch, cache):
        lc, eps = L.cfg, self.config.norm_eps
        P = self._lin(h, L.in_w)
        pre = f"l{L.index}."
        o = ops.hgrn2_scan(P, cache.state[L.index], batch.seqs, heads=lc.heads, dim=lc.dim, vdim=lc.vdim,
                           q_off=L.in_off[pre + "mix.q"][0], f_off=L.in_off[pre + "mix.f"][0],
                           v_off=L.in_off[pre + "mix.v"][0], f_bias=L.f_bias, lower=L.lower)
        on = ops.rmsnorm_rows(o.view(-1, lc.vdim), L.out_norm, eps, out_dtype=self.dtype).view(-1, lc.heads * lc.vdim)
        a, n = L.in_off[pre + "rg1"]
        return self._lin(on, L.o), P[:, a:a + n]

    def _experts(self, L: _Layer, h):
        lc = L.cfg
        T = h.shape[0]
        idx, wt = ops.moe_route(h, L.router, L.router_b, lc.top)
        seg, srt = ops.moe_group(idx, lc.experts)
        act = ops.glinear(h, L.up, groups=lc.experts, seg=seg, a_rows=srt, a_row_div=lc.top, act=ops.ACT_RELU2)
        return ops.glinear(act, L.down, groups=lc.experts, seg=seg, o_rows=srt, row_scale=wt.view(-1),
                           out_dtype=torch.float32, out_rows_total=T * lc.top)

    @torch.inference_mode()
    def forward_step(self, batch, cache, layer_outputs: Optional[list] = None) -> torch.Tensor:
        """Run the rows of `batch` through all layers on top of what `cache` holds; the latent rows and
        recurrent states of the batch are written to the cache.  -> residual stream fp32 [T, width]."""
        eps = self.config.norm_eps
        x = ops.embed_rows(self.embed, batch.ids)
        for L in self.layers:
            h = ops.rmsnorm_rows(x, L.norm1, eps, w_offset=1.0, out_dtype=self.dtype)
            mix = self._latent_mixer if L.cfg.type == "latent_attention" else self._hgrn2_mixer
            y, gate = mix(L, h, batch, cache)
            ops.gated_norm_residual(x, y, gate=gate, gate_bias=L.rg1_b, w=L.norm1b, w_offset=1.0, eps=eps)
            if L.cfg.mlp_kind is not None:
                h = ops.rmsnorm_rows(x, L.norm2, eps, w_offset=1.0, out_dtype=self.dtype)
                gate = self._lin(h, L.rg2)
                if L.cfg.mlp_kind == "dense":
                    y, nparts = self._lin(self._lin(h, L.gu, swiglu=True), L.down), 1
                else:
                    y, nparts = self._experts(L, h), L.cfg.top
                ops.gated_norm_residual(x, y, n_partials=nparts, gate=gate, gate_bias=L.rg2_b, w=L.norm2b,
                                        w_offset=1.0, eps=eps)
            if layer_outputs is not None:
                layer_outputs.append(x.clone())
        return x

    @torch.inference_mode()
    def logits(self, hidden_rows: torch.Tensor) -> torch.Tensor:
        """final norm + output head for the given residual rows fp32 [n, width] -> fp32 [n, vocab]"""
        h = ops.rmsnorm_rows(hidden_rows.contiguous(), self.final_norm, self.config.norm_eps, w_offset=1.0,
                             out_dtype=self.dtype)
        return ops.glinear(h, self.head, out_dtype=torch.float32)

    @torch.inference_mode()
    def generate(self, input_ids, max_new_tokens: int = 20, eos_token_id=None, do_sample: bool = False,
                 temperature: float = 1.0, top_k: int = 0, top_p: float = 1.0, seed: Optional[int] = None,
                 slots: int = 4, **engine_kw) -> List[List[int]]:
        """input_ids: one prompt (list of ids) or a list of prompts -> new ids per prompt, through the
        continuous-batching scheduler (vila_b200.serving.generate_tokens)."""
        from ..serving import generate_tokens
        prompts = [list(map(int, input_ids))] if input_ids and not isinstance(input_ids[0], (list, tuple)) \
            else [list(map(int, p)) for p in input_ids]
        eos = [] if eos_token_id is None else ([eos_token_id] if isinstance(eos_token_id, int) else list(eos_token_id))
        return generate_tokens(self, prompts, max_new_tokens, eos, slots=slots, sample=do_sample,
                               temperature=temperature, top_k=top_k, top_p=top_p, seed=seed, **engine_kw)
