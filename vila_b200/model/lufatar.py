"""Lufatar: a decoder-only language model with parallel sublayers on the ragged-batch kernels.

Residual stream x (fp32).  A token enters as its word row plus a hashed (previous token, token) pair
row.  Layer i updates

    x += m * (attention(c1(n1 x)) + experts(c2(n2 x)))        both sublayers read the same x
    x += m * unit(P_i (gelu(G_i x) * e_i(token))) * s_i        a per-layer slice of a per-token side table

with n = RMS norm in `norm.groups` pieces of the row, c = input + causal short convolution over time
(`canon.taps` taps, the last taps - 1 inputs are per-sequence state), m = `residual_mult`.  A block of
layers (`loop`) can run several times in a row with the same weights; every pass has its own cache and
state, and a per-pass vector is added to x before the block's first layer.

  attention   grouped-query heads, rotary positions on the first `rot.dims` columns (interleaved pairs),
              unit norm of q and k per head after the rotation, scores of all heads mixed by a
              [heads, heads] matrix before the softmax, softmax with 1 added to the denominator
              (a sink with logit 0), K | V rows in a paged pool per (layer, pass)
  experts     sigmoid router with a selection-only correction, group-limited top-k, un-normalised
              weights; experts are clamped gated units  min(g, L) * sigmoid(1.702 min(g, L)) * (clamp(u) + 1)

One step takes a RaggedBatch and a HybridCache owned by the serving engine (vila_b200/serving.py).
dtype bfloat16: projections on the tcgen05 GEMM (shapes it does not take go to the CUDA-core grouped
kernel); positions and angles, norms, scores and softmax, router, residual sums in fp32.  dtype float32:
the same kernels with fp32 tensors and the CUDA-core linear layer throughout.
"""
from __future__ import annotations

import json
from dataclasses import dataclass, field
from pathlib import Path
from typing import Dict, List, Optional, Tuple

import torch

from .. import ops
from .moronex import read_safetensors

ARCHITECTURE = "Lufatar"
GLU_ALPHA = 1.702   # fixed by the architecture: slope of the sigmoid inside the expert's gated unit


@dataclass
class LufatarLayerConfig:
    type: str                       # "attention"
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    rot_dims: int
    rot_base: float
    scale: float
    mlp_kind: Optional[str] = None  # "moe" | None
    ff: int = 0
    limit: float = 0.0
    experts: int = 0
    top: int = 0
    groups: int = 1
    keep: int = 1


@dataclass
class LufatarConfig:
    vocab: int
    width: int
    norm_eps: float
    norm_groups: int
    residual_mult: float
    taps: int
    buckets: int
    mul_prev: int
    mul_cur: int
    side_dim: int                   # 0: no per-token side input
    loop_start: int = 0
    loop_stop: int = 0              # stop <= start: nothing repeats
    loop_times: int = 1
    layers: List[LufatarLayerConfig] = field(default_factory=list)
    architecture: str = ARCHITECTURE

    @staticmethod
    def from_dict(d: dict) -> "LufatarConfig":
        layers = []
        for i, spec in enumerate(d["layers"]):
            if spec["type"] != "attention":
                raise ValueError(f"layer {i}: unknown mixer type {spec['type']!r}")
            m = spec["mixer"]
            lc = LufatarLayerConfig(type="attention", heads=int(m["heads"]), kv_heads=int(m["kv_heads"]),
                                    dim=int(m["dim"]), vdim=int(m["vdim"]), rot_dims=int(m["rot"]["dims"]),
                                    rot_base=float(m["rot"]["base"]), scale=float(m["scale"]))
            mlp = spec.get("mlp")
            if mlp is not None:
                if mlp["kind"] != "moe":
                    raise ValueError(f"layer {i}: unknown feed-forward kind {mlp['kind']!r}")
                r = mlp["router"]
                g = r.get("groups") or {"count": 1, "keep": 1}
                lc.mlp_kind, lc.ff, lc.limit = "moe", int(mlp["expert"]["ff"]), float(mlp["expert"]["limit"])
                lc.experts, lc.top = int(r["experts"]), int(r["top"])
                lc.groups, lc.keep = int(g["count"]), int(g["keep"])
            layers.append(lc)
        lp = d.get("loop") or {}
        side = d.get("token_side") or {}
        bg = d["embedding"]["bigram"]
        cfg = LufatarConfig(vocab=int(d["vocab"]), width=int(d["width"]), norm_eps=float(d["norm"]["eps"]),
                            norm_groups=int(d["norm"].get("groups", 1)), residual_mult=float(d["residual_mult"]),
                            taps=int(d["canon"]["taps"]), buckets=int(bg["buckets"]), mul_prev=int(bg["mul_prev"]),
                            mul_cur=int(bg["mul_cur"]), side_dim=int(side.get("dim", 0)),
                            loop_start=int(lp.get("start", 0)), loop_stop=int(lp.get("stop", 0)),
                            loop_times=int(lp.get("times", 1)), layers=layers)
        cfg.validate()
        return cfg

    def validate(self) -> None:
        if self.width % self.norm_groups:
            raise ValueError(f"width {self.width} is not a multiple of norm.groups {self.norm_groups}")
        if not 1 <= self.taps <= 16:
            raise ValueError(f"canon.taps {self.taps} not in 1..16")
        if self.loops and not (0 <= self.loop_start < self.loop_stop <= len(self.layers) and self.loop_times >= 1):
            raise ValueError(f"loop {self.loop_start}..{self.loop_stop} x {self.loop_times} does not fit "
                             f"{len(self.layers)} layers")
        for i, lc in enumerate(self.layers):
            if lc.heads % lc.kv_heads or lc.rot_dims % 2 or lc.rot_dims > lc.dim:
                raise ValueError(f"layer {i}: heads {lc.heads} / kv_heads {lc.kv_heads} / rot.dims {lc.rot_dims}")
            if lc.mlp_kind == "moe" and (lc.experts % lc.groups or not 1 <= lc.keep <= lc.groups or
                                         not 1 <= lc.top <= lc.keep * (lc.experts // lc.groups)):
                raise ValueError(f"layer {i}: router experts {lc.experts} top {lc.top} groups {lc.groups} keep {lc.keep}")

    @property
    def loops(self) -> bool:
        return self.loop_stop > self.loop_start

    def runs(self) -> List[Tuple[int, int]]:
        """(layer, pass) in execution order; pass -1: a layer outside the repeated block"""
        n, a, b = len(self.layers), self.loop_start, self.loop_stop
        if not self.loops:
            return [(i, -1) for i in range(n)]
        return [(i, -1) for i in range(a)] + [(i, t) for t in range(self.loop_times) for i in range(a, b)] + \
               [(i, -1) for i in range(b, n)]

    def to_dict(self) -> dict:
        out = []
        for lc in self.layers:
            m = {"dim": lc.dim, "heads": lc.heads, "kv_heads": lc.kv_heads,
                 "rot": {"base": lc.rot_base, "dims": lc.rot_dims}, "scale": lc.scale, "vdim": lc.vdim}
            mlp = None
            if lc.mlp_kind == "moe":
                mlp = {"expert": {"ff": lc.ff, "limit": lc.limit}, "kind": "moe",
                       "router": {"experts": lc.experts, "groups": {"count": lc.groups, "keep": lc.keep}, "top": lc.top}}
            out.append({"mixer": m, "mlp": mlp, "type": lc.type})
        d = {"architecture": self.architecture, "canon": {"taps": self.taps},
             "embedding": {"bigram": {"buckets": self.buckets, "mul_cur": self.mul_cur, "mul_prev": self.mul_prev}},
             "layers": out, "norm": {"eps": self.norm_eps, "groups": self.norm_groups},
             "residual_mult": self.residual_mult, "vocab": self.vocab, "width": self.width}
        if self.loops:
            d["loop"] = {"start": self.loop_start, "stop": self.loop_stop, "times": self.loop_times}
        if self.side_dim:
            d["token_side"] = {"dim": self.side_dim}
        return d

    def tensor_shapes(self) -> Dict[str, tuple]:
        """name -> shape of every checkpoint tensor (the layout `load_weights` expects)."""
        W, s = self.width, {}
        s["embed"], s["bigram"] = (self.vocab, W), (self.buckets + 1, W)
        if self.loops:
            s["loop.step"] = (self.loop_times, W)
        if self.side_dim:
            s["side.embed"] = (self.vocab, len(self.layers) * self.side_dim)
        for i, lc in enumerate(self.layers):
            p = f"l{i}."
            s[p + "norm1"], s[p + "canon1"] = (W,), (W, self.taps)
            s[p + "mix.q"], s[p + "mix.k"] = (lc.heads * lc.dim, W), (lc.kv_heads * lc.dim, W)
            s[p + "mix.v"], s[p + "mix.talk"] = (lc.kv_heads * lc.vdim, W), (lc.heads, lc.heads)
            s[p + "mix.o"] = (W, lc.heads * lc.vdim)
            if lc.mlp_kind == "moe":
                s[p + "norm2"], s[p + "canon2"] = (W,), (W, self.taps)
                for e in range(lc.experts):
                    s[p + f"mlp.e{e}.gate"], s[p + f"mlp.e{e}.up"] = (lc.ff, W), (lc.ff, W)
                    s[p + f"mlp.e{e}.down"] = (W, lc.ff)
                s[p + "mlp.router"], s[p + "mlp.correction"] = (lc.experts, W), (lc.experts,)
            if self.side_dim:
                s[p + "side.gate"], s[p + "side.proj"], s[p + "side.norm"] = (self.side_dim, W), (W, self.side_dim), (W,)
        s["final.norm"], s["head"] = (W,), (self.vocab, W)
        return s


class _Layer:
    """Device tensors of one layer in the layout the kernels want."""


class LufatarForCausalLM:
    """Weights + the per-step compute of the architecture.  Sequences, pages, state slots, batching and
    sampling belong to `vila_b200.serving.TokenEngine`, which calls `forward_step` / `logits`."""

    def __init__(self, cfg: LufatarConfig, device="cuda", dtype=torch.bfloat16):
        assert dtype in (torch.bfloat16, torch.float32)
        cfg.validate()
        self.config, self.device, self.dtype = cfg, torch.device(device), dtype
        self.vocab_size = cfg.vocab
        self.weights: Dict[str, torch.Tensor] = {}
        self.layers: List[_Layer] = []
        self._runs = cfg.runs()

    # ---- weights ----------------------------------------------------------------------------------
    @classmethod
    def from_pretrained(cls, model_dir, device="cuda", dtype=torch.bfloat16) -> "LufatarForCausalLM":
        d = Path(model_dir)
        cfg = LufatarConfig.from_dict(json.loads((d / "config.json").read_text()))
        files = sorted(d.glob("*.safetensors"))
        if not files:
            raise FileNotFoundError(f"no *.safetensors under {d}")
        tensors: Dict[str, torch.Tensor] = {}
        for f in files:
            tensors.update(read_safetensors(f))
        return cls(cfg, device, dtype).load_weights(tensors)

    def init_random(self, seed: int = 0, scale: float = 1.0, on_device: bool = False) -> "LufatarForCausalLM":
        """Random bf16-representable weights.  on_device: draw them on the model's device (large models)."""
        dev = self.device if on_device else torch.device("cpu")
        g = torch.Generator(device=dev).manual_seed(seed)
        t = {}
        for name, shape in self.config.tensor_shapes().items():
            if name.endswith(".talk"):
                v = torch.eye(shape[0], device=dev) + torch.randn(shape, generator=g, device=dev) * 0.3
            elif ".canon" in name:
                v = torch.randn(shape, generator=g, device=dev) * 0.3
            elif len(shape) == 2:
                v = torch.randn(shape, generator=g, device=dev) * (scale / shape[1] ** 0.5)
            elif name.endswith(".correction"):
                v = torch.randn(shape, generator=g, device=dev) * 0.2
            elif "norm" in name:
                v = 1.0 + torch.randn(shape, generator=g, device=dev) * 0.1
            else:
                v = torch.randn(shape, generator=g, device=dev) * 0.1
            t[name] = v.to(torch.bfloat16)
        return self.load_weights(t)

    def load_weights(self, tensors: Dict[str, torch.Tensor]) -> "LufatarForCausalLM":
        """tensors: checkpoint name -> tensor ([out, in] linear weights).  Sizes are checked against the
        config; the fused device layouts are built here."""
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

        self.weights = {n: tensors[n] for n in want}
        self.embed, self.pair, self.head, self.final_norm = w("embed"), w("bigram"), w("head"), f32("final.norm")
        self.loop_step = f32("loop.step") if cfg.loops else None
        self.side_embed = w("side.embed") if cfg.side_dim else None
        self.layers = []
        for i, lc in enumerate(cfg.layers):
            p, L = f"l{i}.", _Layer()
            L.cfg, L.index = lc, i
            L.norm1, L.canon1 = f32(p + "norm1"), f32(p + "canon1")
            L.qkv = torch.cat([w(p + "mix.q"), w(p + "mix.k"), w(p + "mix.v")], 0).contiguous()
            L.talk, L.o = f32(p + "mix.talk"), w(p + "mix.o")
            L.sink = torch.zeros(lc.heads, dtype=torch.float32, device=dev)   # exp(0) = the 1 in the denominator
            half = lc.rot_dims // 2
            L.inv_freq = None
            if half:
                L.inv_freq = (torch.tensor(lc.rot_base, dtype=torch.float64) **
                              (-2.0 * torch.arange(half, dtype=torch.float64) / lc.rot_dims)).to(dev)
            if lc.mlp_kind == "moe":
                L.norm2, L.canon2 = f32(p + "norm2"), f32(p + "canon2")
                gu = torch.empty(lc.experts, 2 * lc.ff, cfg.width, device=dev, dtype=dt)  # rows gate_0, up_0, gate_1, ...
                for e in range(lc.experts):
                    gu[e, 0::2], gu[e, 1::2] = w(p + f"mlp.e{e}.gate"), w(p + f"mlp.e{e}.up")
                L.gu = gu
                L.down = torch.stack([w(p + f"mlp.e{e}.down") for e in range(lc.experts)]).contiguous()
                L.router, L.correction = f32(p + "mlp.router"), f32(p + "mlp.correction")
            if cfg.side_dim:
                L.side_gate, L.side_proj, L.side_norm = w(p + "side.gate"), w(p + "side.proj"), f32(p + "side.norm")
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
        """layer run -> width of its paged per-token row: k (kv_heads * dim) | v (kv_heads * vdim)"""
        return {r: self.config.layers[i].kv_heads * (self.config.layers[i].dim + self.config.layers[i].vdim)
                for r, (i, _) in enumerate(self._runs)}

    def state_shapes(self) -> Dict[Tuple[int, int], tuple]:
        """(layer run, sublayer) -> (taps - 1, width): the last inputs of that sublayer's input convolution"""
        back = self.config.taps - 1
        if back == 0:
            return {}
        return {(r, k): (back, self.config.width) for r, (i, _) in enumerate(self._runs)
                for k in range(2 if self.config.layers[i].mlp_kind else 1)}

    # ---- compute --------------------------------------------------------------------------------------
    def _sublayer_inputs(self, L: _Layer, x, batch, cache, run: int):
        """group norm -> + causal short convolution, for the mixer and (if any) the feed-forward at once;
        reads and then advances the sequences' convolution states"""
        cfg = self.config
        norms, convs = [L.norm1], [L.canon1]
        if L.cfg.mlp_kind is not None:
            norms.append(L.norm2)
            convs.append(L.canon2)
        return ops.norm_conv_rows(x, norms, convs, [cache.state.get((run, k)) for k in range(len(norms))],
                                  batch.seqs, batch.row_seq,
                                  groups=cfg.norm_groups, eps=cfg.norm_eps, out_dtype=self.dtype)

    def _attention(self, L: _Layer, a, batch, cache, run: int):
        lc = L.cfg
        pool = cache.latent[run]
        qkv = ops.linear_any(a, L.qkv)
        q = ops.rope_append(qkv, batch.positions, batch.cache_rows, pool, heads=lc.heads, kv_heads=lc.kv_heads,
                            dim=lc.dim, vdim=lc.vdim, inv_freq=L.inv_freq, unit_norm=True, eps=self.config.norm_eps)
        o = torch.empty(a.shape[0], lc.heads * lc.vdim, dtype=self.dtype, device=self.device)
        kw = dict(heads=lc.heads, kv_heads=lc.kv_heads, dim=lc.dim, vdim=lc.vdim, page=cache.page, scale=lc.scale,
                  talk=L.talk, sink=L.sink, out=o)
        if batch.tiles is not None:
            ops.paged_attention(q, pool, cache.page_tables, batch.tiles, max_rows=16, **kw)
        if batch.decode_tiles is not None:
            ops.paged_attention(q, pool, cache.page_tables, batch.decode_tiles, max_rows=1,
                                nsplit=cache.decode_splits, **kw)
        return ops.linear_any(o, L.o)

    def _experts(self, L: _Layer, a):
        lc = L.cfg
        T = a.shape[0]
        idx, wt = ops.moe_route_sigmoid(a, L.router, L.correction, lc.top, lc.groups, lc.keep)
        seg, srt = ops.moe_group(idx, lc.experts)
        act = ops.glinear(a, L.gu, groups=lc.experts, seg=seg, a_rows=srt, a_row_div=lc.top,
                          glu_clamp=(GLU_ALPHA, lc.limit))
        return ops.glinear(act, L.down, groups=lc.experts, seg=seg, o_rows=srt, row_scale=wt.view(-1),
                           out_dtype=torch.float32, out_rows_total=T * lc.top)

    def _token_side(self, L: _Layer, x, xc, batch):
        """xc: x in the compute dtype (the gate projection's operand)"""
        cfg = self.config
        z = ops.linear_any(xc, L.side_gate)
        g = ops.gelu_mul_gather(z, self.side_embed, batch.ids, L.index * cfg.side_dim, out_dtype=self.dtype)
        y = ops.linear_any(g, L.side_proj)
        ops.gated_norm_residual(x, y, w=L.side_norm, eps=cfg.norm_eps, mult=cfg.residual_mult)

    @torch.inference_mode()
    def forward_step(self, batch, cache, layer_outputs: Optional[list] = None) -> torch.Tensor:
        """Run the rows of `batch` through all layer runs on top of what `cache` holds; K | V rows and the
        convolution states of the batch are written to the cache.  -> residual stream fp32 [T, width]."""
        cfg = self.config
        x = ops.embed_pair_rows(self.embed, self.pair, batch.ids, batch.prev_ids, cfg.mul_prev, cfg.mul_cur, cfg.buckets)
        for run, (i, t) in enumerate(self._runs):
            L = self.layers[i]
            if t >= 0 and i == cfg.loop_start:
                ops.add_row_vector(x, self.loop_step[t])
            a = self._sublayer_inputs(L, x, batch, cache, run)
            y = self._attention(L, a[0], batch, cache, run)
            parts, nparts = None, 1
            if L.cfg.mlp_kind is not None:
                parts, nparts = self._experts(L, a[1]), L.cfg.top
            xc = ops.residual_add_rows(x, y, parts, n_partials=nparts, mult=cfg.residual_mult,
                                       copy_dtype=self.dtype if cfg.side_dim else None)
            if cfg.side_dim:
                self._token_side(L, x, xc, batch)
            if layer_outputs is not None:
                layer_outputs.append(x.clone())
        return x

    @torch.inference_mode()
    def logits(self, hidden_rows: torch.Tensor) -> torch.Tensor:
        """final norm + output head for the given residual rows fp32 [n, width] -> fp32 [n, vocab]"""
        cfg = self.config
        h = ops.rmsnorm_rows(hidden_rows.contiguous(), self.final_norm, cfg.norm_eps, groups=cfg.norm_groups,
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
