"""Continuous batching over ONE shared paged KV pool.

The reference serialises requests (`serving/server.py:65-73` semaphore / global lock around
`model.generate_content`, one HF `generate` loop per request).  Decode at batch 1 is a pure weight
stream (14.14 GB per token for NVILA-8B): serving B requests from the same stream multiplies the
tokens per byte by B.  Here:

  * one paged pool `[L, 2, P, 128, Hkv, D]` holds the K/V of every slot; slot s owns the page-table row
    `page_tables[s]` (vLLM-style indirection: the kernels only ever see (pool, page-table row));
  * a request is admitted by prefilling it into a free slot (the ordinary tcgen05 prefill path writes
    straight into that slot's pages), its first token comes from the prefill;
  * ONE CUDA graph advances all slots by one token: per layer RMSNorm → q/k/v GEMM (swap-AB skinny
    tcgen05 kernel, M = slots: every weight byte is read once for the whole batch) → batched decode
    attention (`vila_decode_attention_batch`: one CTA per (query head, slot), RoPE + KV append fused,
    per-slot position and page-table row, idle slots skipped) → o-proj GEMM(+res) → RMSNorm → gate/up
    GEMM (SwiGLU epilogue) → down GEMM(+res); then lm_head GEMM, greedy arg-max, embedding gather and
    position++ — all on the device, no host sync per token;
  * finished slots (EOS / budget) are harvested and refilled between graph replays.
"""
from __future__ import annotations

from collections import deque
from typing import Deque, Dict, List, Optional, Sequence, Tuple

import torch

from . import ops

PAGE = 128


class _SlotCache:
    """The view of one slot that Qwen2ForCausalLM.prefill_hidden needs (PagedKVCache duck type)."""

    def __init__(self, pool: torch.Tensor, page_table: torch.Tensor):
        self.pool, self.page_table = pool, page_table
        self.length = 0
        self.max_tokens = page_table.numel() * PAGE
        self.n_pages = pool.shape[2]

    def k(self, layer: int) -> torch.Tensor:
        return self.pool[layer, 0]

    def v(self, layer: int) -> torch.Tensor:
        return self.pool[layer, 1]


class PageAllocator:
    """Free list over the physical pages of the shared pool (host-side bookkeeping only)."""

    def __init__(self, n_pages: int):
        self.free: List[int] = list(range(n_pages - 1, -1, -1))  # pop() hands out page 0 first
        self.n_pages = n_pages

    def alloc(self, n: int) -> List[int]:
        if n > len(self.free):
            raise MemoryError(f"KV pool exhausted: {n} pages wanted, {len(self.free)} free of {self.n_pages}")
        return [self.free.pop() for _ in range(n)]

    def release(self, pages: Sequence[int]) -> None:
        self.free.extend(reversed(list(pages)))

    @property
    def available(self) -> int:
        return len(self.free)


class BatchedDecoder:
    """`slots` concurrent greedy decodes of one Qwen2ForCausalLM over a shared paged pool.

    Pages are handed out on demand (PageAllocator): a slot holds ceil(tokens / 128) pages, grows page by
    page while it decodes and returns them when it is released, so `total_pages` can be smaller than
    slots * pages_per_slot (long and short requests share the pool).  The page-table rows live on the
    device and are read by the kernels at every launch: changing them needs no graph re-capture."""

    def __init__(self, llm, slots: int = 8, max_tokens_per_slot: int = 2048, max_new: int = 1024,
                 total_pages: Optional[int] = None):
        cfg = llm.config
        self.llm, self.slots = llm, slots
        dev, dt = llm.device, llm.dtype
        Hq, Hkv, D = cfg.num_attention_heads, cfg.num_key_value_heads, cfg.head_dim
        assert D == 128, "batched decode attention is specialised for head_dim 128"
        self.pages_per_slot = (max_tokens_per_slot + PAGE - 1) // PAGE
        assert self.pages_per_slot <= 32, "vila_decode_attention_batch serves contexts up to 4096 tokens"
        P = total_pages if total_pages is not None else slots * self.pages_per_slot
        self.pool = torch.zeros(cfg.num_hidden_layers, 2, P, PAGE, Hkv, D, device=dev, dtype=dt)
        self.allocator = PageAllocator(P)
        self.slot_pages: List[List[int]] = [[] for _ in range(slots)]
        # unassigned entries point at page 0; they are never dereferenced (tokens beyond a slot's length)
        self.page_tables = torch.zeros(slots, self.pages_per_slot, dtype=torch.int32, device=dev)
        self._pos_host = [-1] * slots  # host mirror of `positions` (advanced by run())
        self.positions = torch.full((slots,), -1, dtype=torch.int32, device=dev)  # < 0: idle slot
        self.x = torch.zeros(slots, cfg.hidden_size, device=dev, dtype=dt)
        self.attn = torch.zeros(slots, Hq * D, device=dev, dtype=dt)
        self.tokens = torch.zeros(slots, dtype=torch.int64, device=dev)
        self.max_new = max_new
        self.hist = torch.zeros(slots, max_new + 8, dtype=torch.int64, device=dev)
        self.step_idx = torch.zeros(slots, 1, dtype=torch.int64, device=dev)  # per-slot write column
        self.graph: Optional[torch.cuda.CUDAGraph] = None
        self.launches_per_step = 7 * cfg.num_hidden_layers + 2

    # ---- admission ------------------------------------------------------------------------------
    @torch.inference_mode()
    def admit(self, slot: int, inputs_embeds: torch.Tensor) -> None:
        """Prefill `inputs_embeds` [S, hidden] into the slot's pages and seed its decode state."""
        llm = self.llm
        S = inputs_embeds.shape[0]
        assert S + 1 <= self.pages_per_slot * PAGE, "prompt longer than a slot"
        self._ensure_pages(slot, S + 1)
        cache = _SlotCache(self.pool, self.page_tables[slot])
        hid = llm.prefill_hidden(inputs_embeds, cache)
        logits = llm.logits_from_hidden(hid[-1:])
        tok = torch.argmax(logits[0].float())
        self.tokens[slot] = tok
        self.hist[slot, 0] = tok
        self.step_idx[slot, 0] = 1
        self.x[slot] = llm.model.embed_tokens.weight[tok]
        self.positions[slot] = S  # position of the token just chosen == tokens cached so far
        self._pos_host[slot] = S

    def release(self, slot: int) -> None:
        self.positions[slot] = -1
        self._pos_host[slot] = -1
        self.allocator.release(self.slot_pages[slot])
        self.slot_pages[slot] = []

    def _ensure_pages(self, slot: int, n_tokens: int) -> None:
        """make sure the slot owns pages for its first n_tokens tokens"""
        need = min(self.pages_per_slot, (n_tokens + PAGE - 1) // PAGE) - len(self.slot_pages[slot])
        if need > 0:
            new = self.allocator.alloc(need)
            first = len(self.slot_pages[slot])
            self.slot_pages[slot].extend(new)
            self.page_tables[slot, first:first + need] = torch.tensor(new, dtype=torch.int32,
                                                                      device=self.page_tables.device)

    # ---- one decode step for every active slot ----------------------------------------------------
    def _step(self) -> None:
        llm, cfg = self.llm, self.llm.config
        Hq, Hkv, D = cfg.num_attention_heads, cfg.num_key_value_heads, cfg.head_dim
        x = self.x
        for li, layer in enumerate(llm.model.layers):
            h = ops.rmsnorm(x, layer.input_layernorm.weight, cfg.rms_norm_eps)
            qkv = ops.linear(h, layer._qkv_w, layer._qkv_b, static_w=True)
            ops.decode_attention_batch(qkv, self.positions, self.pool[li, 0], self.pool[li, 1],
                                       self.page_tables, self.attn, llm.inv_freq, Hq, Hkv, D, D ** -0.5)
            ops.linear(self.attn, layer.self_attn.o_proj.weight, residual=x, out=x, static_w=True)
            h = ops.rmsnorm(x, layer.post_attention_layernorm.weight, cfg.rms_norm_eps)
            a = ops.linear(h, layer._gu_w, swiglu=True, static_w=True)
            ops.linear(a, layer.mlp.down_proj.weight, residual=x, out=x, static_w=True)
        h = ops.rmsnorm(x.clone(), llm.model.norm.weight, cfg.rms_norm_eps)
        logits = ops.linear(h, llm.lm_head.weight, static_w=True)
        active = self.positions >= 0
        tok = torch.argmax(logits.float(), dim=-1)
        self.tokens.copy_(torch.where(active, tok, self.tokens))
        col = self.step_idx.clamp(max=self.hist.shape[1] - 1)
        self.hist.scatter_(1, col, self.tokens[:, None])
        self.step_idx.add_(active[:, None].to(torch.int64))
        x.copy_(ops.embed_splice(llm.model.embed_tokens.weight, None, self.tokens.to(torch.int32)))
        self.positions.add_(active.to(torch.int32))

    @torch.inference_mode()
    def run(self, n_tokens: int) -> None:
        if self.graph is None:
            raise RuntimeError("call capture() (with every slot idle) before run()")
        for s_ in range(self.slots):  # pages for the tokens this call will append
            if self._pos_host[s_] >= 0:
                self._ensure_pages(s_, self._pos_host[s_] + n_tokens + 1)
                self._pos_host[s_] += n_tokens
        for _ in range(n_tokens):
            self.graph.replay()

    @torch.inference_mode()
    def capture(self) -> None:
        """Capture the step graph.  Must be called with every slot idle (positions < 0): the capture
        launches the kernels once, idle slots are skipped by the attention kernel and leave no trace."""
        if self.graph is not None:
            return
        assert bool((self.positions < 0).all()), "capture() with idle slots only"
        saved = (self.tokens.clone(), self.hist.clone(), self.step_idx.clone(), self.x.clone())
        self._step()  # eager warm-up (allocator, function attributes); state restored below
        torch.cuda.synchronize()
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g):
            self._step()
        self.graph = g
        for dst, src in zip((self.tokens, self.hist, self.step_idx, self.x), saved):
            dst.copy_(src)

    def generated(self, slot: int) -> List[int]:
        n = int(self.step_idx[slot, 0])
        return self.hist[slot, :n].tolist()


@torch.inference_mode()
def generate_batch(llm, prompts: Sequence[torch.Tensor], max_new_tokens: int, eos_token_ids: Sequence[int] = (),
                   slots: int = 8, max_tokens_per_slot: int = 2048, check_every: int = 8,
                   decoder: Optional[BatchedDecoder] = None, total_pages: Optional[int] = None) -> List[List[int]]:
    """Greedy-decode `prompts` (list of inputs_embeds [S_i, hidden]) with continuous batching: at most
    `slots` requests in flight; a finished request (EOS or max_new_tokens) frees its slot for the next
    one in the queue.  Returns the new ids per request (EOS included), in request order."""
    dec = decoder or BatchedDecoder(llm, slots, max_tokens_per_slot, max_new=max_new_tokens,
                                    total_pages=total_pages)
    dec.capture()
    cap = dec.pages_per_slot * PAGE
    for p in prompts:
        if p.shape[0] + max_new_tokens + check_every > cap:
            raise ValueError(f"prompt of {p.shape[0]} tokens + {max_new_tokens} new tokens exceeds the slot ({cap})")
    queue: Deque[int] = deque(range(len(prompts)))
    owner: Dict[int, int] = {}           # slot -> request
    out: List[Optional[List[int]]] = [None] * len(prompts)
    eos = set(int(e) for e in eos_token_ids)

    def harvest(slot: int, ids: List[int]) -> Optional[List[int]]:
        for i, t in enumerate(ids):
            if t in eos:
                return ids[:i + 1]
        return ids[:max_new_tokens] if len(ids) >= max_new_tokens else None

    while queue or owner:
        for s in range(dec.slots):
            if s not in owner and queue:
                # admit only when the pool can hold the prompt and the request's whole budget
                need = (prompts[queue[0]].shape[0] + max_new_tokens + check_every + PAGE - 1) // PAGE
                if need > dec.allocator.available and owner:
                    break  # wait for a running request to finish and return its pages
                r = queue.popleft()
                dec.admit(s, prompts[r])
                owner[s] = r
        dec.run(check_every)
        for s in list(owner):
            done = harvest(s, dec.generated(s))
            if done is not None:
                out[owner.pop(s)] = done
                dec.release(s)
    return [o or [] for o in out]


# =====================================================================================================
# Ragged-batch token engine: prompt portions and decoded tokens of several sequences in ONE step.
# =====================================================================================================
# The decoders above admit a request by prefilling it alone and then advance all slots one token per
# graph replay.  Models whose per-sequence memory is more than K/V pages (a paged latent for the
# attention layers plus a fixed-size recurrent state for the linear-recurrence layers) are served by
# the engine below: every step is a ragged batch (any number of rows per sequence), sequences own
# pages from the shared free list (PageAllocator, as above) and one state slot each, and both are
# handed back on release and reused by later sequences.  The scheduler on top (generate_tokens) does
# continuous batching with chunked prefill; the model only sees (RaggedBatch, HybridCache).

import numpy as np  # noqa: E402

from .sampling import pick_token  # noqa: E402

LATENT_PAGE = 64
TILE_ROWS = 16  # rows of one sequence per attention tile (vila_latent_attention)


class RaggedBatch:
    """Device-side description of one step.  Row t of the batch is token ids[t]; rows of one sequence
    are consecutive.  seqs [n, 4] = (first row, rows, position of the first row, slot) per sequence;
    tiles = the multi-row sequences cut into <= 16-row pieces, decode_tiles = the single-row ones
    (same 4 columns); cache_rows[t] = pool row of token t in the paged caches; positions[t] = position of
    token t in its sequence; prev_ids[t] = the token before it in its sequence (-1: none; the last token
    of the previous step for a row that starts a portion); row_seq[t] = index of its sequence in seqs."""

    def __init__(self, ids, cache_rows, seqs, tiles, decode_tiles, ctx_rows=None, kv_tiles=None,
                 positions=None, prev_ids=None, row_seq=None):
        self.ids, self.cache_rows, self.seqs = ids, cache_rows, seqs
        self.positions, self.prev_ids, self.row_seq = positions, prev_ids, row_seq
        self.tiles, self.decode_tiles = tiles, decode_tiles
        # un-folded attention for prompt portions that are a large part of their context: ctx_rows = pool
        # rows of ALL positions of those sequences, kv_tiles = their tiles as (row0, rows, pos0, first row
        # of the sequence inside ctx_rows); `tiles` is None then
        self.ctx_rows, self.kv_tiles = ctx_rows, kv_tiles
        self.T = ids.numel()


class HybridCache:
    """Per-sequence memory of a model: paged pools [pages * page, width] of per-token rows (a latent per
    layer that owns one, or k | v rows per attention layer run), state pools [slots, *shape] fp32 of
    fixed-size per-sequence state (a recurrent matrix, the last inputs of a short convolution), one
    page-table row per slot.  The geometry comes from the model: latent_widths() / state_shapes() map a key
    of the model's choosing (a layer index, a (layer, pass) pair) to a row width / a state shape."""

    def __init__(self, model, max_tokens: int, slots: int, page: int = LATENT_PAGE):
        dev = model.device
        self.page, self.slots = page, slots
        self.n_pages = max(1, (max_tokens + page - 1) // page)
        # decoded tokens: CTAs per (row, head) of the attention over the cache; fixed per pool so that a
        # captured decode graph stays valid while the contexts grow (about one CTA per 256 cached tokens)
        self.decode_splits = min(16, max(1, self.n_pages * page // 256))
        self.latent = {i: torch.zeros(self.n_pages * page, r, device=dev, dtype=model.dtype)
                       for i, r in model.latent_widths().items()}
        self.state = {i: torch.zeros(slots, *shape, device=dev, dtype=torch.float32)
                      for i, shape in model.state_shapes().items()}
        self.page_tables = torch.zeros(slots, self.n_pages, dtype=torch.int32, device=dev)
        self.page_tables_host = np.zeros((slots, self.n_pages), dtype=np.int32)
        self.allocator = PageAllocator(self.n_pages)
        self.free_slots: List[int] = list(range(slots - 1, -1, -1))


class _Sequence:
    __slots__ = ("slot", "pages", "length", "last_token")

    def __init__(self, slot: int):
        self.slot, self.pages, self.length = slot, [], 0
        self.last_token = -1   # the token before the next one to come (-1: the sequence is empty)


class TokenEngine:
    """Step function + cache / state manager for token-id language models (model.forward_step,
    model.logits).  `max_tokens` bounds the tokens live sequences hold together (each rounded up to a
    page), `slots` the number of live sequences."""

    def __init__(self, model, max_tokens: int, slots: int = 4, page: int = LATENT_PAGE, graphs: bool = True):
        self.model = model
        self.cache = HybridCache(model, max_tokens, slots, page)
        self.seqs: Dict[object, _Sequence] = {}
        # steps made of single decoded tokens only: one CUDA graph per row count (index arrays live in
        # static buffers, page tables and state pools are static already); a row count is run eagerly
        # the first time it occurs, captured the second time, replayed from then on
        # prompt portions whose rows x unfold_ratio reach the context they attend to are served by expanding
        # keys / values once per step (4x fewer attention flops at kv_rank = 4 x head size); 0: never
        self.unfold_ratio = 4 if getattr(model, "unfolds_attention", False) else 0
        self.graphs = graphs
        self._decode_graphs: Dict[int, tuple] = {}
        self._decode_seen: Dict[int, int] = {}

    # ---- sequences --------------------------------------------------------------------------------
    def admit(self, seq_id) -> _Sequence:
        if seq_id in self.seqs:
            return self.seqs[seq_id]
        if not self.cache.free_slots:
            raise MemoryError(f"no free state slot ({self.cache.slots} live sequences)")
        s = self.seqs[seq_id] = _Sequence(self.cache.free_slots.pop())
        return s

    def release(self, seq_id) -> None:
        s = self.seqs.pop(seq_id, None)
        if s is None:
            return
        self.cache.allocator.release(s.pages)
        self.cache.free_slots.append(s.slot)

    def length(self, seq_id) -> int:
        return self.seqs[seq_id].length

    def _reserve(self, s: _Sequence, tokens: int) -> bool:
        c = self.cache
        need = (tokens + c.page - 1) // c.page - len(s.pages)
        if need <= 0:
            return False
        new = c.allocator.alloc(need)
        c.page_tables_host[s.slot, len(s.pages):len(s.pages) + need] = new
        s.pages.extend(new)
        return True

    # ---- one step -----------------------------------------------------------------------------------
    def _build(self, entries):
        c, dev = self.cache, self.model.device
        ids, rows, seqs, tiles, dec, want_rows = [], [], [], [], [], []
        poss, prevs, rseq = [], [], []
        ctx, kv_tiles, ctx_at = [], [], 0
        dirty, at = False, 0
        for seq_id, tokens, want in entries:
            n = len(tokens)
            if n == 0:
                continue
            s = self.admit(seq_id)
            dirty |= self._reserve(s, s.length + n)
            pos = np.arange(s.length, s.length + n)
            pages = np.asarray(s.pages, dtype=np.int64)
            rows.append(pages[pos // c.page] * c.page + pos % c.page)
            ids.append(np.asarray(tokens, dtype=np.int64))
            poss.append(pos)
            prevs.append(np.concatenate(([s.last_token], ids[-1][:-1])))
            rseq.append(np.full(n, len(seqs)))
            s.last_token = int(tokens[-1])
            seqs.append((at, n, s.length, s.slot))
            if n == 1:
                dec.append((at, 1, s.length, s.slot))
            else:
                for o in range(0, n, TILE_ROWS):
                    tiles.append((at + o, min(TILE_ROWS, n - o), s.length + o, s.slot))
                    if self.unfold_ratio > 0:
                        kv_tiles.append((at + o, min(TILE_ROWS, n - o), s.length + o, ctx_at))
                if self.unfold_ratio > 0:
                    allpos = np.arange(0, s.length + n)
                    ctx.append(pages[allpos // c.page] * c.page + allpos % c.page)
                    ctx_at += s.length + n
            want_rows.extend(at + int(k) for k in want)
            s.length += n
            at += n
        if dirty:
            c.page_tables.copy_(torch.from_numpy(c.page_tables_host))
        tile_rows = sum(t[1] for t in tiles)
        unfold = bool(tiles) and self.unfold_ratio > 0 and tile_rows * self.unfold_ratio >= ctx_at
        if unfold:
            tiles = []
        else:
            ctx, kv_tiles = [], []
        # one host->device copy for all index arrays of the step
        parts = [np.concatenate(ids), np.concatenate(rows), np.asarray(seqs).reshape(-1),
                 np.asarray(tiles).reshape(-1), np.asarray(dec).reshape(-1),
                 np.concatenate(ctx) if ctx else np.zeros(0), np.asarray(kv_tiles).reshape(-1),
                 np.concatenate(poss), np.concatenate(prevs), np.concatenate(rseq)]
        flat = torch.from_numpy(np.concatenate(parts).astype(np.int32))
        return flat, [p.size for p in parts], want_rows

    @staticmethod
    def _views(flat: torch.Tensor, sizes) -> RaggedBatch:
        cuts = np.cumsum([0] + list(sizes))
        v = [flat[cuts[i]:cuts[i + 1]] for i in range(len(sizes))]
        return RaggedBatch(v[0], v[1], v[2].view(-1, 4), v[3].view(-1, 4) if sizes[3] else None,
                           v[4].view(-1, 4) if sizes[4] else None, v[5] if sizes[5] else None,
                           v[6].view(-1, 4) if sizes[6] else None, v[7], v[8], v[9])

    def _decode_step_graphed(self, flat, sizes) -> Tuple[torch.Tensor, torch.Tensor]:
        """All rows are single decoded tokens: replay (or capture) the graph of this row count.
        -> (residual rows, logits of ALL rows); both are static graph outputs."""
        T = sizes[0]
        ent = self._decode_graphs.get(T)
        if ent is None:
            static = torch.empty(flat.numel(), dtype=torch.int32, device=self.model.device)
            static.copy_(flat)
            batch = self._views(static, sizes)
            torch.cuda.synchronize()
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g):
                x = self.model.forward_step(batch, self.cache)
                lg = self.model.logits(x)
            ent = self._decode_graphs[T] = (g, static, x, lg)
        g, static, x, lg = ent
        static.copy_(flat)
        g.replay()
        return x, lg

    @torch.inference_mode()
    def step(self, entries, layer_outputs: Optional[list] = None) -> Optional[torch.Tensor]:
        """entries: (sequence id, next token ids, indices among them whose logits are wanted).  All
        entries run as one batch on top of what earlier steps cached.  -> fp32 logits [wanted, vocab]
        in entry / index order (None if nothing is wanted)."""
        entries = [e for e in entries if len(e[1])]
        if not entries:
            return None
        flat, sizes, want_rows = self._build(entries)
        T = sizes[0]
        decode_only = sizes[3] == 0 and sizes[6] == 0 and layer_outputs is None
        if self.graphs and decode_only and self._decode_seen.get(T, 0) >= 1:
            x, all_logits = self._decode_step_graphed(flat, sizes)
            if not want_rows:
                return None
            sel = torch.tensor(want_rows, dtype=torch.long, device=x.device)
            return all_logits.index_select(0, sel)
        if decode_only:
            self._decode_seen[T] = self._decode_seen.get(T, 0) + 1
        x = self.model.forward_step(self._views(flat.to(self.model.device), sizes), self.cache, layer_outputs)
        if not want_rows:
            return None
        sel = torch.tensor(want_rows, dtype=torch.long, device=x.device)
        return self.model.logits(x.index_select(0, sel))


@torch.inference_mode()
def generate_tokens(model, prompts: Sequence[Sequence[int]], max_new_tokens: int,
                    eos_token_ids: Sequence[int] = (), *, slots: int = 4, max_tokens: Optional[int] = None,
                    max_step_tokens: int = 2048, sample: bool = False, temperature: float = 1.0,
                    top_k: int = 0, top_p: float = 1.0, seed: Optional[int] = None,
                    engine: Optional[TokenEngine] = None) -> List[List[int]]:
    """Continuous batching with chunked prefill over a TokenEngine: at most `slots` sequences live; each
    step carries one token of every decoding sequence plus prompt portions of the others up to
    `max_step_tokens` rows; a sequence is admitted when a slot is free and the pool can hold its prompt
    and its whole budget; finished ones (EOS / budget) hand pages and slot to the queue.
    -> new ids per prompt (EOS included), in prompt order."""
    page = engine.cache.page if engine is not None else LATENT_PAGE

    def pages_for(r):
        return (len(prompts[r]) + max_new_tokens + page - 1) // page

    if engine is None:
        live = sorted((pages_for(r) for r in range(len(prompts))), reverse=True)[:slots]
        engine = TokenEngine(model, max_tokens or max(1, sum(live)) * page, slots, page)
    for r in range(len(prompts)):
        if len(prompts[r]) == 0:
            raise ValueError("empty prompt")
        if pages_for(r) > engine.cache.n_pages:
            raise ValueError(f"prompt {r}: {len(prompts[r])} + {max_new_tokens} tokens exceed the cache pool")
    gen = torch.Generator(device=model.device).manual_seed(seed) if (sample and seed is not None) else None
    eos = set(int(e) for e in eos_token_ids)
    queue: Deque[int] = deque(range(len(prompts)))
    live: Dict[int, dict] = {}
    out: List[List[int]] = [[] for _ in prompts]
    reserved = 0
    while queue or live:
        while queue and engine.cache.free_slots and len(live) < slots and \
                reserved + pages_for(queue[0]) <= engine.cache.n_pages:
            r = queue.popleft()
            engine.admit(("gen", r))
            live[r] = {"tokens": list(prompts[r]), "fed": 0}
            reserved += pages_for(r)
        budget, entries, asked = max_step_tokens, [], []
        for r, st in sorted(live.items(), key=lambda kv: len(kv[1]["tokens"]) - kv[1]["fed"]):
            n = min(len(st["tokens"]) - st["fed"], budget)  # decoding sequences (1 row) come first
            if n <= 0:
                continue
            chunk = st["tokens"][st["fed"]:st["fed"] + n]
            last = st["fed"] + n == len(st["tokens"])
            entries.append((("gen", r), chunk, [n - 1] if last else []))
            if last:
                asked.append(r)
            st["fed"] += n
            budget -= n
        logits = engine.step(entries)
        for k, r in enumerate(asked):
            tok = pick_token(logits[k], sample, temperature, top_k, top_p, gen)
            out[r].append(tok)
            live[r]["tokens"].append(tok)
            if tok in eos or len(out[r]) >= max_new_tokens:
                engine.release(("gen", r))
                reserved -= pages_for(r)
                del live[r]
    return out
