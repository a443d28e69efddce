"""Grouped-query attention over the cache, with optional per-head q/k RMSNorm.

For the new tokens of a step (skyla-ref/src/model.rs:124-172):
``q = Wq h``, ``k = Wk h``, ``v = Wv h`` (no bias); each q and k head is
RMS-normed with one ``[head_dim]`` weight, then rotated at its absolute position;
k and v go to the cache; query head ``h`` attends the cache of key/value head
``h // (heads / kv_heads)`` with ``softmax(q.k * scale)`` over the positions it
may see; the heads are concatenated, projected by ``Wo`` and added to the
residual stream (the add is fused into the product's epilogue, as the reference
does with its ACCUM matvec, skyla-engine/src/graph.rs:110-112).

Parameters: ``hidden_size``, ``num_heads``, ``num_kv_heads``, ``head_dim``,
``qk_norm``, ``qk_norm_eps``, ``scale`` (``None``: ``1/sqrt(head_dim)``),
``window`` (``None``: all earlier positions), ``position`` (a position part spec),
``cache_dtype`` (``None``: the runtime's; ``"float32"`` keeps this mixer's keys and values
in 32-bit even where activations are 16-bit: its layers then form a cache group of
their own and run on the plain kernels).
The three input projections are stored as one matrix so that a step needs one
product for them.
"""
from __future__ import annotations

import math
from typing import Dict, Optional

import torch

from ..cache.kv import KVNeed
from ..kernels import ops
from ..weights.loader import TensorDecl
from .base import NormedInput, Part, StepPlan, build_part, register_mixer
from .linear import ACCUMULATE, STORE, Linear


class DecodePages(StepPlan):
    """Which pages each block of a decode attention launch reads (``ops.decode_plan``): the same for
    every layer with these key/value heads and this window, so it is made once a step, on the host."""

    def __init__(self, nkv: int, window: int, n_sms: int):
        self.nkv, self.window, self.n_sms = nkv, window, n_sms
        self.key = ("decode pages", nkv, window)
        self._blocks = {}

    def blocks(self, n_seqs: int, pages_width: int) -> int:
        """How many blocks share a decode step's pages.

        Two blocks share an SM, and all of them run at once.  A block costs about three pages' time
        beside its pages (a page takes about 1 us), each further item that it starts about as much
        again, and every piece that an item is read in about 0.3 more in the merge (fitted to
        measurements at batch 1 to 64).  The count is fixed per (batch, width of the page lists), so
        that a recorded launch keeps its grid; which pages a block reads follows the step's lengths.
        """
        got = self._blocks.get((n_seqs, pages_width))
        if got is None:
            items = max(1, self.nkv * n_seqs)
            total = items * max(1.0, 0.75 * pages_width)
            best_cost = None
            for n in range(1, 2 * self.n_sms + 1):
                cost = 3.0 + -(-total // n) + 0.3 * (n / items + 1) + 2.5 * max(0.0, items / n - 1)
                if best_cost is None or cost < best_cost:
                    got, best_cost = n, cost
            self._blocks[(n_seqs, pages_width)] = got
        return got

    def size(self, n_seqs: int, pages_width: int, decode: bool) -> int:
        return ops.decode_plan_ints(n_seqs, self.nkv, self.blocks(n_seqs, pages_width)) if decode else 0

    def fill(self, out, starts, ns, page_size: int) -> None:
        n_blocks = (out.size - 2 * len(starts) * self.nkv) // ops.DECODE_PLAN_INTS
        ops.decode_plan(starts, self.nkv, self.window, page_size, n_blocks, out)


class GQAttention(Part):
    graph_safe = True
    takes_normed_input = True
    kernel_modules = Linear.kernel_modules + ("attn_prep", "attention_plain", "attention_mma", "attention_tc")

    def __init__(self, spec, rt):
        super().__init__(spec, rt)
        p = spec.params
        self.hidden = int(p["hidden_size"])
        self.nq = int(p["num_heads"])
        self.nkv = int(p["num_kv_heads"])
        self.hd = int(p["head_dim"])
        if self.nq % self.nkv:
            raise ValueError(f"{self.nq} query heads do not divide into {self.nkv} key/value heads")
        self.qk_norm = bool(p.get("qk_norm", False))
        self.eps = float(p.get("qk_norm_eps", 0.0))
        self.scale = float(p["scale"]) if p.get("scale") is not None else 1.0 / math.sqrt(self.hd)
        self.window = int(p["window"]) if p.get("window") else 0
        cdt = p.get("cache_dtype")
        if cdt not in (None, "float32", "bfloat16"):
            raise ValueError(f"cache_dtype must be float32 or bfloat16, not {cdt!r}")
        self.cache_dtype = None if cdt is None else getattr(torch, cdt)
        pos = p.get("position")
        self.position = build_part("position", pos, rt) if pos is not None else None
        self.q_norm_w = self.k_norm_w = None
        # tensor-core attention: head sizes 16..128 in steps of 16 (prompts: 1); decode also
        # needs the query heads of a key/value head to fit one 16-row tile (2)
        self._fast = 0
        if not rt.full_precision and self.hd % 16 == 0 and 16 <= self.hd <= 128:
            self._fast = 2 if self.nq // self.nkv <= 16 else 1
        #: the prompt attention kernels work on tiles of consecutive new tokens of one sequence; the step's
        #: batch builder makes the tile lists that the model's mixers ask for here
        self.token_tiles = (ops.PREFILL_TILE,) if self._fast else ()
        #: and, for steps of one token per sequence, which pages each block of the decode kernel reads
        self._pages_plan = DecodePages(self.nkv, self.window, rt.sm_count) if self._fast == 2 else None
        self.step_plans = (self._pages_plan,) if self._pages_plan is not None else ()
        self.qkv: Optional[Linear] = None
        self.q_only: Optional[Linear] = None
        self.out: Optional[Linear] = None

    # ------------------------------------------------------------------ tensors
    @classmethod
    def declare(cls, spec) -> Dict[str, TensorDecl]:
        p, t = spec.params, spec.tensors
        h, nq, nkv, hd = (int(p[k]) for k in ("hidden_size", "num_heads", "num_kv_heads", "head_dim"))
        d = {
            t["q_proj"]: TensorDecl((nq * hd, h)),
            t["k_proj"]: TensorDecl((nkv * hd, h)),
            t["v_proj"]: TensorDecl((nkv * hd, h)),
            t["o_proj"]: TensorDecl((h, nq * hd)),
        }
        if p.get("qk_norm", False):
            d[t["q_norm"]] = TensorDecl((hd,), "norm")
            d[t["k_norm"]] = TensorDecl((hd,), "norm")
        return d

    def load(self, tensors) -> None:
        t = self.spec.tensors
        # the three matrices become one of this part's own: they are taken OUT of the table, so that
        # whoever filled it keeps no second copy of them alive (a 32B model and its cache share one GPU)
        parts = [tensors.pop(t[k]) for k in ("q_proj", "k_proj", "v_proj")]
        if len({w.dtype for w in parts}) > 1:
            parts = [w.to(torch.float32) for w in parts]
        fused = self.rt.matrix(torch.cat(parts, dim=0))
        del parts
        self.qkv = Linear(fused, self.rt)
        self.q_only = Linear(fused[: self.nq * self.hd], self.rt)
        self.out = Linear(self.rt.matrix(tensors[t["o_proj"]]), self.rt)
        if self.qk_norm:
            self.q_norm_w = self.rt.vector(tensors[t["q_norm"]])
            self.k_norm_w = self.rt.vector(tensors[t["k_norm"]])

    def weight_bytes(self) -> int:
        return self.qkv.bytes() + self.out.bytes()

    def kernels_needed(self):
        return self.kernel_modules

    # -------------------------------------------------------------------- cache
    def _decode_plan(self, ctx, pages):
        """(plan, blocks, from the host): the step's plan if its builder made one, else one made here by
        a kernel (which the kernel that finishes q, k and v itself must not be given: it reads the plan
        before it waits for the kernels ahead of it)."""
        plan = ctx.plans.get(self._pages_plan.key) if getattr(ctx, "plans", None) else None
        if plan is not None:
            return plan, (plan.numel() - 2 * ctx.n_seqs * self.nkv) // ops.DECODE_PLAN_INTS, True
        n_blocks = self._pages_plan.blocks(ctx.n_seqs, pages.shape[1])
        plan = ctx.buffer("attn.decode_plan", (ops.decode_plan_ints(ctx.n_seqs, self.nkv, n_blocks),), torch.int32)
        ops.attention_decode_plan(ctx.tok_pos, self.nkv, self.window, n_blocks, plan)
        return plan, n_blocks, False

    def cache_need(self) -> Optional[KVNeed]:
        return KVNeed(self.nkv, self.hd, self.window or None, self.cache_dtype)

    def state_need(self):
        return None

    # --------------------------------------------------------------------- step
    def forward(self, ctx, h, x: torch.Tensor, entry) -> None:
        n = ctx.n_tokens
        state = self.rt.kernel_state
        # few tokens (the weight-streaming product takes them): it leaves whole float32 rows, which the
        # kernels after it finish
        few = entry.owns_cache and self.qkv.streams(n) and self.rt.act_dtype == torch.bfloat16
        scale_in = None
        if isinstance(h, NormedInput):
            if ((few or (entry.owns_cache and self.qkv.prompts(n))) and h.ahead is not None
                    and ops.tc_linear_ok(h.ahead[0], self.qkv.weight)):
                scale_in = (h.ahead[1], h.norm.rms_scale_form()[1])  # the product that wrote x last left x * norm weight
                h = h.ahead[0]
            else:
                h = h.tensor()
        nq, nkv, hd = self.nq, self.nkv, self.hd
        group, k_pool, v_pool = ctx.cache.kv_of_entry(entry.cache_entry)
        pages = ctx.pages[group]
        cos = sin = None
        n_rot = 0
        if self.position is not None:
            cos, sin, n_rot = self.position.tables(ctx.max_position + 1)
        if few:
            whole = ctx.buffer("attn.qkv32", (n, (nq + 2 * nkv) * hd), torch.float32)
            self.qkv.forward(h, whole, STORE, scale_in=scale_in)
            ctx.mark("matvec qkv")
            # (up to 16 sequences; with more, every block's repeating the preparation costs more than the
            # kernel it saves: 7,560 against 7,800 to 7,980 tokens/s at batch 64)
            plan = None
            if (self._fast == 2 and ctx.is_decode and n <= self.qkv.STACKED_MAX_TOKENS
                    and k_pool.dtype == torch.bfloat16 and self.rt.act_dtype == torch.bfloat16):
                plan, n_blocks, from_host = self._decode_plan(ctx, pages)
            if plan is not None and from_host:
                # one new token per sequence: its q, k and v are finished inside the attention kernel
                attn = ctx.buffer("attn.out", (n, nq * hd), self.rt.act_dtype)
                scratch = ctx.buffer("attn.partials", (ops.attention_decode_scratch(n, nq, nkv, hd, n_blocks),), torch.float32)
                ops.attention_decode_fused(whole, 0, nq * hd, (nq + nkv) * hd,
                                           self.q_norm_w, self.k_norm_w, self.eps, cos, sin, n_rot, attn, scratch,
                                           nq, nkv, hd, k_pool, v_pool, pages, ctx.page_size, ctx.tok_pos,
                                           self.scale, self.window, n_blocks, plan, state=state)
                ctx.mark("attention")
                self.out.forward(attn, x, ACCUMULATE, ctx=ctx)
                ctx.mark("matvec o")
                return
            qkv = ctx.buffer("attn.q", (n, nq * hd), self.rt.act_dtype)
            ops.qk_norm_rope_cache(whole, 0, nq * hd, (nq + nkv) * hd, nq, nkv, hd, self.q_norm_w,
                                   self.k_norm_w, self.eps, cos, sin, n_rot, ctx.tok_pos, ctx.tok_seq,
                                   k_pool, v_pool, pages, ctx.page_size, q_out=qkv)
        elif (entry.owns_cache and self.qkv.prompts(n) and ops.tc_linear_ok(h, self.qkv.weight)
              and self.hd in (32, 64, 128, 256) and (cos is None or n_rot == self.hd)
              and k_pool.dtype == torch.bfloat16 and self.rt.act_dtype == torch.bfloat16):
            # a prompt: the heads are normed, rotated and put into the cache in the product's epilogue
            qkv = ctx.buffer("attn.q", (n, nq * hd), self.rt.act_dtype)
            self.qkv.forward_heads(h, qkv, dict(
                nq=nq, nkv=nkv, hd=hd, q_norm=self.q_norm_w, k_norm=self.k_norm_w, eps=self.eps, cos=cos, sin=sin,
                tok_pos=ctx.tok_pos, tok_slot=ctx.tok_seq, k_pool=k_pool, v_pool=v_pool, page_table=pages,
                page_size=ctx.page_size), scale_in=scale_in)
            ctx.mark("matvec qkv")
        elif entry.owns_cache:
            qkv = ctx.buffer("attn.qkv", (n, (nq + 2 * nkv) * hd), self.rt.act_dtype)
            self.qkv.forward(h, qkv, STORE, scale_in=scale_in)
            ctx.mark("matvec qkv")
            ops.qk_norm_rope_cache(qkv, 0, nq * hd, (nq + nkv) * hd, nq, nkv, hd, self.q_norm_w,
                                   self.k_norm_w, self.eps, cos, sin, n_rot, ctx.tok_pos, ctx.tok_seq,
                                   k_pool, v_pool, pages, ctx.page_size)
        else:  # reads the cache another run wrote: only queries are needed
            qkv = ctx.buffer("attn.q", (n, nq * hd), self.rt.act_dtype)
            self.q_only.forward(h, qkv, STORE)
            ctx.mark("matvec qkv")
            ops.qk_norm_rope_cache(qkv, 0, 0, 0, nq, 0, hd, self.q_norm_w, None, self.eps, cos, sin,
                                   n_rot, ctx.tok_pos, ctx.tok_seq, None, None, pages, ctx.page_size)
        ctx.mark("qk norm + rope")
        attn = ctx.buffer("attn.out", (n, nq * hd), self.rt.act_dtype)
        q = qkv[:, : nq * hd]
        fast = self._fast if k_pool.dtype == torch.bfloat16 and q.dtype == torch.bfloat16 else 0
        if fast == 2 and ctx.is_decode:
            plan, n_blocks, _ = self._decode_plan(ctx, pages)
            scratch = ctx.buffer("attn.partials", (ops.attention_decode_scratch(n, nq, nkv, hd, n_blocks),), torch.float32)
            ops.attention_decode(q, attn, scratch, nq, nkv, hd, k_pool, v_pool, pages, ctx.page_size,
                                 ctx.tok_pos, self.scale, self.window, n_blocks, plan, state=state)
        elif fast:
            tile_seq, tile_tok0, tile_rows = ctx.tiles[ops.PREFILL_TILE]
            ops.attention_prefill(q, attn, nq, nkv, hd, k_pool, v_pool, pages, ctx.page_size, ctx.tok_pos,
                                  tile_seq, tile_tok0, tile_rows, self.scale, self.window, state=state)
        else:
            ops.attention_plain(q, attn, nq, nkv, hd, k_pool, v_pool, pages, ctx.page_size, ctx.tok_pos,
                                ctx.tok_seq, self.scale, self.window)
        ctx.mark("attention")
        self.out.forward(attn, x, ACCUMULATE, ctx=ctx)
        ctx.mark("matvec o")


register_mixer("gqa_attention", GQAttention)
