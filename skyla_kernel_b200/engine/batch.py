"""One step's batch as the kernels see it.

The reference keeps three control words in GPU-visible memory -- first token,
position, token count -- so that its recorded command buffers never change
(skyla-engine/src/engine.rs:121-123, README.md:161-162).  With many sequences of
unequal length the control block becomes a set of int32 arrays, packed in one
pinned host buffer and sent with one copy per step:

  tokens[T]    the new tokens of all sequences, packed without padding
  tok_pos[T]   absolute position of each token in its sequence
  tok_seq[T]   row of its sequence in this batch
  seq_slot[B]  cache slot of each sequence (for parts with per-slot state)
  seq_start[B] positions already cached, seq_n[B] new tokens, cu[B+1] packed offsets
  want[R]      rows (packed token indices) whose logits are asked for
  tiles[h] = (tile_seq, tile_tok0, tile_rows)[Q]  for every tile height h that a mixer of the
               model asked for (``Part.token_tiles``): tiles of up to h consecutive new tokens of
               one sequence, the units a prompt attention kernel works in, in ascending order of
               the last position they see
  pages[G][B,P] for each cache group the page list of each sequence
  plans[key]   what a part of the model asked to have worked out on the host from the step's
               positions (``parts.base.StepPlan``), e.g. which pages each block of a decode
               attention launch reads
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Dict, List, Optional, Sequence, Tuple

import numpy as np
import torch


@dataclass
class StepItem:
    """One sequence's share of a step: its slot, its next tokens, the wanted places."""

    slot: int
    tokens: Sequence[int]
    want: Sequence[int] = ()
    #: (handle, row): the item's one token is row ``row`` of ``handle.device_tokens`` (int32 on
    #: the device, e.g. what a sampler just wrote) and ``tokens`` is a placeholder of length 1
    device_token: Optional[tuple] = None


class Workspace:
    """Named device buffers that grow and are reused from step to step."""

    def __init__(self, device):
        self.device = device
        self._bufs: Dict[Tuple[str, torch.dtype], torch.Tensor] = {}

    def get(self, name: str, shape: Tuple[int, ...], dtype: torch.dtype) -> torch.Tensor:
        n = 1
        for s in shape:
            n *= int(s)
        key = (name, dtype)
        buf = self._bufs.get(key)
        if buf is None or buf.numel() < n:
            buf = torch.empty(max(n, 1), dtype=dtype, device=self.device)
            self._bufs[key] = buf
        return buf[:n].view(shape)

    def bytes(self) -> int:
        return sum(b.numel() * b.element_size() for b in self._bufs.values())


@dataclass
class StepContext:
    """Everything a part may read during a step."""

    rt: object
    cache: object
    workspace: Workspace
    n_tokens: int
    n_seqs: int
    n_want: int
    max_position: int          # largest absolute position among the new tokens
    max_context: int           # largest sequence length after this step
    max_new: int               # most new tokens of one sequence
    page_size: int
    tokens: torch.Tensor
    tok_pos: torch.Tensor
    tok_seq: torch.Tensor
    seq_slot: torch.Tensor
    seq_start: torch.Tensor
    seq_n: torch.Tensor
    cu: torch.Tensor
    want: torch.Tensor
    pages: List[torch.Tensor]
    #: key of a part's :class:`~skyla_kernel_b200.parts.base.StepPlan` -> its ints on the device
    plans: Dict[object, torch.Tensor] = field(default_factory=dict)
    #: tile height -> (sequence row, first packed token, rows) of every tile, for the heights the
    #: model's mixers asked for
    tiles: Dict[int, Tuple[torch.Tensor, torch.Tensor, torch.Tensor]] = field(default_factory=dict)
    host: Dict[str, np.ndarray] = field(default_factory=dict)
    #: when profiling: (label, event) pairs, an event after each stage
    #: (the reference's timestamp marks, skyla-engine/src/graph.rs:54-57)
    marks: Optional[list] = None
    #: hints for "norm ahead": the norm that reads the residual stream after the part now running
    #: (set by the block), and the norm that reads it after the block now running (set by the model)
    next_norm: Optional[object] = None
    after_block_norm: Optional[object] = None
    #: what the last writer of the residual stream left for its next reader:
    #: (norm, x, x * norm.weight in bfloat16, shares of the rows' sums of squares)
    ahead: Optional[tuple] = None

    @property
    def is_decode(self) -> bool:
        return self.max_new == 1

    def take_ahead(self, norm, x: torch.Tensor):
        """(x * norm.weight in bfloat16, shares of the sums of squares) if the last writer of ``x``
        left them for this very norm, else ``None``; either way they are gone afterwards."""
        a, self.ahead = self.ahead, None
        if a is not None and a[0] is norm and a[1] is x:
            return a[2], a[3]
        return None

    def mark(self, label: str) -> None:
        """End of a stage; a no-op unless the step is profiled."""
        if self.marks is not None:
            ev = torch.cuda.Event(enable_timing=True)
            ev.record()
            self.marks.append((label, ev))

    def buffer(self, name: str, shape, dtype) -> torch.Tensor:
        return self.workspace.get(name, tuple(shape), dtype)


class BatchBuilder:
    """Packs a step's arrays on the host and moves them with one copy."""

    #: bytes that all builders of this process have copied to devices so far (for measurements)
    h2d_bytes = 0

    def _feed_device_tokens(self, items, dev_tokens: torch.Tensor, ns) -> None:
        """Tokens that only exist on the device are copied into place there."""
        fed = [(b, it.device_token) for b, it in enumerate(items) if it.device_token is not None]
        if not fed:
            return
        if len(fed) != len(items) or any(n != 1 for n in ns):
            raise ValueError("device-fed tokens: every item of the step must bring exactly one such token")
        src = fed[0][1][0].device_tokens
        rows = [ref[1] for _, ref in fed]
        if any(ref[0].device_tokens is not src for _, ref in fed):
            raise ValueError("device-fed tokens must come from one step's sampler output")
        if rows == list(range(len(rows))):
            dev_tokens.copy_(src[: len(rows)])
        else:
            idx = torch.tensor(rows, dtype=torch.int64).to(self.rt.device, non_blocking=True)
            dev_tokens.copy_(src.index_select(0, idx))

    def __init__(self, rt, cache, tile_heights: Sequence[int] = (), plans: Sequence[object] = ()):
        """``tile_heights``: the heights of token tiles that the model's mixers want listed every step;
        ``plans``: the ``StepPlan`` objects of its parts."""
        self.rt = rt
        self.plans = tuple(plans)
        self.cache = cache
        self.tile_heights = tuple(sorted(set(int(h) for h in tile_heights)))
        self.workspace = Workspace(rt.device)
        self._pinned: Optional[torch.Tensor] = None
        self._device: Optional[torch.Tensor] = None
        self._copied = None  # event after the last copy out of the pinned buffer

    def _staging(self, n: int):
        if self._pinned is None or self._pinned.numel() < n:
            cap = max(1024, 1 << (n - 1).bit_length())
            self._pinned = torch.empty(cap, dtype=torch.int32, pin_memory=self.rt.device.type == "cuda")
            self._device = torch.empty(cap, dtype=torch.int32, device=self.rt.device)
        return self._pinned, self._device

    def build(self, items: List[StepItem], pages_width: Optional[int] = None) -> StepContext:
        """``pages_width``: columns of the page lists (default: what the longest sequence needs);
        a fixed width keeps the layout of the arrays the same from step to step."""
        cache = self.cache
        B = len(items)
        ns = [len(it.tokens) for it in items]
        T = sum(ns)
        starts = [cache.length(it.slot) for it in items]
        R = sum(len(it.want) for it in items)
        G = len(cache.groups)
        P = max(1, max(-(-(s + n) // cache.page_size) for s, n in zip(starts, ns)))
        if pages_width is not None:
            if pages_width < P:
                raise ValueError(f"page lists need {P} columns, {pages_width} were given")
            P = pages_width
        n_tiles = {th: sum(-(-n // th) for n in ns) for th in self.tile_heights}
        plan_sizes = [int(p.size(B, P, max(ns) == 1)) for p in self.plans]
        total = 3 * T + 3 * B + (B + 1) + R + 3 * sum(n_tiles.values()) + G * B * P + sum(s + 3 for s in plan_sizes if s)
        if self._copied is not None:
            self._copied.synchronize()  # the last step's copy has left the pinned buffer
        host, dev = self._staging(total)
        h = host.numpy()
        o = 0

        def take(n):
            nonlocal o
            v = h[o:o + n]
            o += n
            return v, (o - n, o)

        tokens, r_tokens = take(T)
        tok_pos, r_pos = take(T)
        tok_seq, r_seq = take(T)
        seq_slot, r_slot = take(B)
        seq_start, r_start = take(B)
        seq_n, r_n = take(B)
        cu, r_cu = take(B + 1)
        want, r_want = take(R)
        tiles = {th: [take(q) for _ in range(3)] for th, q in n_tiles.items()}
        q = {th: 0 for th in tiles}
        t = 0
        w = 0
        cu[0] = 0
        for b, it in enumerate(items):
            n = ns[b]
            tokens[t:t + n] = np.asarray(it.tokens, dtype=np.int64)
            tok_pos[t:t + n] = np.arange(starts[b], starts[b] + n)
            tok_seq[t:t + n] = b
            seq_slot[b], seq_start[b], seq_n[b] = it.slot, starts[b], n
            for j in it.want:
                if not 0 <= j < n:
                    raise IndexError(f"wanted place {j} is outside the {n} tokens of this step")
                want[w] = t + j
                w += 1
            for th, ((tile_seq, _), (tile_tok0, _), (tile_rows, _)) in tiles.items():
                for j in range(0, n, th):
                    tile_seq[q[th]], tile_tok0[q[th]], tile_rows[q[th]] = b, t + j, min(th, n - j)
                    q[th] += 1
            t += n
            cu[b + 1] = t
        # The prompt attention kernels start the tiles from the list's end: the tiles that see the most keys go
        # last in the list, so that the longest blocks start first whichever sequences they belong to.
        for th, ((tile_seq, _), (tile_tok0, _), (tile_rows, _)) in tiles.items():
            if len(tile_seq) > 1:
                ends = np.asarray(starts)[tile_seq] + (tile_tok0 - cu[tile_seq]) + tile_rows
                order = np.argsort(ends, kind="stable")
                tile_seq[:], tile_tok0[:], tile_rows[:] = tile_seq[order], tile_tok0[order], tile_rows[order]
        r_pages = []
        for g in range(G):
            pg, r = take(B * P)
            pg = pg.reshape(B, P)
            pg[:] = 0
            for b, it in enumerate(items):
                lst = cache.pages_of(g, it.slot)
                m = min(len(lst), P)
                pg[b, :m] = np.maximum(np.asarray(lst[:m], dtype=np.int64), 0)
            r_pages.append(r)
        r_plans = {}
        for plan, size in zip(self.plans, plan_sizes):
            if size:
                o = -(-o // 4) * 4  # 16-byte aligned: kernels read plan rows as vectors
                arr, r = take(size)
                plan.fill(arr, np.asarray(starts), np.asarray(ns), cache.page_size)
                r_plans[plan.key] = r
        dev[:total].copy_(host[:total], non_blocking=True)
        BatchBuilder.h2d_bytes += 4 * total
        if self.rt.device.type == "cuda":
            self._copied = torch.cuda.Event()
            self._copied.record()
        self._feed_device_tokens(items, dev[r_tokens[0]:r_tokens[1]], ns)

        def view(r):
            return dev[r[0]:r[1]]

        return StepContext(
            rt=self.rt, cache=cache, workspace=self.workspace, n_tokens=T, n_seqs=B, n_want=R,
            max_position=max(s + n - 1 for s, n in zip(starts, ns)),
            max_context=max(s + n for s, n in zip(starts, ns)), max_new=max(ns),
            page_size=cache.page_size, tokens=view(r_tokens), tok_pos=view(r_pos),
            tok_seq=view(r_seq), seq_slot=view(r_slot), seq_start=view(r_start), seq_n=view(r_n),
            cu=view(r_cu), want=view(r_want), pages=[view(r).view(B, P) for r in r_pages],
            tiles={th: tuple(view(r) for _, r in three) for th, three in tiles.items()},
            plans={k: view(r) for k, r in r_plans.items()},
            host={"starts": np.asarray(starts), "ns": np.asarray(ns)},
        )
