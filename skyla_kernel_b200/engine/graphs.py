"""Decode steps as CUDA graphs.

The reference records its command buffer once and replays it for every token,
with token, position and count in GPU-visible memory so that the recording never
changes (skyla-engine/src/graph.rs:195-233, README.md:161-162).  Here a decode
step -- one new token for each of B sequences -- is captured once per
(B, width of the page lists) as a CUDA graph over static buffers: the step's
int32 arrays, the workspace and the logits.  A replay fills the arrays on the host,
copies them in one transfer and launches the graph.
"""
from __future__ import annotations

from typing import Dict, List, Tuple

import torch

from .batch import BatchBuilder, StepItem


def page_bucket(pages: int) -> int:
    """Widths of the page lists come in powers of two (at least 8), so few graphs are captured."""
    b = 8
    while b < pages:
        b *= 2
    return b


class _Captured:
    def __init__(self, batcher, graph, logits):
        self.batcher, self.graph, self.logits = batcher, graph, logits


class DecodeGraphs:
    #: graphs kept at a time; each owns its arrays, its workspace and a [batch, vocabulary] logits
    #: buffer, so a batch that shrinks from 64 to 1 across several widths must not keep them all for ever
    MAX_GRAPHS = 24

    def __init__(self, model, rt, cache):
        self.model, self.rt, self.cache = model, rt, cache
        self._graphs: Dict[Tuple[int, int], _Captured] = {}  # in order of last use
        self.replays = 0
        self.captures = 0

    def run(self, items: List[StepItem]) -> torch.Tensor:
        """``items``: one token each, logits wanted for it.  Returns the graph's own
        logits buffer (valid until this graph is replayed again)."""
        from ..kernels import ops
        B = len(items)
        pages = max(-(-(self.cache.length(it.slot) + 1) // self.cache.page_size) for it in items)
        width = page_bucket(pages)
        key = (B, width)
        cap = self._graphs.pop(key, None)
        if cap is None:
            while len(self._graphs) >= self.MAX_GRAPHS:  # the one used longest ago goes
                old = self._graphs.pop(next(iter(self._graphs)))
                torch.cuda.synchronize(self.rt.device)    # it may still be running
                del old
            cap = self._capture(items, width)
            self.captures += 1
        self._graphs[key] = cap
        cap.batcher.build(items, pages_width=width)  # refills the static arrays
        cap.graph.replay()
        self.replays += 1
        ops.LAUNCHES += cap.launches  # the kernels the replay launched
        self.last_key = key
        return cap.logits

    def _capture(self, items: List[StepItem], width: int) -> _Captured:
        from ..kernels import ops
        # arrays and workspace of this graph alone
        batcher = BatchBuilder(self.rt, self.cache, self.model.tile_heights(), self.model.step_plans())
        ctx = batcher.build(items, pages_width=width)
        ctx.max_position = width * self.cache.page_size - 1  # position tables must cover the bucket
        ctx.max_context = width * self.cache.page_size
        # one eager run: loads every kernel, sizes the workspace, grows position tables
        side = torch.cuda.Stream(device=self.rt.device)
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            self.model.forward(ctx)
        torch.cuda.current_stream().wait_stream(side)
        torch.cuda.synchronize(self.rt.device)
        graph = torch.cuda.CUDAGraph()
        before = ops.LAUNCHES
        with torch.cuda.graph(graph):
            logits = self.model.forward(ctx)
        cap = _Captured(batcher, graph, logits)
        cap.launches = ops.LAUNCHES - before
        return cap
