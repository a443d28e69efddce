"""Matrix products of the parts: picks the kernel for a weight, a precision and a row count.

``y = x W^T`` with ``W`` stored ``[outputs, inputs]`` (skyla-ref/src/matrix.rs:38-58).
The plain 32-bit kernel takes every shape and dtype; the tensor-core and
bandwidth-bound bfloat16 kernels take the shapes they are written for and are
chosen here, never by the caller.
"""
from __future__ import annotations

import torch

from ..kernels import ops

STORE, ACCUMULATE, GATED = ops.STORE, ops.ACCUMULATE, ops.GATED


class Linear:
    kernel_modules = ("linear_plain", "gemm_tc", "gemm_prompt")

    #: inputs from which a product of 65 to 128 tokens that the weight-streaming kernel does not take goes to
    #: the prompt kernel
    PROMPT_LONG_K = 8192
    #: the weight-streaming kernel takes over up to this many tokens: with tall tiles (gated products,
    #: products of many waves) or with tiles whose K is cut into a cluster of splits ...
    ROWS_MAX_TOKENS = ops.ROWS_MAX_TOKENS
    #: ... but where its blocks each read every token's whole row (short tiles, K blocks stacked, no K
    #: split) only up to this many: beyond, the token rows outweigh the block's weights
    STACKED_MAX_TOKENS = 16

    def __init__(self, weight: torch.Tensor, rt, gated: bool = False):
        """``weight`` on the device; ``gated`` marks a fused matrix: all gate rows, then all up rows."""
        self.weight = weight
        self.rt = rt
        self.gated = gated
        self.n_in = weight.shape[1]
        self.n_out = weight.shape[0] // 2 if gated else weight.shape[0]
        self._map = None
        self._rows_maps = {}
        self.tensor_cores = (not rt.full_precision and weight.dtype == torch.bfloat16 and self.n_in % 8 == 0
                             and weight.is_contiguous() and weight.data_ptr() % 16 == 0)
        #: token tile -> (rows per block, K splits, K blocks per box, K blocks per MMA) of the weight-streaming kernel
        self.rows_plans = {bn: ops.rows_plan(self.n_out, self.n_in, gated, bn, rt.sm_count) for bn in (16, 32, 64, 128)}
        self.streams_wide = self.rows_plans[64][0] > 64  # tall tiles: gated products, many-wave products
        if self.tensor_cores and not self.streams_wide and not gated:
            # 17 to 128 tokens: tiles whose K is cut into a cluster of splits, where K is long enough to cut
            for bn in (32, 64, 128):
                plan = ops.rows_cluster_plan(self.n_out, self.n_in, bn, rt.clusters)
                if plan is not None:
                    self.rows_plans[bn] = plan
        #: the most tokens that the weight-streaming kernel takes for this weight
        self.rows_limit = (self.ROWS_MAX_TOKENS if self.streams_wide or all(self.rows_plans[bn][1] > 1 for bn in (32, 64, 128))
                           else self.STACKED_MAX_TOKENS)

    def weight_map(self):
        if self._map is None:
            self._map = ops.TensorMap(self.weight, 128)
        return self._map

    def streams(self, m: int) -> bool:
        """Whether ``m`` tokens go to the weight-streaming kernel (given operands it takes)."""
        return self.tensor_cores and m <= self.rows_limit

    def prompts(self, m: int) -> bool:
        """Whether ``m`` tokens go to the prompt kernel (tokens are the tile's rows; given operands it takes)."""
        if not self.tensor_cores:
            return False
        # from 65 tokens already where the reduction is long and the weight-streaming kernel does not take the
        # product: the prompt kernel cuts few tiles along K (a down product of the 8B shape at 96 and 128
        # tokens: 41 against 60 us for the tile kernel; the products with 4,096 inputs are even or lose)
        return m >= ops.PROMPT_MIN_TOKENS or (m > 64 and not self.streams(m) and self.n_in >= self.PROMPT_LONG_K
                                              and not self.gated)

    def takes_scale_in(self, m: int) -> bool:
        """Whether :meth:`forward` of ``m`` tokens accepts ``scale_in``."""
        return self.streams(m) or self.prompts(m)

    def _rows_map(self, m: int):
        rows, splits, kkb, kstack = self.rows_plans[ops.token_tile(m)]
        w_map = self._rows_maps.get((rows, kkb))
        if w_map is None:
            w_map = self._rows_maps[(rows, kkb)] = ops.TensorMap(self.weight, rows, kkb)
        return w_map

    def _stream(self, x, y, tc, norm_ahead=None, scale_in=None):
        m = x.shape[0]
        rows, splits, kkb, kstack = self.rows_plans[ops.token_tile(m)]
        return ops.gemm_tc_rows(x, self._rows_map(m), rows, self.n_out, y, tc, kkb=kkb, splits=splits, kstack=kstack,
                                norm_ahead=norm_ahead, scale_in=scale_in, state=self.rt.kernel_state)

    def _norm_ahead(self, ctx, x, y, parts: int):
        """Buffers for "norm ahead" if this product adds into the residual stream ``y`` and the norm
        that reads it next says that it has the form ``x * w / sqrt(mean(x^2) + eps)`` over this
        width (``norm.rms_scale_form()``); the kernel leaves ``parts`` shares of a row's sum of
        squares (0: it cannot)."""
        norm = getattr(ctx, "next_norm", None) if ctx is not None else None
        if ctx is not None:
            ctx.next_norm = None
        m = x.shape[0]
        form = getattr(norm, "rms_scale_form", None)
        form = form() if form is not None else None
        if form is None or y.dtype != torch.float32 or form[0].numel() != self.n_out or self.n_out % 8 or parts < 1:
            return None, None
        xw = ctx.buffer("x.times_norm_weight", (m, self.n_out), torch.bfloat16)
        ssq = ctx.buffer("x.ssq_shares", (parts, m), torch.float32)
        return norm, (form[0], xw, ssq)

    def forward(self, x: torch.Tensor, y: torch.Tensor, mode: int = STORE, scale_in=None, ctx=None) -> torch.Tensor:
        """``scale_in=(shares of the rows' sums of squares, eps)``: ``x`` is a residual stream times
        its norm's weight (see ``NormedInput.ahead``); only where :meth:`takes_scale_in` holds.
        ``ctx`` with ``mode=ACCUMULATE``: ``y`` is the residual stream, and if ``ctx.next_norm``
        names the RMSNorm that reads it next, its input is prepared on the way (``ctx.ahead``)."""
        if self.gated:
            mode = GATED
        if self.tensor_cores and ops.tc_linear_ok(x, self.weight):
            m = x.shape[0]
            tc = {GATED: ops.TC_GLU_BF16, ACCUMULATE: ops.TC_ACCUM_F32}.get(
                mode, ops.TC_STORE_BF16 if y.dtype == torch.bfloat16 else ops.TC_STORE_F32)
            if self.streams(m):
                rows = self.rows_plans[ops.token_tile(m)][0]
                norm, ahead = self._norm_ahead(ctx, x, y, -(-self.n_out // rows)) if mode == ACCUMULATE else (None, None)
                self._stream(x, y, tc, norm_ahead=ahead, scale_in=scale_in)
                if ahead is not None:
                    ctx.ahead = (norm, y, ahead[1], ahead[2])
                return y
            if self.prompts(m):
                # (Prompts add into the residual stream by TMA reduce, which never reads it; preparing the next
                # norm's input on the way would need the rows back in the threads: 106 against 65 us for the O
                # product of 2,048 tokens of the 8B shape, more than the norm kernel it saves.)
                if ctx is not None:
                    ctx.next_norm = None
                ops.gemm_prompt(x, self.weight_map(), self.n_out, y, tc, scale_in=scale_in, state=self.rt.kernel_state)
                return y
            if scale_in is not None:
                raise ValueError("scale_in goes with the weight-streaming and the prompt kernel only (Linear.takes_scale_in)")
            return ops.gemm_tc(x, self.weight_map(), self.n_out, y, tc, state=self.rt.kernel_state)
        if scale_in is not None:
            raise ValueError("scale_in goes with the weight-streaming and the prompt kernel only (Linear.takes_scale_in)")
        return ops.linear_plain(x, self.weight, y, mode, 0)

    def forward_heads(self, x: torch.Tensor, q_out: torch.Tensor, prep: dict, scale_in=None) -> torch.Tensor:
        """The product of a fused q/k/v weight whose heads are finished in its epilogue
        (``ops.gemm_prompt`` with TC_QKV_PREP); only where :meth:`prompts` holds."""
        return ops.gemm_prompt(x, self.weight_map(), self.n_out, q_out, ops.TC_QKV_PREP, scale_in=scale_in, prep=prep,
                               state=self.rt.kernel_state)

    def bytes(self) -> int:
        return self.weight.numel() * self.weight.element_size()
