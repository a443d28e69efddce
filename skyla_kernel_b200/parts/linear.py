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
    kernel_modules = ("linear_plain", "gemm_tc")

    #: rows of gate and of up that alternate in a fused gate/up matrix for the tensor-core kernel
    TC_GATED_GROUP = 128

    def __init__(self, weight: torch.Tensor, rt, gated_group: int = 0):
        """``weight`` on the device; ``gated_group`` > 0 marks a fused gate/up matrix."""
        self.weight = weight
        self.rt = rt
        self.gated_group = gated_group
        self.n_in = weight.shape[1]
        self.n_out = weight.shape[0] // 2 if gated_group else weight.shape[0]
        self._map = None
        self.tensor_cores = (not rt.full_precision and weight.dtype == torch.bfloat16 and self.n_in % 8 == 0
                             and weight.is_contiguous() and weight.data_ptr() % 16 == 0
                             and (not gated_group or gated_group == self.TC_GATED_GROUP))

    @classmethod
    def gated_group_for(cls, rt, gate: torch.Tensor) -> int:
        """The gate/up grouping to fuse with: 128 where the tensor-core kernel will run, else one block."""
        n, k = gate.shape
        fast = not rt.full_precision and gate.dtype == torch.bfloat16 and n % cls.TC_GATED_GROUP == 0 and k % 8 == 0
        return cls.TC_GATED_GROUP if fast else n

    def weight_map(self):
        if self._map is None:
            self._map = ops.TensorMap(self.weight, 256 if self.gated_group else 128)
        return self._map

    def forward(self, x: torch.Tensor, y: torch.Tensor, mode: int = STORE) -> torch.Tensor:
        if self.gated_group:
            mode = GATED
        if self.tensor_cores and ops.tc_linear_ok(x, self.weight):
            if mode == GATED:
                tc = ops.TC_GLU_BF16
            elif mode == ACCUMULATE:
                splits = self.choose_splits(x.shape[0])
                if splits > 8:  # more splits than a portable cluster holds: they meet through scratch
                    scratch = ops.accum_scratch(x.device, splits * x.shape[0] * self.n_out)
                    return ops.gemm_tc(x, self.weight_map(), self.n_out, y, ops.TC_ACCUM_LAST, splits=splits,
                                       scratch=scratch)
                if splits > 1:  # few tokens: K is cut across a cluster of blocks so that every SM streams
                    return ops.gemm_tc(x, self.weight_map(), self.n_out, y, ops.TC_ACCUM_CLUSTER, splits=splits)
                tc = ops.TC_ACCUM_F32
            else:
                tc = ops.TC_STORE_BF16 if y.dtype == torch.bfloat16 else ops.TC_STORE_F32
            return ops.gemm_tc(x, self.weight_map(), self.n_out, y, tc)
        return ops.linear_plain(x, self.weight, y, mode, self.gated_group)

    # ---- K-split products for small batches
    N_SMS = 148
    # How the K splits of "y += x W^T" meet: up to 8 splits form a thread-block cluster and add up
    # through distributed shared memory (ops.TC_ACCUM_CLUSTER); more than 8 leave their tiles in
    # scratch and the one that finishes last adds them up (ops.TC_ACCUM_LAST).  Measured at the
    # 8B shape the two cost the same for 8 tokens (10.7 and 21.8 us for the O and down
    # products); the cluster is faster for 64 (15.4 against 23.5 us, 28.0 against 35.8).

    def choose_splits(self, m: int) -> int:
        """How many K splits make a small batch's product fill the GPU (1: do not split).

        One block per SM is resident; a block costs its K blocks plus about six more
        for filling and draining its pipeline; at least 16 K blocks stay per split.
        """
        if m > 64:
            return 1
        bn = ops.token_tile(m)
        tiles = -(-self.n_out // 128) * -(-m // bn)
        total = -(-self.n_in // 64)
        best, best_cost = 1, None
        for s in range(1, max(1, total // 16) + 1):
            per = -(-total // s)
            if (s - 1) * per >= total:
                continue
            cost = -(-tiles * s // self.N_SMS) * (per + 6)
            if best_cost is None or cost < best_cost:
                best, best_cost = s, cost
        return best

    def forward_partial(self, x: torch.Tensor, ctx, name: str, fold=None):
        """The product as K-split partial sums [splits, tokens, n_out] (float32) in a workspace
        buffer, or ``None`` when splitting does not pay or the tensor-core kernel does not
        take these operands; the reader adds the splits up in ascending order.
        ``fold=(r, partials)`` rides along (``r += sum partials``) when the product is made."""
        if self.gated_group or not self.tensor_cores or not ops.tc_linear_ok(x, self.weight):
            return None
        m = x.shape[0]
        splits = self.choose_splits(m)
        if splits <= 1:
            return None
        part = ctx.buffer(name, (splits, m, self.n_out), torch.float32)
        ops.gemm_tc(x, self.weight_map(), self.n_out, part, ops.TC_PARTIAL_F32, splits=splits, fold=fold)
        return part

    # ---- the RMSNorm of the input made inside the product
    FUSED_NORM_MAX_TOKENS = 16  # every block re-reads the rows it normalises: only worth it for few

    def can_fuse_norm(self, normed) -> bool:
        """Whether ``norm(x + pending)`` can be made inside this product: RMSNorm, float32 rows
        with 16-byte alignment, few tokens, and a weight the tensor-core kernel takes."""
        x, norm, pend = normed.x, normed.norm, normed.ctx.pending
        return (self.tensor_cores and type(norm).__name__ == "RMSNorm" and x.dtype == torch.float32
                and x.shape[0] <= self.FUSED_NORM_MAX_TOKENS and x.shape[1] == self.n_in
                and x.stride(1) == 1 and x.stride(0) % 4 == 0 and x.data_ptr() % 16 == 0
                and (pend is None or (pend.dim() == 3 and tuple(pend.shape[1:]) == tuple(x.shape))))

    def forward_normed_partial(self, normed, ctx, name: str):
        """(partial sums [splits, tokens, n_out], row sums of squares [splits, tokens]) of the
        product of the *un-scaled* normed input; the reader applies the rows' scalars.
        ``x`` and ``ctx.pending`` are left as they are."""
        x, norm = normed.x, normed.norm
        m = x.shape[0]
        splits = self.choose_splits(m)
        part = ctx.buffer(name, (splits, m, self.n_out), torch.float32)
        ssq = ctx.buffer(name + ".ssq", (splits, m), torch.float32)
        ops.gemm_tc_norm(x, ctx.pending, norm.weight, norm.eps, self.weight_map(), self.n_out, part,
                         ops.TC_PARTIAL_F32, splits=splits, ssq_out=ssq)
        return part, ssq

    def forward_normed(self, normed, ctx, y: torch.Tensor) -> torch.Tensor:
        """``y = f(norm(x + pending) W^T)`` in one kernel (gated or plain store)."""
        x, norm = normed.x, normed.norm
        mode = ops.TC_GLU_BF16 if self.gated_group else (ops.TC_STORE_BF16 if y.dtype == torch.bfloat16 else ops.TC_STORE_F32)
        return ops.gemm_tc_norm(x, ctx.pending, norm.weight, norm.eps, self.weight_map(), self.n_out, y, mode)

    def bytes(self) -> int:
        return self.weight.numel() * self.weight.element_size()
