"""Python faces of the CUDA launchers: tensors in, one kernel launch each.

Every function checks device, dtype and layout, passes raw pointers and the
current CUDA stream to an ``extern "C"`` launcher, and raises
:class:`KernelError` with the launcher's message on a refused size or a failed
launch.  Nothing here computes on the host or falls back to library code.
"""
from __future__ import annotations

import ctypes
from ctypes import c_float, c_int, c_int64, c_size_t, c_uint64, c_void_p
from typing import Optional

import torch

from . import build

F32, BF16 = 0, 1
_CODES = {torch.float32: F32, torch.bfloat16: BF16}


class KernelError(RuntimeError):
    pass


def dtype_code(t: torch.Tensor) -> int:
    try:
        return _CODES[t.dtype]
    except KeyError:
        raise KernelError(f"kernels take float32 or bfloat16 tensors, not {t.dtype}") from None


def _ptr(t: Optional[torch.Tensor]):
    return c_void_p(0 if t is None else t.data_ptr())


def _stream():
    return c_void_p(torch.cuda.current_stream().cuda_stream)


def _cuda(*tensors):
    for t in tensors:
        if t is not None and not t.is_cuda:
            raise KernelError("kernel operands must be CUDA tensors; there is no host path")


def _rows(t: torch.Tensor, what: str) -> int:
    """Row stride of a 2-D tensor whose rows are contiguous."""
    if t.dim() != 2 or (t.shape[1] > 1 and t.stride(1) != 1):
        raise KernelError(f"{what}: expected a 2-D tensor with contiguous rows, got shape "
                          f"{tuple(t.shape)} strides {t.stride()}")
    return t.stride(0) if t.shape[0] > 1 else max(t.stride(0), t.shape[1])


def _i32(t: Optional[torch.Tensor], what: str):
    if t is not None and (t.dtype != torch.int32 or not t.is_contiguous()):
        raise KernelError(f"{what}: expected a contiguous int32 tensor")
    return t


_FUNCS = {}


def _fn(module: str, name: str, argtypes):
    key = (module, name)
    f = _FUNCS.get(key)
    if f is None:
        lib = build.load(module)
        f = getattr(lib, name)
        f.argtypes = argtypes
        f.restype = c_int
        _FUNCS[key] = f
    return f


#: kernel launches made through this module since import (bench.py reports the difference)
LAUNCHES = 0
#: the same per kernel library, for tests that want to know which kernels a step went through
LAUNCHES_BY_MODULE = {}


def _check_nolaunch(module: str, rc: int):
    if rc != 0:
        msg = build.load(module).skyla_error_message().decode("utf-8", "replace")
        raise KernelError(msg or f"{module}: error {rc}")


def _check(module: str, rc: int):
    global LAUNCHES
    LAUNCHES += 1
    LAUNCHES_BY_MODULE[module] = LAUNCHES_BY_MODULE.get(module, 0) + 1
    if rc != 0:
        msg = build.load(module).skyla_error_message().decode("utf-8", "replace")
        raise KernelError(msg or f"{module}: error {rc}")


# ------------------------------------------------------------------ embedding
def embed_gather(tokens: torch.Tensor, table: torch.Tensor, out: torch.Tensor,
                 state: Optional["KernelState"] = None) -> torch.Tensor:
    """out[t, :] = table[tokens[t], :].  A token outside the table gets a row of zeros and raises the
    state's error word (the host checks the tokens it feeds; a sampler's output is checked here)."""
    _cuda(tokens, table, out)
    _i32(tokens, "tokens")
    if not table.is_contiguous():
        raise KernelError("embedding table must be contiguous")
    n, hidden = tokens.numel(), table.shape[1]
    if out.shape[0] < n or out.shape[1] != hidden:
        raise KernelError(f"embed_gather: out {tuple(out.shape)} does not hold [{n}, {hidden}]")
    f = _fn("embed", "skyla_embed_gather",
            [c_void_p, c_int, c_void_p, c_int, c_int, c_int, c_void_p, c_int, c_int64, c_void_p, c_void_p])
    _check("embed", f(_ptr(tokens), n, _ptr(table), dtype_code(table), table.shape[0], hidden, _ptr(out),
                      dtype_code(out), _rows(out, "out"), _ptr(_state(state, out).error_flag), _stream()))
    return out


# ----------------------------------------------------------------------- norm
def rmsnorm(x: torch.Tensor, weight: torch.Tensor, eps: float, out: torch.Tensor,
            rows: Optional[torch.Tensor] = None) -> torch.Tensor:
    """out[r] = rmsnorm(x[rows[r]] or x[r]) * weight, computed in 32-bit."""
    _cuda(x, weight, out, rows)
    _i32(rows, "rows")
    if weight.dtype != torch.float32 or not weight.is_contiguous():
        raise KernelError("rmsnorm: the weight must be a contiguous float32 vector")
    width = weight.numel()
    n = rows.numel() if rows is not None else x.shape[0]
    if x.shape[1] != width or out.shape[1] != width or out.shape[0] < n:
        raise KernelError(f"rmsnorm: shapes x {tuple(x.shape)} out {tuple(out.shape)} weight [{width}]")
    f = _fn("norm", "skyla_rmsnorm",
            [c_void_p, c_int, c_int64, c_void_p, c_int, c_int, c_void_p, c_float, c_void_p, c_int,
             c_int64, c_void_p])
    _check("norm", f(_ptr(x), dtype_code(x), _rows(x, "x"), _ptr(rows), n, width, _ptr(weight),
                     float(eps), _ptr(out), dtype_code(out), _rows(out, "out"), _stream()))
    return out


# --------------------------------------------------------------------- linear
STORE, ACCUMULATE, GATED = 0, 1, 2


def linear_plain(x: torch.Tensor, w: torch.Tensor, y: torch.Tensor, mode: int = STORE,
                 glu_group: int = 0) -> torch.Tensor:
    """y = x @ w.T (store), y += x @ w.T (accumulate, y float32) or the gated product.

    In gated mode ``w`` has ``2 * y.shape[1]`` rows in groups of ``glu_group``
    gate rows followed by the ``glu_group`` up rows of the same outputs (0: all
    gate rows, then all up rows).
    """
    _cuda(x, w, y)
    if not w.is_contiguous() or w.dim() != 2:
        raise KernelError("linear: the weight must be a contiguous matrix")
    m, k = x.shape
    n = y.shape[1]
    if w.shape[1] != k or w.shape[0] != (2 * n if mode == GATED else n) or y.shape[0] != m:
        raise KernelError(f"linear: shapes x {tuple(x.shape)} w {tuple(w.shape)} y {tuple(y.shape)} mode {mode}")
    f = _fn("linear_plain", "skyla_linear_plain",
            [c_void_p, c_int, c_int64, c_void_p, c_int, c_int, c_int, c_int, c_void_p, c_int, c_int64,
             c_int, c_int, c_void_p])
    _check("linear_plain", f(_ptr(x), dtype_code(x), _rows(x, "x"), _ptr(w), dtype_code(w), m, n, k,
                             _ptr(y), dtype_code(y), _rows(y, "y"), mode, glu_group or n, _stream()))
    return y


# ---------------------------------------------------------- tensor-core linear
TC_STORE_BF16, TC_STORE_F32, TC_ACCUM_F32, TC_GLU_BF16 = 0, 1, 2, 3
TC_TOKEN_TILES = (16, 32, 64, 128, 256)


class KernelState:
    """Device memory that the kernels of ONE engine keep between their launches.

    * ``error_flag``: one int32 that a kernel raises when a bounded wait ran out (codes 1 to 19),
      when the sampler found no token in a row of logits (31: every logit NaN) or when a token fed
      on the device lies outside the embedding table (32);
    * counters with which the blocks of a launch find out which of them finishes last (the pieces of a
      sequence in decode attention): zero between launches;
    * the scratch and the flags of the prompt product's tiles that are cut along K.

    An engine owns one (``Runtime.kernel_state``) and hands it to every launch, so two engines on
    two streams share nothing.  The launches of one state must not overlap on the device: one
    engine runs its steps on one stream.  Launches that name no state (kernel tests, the kernel
    benchmark) use the device's default state.  Buffers that had to grow stay alive, because a
    recorded CUDA graph may still point at the old ones.
    """

    MERGE_COUNTERS = 1 << 16

    def __init__(self, device):
        self.device = torch.device(device)
        self.error_flag = torch.zeros(1, dtype=torch.int32, device=self.device)
        self._merge = None
        self._shares = None

    @property
    def sm_count(self) -> int:
        return torch.cuda.get_device_properties(self.device).multi_processor_count

    def merge_counters(self) -> torch.Tensor:
        """One zeroed int32 per (sequence, key/value head) of a decode step."""
        if self._merge is None:
            self._merge = torch.zeros(self.MERGE_COUNTERS, dtype=torch.int32, device=self.device)
        return self._merge

    def prompt_shares(self):
        """(scratch for one accumulator tile per SM, a flag per SM, SMs) for ``gemm_prompt``'s tiles
        that are cut along K."""
        if self._shares is None:
            n = self.sm_count
            self._shares = (torch.empty(n * 128 * 256, dtype=torch.float32, device=self.device),
                            torch.zeros(n, dtype=torch.int32, device=self.device), n)
        return self._shares

    def reset(self) -> None:
        """Everything that has to be zero between launches is zero again (after a kernel gave up,
        any of it may have been left raised)."""
        self.error_flag.zero_()
        if self._merge is not None:
            self._merge.zero_()
        if self._shares is not None:
            self._shares[1].zero_()

    def raise_if(self, code: int) -> None:
        """``code`` is the error word as read on the host (0: nothing happened)."""
        if not code:
            return
        self.reset()
        if code == 31:
            what = "the sampler found no token in a row of logits (all NaN?) and gave token 0"
        elif code == 32:
            what = "a token fed on the device lies outside the embedding table; its row was zero-filled"
        else:
            what = f"a kernel's bounded wait ran out (code {code})"
        raise KernelError(f"{what}; the results since the last check are not valid")

    def check(self) -> None:
        """Raise if a kernel reported an error since the last check (synchronizes)."""
        self.raise_if(int(self.error_flag.item()))


_DEFAULT_STATES = {}


def default_state(device) -> KernelState:
    dev = torch.device(device)
    if dev.index is None:
        dev = torch.device(dev.type, torch.cuda.current_device())
    st = _DEFAULT_STATES.get(dev)
    if st is None:
        st = _DEFAULT_STATES[dev] = KernelState(dev)
    return st


def _state(state: Optional[KernelState], t: torch.Tensor) -> KernelState:
    return state if state is not None else default_state(t.device)


def check_device_errors(device) -> None:
    """Raise if a kernel launched without a state of its own gave up since the last check."""
    default_state(device).check()


class TensorMap:
    """A TMA descriptor of a row-major bfloat16 matrix, boxes of [box_rows x 64]; with
    ``box_kblocks`` > 1 a box brings that many 64-column blocks of its rows (the width must
    then be a multiple of 64)."""

    __slots__ = ("buf", "key", "keep")

    def __init__(self, t: torch.Tensor, box_rows: int, box_kblocks: int = 1):
        _cuda(t)
        if t.dtype != torch.bfloat16 or t.dim() != 2:
            raise KernelError("tensor maps are built for 2-D bfloat16 tensors")
        ld = _rows(t, "tensor map")
        self.buf = ctypes.create_string_buffer(128)
        self.keep = t
        f = _fn("gemm_tc", "skyla_tensor_map_bf16",
                [c_void_p, c_void_p, c_uint64, c_uint64, c_uint64, ctypes.c_uint32, ctypes.c_uint32])
        _check_nolaunch("gemm_tc", f(self.buf, _ptr(t), t.shape[0], t.shape[1], ld, box_rows, box_kblocks))


_X_MAPS = {}


def activation_map(x: torch.Tensor, box_rows: int, box_kblocks: int = 1) -> TensorMap:
    """Tensor maps of workspace buffers are few (the buffers are reused) and cached."""
    key = (x.data_ptr(), x.shape[0], x.shape[1], x.stride(0), box_rows, box_kblocks)
    m = _X_MAPS.get(key)
    if m is None:
        if len(_X_MAPS) > 4096:
            _X_MAPS.clear()
        m = _X_MAPS[key] = TensorMap(x, box_rows, box_kblocks)
        m.keep = None  # do not pin workspace memory; the key holds the address
    return m


def tc_linear_ok(x: torch.Tensor, w: torch.Tensor) -> bool:
    """Whether the tensor-core kernel takes these operands (bfloat16, 16-byte rows)."""
    return (x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and x.dim() == 2 and w.is_contiguous()
            and x.shape[1] % 8 == 0 and x.stride(1) == 1 and (x.shape[0] == 1 or x.stride(0) % 8 == 0)
            and x.data_ptr() % 16 == 0 and w.data_ptr() % 16 == 0)


def token_tile(m: int, gated: bool = False) -> int:
    """Tokens per tile of the weight-major kernels (128 at most for the gated product, whose two
    accumulators are twice as wide).  From 129 tokens on the parts use :func:`gemm_prompt` instead."""
    for bn in TC_TOKEN_TILES:
        if m <= bn:
            return 128 if gated and bn == 256 else bn
    return 128 if gated else 256


def gemm_tc(x: torch.Tensor, w_map: TensorMap, n_out: int, y: torch.Tensor, mode: int, bn: Optional[int] = None,
            state: Optional[KernelState] = None) -> torch.Tensor:
    """y = x W^T on the tensor cores, whole K in every block.  ``w_map`` has boxes of 128 rows; a gated
    weight holds the ``n_out`` gate rows, then the up rows.
    ``mode``: TC_STORE_BF16 / TC_STORE_F32 / TC_ACCUM_F32 (``y += x W^T``, the residual add) / TC_GLU_BF16.
    """
    m, k = x.shape
    bn = bn or token_tile(m, mode == TC_GLU_BF16)
    want = {TC_STORE_BF16: torch.bfloat16, TC_GLU_BF16: torch.bfloat16}.get(mode, torch.float32)
    if y.dtype != want:
        raise KernelError(f"gemm_tc: epilogue {mode} writes {want}, y is {y.dtype}")
    if y.shape[0] != m or y.shape[1] != n_out:
        raise KernelError(f"gemm_tc: y {tuple(y.shape)} is not [{m}, {n_out}]")
    xm = activation_map(x, bn)
    f = _fn("gemm_tc", "skyla_gemm_tc",
            [c_void_p, c_void_p, c_void_p, c_int64, c_int, c_int, c_int, c_int, c_int, c_void_p, c_void_p])
    _check("gemm_tc", f(w_map.buf, xm.buf, _ptr(y), _rows(y, "y"), m, n_out, k, bn, mode,
                        _ptr(_state(state, x).error_flag), _stream()))
    return y


ROWS_MAX_TOKENS = 128
ROWS_MAX_SPLITS = 8


_CLUSTER_ROOM = {}


def rows_cluster_room(device) -> dict:
    """{blocks per cluster: clusters that the device holds at a time} for the weight-streaming kernel,
    asked from the occupancy calculator once per device (clusters stay inside a GPC, so it is less
    than SMs / size: on a B200 33 clusters of four)."""
    dev = torch.device(device)
    room = _CLUSTER_ROOM.get(dev)
    if room is None:
        f = _fn("gemm_tc", "skyla_gemm_tc_rows_max_clusters", [c_int])
        room = {}
        with torch.cuda.device(dev):
            for size in (2, 4):
                n = int(f(size))
                if n < 0:
                    _check_nolaunch("gemm_tc", n)
                room[size] = n
        _CLUSTER_ROOM[dev] = room
    return room


def rows_cluster_plan(n_out: int, n_in: int, bn: int, room: dict):
    """The plan for 17 to 128 tokens of a product that is not gated: tiles of up to 128 rows whose K is
    cut into a cluster of 2 or 4 splits, chosen so that all blocks run at once (``room``: clusters of
    each size that fit) and a block moves as few bytes as possible (its share of the weight and of the
    tokens' rows, which every tile reads whole).  ``None`` where K is too short to cut."""
    if n_in % 64 or n_out % 4:  # (the owners of a cluster write four neighbouring outputs at once)
        return None
    n_kb = n_in // 64
    best, best_cost = None, None
    for splits in (2, 4):
        if n_kb < 8 * splits or room.get(splits, 0) < 1:
            continue
        rows = -(-n_out // room[splits])              # the fewest rows whose tiles fit at once
        rows = max(8, -(-rows // 8) * 8)
        if rows > 128:
            continue
        cost = (rows + bn) * -(-n_kb // splits)
        if best_cost is None or cost < best_cost:
            # boxes of two K blocks; of one for the widest token tile, whose landing zone leaves the ring less room
            best, best_cost = (rows, splits, 2 if bn <= 64 else 1, 1), cost
    return best


def rows_plan(n_out: int, n_in: int, gated: bool = False, bn: int = 16, n_sms: int = 148):
    """(rows per block, K splits, K blocks per box, K blocks per MMA) for the few-token product
    of a weight [n_out (x2 when gated), n_in] with token tiles of ``bn``.

    The tile height is the smallest multiple of 8 whose tiles fill the ``n_sms`` SMs in whole waves.
    Tiles of at most 64 rows stack 128 / rows K blocks into one MMA, so that a block covers
    all of K without a K split; a box brings about 32 KB of weights (a TMA load costs the
    same 0.16 us whatever it brings).  K that is no multiple of 64 has to do with one K
    block per box (two-dimensional tensor maps).
    """
    waves = -(-n_out // (n_sms * 128))
    rows = -(-n_out // (n_sms * waves))
    rows = min(128, max(8, -(-rows // 8) * 8))
    if n_in % 64:
        return rows, 1, 1, 1
    if gated:
        return rows, 1, 2 if bn <= 64 else 1, 1        # (a stage holds both halves of the weight tile and the tokens)
    n_kb = n_in // 64
    kstack = max(1, min(128 // rows, 256 // bn, n_kb))
    group = kstack * rows * 128                     # bytes of weights that one MMA takes
    per_box = max(1, min(-(-28 * 1024 // group), 16 // kstack, -(-n_kb // kstack)))
    while per_box > 1 and per_box * kstack * (rows + bn) * 128 > 48 * 1024:
        per_box -= 1                                 # four stages or more in the ring
    return rows, 1, per_box * kstack, kstack


def gemm_tc_rows(x: torch.Tensor, w_map: TensorMap, rows: int, n_out: int, y: torch.Tensor, mode: int,
                 kkb: int = 1, splits: int = 1, kstack: int = 1, norm_ahead=None, scale_in=None,
                 state: Optional[KernelState] = None) -> torch.Tensor:
    """y = x W^T for at most 128 tokens, streaming the weight: blocks of ``rows`` weight rows
    (a multiple of 8 up to 128), K cut into ``splits`` that meet in a thread-block cluster.

    ``w_map`` has boxes of ``rows`` rows and ``kkb`` K blocks, of which one MMA takes ``kstack``
    at once (then ``kstack * rows <= 128``, one split, not gated); a gated weight holds the
    ``n_out`` gate rows, then the up rows.  Modes TC_STORE_BF16 / TC_STORE_F32 / TC_ACCUM_F32 /
    TC_GLU_BF16 (one split).
    ``norm_ahead=(w, xw, ssq_parts)`` with TC_ACCUM_F32: ``y`` being the residual stream, also leave
    ``xw = bf16(y_new * w)`` [tokens, n_out] and ``ssq_parts`` [blocks, tokens], every block's share of
    the new rows' sums of squares, for the RMSNorm (weight ``w``) that reads ``y`` next.
    ``scale_in=(ssq_parts, eps)``: ``x`` is such an ``xw``; the result is multiplied by the rows'
    ``1/sqrt(sum(ssq_parts) / K + eps)``.
    """
    want = {TC_STORE_BF16: torch.bfloat16, TC_GLU_BF16: torch.bfloat16}.get(mode, torch.float32)
    if y.dtype != want:
        raise KernelError(f"gemm_tc_rows: epilogue {mode} writes {want}, y is {y.dtype}")
    _cuda(x, y)
    m, k = x.shape
    if m > ROWS_MAX_TOKENS:
        raise KernelError(f"gemm_tc_rows: at most {ROWS_MAX_TOKENS} tokens")
    bn = token_tile(m)
    xm = activation_map(x, bn, kkb)
    if tuple(y.shape) != (m, n_out):
        raise KernelError(f"gemm_tc_rows: y {tuple(y.shape)} is not [{m}, {n_out}]")
    blocks = -(-n_out // rows)
    ahead_args = [c_void_p(0), c_void_p(0), 0, c_void_p(0)]
    if norm_ahead is not None:
        aw, axw, assq = norm_ahead
        _cuda(aw, axw, assq)
        if (aw.dtype != torch.float32 or aw.numel() != n_out or not aw.is_contiguous() or axw.dtype != torch.bfloat16
                or tuple(axw.shape) != (m, n_out) or axw.stride(1) != 1 or assq.dtype != torch.float32
                or tuple(assq.shape) != (blocks, m) or not assq.is_contiguous()):
            raise KernelError(f"gemm_tc_rows: norm-ahead wants w [{n_out}] float32, xw [{m}, {n_out}] bfloat16, "
                              f"ssq_parts [{blocks}, {m}] float32")
        ahead_args = [_ptr(aw), _ptr(axw), axw.stride(0), _ptr(assq)]
    scale_args = [c_void_p(0), 0, 0.0]
    if scale_in is not None:
        sssq, seps = scale_in
        _cuda(sssq)
        if sssq.dtype != torch.float32 or sssq.dim() != 2 or sssq.shape[1] != m or not sssq.is_contiguous():
            raise KernelError(f"gemm_tc_rows: handed-in sums of squares are float32 [parts, {m}]")
        scale_args = [_ptr(sssq), sssq.shape[0], float(seps)]
    f = _fn("gemm_tc", "skyla_gemm_tc_rows",
            [c_void_p, c_void_p, c_void_p, c_int64, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_int,
             c_void_p, c_void_p, c_void_p, c_int64, c_void_p, c_void_p, c_int, c_float, c_void_p])
    _check("gemm_tc", f(w_map.buf, xm.buf, _ptr(y), _rows(y, "y"), m, n_out, k, bn, mode, rows, kkb, kstack, splits,
                        _ptr(_state(state, x).error_flag), *ahead_args, *scale_args, _stream()))
    return y


# ------------------------------------------------------- tensor-core linear, prompts
TC_QKV_PREP = 4  # gemm_prompt only: the product's heads go through norm and rotation into q and the cache
# Fewer tokens leave most of a 128-token tile empty, and the weight-major kernels take them.  (At 96 and
# 128 tokens of the 8B shape the two are about even: QKV 28 against 21 us, O 26 against 25, gate/up 48
# against 48, down 41 against 60.)
PROMPT_MIN_TOKENS = 129


_Y_MAPS = {}


def _output_map(y: torch.Tensor):
    """The tensor map through which ``gemm_prompt`` adds into ``y`` (cached: workspace buffers are few)."""
    key = (y.data_ptr(), y.shape[0], y.shape[1], y.stride(0))
    buf = _Y_MAPS.get(key)
    if buf is None:
        if len(_Y_MAPS) > 1024:
            _Y_MAPS.clear()
        buf = ctypes.create_string_buffer(128)
        f = _fn("gemm_prompt", "skyla_output_map_f32", [c_void_p, c_void_p, c_uint64, c_uint64, c_uint64])
        _check_nolaunch("gemm_prompt", f(buf, _ptr(y), y.shape[0], y.shape[1], _rows(y, "y")))
        _Y_MAPS[key] = buf
    return buf


def prompt_cut_blocks(m: int, n_out: int, k: int, gated: bool, device) -> int:
    """Over how many blocks ``gemm_prompt`` cuts this product's tiles along K (0: whole tiles)."""
    f = _fn("gemm_prompt", "skyla_gemm_prompt_cut_blocks", [c_int, c_int, c_int, c_int, c_int])
    return int(f(m, n_out, k, int(gated), torch.cuda.get_device_properties(device).multi_processor_count))


def prompt_ahead_parts(n_out: int) -> int:
    """Shares of a row's sum of squares that ``gemm_prompt(..., norm_ahead=...)`` leaves: one per tile of 256 outputs."""
    return -(-n_out // 256)


def gemm_prompt(x: torch.Tensor, w_map: TensorMap, n_out: int, y: torch.Tensor, mode: int, scale_in=None,
                norm_ahead=None, prep=None, tma_add: bool = True, cut_k: bool = True,
                state: Optional[KernelState] = None) -> torch.Tensor:
    """y = x W^T for a prompt's tokens, a token's row of a tile in one thread of the epilogue.

    ``w_map`` has boxes of 128 rows; a gated weight holds the ``n_out`` gate rows, then the up rows.
    Modes TC_STORE_BF16 / TC_STORE_F32 / TC_ACCUM_F32 / TC_GLU_BF16 as in :func:`gemm_tc`.
    ``scale_in=(ssq_parts [parts, tokens], eps)``: ``x`` is ``bf16(rows * norm weight)`` of rows whose
    sums of squares lie in ``ssq_parts``; the result is multiplied by ``1/sqrt(sum / K + eps)``.
    ``norm_ahead=(w, xw, ssq_parts)`` with TC_ACCUM_F32: also leave ``xw = bf16(y_new * w)`` and the
    tiles' shares of the new rows' sums of squares, ``ssq_parts`` [prompt_ahead_parts(n_out), tokens].
    Mode TC_QKV_PREP with ``prep=dict(nq, nkv, hd, q_norm, k_norm, eps, cos, sin, tok_pos, tok_slot, k_pool,
    v_pool, page_table, page_size)``: the outputs are ``nq`` query, ``nkv`` key and ``nkv`` value heads of
    ``hd``; q and k heads are RMS-normed (weights may be ``None``) and rotated whole (tables may be
    ``None``), the queries go to ``y`` [tokens, nq * hd] bfloat16, keys and values to the tokens' places
    in the pools (``None``: not written).
    ``tma_add=False``: the accumulate epilogue's threads read, add and write ``y`` themselves (the path
    that ``y`` without 16-byte rows takes anyway); ``cut_k=False``: few tiles stay whole tiles on few SMs.
    """
    _cuda(x, y)
    m, k = x.shape
    want = {TC_STORE_BF16: torch.bfloat16, TC_GLU_BF16: torch.bfloat16, TC_QKV_PREP: torch.bfloat16}.get(mode, torch.float32)
    if y.dtype != want:
        raise KernelError(f"gemm_prompt: epilogue {mode} writes {want}, y is {y.dtype}")
    scale_args = [c_void_p(0), 0, 0.0]
    if scale_in is not None:
        sssq, seps = scale_in
        _cuda(sssq)
        if sssq.dtype != torch.float32 or sssq.dim() != 2 or sssq.shape[1] != m or not sssq.is_contiguous():
            raise KernelError(f"gemm_prompt: handed-in sums of squares are float32 [parts, {m}]")
        scale_args = [_ptr(sssq), sssq.shape[0], float(seps)]
    ahead_args = [c_void_p(0), c_void_p(0), 0, c_void_p(0)]
    if norm_ahead is not None:
        aw, axw, assq = norm_ahead
        _cuda(aw, axw, assq)
        parts = prompt_ahead_parts(n_out)
        if (mode != TC_ACCUM_F32 or aw.dtype != torch.float32 or aw.numel() != n_out or not aw.is_contiguous()
                or axw.dtype != torch.bfloat16 or tuple(axw.shape) != (m, n_out) or axw.stride(1) != 1
                or assq.dtype != torch.float32 or tuple(assq.shape) != (parts, m) or not assq.is_contiguous()):
            raise KernelError(f"gemm_prompt: norm-ahead goes with TC_ACCUM_F32 and wants w [{n_out}] float32, "
                              f"xw [{m}, {n_out}] bfloat16, ssq_parts [{parts}, {m}] float32")
        ahead_args = [_ptr(aw), _ptr(axw), axw.stride(0), _ptr(assq)]
    prep_args = [0, 0, 0, c_void_p(0), c_void_p(0), 0.0, c_void_p(0), c_void_p(0), c_void_p(0), c_void_p(0),
                 c_void_p(0), c_void_p(0), c_void_p(0), 0, 0]
    if mode == TC_QKV_PREP:
        if prep is None:
            raise KernelError("gemm_prompt: TC_QKV_PREP needs prep")
        nq, nkv, hd = int(prep["nq"]), int(prep["nkv"]), int(prep["hd"])
        q_norm, k_norm, cos, sin = prep.get("q_norm"), prep.get("k_norm"), prep.get("cos"), prep.get("sin")
        tok_pos, tok_slot, page_table = prep["tok_pos"], prep.get("tok_slot"), prep.get("page_table")
        k_pool, v_pool, page_size = prep.get("k_pool"), prep.get("v_pool"), int(prep.get("page_size") or 0)
        _cuda(q_norm, k_norm, cos, sin, tok_pos, tok_slot, page_table, k_pool, v_pool)
        if (nq + 2 * nkv) * hd != n_out or tuple(y.shape) != (m, nq * hd):
            raise KernelError(f"gemm_prompt: {nq} + 2 x {nkv} heads of {hd} against {n_out} outputs and y {tuple(y.shape)}")
        for t, what in ((tok_pos, "tok_pos"), (tok_slot, "tok_slot"), (page_table, "page_table")):
            if t is not None:
                _i32(t, what)
        if tok_pos.numel() != m:
            raise KernelError("gemm_prompt: one position per token")
        for t, what, shape in ((q_norm, "q_norm", (hd,)), (k_norm, "k_norm", (hd,)), (cos, "cos", None), (sin, "sin", None)):
            if t is not None and (t.dtype != torch.float32 or not t.is_contiguous() or (shape and tuple(t.shape) != shape)):
                raise KernelError(f"gemm_prompt: {what} must be a contiguous float32 tensor" + (f" {shape}" if shape else ""))
        if cos is not None and (sin is None or cos.shape != sin.shape or cos.dim() != 2 or cos.shape[1] != hd // 2):
            raise KernelError("gemm_prompt: the rotary tables must be [positions, head size / 2]: the whole head rotates")
        max_pages = 0
        if k_pool is not None:
            if (v_pool is None or k_pool.shape != v_pool.shape or tuple(k_pool.shape[1:]) != (nkv, page_size, hd)
                    or k_pool.dtype != torch.bfloat16 or v_pool.dtype != torch.bfloat16
                    or not k_pool.is_contiguous() or not v_pool.is_contiguous() or tok_slot is None or page_table is None
                    or page_table.dim() != 2 or tok_slot.numel() != m):
                raise KernelError(f"gemm_prompt: bfloat16 cache pools [pages, {nkv}, {page_size}, {hd}] with slots and a page table")
            max_pages = page_table.shape[1]
        prep_args = [nq, nkv, hd, _ptr(q_norm), _ptr(k_norm), float(prep.get("eps") or 0.0), _ptr(cos), _ptr(sin),
                     _ptr(tok_pos), _ptr(tok_slot), _ptr(k_pool), _ptr(v_pool), _ptr(page_table), max_pages, page_size]
    elif tuple(y.shape) != (m, n_out):
        raise KernelError(f"gemm_prompt: y {tuple(y.shape)} is not [{m}, {n_out}]")
    xm = activation_map(x, 128)
    ym = None
    if (mode == TC_ACCUM_F32 and norm_ahead is None and tma_add and y.data_ptr() % 16 == 0
            and _rows(y, "y") % 4 == 0):
        ym = _output_map(y)
    f = _fn("gemm_prompt", "skyla_gemm_prompt",
            [c_void_p, c_void_p, c_void_p, c_void_p, c_int64, c_int, c_int, c_int, c_int, c_void_p, c_void_p, c_int, c_float,
             c_void_p, c_void_p, c_int64, c_void_p,
             c_int, c_int, c_int, c_void_p, c_void_p, c_float, c_void_p, c_void_p, c_void_p, c_void_p,
             c_void_p, c_void_p, c_void_p, c_int, c_int, c_void_p, c_void_p, c_int, c_void_p])
    st = _state(state, x)
    share, flags, n_share = st.prompt_shares() if cut_k else (None, None, 0)
    _check("gemm_prompt", f(xm.buf, w_map.buf, ym, _ptr(y), _rows(y, "y"), m, n_out, k, mode, _ptr(st.error_flag),
                            *scale_args, *ahead_args, *prep_args, _ptr(share), _ptr(flags), n_share, _stream()))
    return y


# ------------------------------------------------------------ attention parts
def qk_norm_rope_cache(qkv: torch.Tensor, q_off: int, k_off: int, v_off: int, nq: int, nkv: int,
                       hd: int, q_norm: Optional[torch.Tensor], k_norm: Optional[torch.Tensor],
                       eps: float, cos: Optional[torch.Tensor], sin: Optional[torch.Tensor],
                       n_rot: int, tok_pos: torch.Tensor, tok_slot: torch.Tensor,
                       k_pool: Optional[torch.Tensor], v_pool: Optional[torch.Tensor],
                       page_table: torch.Tensor, page_size: int, q_out: Optional[torch.Tensor] = None) -> None:
    """Per-head norm and rotation of the new tokens; q to ``q_out`` (default: in place), k and
    v into the cache.

    ``qkv``: [tokens, width] rows of the q/k/v product in any precision (32-bit rows go with a
    ``q_out`` of the activations' precision).  ``k_pool``/``v_pool`` of shape
    [pages, nkv, page_size, hd]; ``None`` skips the cache write (a run that reads another
    entry's cache).
    """
    _cuda(qkv, q_norm, k_norm, cos, sin, tok_pos, tok_slot, k_pool, v_pool, page_table, q_out)
    for t, what in ((tok_pos, "tok_pos"), (tok_slot, "tok_slot"), (page_table, "page_table")):
        _i32(t, what)
    for t, what in ((q_norm, "q_norm"), (k_norm, "k_norm"), (cos, "cos"), (sin, "sin")):
        if t is not None and (t.dtype != torch.float32 or not t.is_contiguous()):
            raise KernelError(f"{what}: expected a contiguous float32 tensor")
    n = tok_pos.numel()
    ld = _rows(qkv, "qkv")
    if q_out is None:
        q_ptr, q_dt, ldq = c_void_p(qkv.data_ptr() + q_off * qkv.element_size()), dtype_code(qkv), ld
    else:
        if q_out.shape[0] < n or q_out.shape[1] < nq * hd:
            raise KernelError("qk_norm_rope_cache: q_out too small")
        q_ptr, q_dt, ldq = _ptr(q_out), dtype_code(q_out), _rows(q_out, "q_out")
    if k_pool is not None:
        if (k_pool.shape != v_pool.shape or tuple(k_pool.shape[1:]) != (nkv, page_size, hd)
                or not k_pool.is_contiguous() or not v_pool.is_contiguous()):
            raise KernelError(f"cache pools {tuple(k_pool.shape)} do not match [pages, {nkv}, {page_size}, {hd}]")
        cdt = dtype_code(k_pool)
    else:
        cdt = q_dt
    if cos is not None and (cos.shape != sin.shape or cos.shape[1] != n_rot // 2):
        raise KernelError("rotary table does not match the rotary width")
    f = _fn("attn_prep", "skyla_qk_norm_rope_cache",
            [c_void_p, c_int, c_int64, c_void_p, c_int, c_int64, c_int, c_int, c_int, c_int, c_int,
             c_int, c_int, c_void_p, c_void_p, c_float, c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_void_p,
             c_void_p, c_int, c_void_p, c_int, c_int, c_void_p])
    _check("attn_prep", f(_ptr(qkv), dtype_code(qkv), ld, q_ptr, q_dt, ldq, q_off, k_off,
                          v_off, n, nq, nkv, hd, _ptr(q_norm), _ptr(k_norm), float(eps), _ptr(cos), _ptr(sin),
                          n_rot if cos is not None else 0, _ptr(tok_pos), _ptr(tok_slot),
                          _ptr(k_pool), _ptr(v_pool), cdt, _ptr(page_table), page_table.shape[1],
                          page_size, _stream()))


def attention_plain(q: torch.Tensor, out: torch.Tensor, nq: int, nkv: int, hd: int,
                    k_pool: torch.Tensor, v_pool: torch.Tensor, page_table: torch.Tensor,
                    page_size: int, tok_pos: torch.Tensor, tok_slot: torch.Tensor, scale: float,
                    window: int = 0) -> torch.Tensor:
    """Causal (optionally windowed) attention of each token over its own sequence's cache.

    ``q`` is [tokens, >= nq*hd] with contiguous rows (a view into a fused buffer
    is fine), ``out`` [tokens, nq*hd].
    """
    _cuda(q, out, k_pool, v_pool, page_table, tok_pos, tok_slot)
    for t, what in ((tok_pos, "tok_pos"), (tok_slot, "tok_slot"), (page_table, "page_table")):
        _i32(t, what)
    if q.dtype != out.dtype:
        raise KernelError("attention: q and out must share a dtype")
    if tuple(k_pool.shape[1:]) != (nkv, page_size, hd) or k_pool.shape != v_pool.shape:
        raise KernelError(f"cache pools {tuple(k_pool.shape)} do not match [pages, {nkv}, {page_size}, {hd}]")
    n = tok_pos.numel()
    f = _fn("attention_plain", "skyla_attention_plain",
            [c_void_p, c_int, c_int64, c_void_p, c_int64, c_int, c_int, c_int, c_int, c_void_p,
             c_void_p, c_int, c_void_p, c_int, c_int, c_void_p, c_void_p, c_float, c_int, c_void_p])
    _check("attention_plain", f(_ptr(q), dtype_code(q), _rows(q, "q"), _ptr(out), _rows(out, "out"), n,
                                nq, nkv, hd, _ptr(k_pool), _ptr(v_pool), dtype_code(k_pool),
                                _ptr(page_table), page_table.shape[1], page_size, _ptr(tok_pos),
                                _ptr(tok_slot), float(scale), int(window or 0), _stream()))
    return out


def attention_mma_supports(hd: int, group: int) -> int:
    """0: the tensor-core attention does not take this head size; 1: prefill only; 2: prefill and decode."""
    f = _fn("attention_mma", "skyla_attention_mma_supports", [c_int, c_int])
    return int(f(hd, group))


def _attn_common(q, out, k_pool, v_pool, nq, nkv, hd, page_size, *ints):
    _cuda(q, out, k_pool, v_pool, *ints)
    for t in ints:
        _i32(t, "index array")
    if q.dtype != torch.bfloat16 or out.dtype != torch.bfloat16 or k_pool.dtype != torch.bfloat16:
        raise KernelError("tensor-core attention takes bfloat16 queries, outputs and cache")
    if (tuple(k_pool.shape[1:]) != (nkv, page_size, hd) or k_pool.shape != v_pool.shape
            or not k_pool.is_contiguous() or not v_pool.is_contiguous()):
        raise KernelError(f"cache pools {tuple(k_pool.shape)} do not match [pages, {nkv}, {page_size}, {hd}]")


#: ints per row of a decode plan
DECODE_PLAN_INTS = 8
#: what starting another item costs a block, and what a block costs beside its pages, in pages' time
#: (a page of 64 positions of one key/value head takes about a microsecond)
_PIECE_COST, _BLOCK_COST = 3, 3
_plan_memo: dict = {}


def decode_plan_ints(n_seqs: int, nkv: int, n_blocks: int) -> int:
    """Ints of a decode plan: a row per block, then (first block, pieces) per item."""
    return DECODE_PLAN_INTS * n_blocks + 2 * n_seqs * nkv


def _plan_layout(n_pages, nkv: int, n_blocks: int, even_only: bool):
    """Rows (without the positions) and item table of :func:`decode_plan` for sequences of ``n_pages[b]`` pages."""
    import numpy as np
    B = len(n_pages)
    items = B * nkv
    rows = np.zeros((n_blocks, DECODE_PLAN_INTS), dtype=np.int32)
    table = np.zeros((items, 2), dtype=np.int32)
    total = int(n_pages.sum()) * nkv
    per = max(1, -(-total // n_blocks))
    # even runs: cost of the slowest block
    ends = np.cumsum(n_pages) * nkv                       # where each sequence's items end
    starts = ends - n_pages * nkv
    u0 = np.arange(n_blocks, dtype=np.int64) * per
    live = u0 < total
    u0 = np.where(live, u0, 0)
    u1 = np.minimum(u0 + per, total) - 1                  # a block's last page

    def item_of(u):
        b = np.minimum(np.searchsorted(ends, u, side="right"), B - 1)
        r = u - starts[b]
        return b, r // n_pages[b], r % n_pages[b]
    b0, h0, p0 = item_of(u0)
    b1, h1, _ = item_of(np.maximum(u1, u0))
    pieces = (b1 * nkv + h1) - (b0 * nkv + h0) + 1
    even_cost = _BLOCK_COST + per + _PIECE_COST * (int(pieces[live].max()) - 1)
    # runs that end with their item: every item in k equal pieces, as few pages a piece as the blocks allow
    m = n_blocks // nkv
    if m >= B and not even_only:
        size = max(1, -(-int(n_pages.sum()) // m))
        while int((-(-n_pages // size)).sum()) > m:
            size += 1
        k = -(-n_pages // size)
        if _BLOCK_COST + int((-(-n_pages // k)).max()) <= even_cost:
            first_block = (np.cumsum(k) - k) * nkv       # of each sequence's first item
            # piece c of an item of n pages and k pieces starts at page c * n // k
            seq = np.repeat(np.arange(B), k * nkv)
            head = np.concatenate([np.repeat(np.arange(nkv), kb) for kb in k])
            piece = np.concatenate([np.tile(np.arange(kb), nkv) for kb in k])
            n_of, k_of = n_pages[seq], k[seq]
            lo = piece * n_of // k_of
            used = len(seq)
            rows[:used, 0], rows[:used, 1], rows[:used, 2] = seq, head, lo
            rows[:used, 3] = (piece + 1) * n_of // k_of - lo
            rows[:used, 5] = first_block[seq] + head * k_of
            rows[:used, 6] = k_of
            item_seq = np.repeat(np.arange(B), nkv)
            table[:, 0] = first_block[item_seq] + np.tile(np.arange(nkv), B) * k[item_seq]
            table[:, 1] = k[item_seq]
            return rows, table
    rows[:, 0], rows[:, 1], rows[:, 2] = np.where(live, b0, 0), np.where(live, h0, 0), np.where(live, p0, 0)
    rows[:, 3] = np.where(live, u1 - u0 + 1, 0)
    item_seq = np.repeat(np.arange(B), nkv)
    lo = starts[item_seq] + np.tile(np.arange(nkv), B) * n_pages[item_seq]
    table[:, 0] = lo // per
    table[:, 1] = (lo + n_pages[item_seq] - 1) // per - lo // per + 1
    first_item = b0 * nkv + h0
    rows[:, 5] = np.where(live, table[first_item, 0], 0)
    rows[:, 6] = np.where(live, table[first_item, 1], 0)
    return rows, table


def decode_plan(positions, nkv: int, window: int, page_size: int, n_blocks: int, out=None, even_only: bool = False):
    """Which pages each block of a decode launch reads, made on the host: int32, :func:`decode_plan_ints` long.

    ``positions[b]`` is the position of sequence b's new token.  The items of the step are its
    (sequence, key/value head) pairs, item = sequence * nkv + head, each with the pages from the
    window's first to the new token's.  Blocks take runs of consecutive pages of consecutive items:
    row j = (sequence, head, page of that item where the run starts, pages of the run, position of that
    sequence's new token, first block and number of pieces of that item, 0).  After the rows, for every
    item, (first block, pieces): the blocks that read pieces of one item are consecutive.
    Two ways of cutting, whichever makes the slowest block faster: every item in equal pieces, so that no
    block has to start a second item (few long sequences); or all pages laid end to end and cut into
    even runs, whatever the lengths are (more items than blocks, unequal lengths).
    ``attn_decode_plan_kernel`` writes a plan of the second kind (``even_only``) from positions that only
    the device has.
    """
    import numpy as np
    pos = np.asarray(positions, dtype=np.int64)
    first = np.maximum(pos - window + 1, 0) if window and window > 0 else np.zeros_like(pos)
    n_pages = pos // page_size + 1 - first // page_size
    key = (nkv, n_blocks, even_only, n_pages.tobytes())
    got = _plan_memo.get(key)
    if got is None:                                       # the cuts change only when a sequence gains a page
        if len(_plan_memo) > 256:
            _plan_memo.clear()
        got = _plan_memo[key] = _plan_layout(n_pages, nkv, n_blocks, even_only)
    rows, table = got
    if out is None:
        out = np.empty(decode_plan_ints(len(pos), nkv, n_blocks), dtype=np.int32)
    out_rows = out[: rows.size].reshape(rows.shape)
    out_rows[:] = rows
    out_rows[:, 4] = np.where(rows[:, 3] > 0, pos[rows[:, 0]], 0)
    out[rows.size:] = table.reshape(-1)
    return out


def attention_decode_plan(tok_pos: torch.Tensor, nkv: int, window: int, n_blocks: int,
                          plan: Optional[torch.Tensor] = None) -> torch.Tensor:
    """:func:`decode_plan` by a kernel, from positions on the device (pages of 64 positions)."""
    _cuda(tok_pos, plan); _i32(tok_pos, "tok_pos")
    need = decode_plan_ints(tok_pos.numel(), nkv, n_blocks)
    if plan is None:
        plan = torch.empty(need, dtype=torch.int32, device=tok_pos.device)
    _i32(plan, "plan")
    if plan.numel() < need:
        raise KernelError("attention_decode_plan: plan too small")
    f = _fn("attention_mma", "skyla_attention_decode_plan", [c_void_p, c_int, c_int, c_int, c_int, c_void_p, c_void_p])
    _check("attention_mma", f(_ptr(tok_pos), tok_pos.numel(), nkv, int(window or 0), n_blocks, _ptr(plan), _stream()))
    return plan


def attention_decode_scratch(n_seqs: int, nq: int, nkv: int, hd: int, n_blocks: int) -> int:
    """Floats of scratch that a decode launch needs: a partial result for every piece of an item that a
    block reads, and two ints per item for the merge kernel."""
    return (n_blocks + n_seqs * nkv) * (nq // nkv) * (hd + 2) + 2 * n_seqs * nkv


def _decode_plan_arg(plan, n_seqs, nkv, n_blocks, what):
    _cuda(plan); _i32(plan, "plan")
    if plan.numel() < decode_plan_ints(n_seqs, nkv, n_blocks) or plan.data_ptr() % 16:
        raise KernelError(f"{what}: a plan of {n_blocks} rows of {DECODE_PLAN_INTS} ints and two ints per item, 16-byte aligned")


def attention_decode(q: torch.Tensor, out: torch.Tensor, scratch: torch.Tensor, nq: int, nkv: int, hd: int,
                     k_pool: torch.Tensor, v_pool: torch.Tensor, pages: torch.Tensor, page_size: int,
                     tok_pos: torch.Tensor, scale: float, window: int, n_blocks: int,
                     plan: Optional[torch.Tensor] = None, state: Optional[KernelState] = None) -> torch.Tensor:
    """One new token per sequence (token b belongs to sequence b): attention over the cache for all
    query heads of a key/value head at once, the step's pages dealt evenly to ``n_blocks`` blocks.

    ``scratch``: float32, at least :func:`attention_decode_scratch` elements.
    ``plan``: :func:`decode_plan` on the device (default: made here by :func:`attention_decode_plan`).
    """
    _attn_common(q, out, k_pool, v_pool, nq, nkv, hd, page_size, pages, tok_pos)
    n = tok_pos.numel()
    if plan is None:
        plan = attention_decode_plan(tok_pos, nkv, window, n_blocks)
    _decode_plan_arg(plan, n, nkv, n_blocks, "attention_decode")
    if scratch.dtype != torch.float32 or scratch.numel() < attention_decode_scratch(n, nq, nkv, hd, n_blocks):
        raise KernelError("attention_decode: scratch too small")
    f = _fn("attention_mma", "skyla_attention_decode",
            [c_void_p, c_int64, c_void_p, c_int64, c_void_p, c_int64, c_int, c_int, c_int, c_int, c_void_p, c_void_p,
             c_void_p, c_int, c_int, c_void_p, c_float, c_int, c_void_p, c_int, c_void_p, c_int, c_void_p])
    counters = _state(state, q).merge_counters()
    _check("attention_mma", f(_ptr(q), _rows(q, "q"), _ptr(out), _rows(out, "out"), _ptr(scratch), scratch.numel(),
                              n, nq, nkv, hd, _ptr(k_pool), _ptr(v_pool), _ptr(pages), pages.shape[1], page_size,
                              _ptr(tok_pos), float(scale), int(window or 0), _ptr(plan), n_blocks,
                              _ptr(counters), counters.numel(), _stream()))
    if tok_pos.numel() * nkv > counters.numel():
        global LAUNCHES
        LAUNCHES += 1  # the merge kernel, which otherwise is part of the attention kernel
    return out


def attention_decode_fused(qkv: torch.Tensor, q_off: int, k_off: int, v_off: int, q_norm: Optional[torch.Tensor],
                           k_norm: Optional[torch.Tensor], eps: float, cos: Optional[torch.Tensor],
                           sin: Optional[torch.Tensor], n_rot: int, out: torch.Tensor, scratch: torch.Tensor,
                           nq: int, nkv: int, hd: int, k_pool: torch.Tensor, v_pool: torch.Tensor,
                           pages: torch.Tensor, page_size: int, tok_pos: torch.Tensor, scale: float, window: int,
                           n_blocks: int, plan: torch.Tensor, state: Optional[KernelState] = None) -> torch.Tensor:
    """Decode attention that also finishes the new token's q, k and v (what
    ``qk_norm_rope_cache`` does) from the float32 rows ``qkv`` [tokens, width] of the q/k/v
    product, and writes k and v to the cache.

    The kernel reads ``plan`` while the kernel launched before it may still run, so the plan must
    be older than that one: copied from the host (:func:`decode_plan`), or written by
    :func:`attention_decode_plan` and waited for."""
    _cuda(qkv, q_norm, k_norm, cos, sin, out, scratch, k_pool, v_pool, pages, tok_pos)
    _i32(pages, "pages"); _i32(tok_pos, "tok_pos")
    n = tok_pos.numel()
    _decode_plan_arg(plan, n, nkv, n_blocks, "attention_decode_fused")
    if qkv.dtype != torch.float32 or qkv.dim() != 2 or qkv.shape[0] != n or qkv.stride(1) != 1:
        raise KernelError("attention_decode_fused: the q/k/v rows are float32 [tokens, width]")
    if out.dtype != torch.bfloat16 or k_pool.dtype != torch.bfloat16 or tuple(k_pool.shape[1:]) != (nkv, page_size, hd) \
            or k_pool.shape != v_pool.shape or not k_pool.is_contiguous() or not v_pool.is_contiguous():
        raise KernelError("attention_decode_fused: bfloat16 output and cache pools [pages, kv heads, page, head]")
    for t_, what in ((q_norm, "q_norm"), (k_norm, "k_norm"), (cos, "cos"), (sin, "sin")):
        if t_ is not None and (t_.dtype != torch.float32 or not t_.is_contiguous()):
            raise KernelError(f"{what}: expected a contiguous float32 tensor")
    if scratch.dtype != torch.float32 or scratch.numel() < attention_decode_scratch(n, nq, nkv, hd, n_blocks):
        raise KernelError("attention_decode_fused: scratch too small")
    f = _fn("attention_mma", "skyla_attention_decode_fused",
            [c_void_p, c_int64, c_int, c_int, c_int, c_void_p, c_void_p,
             c_float, c_void_p, c_void_p, c_int, c_void_p, c_int64, c_void_p, c_int64, c_int, c_int, c_int, c_int, c_void_p,
             c_void_p, c_void_p, c_int, c_int, c_void_p, c_float, c_int, c_void_p, c_int, c_void_p, c_int, c_void_p])
    counters = _state(state, out).merge_counters()
    _check("attention_mma", f(_ptr(qkv), _rows(qkv, "qkv"), q_off, k_off, v_off,
                              _ptr(q_norm), _ptr(k_norm), float(eps), _ptr(cos), _ptr(sin), n_rot if cos is not None else 0,
                              _ptr(out), _rows(out, "out"), _ptr(scratch), scratch.numel(), n, nq, nkv, hd,
                              _ptr(k_pool), _ptr(v_pool), _ptr(pages), pages.shape[1], page_size, _ptr(tok_pos),
                              float(scale), int(window or 0), _ptr(plan), n_blocks, _ptr(counters), counters.numel(),
                              _stream()))
    if tok_pos.numel() * nkv > counters.numel():
        global LAUNCHES
        LAUNCHES += 1  # the merge kernel, which otherwise is part of the attention kernel
    return out


def attention_prefill(q: torch.Tensor, out: torch.Tensor, nq: int, nkv: int, hd: int, k_pool: torch.Tensor,
                      v_pool: torch.Tensor, pages: torch.Tensor, page_size: int, tok_pos: torch.Tensor,
                      tile_seq: torch.Tensor, tile_tok0: torch.Tensor, tile_rows: torch.Tensor, scale: float,
                      window: int = 0, tcgen05: bool = True, state: Optional[KernelState] = None) -> torch.Tensor:
    """Causal attention of new tokens in tiles of up to ``PREFILL_TILE`` tokens of one sequence.  Heads of
    128 with an even number of query heads per key/value head run on the tcgen05 kernel (unless
    ``tcgen05=False``), the others on the mma.sync one."""
    _attn_common(q, out, k_pool, v_pool, nq, nkv, hd, page_size, pages, tok_pos, tile_seq, tile_tok0, tile_rows)
    if (tcgen05 and hd == 128 and page_size == 64 and (nq // nkv) % 2 == 0 and q.dtype == torch.bfloat16
            and q.stride(1) == 1 and q.stride(0) % 8 == 0 and q.data_ptr() % 16 == 0 and q.shape[1] == nq * hd
            and out.stride(0) % 8 == 0 and out.data_ptr() % 16 == 0):
        key = (k_pool.data_ptr(), v_pool.data_ptr(), k_pool.numel())
        maps = _POOL_MAPS.get(key)
        if maps is None:
            if len(_POOL_MAPS) > 1024:
                _POOL_MAPS.clear()
            maps = _POOL_MAPS[key] = (TensorMap(k_pool.view(-1, hd), 64, 2), TensorMap(v_pool.view(-1, hd), 64, 2))
            maps[0].keep = maps[1].keep = None  # the key holds the addresses; do not pin the pools
        q_map = activation_map(q, 64)
        f = _fn("attention_tc", "skyla_attention_prefill_tc",
                [c_void_p, c_void_p, c_void_p, c_void_p, c_int64, c_int, c_int, c_int, c_int, c_void_p, c_int, c_int,
                 c_void_p, c_void_p, c_void_p, c_void_p, c_float, c_int, c_void_p, c_void_p])
        _check("attention_tc", f(q_map.buf, maps[0].buf, maps[1].buf, _ptr(out), _rows(out, "out"), tile_seq.numel(), nq,
                                 nkv, hd, _ptr(pages), pages.shape[1], page_size, _ptr(tok_pos), _ptr(tile_seq),
                                 _ptr(tile_tok0), _ptr(tile_rows), float(scale), int(window or 0),
                                 _ptr(_state(state, q).error_flag), _stream()))
        return out
    f = _fn("attention_mma", "skyla_attention_prefill",
            [c_void_p, c_int64, c_void_p, c_int64, c_int, c_int, c_int, c_int, c_void_p, c_void_p, c_void_p,
             c_int, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_float, c_int, c_void_p])
    _check("attention_mma", f(_ptr(q), _rows(q, "q"), _ptr(out), _rows(out, "out"), tile_seq.numel(), nq, nkv, hd,
                              _ptr(k_pool), _ptr(v_pool), _ptr(pages), pages.shape[1], page_size, _ptr(tok_pos),
                              _ptr(tile_seq), _ptr(tile_tok0), _ptr(tile_rows), float(scale), int(window or 0),
                              _stream()))
    return out


#: the prefill attention kernels work on tiles of this many consecutive new tokens of one sequence
PREFILL_TILE = 64
_POOL_MAPS = {}


# ------------------------------------------------------------------- sampling
def sample(logits: torch.Tensor, out: torch.Tensor, temperature: float = 0.0, top_k: int = 0,
           top_p: float = 1.0, seed: int = 0, req_ids: Optional[torch.Tensor] = None,
           steps: Optional[torch.Tensor] = None, state: Optional[KernelState] = None) -> torch.Tensor:
    """One token per row of float32 logits: argmax when ``temperature`` is 0, else a seeded draw.
    A row in which nothing compares (all NaN) gives token 0 and raises the state's error word."""
    _cuda(logits, out, req_ids, steps)
    _i32(out, "out"); _i32(req_ids, "req_ids"); _i32(steps, "steps")
    if logits.dtype != torch.float32:
        raise KernelError("sample: logits must be float32")
    n, vocab = logits.shape
    if out.numel() < n:
        raise KernelError("sample: output too small")
    f = _fn("sampling", "skyla_sample",
            [c_void_p, c_int64, c_int, c_int, c_float, c_int, c_float, c_uint64, c_void_p, c_void_p,
             c_void_p, c_void_p, c_void_p])
    _check("sampling", f(_ptr(logits), _rows(logits, "logits"), n, vocab, float(temperature),
                         int(top_k), float(top_p), int(seed) & 0xFFFFFFFFFFFFFFFF, _ptr(req_ids),
                         _ptr(steps), _ptr(out), _ptr(_state(state, logits).error_flag), _stream()))
    return out


# ------------------------------------------------------------------ utilities
def bandwidth_read(buf: torch.Tensor, blocks: int, sink: torch.Tensor) -> None:
    _cuda(buf, sink)
    f = _fn("util", "skyla_bandwidth_read", [c_void_p, c_size_t, c_int, c_void_p, c_void_p])
    _check("util", f(_ptr(buf), buf.numel() * buf.element_size(), blocks, _ptr(sink), _stream()))


def fill_normal(out: torch.Tensor, mean: float, std: float, seed: int) -> torch.Tensor:
    _cuda(out)
    if not out.is_contiguous():
        raise KernelError("fill_normal: tensor must be contiguous")
    f = _fn("util", "skyla_fill_normal", [c_void_p, c_int, c_size_t, c_float, c_float, c_uint64, c_void_p])
    _check("util", f(_ptr(out), dtype_code(out), out.numel(), float(mean), float(std),
                     int(seed) & 0xFFFFFFFFFFFFFFFF, _stream()))
    return out
