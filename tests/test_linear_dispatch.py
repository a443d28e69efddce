"""Which kernel a matrix product goes to is decided from shapes alone (``parts/linear.py``): these
decisions are checked here without a GPU, at the layer sizes of the benchmark model."""
import torch

from skyla_kernel_b200.kernels import ops
from skyla_kernel_b200.parts.base import Runtime
from skyla_kernel_b200.parts.linear import Linear

H, QKV, INTER = 4096, 6144, 12288


def _lin(n_out, n_in, gated=False, dtype="bfloat16"):
    # a meta tensor: only its shape, dtype and (absent) address are looked at
    rows = 2 * n_out if gated else n_out
    w = torch.empty(rows, n_in, dtype=torch.bfloat16 if dtype == "bfloat16" else torch.float32, device="meta")
    # the machine the decisions are checked for: a B200's SMs and its room for clusters of two and four blocks
    return Linear(w, Runtime(torch.device("cpu"), dtype, n_sms=148, cluster_room={2: 72, 4: 33}), gated=gated)


def test_few_tokens_stream_the_weight_and_many_go_to_the_prompt_kernel():
    qkv, o, gate_up, down = _lin(QKV, H), _lin(H, H), _lin(INTER, H, gated=True), _lin(H, INTER)
    for lin in (qkv, o, gate_up, down):
        assert lin.tensor_cores
        assert all(lin.streams(m) for m in (1, 8, 16))
        assert all(lin.prompts(m) and not lin.streams(m) for m in (129, 2048))
        assert all(lin.takes_scale_in(m) for m in (1, 16, 129, 4096))
    # 17 to 128 tokens: the tall tiles of the gated product still stream; the others stream as tiles whose K is
    # cut into a cluster of splits, all of whose blocks run at once
    assert gate_up.streams(17) and gate_up.streams(128) and not gate_up.streams(129)
    for lin in (qkv, o, down):
        assert lin.streams(17) and lin.streams(64) and lin.streams(128) and not lin.streams(129)
        for bn in (32, 64, 128):
            rows, splits, kkb, kstack = lin.rows_plans[bn]
            assert splits in (2, 4) and kstack == 1 and rows % 8 == 0 and rows <= 128
            assert -(-lin.n_out // rows) <= {2: 72, 4: 33}[splits]
            assert kkb == (1 if bn == 128 else 2)  # the widest tile's landing zone leaves room for boxes of one K block
        assert lin.rows_plans[16][1] == 1          # up to 16 tokens: short tiles, K blocks stacked, no split
    assert o.rows_plans[64][:2] == (128, 4) and down.rows_plans[64][:2] == (128, 4) and qkv.rows_plans[64][1] == 2
    assert o.rows_plans[128][:2] == (128, 4) and gate_up.rows_plans[128][2:] == (1, 1)
    # a reduction too short to cut stays with the kernels it had: the tile kernel up to 128 tokens, or, where
    # the reduction is long, the prompt kernel from 65
    short = _lin(H, 512)
    assert short.streams(16) and not short.streams(17) and not short.prompts(128)
    odd = _lin(4098, INTER)                        # outputs that are no multiple of four: no cluster plan
    assert not odd.streams(17) and odd.prompts(65) and not odd.prompts(64)
    assert not any(lin.prompts(m) for lin in (qkv, o, gate_up, down) for m in (65, 128))


def test_the_32_bit_path_never_takes_a_tensor_core_kernel():
    lin = _lin(H, H, dtype="float32")
    assert not lin.tensor_cores
    assert not any(lin.streams(m) or lin.prompts(m) or lin.takes_scale_in(m) for m in (1, 16, 64, 129, 4096))


def test_widths_that_are_no_multiple_of_eight_stay_on_the_plain_kernel():
    lin = _lin(200, 84)
    assert not lin.tensor_cores and not lin.streams(4) and not lin.prompts(500)


def test_rows_plans_fill_the_sms_with_one_wave():
    for n_out, n_in, gated in ((QKV, H, False), (H, H, False), (INTER, H, True), (H, INTER, False), (151936, H, False)):
        rows, splits, kkb, kstack = ops.rows_plan(n_out, n_in, gated, 16, 148)
        assert rows % 8 == 0 and 8 <= rows <= 128 and splits == 1
        blocks = -(-n_out // rows)
        if n_out <= 148 * 128:
            assert blocks <= 148, (n_out, rows, blocks)   # one block per SM at most: a single wave
        assert kstack * rows <= 128 and kkb % kstack == 0
