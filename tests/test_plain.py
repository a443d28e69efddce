"""The plain implementation checked against itself and against closed forms (no GPU)."""
import math

import numpy as np
import torch

import plain_qwen3 as plain
from helpers import TINY, make_folder, random_tokens


def test_rmsnorm_and_softmax_closed_forms():
    x = torch.tensor([[3.0, 4.0]])
    out = plain.rmsnorm(x, torch.tensor([1.0, 2.0]), 0.0)
    r = 1 / math.sqrt(12.5)
    assert torch.allclose(out, torch.tensor([[3 * r, 8 * r]]))
    p = plain.softmax(torch.tensor([0.0, math.log(3.0)]))
    assert torch.allclose(p, torch.tensor([0.25, 0.75]))
    assert abs(plain.silu(torch.tensor(1.0)).item() - 1 / (1 + math.exp(-1))) < 1e-7


def test_rope_is_a_rotation_and_relative():
    freqs, m = plain.rope_frequencies(8, 100.0)
    assert m == 1.0 and torch.allclose(freqs, torch.tensor([1.0, 100 ** -0.25, 100 ** -0.5, 100 ** -0.75]))
    g = torch.Generator().manual_seed(0)
    q, k = torch.randn(1, 1, 8, generator=g), torch.randn(1, 1, 8, generator=g)
    def dot(pq, pk):
        a = plain.rope_neox(q, torch.tensor([pq]), freqs, 1.0, 8)
        b = plain.rope_neox(k, torch.tensor([pk]), freqs, 1.0, 8)
        return (a * b).sum().item()
    assert abs(dot(5, 3) - dot(12, 10)) < 1e-4          # depends on the distance only
    a = plain.rope_neox(q, torch.tensor([7]), freqs, 1.0, 8)
    assert abs(a.norm().item() - q.norm().item()) < 1e-5  # lengths are kept
    part = plain.rope_neox(q, torch.tensor([7]), freqs[:2], 1.0, 4)
    assert torch.equal(part[..., 4:], q[..., 4:])          # elements past n_rot stay


def test_yarn_frequencies():
    sc = {"factor": 4.0, "original_max_position_embeddings": 64, "attn_factor": 1.0}
    f, m = plain.rope_frequencies(48, 5000.0, sc)
    base, _ = plain.rope_frequencies(48, 5000.0)
    assert abs(m - (1 + 0.1 * math.log(4.0))) < 1e-6
    assert torch.allclose(f[0], base[0]) and torch.allclose(f[-1], base[-1] / 4)
    assert ((f <= base + 1e-9) & (f >= base / 4 - 1e-9)).all()


def test_causality_and_prefix_property(tmp_path):
    folder = make_folder(tmp_path, "B")
    cfg, w = plain.read_folder(folder)
    toks = random_tokens(40, cfg["vocab_size"], 1)
    full = plain.forward(cfg, w, toks)
    part = plain.forward(cfg, w, toks[:23])
    assert torch.allclose(full[:23], part, atol=1e-5)
    other = list(toks)
    other[30] = (other[30] + 1) % cfg["vocab_size"]
    assert torch.allclose(plain.forward(cfg, w, other)[:30], full[:30], atol=1e-5)
    assert not torch.allclose(plain.forward(cfg, w, other)[30:], full[30:], atol=1e-3)


def test_float64_agrees_and_far_keys_matter(tmp_path):
    folder = make_folder(tmp_path, "A")
    cfg, w = plain.read_folder(folder)
    toks = random_tokens(90, cfg["vocab_size"], 2)
    a = plain.forward(cfg, w, toks)
    b = plain.forward(cfg, w, toks, dtype=torch.float64).float()
    assert (a - b).abs().max() < 1e-4
    # the sharpened models look far back: changing the first token changes the last logits
    other = [(toks[0] + 7) % cfg["vocab_size"]] + toks[1:]
    c = plain.forward(cfg, w, other)
    assert (a[-1] - c[-1]).abs().max() > 1e-3


def test_window_mask():
    g = torch.Generator().manual_seed(3)
    n = torch.randn(10, 8, generator=g)
    wq, wk, wv, wo = (torch.randn(8, 8, generator=g) for _ in range(4))
    freqs, m = plain.rope_frequencies(4, 10.0)
    full = plain.attention(n, wq, wk, wv, wo, None, None, 2, 2, 4, 0.0, freqs, m, 4)
    win = plain.attention(n, wq, wk, wv, wo, None, None, 2, 2, 4, 0.0, freqs, m, 4, window=3)
    assert torch.allclose(full[:3], win[:3], atol=1e-6) and not torch.allclose(full[5:], win[5:], atol=1e-4)
    # with a window of 3, token 9 must not depend on token 5's input
    n2 = n.clone(); n2[5] += 1.0
    win2 = plain.attention(n2, wq, wk, wv, wo, None, None, 2, 2, 4, 0.0, freqs, m, 4, window=3)
    assert torch.allclose(win[9], win2[9], atol=1e-6) and not torch.allclose(win[7], win2[7], atol=1e-4)


def test_sampling_twin_filters():
    logits = torch.tensor([0.0, 3.0, 1.0, 2.9, -1.0, 2.0])
    s, keep = plain.sample_scores(logits, 1.0, 3, 1.0, 0, 0, 0)
    assert keep.tolist() == [False, True, False, True, False, True]
    s, keep = plain.sample_scores(logits, 1.0, 0, 0.5, 0, 0, 0)
    assert keep.tolist() == [False, True, False, True, False, False]
    u = plain.uniforms(5, 1, 2, 1000)
    assert 0 < u.min() and u.max() < 1 and abs(u.mean() - 0.5) < 0.05
    assert not np.allclose(u, plain.uniforms(5, 1, 3, 1000))
    # frequencies follow softmax
    counts = np.zeros(6)
    for step in range(4000):
        s, _ = plain.sample_scores(logits, 1.0, 0, 1.0, 9, 0, step)
        counts[int(np.argmax(s))] += 1
    p = torch.softmax(logits, 0).numpy()
    assert np.abs(counts / 4000 - p).max() < 0.03


import pytest


@pytest.mark.parametrize("name", ["A", "B", "C"])
def test_two_independent_restatements_agree(tmp_path, name):
    """``plain_qwen3`` (whole sequences, torch, a mask) against ``plain_numpy64`` (token by token with
    a growing cache, 64-bit NumPy, loops), written apart from the same cited lines of the reference:
    logits and the residual stream after every layer."""
    import plain_numpy64 as second
    folder = make_folder(tmp_path, name)
    cfg, w = plain.read_folder(folder)
    toks = random_tokens(70 if name != "C" else 90, cfg["vocab_size"], 5)   # C: past YaRN's original 64 positions
    taps = []
    ref = plain.forward(cfg, w, toks, dtype=torch.float64, taps=taps)
    dec = second.Decoder(cfg, {k: v.numpy() for k, v in w.items()})
    taps2 = []
    got = np.stack([dec.step(t, taps2) for t in toks])
    scale = ref.abs().max().item()
    assert np.abs(got - ref.numpy()).max() / scale < 3e-6     # 32-bit frequencies and angles on both sides
    L = cfg["num_hidden_layers"]
    for pos, l, x in taps2:
        assert np.abs(x - taps[l][pos].numpy()).max() < 3e-6 * max(1.0, taps[l].abs().max().item())
    assert len(taps2) == L * len(toks)
    # and the 32-bit run of the first stays within rounding of the 64-bit run of the second
    ref32 = plain.forward(cfg, w, toks)
    assert np.abs(got - ref32.numpy().astype(np.float64)).max() / scale < 2e-5
