"""A plain, slow implementation of the Qwen3 dense decoder for the tests.

It rests on the formulas of the reference's CPU model (maulanasdqn/skyla-kernel,
``skyla-ref``), cited function by function below; the reference's own code is
Rust and cannot be compiled or imported where these tests run, so there is no
comparison against its binaries.  Whole sequences, no cache, one function per
part, 32-bit torch on the CPU (64-bit on request).  It shares no code with the
package under test: it reads config.json with ``json`` and the weights with the
``safetensors`` package.
"""
from __future__ import annotations

import json
import math
import os

import numpy as np
import torch


def read_folder(folder):
    """(config dict, {name: float32 tensor}) of a model folder."""
    from safetensors.torch import load_file
    with open(os.path.join(folder, "config.json")) as f:
        cfg = json.load(f)
    w = load_file(os.path.join(folder, "model.safetensors"))
    return cfg, {k: v.to(torch.float32) for k, v in w.items()}


# skyla-ref/src/ops.rs:1-16 -- y = x * r * w with r = 1/sqrt(mean(x^2) + eps)
def rmsnorm(x, w, eps):
    ms = (x * x).sum(-1, keepdim=True) / x.shape[-1]
    r = 1.0 / torch.sqrt(ms + eps)
    return x * r * w


# skyla-ref/src/rope.rs:33-57 -- theta^(-2i/d), optional YaRN blend and mscale
def rope_frequencies(n_rot, theta, scaling=None):
    d = float(n_rot)
    i = torch.arange(n_rot // 2, dtype=torch.float32)
    base = torch.tensor(theta, dtype=torch.float32) ** (-2.0 * i / torch.tensor(d, dtype=torch.float32))
    if not scaling:
        return base, 1.0
    factor = float(scaling["factor"])
    orig = float(scaling["original_max_position_embeddings"])
    attn_factor = float(scaling.get("attn_factor", 1.0))
    beta_fast, beta_slow = 32.0, 1.0  # rope.rs:4-5

    def corr_dim(n_rotations):  # rope.rs:33-35
        return d * math.log(orig / (n_rotations * 2.0 * math.pi)) / (2.0 * math.log(theta))

    freq_scale = 1.0 / factor
    low = max(math.floor(corr_dim(beta_fast)), 0.0)
    high = min(math.ceil(corr_dim(beta_slow)), d - 1.0)
    y = (i - low) / max(high - low, 0.001)
    mix = 1.0 - torch.clamp(y, 0.0, 1.0)
    freqs = base * (freq_scale * (1.0 - mix) + mix)
    mscale = attn_factor * (1.0 + 0.1 * math.log(1.0 / freq_scale))
    return freqs.to(torch.float32), mscale


# skyla-ref/src/rope.rs:59-68 -- pairs (x_i, x_{i+half}) turn by pos * f_i (a 32-bit product)
def rope_neox(x, positions, freqs, mscale, n_rot):
    """x: [T, heads, hd]; positions: [T] ints."""
    half = n_rot // 2
    ang32 = positions.to(torch.float32)[:, None] * freqs[None, :].to(torch.float32)
    ang = ang32.to(torch.float64)
    cos = (torch.cos(ang) * mscale).to(x.dtype)[:, None, :]
    sin = (torch.sin(ang) * mscale).to(x.dtype)[:, None, :]
    a, b = x[..., :half], x[..., half:n_rot]
    out = x.clone()
    out[..., :half] = a * cos - b * sin
    out[..., half:n_rot] = a * sin + b * cos
    return out


# skyla-ref/src/ops.rs:18-26 -- subtract the maximum, exponentiate, divide by the sum
def softmax(s):
    m = s.max(-1, keepdim=True).values
    e = torch.exp(s - m)
    return e / e.sum(-1, keepdim=True)


# skyla-ref/src/ops.rs:28-30
def silu(z):
    return z / (1.0 + torch.exp(-z))


# skyla-ref/src/model.rs:124-172 -- one sequence, all positions at once, causal
def attention(n, wq, wk, wv, wo, q_norm, k_norm, nq, nkv, hd, eps, freqs, mscale, n_rot,
              scale=None, window=None, positions=None, rnd=lambda t: t):
    """``rnd`` rounds stored intermediates (identity: everything stays 32-bit); with a
    bfloat16 round trip it imitates where a 16-bit engine stores activations."""
    T = n.shape[0]
    positions = torch.arange(T) if positions is None else positions
    q = rnd(n @ wq.T).view(T, nq, hd)
    k = rnd(n @ wk.T).view(T, nkv, hd)
    v = rnd(n @ wv.T).view(T, nkv, hd)
    if q_norm is not None:  # model.rs:138-145: norm over the head, then rotation
        q = rmsnorm(q, q_norm, eps)
        k = rmsnorm(k, k_norm, eps)
    if freqs is not None:
        q = rope_neox(q, positions, freqs, mscale, n_rot)
        k = rope_neox(k, positions, freqs, mscale, n_rot)
    q, k = rnd(q), rnd(k)
    n_rep = nq // nkv                       # model.rs:149
    scale = 1.0 / math.sqrt(hd) if scale is None else scale  # model.rs:150
    out = torch.zeros(T, nq, hd, dtype=n.dtype)
    for h in range(nq):
        kvh = h // n_rep                    # model.rs:154
        s = (q[:, h, :] @ k[:, kvh, :].T) * scale  # model.rs:156-158
        i = torch.arange(T)
        mask = i[None, :] > i[:, None]       # a token sees positions 0..=its own
        if window:
            mask = mask | (i[None, :] < i[:, None] - window + 1)
        s = s.masked_fill(mask, float("-inf"))
        out[:, h, :] = rnd(softmax(s)) @ v[:, kvh, :]   # model.rs:159-165 (a 16-bit engine rounds the weights too)
    return rnd(out.reshape(T, nq * hd)) @ wo.T   # model.rs:171


# skyla-ref/src/ffn.rs:21-28
def swiglu(n, w_gate, w_up, w_down, rnd=lambda t: t):
    return rnd(silu(n @ w_gate.T) * (n @ w_up.T)) @ w_down.T


# skyla-ref/src/model.rs:97-122
def bf16_round(t):
    return t.to(torch.bfloat16).to(t.dtype)


def forward(cfg, w, tokens, dtype=torch.float32, taps=None, rnd=lambda t: t):
    """Logits [T, vocab] for one whole sequence of token ids."""
    w = {k: v.to(dtype) for k, v in w.items()}
    H, nq = cfg["hidden_size"], cfg["num_attention_heads"]
    nkv = cfg.get("num_key_value_heads", nq)
    hd = cfg.get("head_dim") or H // nq     # skyla-ref/src/lib.rs:88-90
    eps = cfg["rms_norm_eps"]
    freqs, mscale = rope_frequencies(hd, cfg["rope_theta"], _scaling(cfg))
    x = w["model.embed_tokens.weight"][torch.as_tensor(tokens, dtype=torch.long)]  # model.rs:99-100
    for l in range(cfg["num_hidden_layers"]):
        p = f"model.layers.{l}."
        n = rnd(rmsnorm(x, w[p + "input_layernorm.weight"], eps))   # model.rs:105
        x = x + attention(n, w[p + "self_attn.q_proj.weight"], w[p + "self_attn.k_proj.weight"],
                          w[p + "self_attn.v_proj.weight"], w[p + "self_attn.o_proj.weight"],
                          w[p + "self_attn.q_norm.weight"], w[p + "self_attn.k_norm.weight"],
                          nq, nkv, hd, eps, freqs, mscale, hd, rnd=rnd)  # model.rs:108-110
        n = rnd(rmsnorm(x, w[p + "post_attention_layernorm.weight"], eps))  # model.rs:112
        x = x + swiglu(n, w[p + "mlp.gate_proj.weight"], w[p + "mlp.up_proj.weight"],
                       w[p + "mlp.down_proj.weight"], rnd)            # model.rs:113-114
        if taps is not None:
            taps.append(x.clone())
    x = rnd(rmsnorm(x, w["model.norm.weight"], eps))                 # model.rs:117
    head = w["lm_head.weight"] if not cfg.get("tie_word_embeddings", False) else w["model.embed_tokens.weight"]
    return x @ head.T                                                # model.rs:118-119, 70-73


def _scaling(cfg):
    rs = cfg.get("rope_scaling")
    if not rs or rs.get("rope_type", rs.get("type")) in (None, "none", "default"):
        return None
    return rs


# skyla-ref/src/ops.rs:36-41 (ties: the library under test documents "lowest index")
def argmax(logits):
    return int(torch.argmax(logits))


def greedy(cfg, w, prompt, n_new, dtype=torch.float32):
    """Greedy continuation by re-running the whole sequence for every token."""
    seq = list(prompt)
    out = []
    for _ in range(n_new):
        tok = argmax(forward(cfg, w, seq, dtype)[-1])
        out.append(tok)
        seq.append(tok)
    return out


# ---- sampling twin (the library's own definition; the reference samples outside its repository)
def _mix32(x):
    x = np.asarray(x, dtype=np.uint64)
    x ^= x >> np.uint64(16); x = (x * np.uint64(0x7feb352d)) & np.uint64(0xFFFFFFFF)
    x ^= x >> np.uint64(15); x = (x * np.uint64(0x846ca68b)) & np.uint64(0xFFFFFFFF)
    x ^= x >> np.uint64(16)
    return x


def uniforms(seed, req, step, n):
    h = _mix32(np.uint64((seed & 0xFFFFFFFF) ^ 0x9e3779b9))
    h = _mix32(h ^ np.uint64((seed >> 32) & 0xFFFFFFFF))
    h = _mix32(h ^ np.uint64(req & 0xFFFFFFFF))
    h = _mix32(h ^ np.uint64(step & 0xFFFFFFFF))
    h = _mix32(np.uint64(h) ^ np.arange(n, dtype=np.uint64))
    return ((h >> np.uint64(8)).astype(np.float64) + 0.5) / 16777216.0


def sample_scores(logits, temperature, top_k, top_p, seed, req, step):
    """Perturbed scores (float64) of the kept tokens, -inf elsewhere; the draw is their argmax."""
    z = (logits.to(torch.float32) / torch.tensor(temperature, dtype=torch.float32)).numpy().astype(np.float64)
    keep = np.ones_like(z, dtype=bool)
    if 0 < top_k < len(z):
        kth = np.sort(z)[::-1][top_k - 1]
        keep &= z >= kth
    if top_p < 1.0:
        e = np.where(keep, np.exp(z - z.max()), 0.0)
        order = np.argsort(-z, kind="stable")
        c = np.cumsum(e[order])
        j = int(np.searchsorted(c, top_p * e.sum(), side="left"))
        keep &= z >= z[order[min(j, len(z) - 1)]]
    u = uniforms(seed, req, step, len(z))
    return np.where(keep, z - np.log(-np.log(u)), -np.inf), keep
