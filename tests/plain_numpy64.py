"""A second restatement of the reference's formulas, written apart from ``plain_qwen3``.

``plain_qwen3`` runs a whole sequence at once with torch matrices and a mask.  This one
does what the reference's CPU model does (skyla-ref/src/model.rs:97-172): ONE token at a
time, 64-bit NumPy, keys and values appended to per-layer lists, scores over the cached
positions only (so no mask exists that could be wrong), every head in a Python loop.  The
two share no code and no algorithm; a misreading of a formula would have to be made twice,
in two different shapes, to go unseen.  Weights come in as a dict of arrays, the
configuration as the plain config.json dict.
"""
from __future__ import annotations

import math

import numpy as np


def _rms(v, w, eps):
    # skyla-ref/src/ops.rs:1-11: sum of squares over the vector's length, plus eps, inverse root
    ss = 0.0
    for a in v:
        ss += float(a) * float(a)
    r = 1.0 / math.sqrt(ss / len(v) + eps)
    return np.array([float(a) * r * float(b) for a, b in zip(v, w)], dtype=np.float64)


def _frequencies(cfg, d):
    # skyla-ref/src/rope.rs:37-57; the table is 32-bit in the reference, and so is pos * f below
    theta = float(cfg["rope_theta"])
    f = np.empty(d // 2, dtype=np.float32)
    for i in range(d // 2):
        f[i] = np.float32(theta) ** np.float32(-2.0 * i / d)
    rs = cfg.get("rope_scaling")
    kind = (rs or {}).get("rope_type", (rs or {}).get("type"))
    if not rs or kind in (None, "none", "default"):
        return f, 1.0
    assert kind == "yarn", kind            # rope.rs:14-31: anything else is an error
    factor = float(rs["factor"])
    orig = float(rs["original_max_position_embeddings"])

    def corr(beta):                        # rope.rs:33-35
        return d * math.log(orig / (beta * 2.0 * math.pi)) / (2.0 * math.log(theta))

    low = max(math.floor(corr(32.0)), 0)   # rope.rs:4-5: BETA_FAST 32, BETA_SLOW 1
    high = min(math.ceil(corr(1.0)), d - 1)
    one, fs = np.float32(1.0), np.float32(1.0) / np.float32(factor)
    for i in range(d // 2):                # every step in 32-bit, as rope.rs:46-54 has it
        y = (np.float32(i) - np.float32(low)) / np.float32(max(high - low, 0.001))
        mix = one - np.float32(min(max(y, np.float32(0.0)), one))
        f[i] = f[i] * (fs * (one - mix) + mix)
    return f, float(rs.get("attn_factor", 1.0)) * (1.0 + 0.1 * math.log(factor))


def _rotate(v, pos, freqs, mscale):
    # skyla-ref/src/rope.rs:59-68: element i pairs with element i + half
    half = len(freqs)
    out = v.copy()
    for i in range(half):
        ang = float(np.float32(pos) * freqs[i])     # a 32-bit product
        c, s = math.cos(ang) * mscale, math.sin(ang) * mscale
        a, b = v[i], v[i + half]
        out[i] = a * c - b * s
        out[i + half] = a * s + b * c
    return out


class Decoder:
    """One sequence; ``step(token)`` returns the logits after it (skyla-ref/src/model.rs:97-122)."""

    def __init__(self, cfg, weights):
        self.cfg = cfg
        self.w = {k: np.asarray(v, dtype=np.float64) for k, v in weights.items()}
        self.H = cfg["hidden_size"]
        self.nq = cfg["num_attention_heads"]
        self.nkv = cfg.get("num_key_value_heads", self.nq)
        self.hd = cfg.get("head_dim") or self.H // self.nq      # skyla-ref/src/lib.rs:88-90
        self.eps = cfg["rms_norm_eps"]
        self.L = cfg["num_hidden_layers"]
        self.freqs, self.mscale = _frequencies(cfg, self.hd)
        self.keys = [[] for _ in range(self.L)]                  # model.rs:58-59: they grow by a token
        self.values = [[] for _ in range(self.L)]
        self.pos = 0

    def _attention(self, l, n):
        # model.rs:124-172
        w, p = self.w, f"model.layers.{l}.self_attn."
        nq, nkv, hd = self.nq, self.nkv, self.hd
        q = w[p + "q_proj.weight"] @ n
        k = w[p + "k_proj.weight"] @ n
        v = w[p + "v_proj.weight"] @ n
        qs = [_rotate(_rms(q[h * hd:(h + 1) * hd], w[p + "q_norm.weight"], self.eps), self.pos, self.freqs, self.mscale)
              for h in range(nq)]
        ks = [_rotate(_rms(k[h * hd:(h + 1) * hd], w[p + "k_norm.weight"], self.eps), self.pos, self.freqs, self.mscale)
              for h in range(nkv)]
        self.keys[l].append(ks)
        self.values[l].append([v[h * hd:(h + 1) * hd] for h in range(nkv)])
        n_rep = nq // nkv
        scale = 1.0 / math.sqrt(hd)
        out = np.zeros(nq * hd)
        for h in range(nq):
            kvh = h // n_rep
            scores = [float(qs[h] @ self.keys[l][t][kvh]) * scale for t in range(self.pos + 1)]
            m = max(scores)                                       # ops.rs:18-26
            e = [math.exp(s - m) for s in scores]
            tot = sum(e)
            acc = np.zeros(hd)
            for t in range(self.pos + 1):
                acc += (e[t] / tot) * self.values[l][t][kvh]
            out[h * hd:(h + 1) * hd] = acc
        return w[p + "o_proj.weight"] @ out

    def step(self, token, taps=None):
        w = self.w
        x = w["model.embed_tokens.weight"][token].copy()         # model.rs:99-100, no scaling
        for l in range(self.L):
            p = f"model.layers.{l}."
            x = x + self._attention(l, _rms(x, w[p + "input_layernorm.weight"], self.eps))
            n = _rms(x, w[p + "post_attention_layernorm.weight"], self.eps)
            g = w[p + "mlp.gate_proj.weight"] @ n                 # ffn.rs:21-28
            u = w[p + "mlp.up_proj.weight"] @ n
            a = np.array([gi / (1.0 + math.exp(-gi)) * ui for gi, ui in zip(g, u)])
            x = x + w[p + "mlp.down_proj.weight"] @ a
            if taps is not None:
                taps.append((self.pos, l, x.copy()))
        x = _rms(x, w["model.norm.weight"], self.eps)
        head = w["model.embed_tokens.weight"] if self.cfg.get("tie_word_embeddings", False) else w["lm_head.weight"]
        self.pos += 1
        return head @ x                                           # model.rs:118-119, 70-73


def forward(cfg, weights, tokens):
    """Logits [T, vocab] (float64) by feeding the tokens one by one."""
    d = Decoder(cfg, weights)
    return np.stack([d.step(int(t)) for t in tokens])
