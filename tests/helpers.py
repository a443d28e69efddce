"""Shared by the tests: tiny configurations, model folders, ways of cutting a run."""
from __future__ import annotations

import json
import os

import torch

# Two tiny configurations that differ in every size and option, and a third
# with sizes that are no powers of two anywhere and YaRN scaling.
TINY_A = dict(hidden_size=64, num_hidden_layers=2, num_attention_heads=4, num_key_value_heads=2,
              head_dim=16, intermediate_size=128, vocab_size=256, rope_theta=10000.0,
              rms_norm_eps=1e-6, max_position_embeddings=128, tie_word_embeddings=True)
TINY_B = dict(hidden_size=96, num_hidden_layers=3, num_attention_heads=6, num_key_value_heads=1,
              head_dim=32, intermediate_size=160, vocab_size=509, rope_theta=1000000.0,
              rms_norm_eps=1e-5, max_position_embeddings=256, tie_word_embeddings=False)
TINY_C = dict(hidden_size=80, num_hidden_layers=1, num_attention_heads=3, num_key_value_heads=3,
              head_dim=48, intermediate_size=112, vocab_size=131, rope_theta=5000.0,
              rms_norm_eps=3e-6, max_position_embeddings=512, tie_word_embeddings=False,
              rope_scaling={"rope_type": "yarn", "factor": 4.0,
                            "original_max_position_embeddings": 64, "attn_factor": 1.0})
# Not tiny in width: heads of 128 in pairs and a width of 2048 bring in the kernels that the small
# ones never reach (tcgen05 attention, heads finished in the q/k/v product, tiles cut along K,
# K-split products of mid-size batches).
WIDE_D = dict(hidden_size=2048, num_hidden_layers=2, num_attention_heads=4, num_key_value_heads=2,
              head_dim=128, intermediate_size=1280, vocab_size=300, rope_theta=20000.0,
              rms_norm_eps=2e-6, max_position_embeddings=1024, tie_word_embeddings=False)
TINY = {"A": (TINY_A, "float32", 0), "B": (TINY_B, "bfloat16", 1), "C": (TINY_C, "bfloat16", 2),
        "D": (WIDE_D, "bfloat16", 3)}


def config_dict(base: dict) -> dict:
    d = dict(base)
    d["architectures"] = ["Qwen3ForCausalLM"]
    d["model_type"] = "qwen3"
    d["hidden_act"] = "silu"
    return d


def make_folder(tmpdir, name: str, sharp: float = 2.0, linear_std: float = 0.05) -> str:
    """A model folder for tiny configuration ``name``.

    ``sharp`` multiplies the q/k norm weights so that attention scores spread over
    several units and a wrong or missing key changes the result visibly (with unit
    norm weights every softmax is nearly flat and hides such faults).
    """
    from safetensors.torch import save_file
    base, store, seed = TINY[name]
    cfg = config_dict(base)
    cfg["torch_dtype"] = store
    g = torch.Generator().manual_seed(1000 + seed)
    H, nq, nkv, hd = base["hidden_size"], base["num_attention_heads"], base["num_key_value_heads"], base["head_dim"]
    I, V, L = base["intermediate_size"], base["vocab_size"], base["num_hidden_layers"]

    def lin(*shape):
        return torch.randn(*shape, generator=g) * linear_std

    def norm(n, mul=1.0):
        return (1.0 + 0.1 * torch.randn(n, generator=g)) * mul

    w = {"model.embed_tokens.weight": lin(V, H), "model.norm.weight": norm(H)}
    if not base["tie_word_embeddings"]:
        w["lm_head.weight"] = lin(V, H)
    for l in range(L):
        p = f"model.layers.{l}."
        w[p + "input_layernorm.weight"] = norm(H)
        w[p + "post_attention_layernorm.weight"] = norm(H)
        w[p + "self_attn.q_proj.weight"] = lin(nq * hd, H)
        w[p + "self_attn.k_proj.weight"] = lin(nkv * hd, H)
        w[p + "self_attn.v_proj.weight"] = lin(nkv * hd, H)
        w[p + "self_attn.o_proj.weight"] = lin(H, nq * hd)
        w[p + "self_attn.q_norm.weight"] = norm(hd, sharp)
        w[p + "self_attn.k_norm.weight"] = norm(hd, sharp)
        w[p + "mlp.gate_proj.weight"] = lin(I, H)
        w[p + "mlp.up_proj.weight"] = lin(I, H)
        w[p + "mlp.down_proj.weight"] = lin(H, I)
    tdt = torch.float32 if store == "float32" else torch.bfloat16
    w = {k: v.to(tdt).contiguous() for k, v in w.items()}
    folder = os.path.join(str(tmpdir), f"tiny_{name}")
    os.makedirs(folder, exist_ok=True)
    with open(os.path.join(folder, "config.json"), "w") as f:
        json.dump(cfg, f)
    save_file(w, os.path.join(folder, "model.safetensors"))
    return folder


def random_tokens(n: int, vocab: int, seed: int):
    g = torch.Generator().manual_seed(seed)
    return torch.randint(0, vocab, (n,), generator=g).tolist()


# Tolerances; the error is measured against the largest reference logit of the
# compared block.
#   float32: engine against the plain 32-bit implementation.
#   bfloat16: engine against the plain 32-bit implementation.  How much of that
#     difference is rounding alone was measured with the plain implementation itself:
#     run with a bfloat16 round trip where a 16-bit engine stores activations
#     (plain.forward(..., rnd=plain.bf16_round): normed inputs, q/k/v, rotated q/k,
#     softmax weights, attention output, gated activation, final norm) it differs
#     from its own 32-bit run by up to 9.7e-2 (worst element) and 4.4e-3 (mean) of the
#     largest logit over 60 sequences of these tiny, deliberately sharp models.  The
#     limits sit just above that.  A fault in a key, a position or a slot moves
#     logits by the order of the largest logit itself and is far outside them.
#     (The engine is not compared with that rounded run: its kernels round at other
#     scales -- attention weights relative to a running maximum -- so every stored
#     value draws its rounding anew and the two differ by as much as either differs
#     from the 32-bit run.)
#   "bfloat16 flat": the same comparison on models made with sharp=1.0 (unit q/k norm weights: flatter
#     attention, less rounding noise).  There the rounded plain run differs from the 32-bit one by up to
#     1.14e-2 (worst) and 1.91e-3 (mean) over the four configurations, and the engine by 1.06e-2 and
#     1.90e-3: the limits are about twice that, six times tighter than for the sharp models.
TOL = {"float32": 1e-4, "bfloat16": 1.5e-1, "bfloat16 flat": 2.5e-2}
TOL_MEAN = {"float32": 2e-5, "bfloat16": 1e-2, "bfloat16 flat": 4e-3}


def assert_close(got: torch.Tensor, ref: torch.Tensor, dtype: str, what: str = ""):
    """``dtype`` names the limits: "float32", "bfloat16" or "bfloat16 flat"."""
    got, ref = got.detach().cpu().to(torch.float64), ref.detach().cpu().to(torch.float64)
    assert got.shape == ref.shape, f"{what}: shape {tuple(got.shape)} vs {tuple(ref.shape)}"
    assert torch.isfinite(got).all(), f"{what}: non-finite logits"
    scale = max(ref.abs().max().item(), 1e-6)
    err = (got - ref).abs()
    worst = err.max().item() / scale
    mean = err.mean().item() / scale
    if worst > TOL[dtype] or mean > TOL_MEAN[dtype]:
        row = int(err.max(dim=-1).values.argmax()) if err.dim() == 2 else 0
        raise AssertionError(f"{what}: worst error {worst:.3e} (limit {TOL[dtype]:.0e}), mean {mean:.3e} "
                             f"(limit {TOL_MEAN[dtype]:.0e}) of the largest logit {scale:.3f}; "
                             f"first bad row {first_bad_row(err, scale, TOL[dtype])}, worst row {row}")
    return worst


def first_bad_row(err, scale, tol):
    if err.dim() != 2:
        return None
    bad = (err.max(dim=-1).values / scale > tol).nonzero()
    return int(bad[0]) if len(bad) else None
