"""Each part alone, and schedules that name a layer twice or share a cache."""
import math

import pytest
import torch

import plain_qwen3 as plain

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def _rt(dtype):
    from skyla_kernel_b200.parts import Runtime
    return Runtime(torch.device(DEV), dtype)


def _tensors(decl, seed, std=0.08, sharp=1.0):
    g = torch.Generator().manual_seed(seed)
    out = {}
    for name, d in decl.items():
        t = torch.randn(d.shape, generator=g)
        out[name] = (1 + 0.1 * t) * (sharp if "q_norm" in name or "k_norm" in name else 1.0) if d.init == "norm" else t * std
    return out


def _ctx(rt, needs, states, items, max_tokens=1024, tiles=(64,), plans=()):
    from skyla_kernel_b200.cache import SequenceCache
    from skyla_kernel_b200.engine.batch import BatchBuilder
    cache = SequenceCache(needs, states, max_tokens, None, rt.cache_dtype, rt.device)
    # the token tiles and the host-made plans that a mixer asks for (Part.token_tiles, Part.step_plans)
    return cache, BatchBuilder(rt, cache, tiles, plans)


def _tol(dtype):
    return dict(rtol=3e-2, atol=3e-2) if dtype == "bfloat16" else dict(rtol=2e-5, atol=2e-5)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_rmsnorm_part(dtype):
    from skyla_kernel_b200.config import PartSpec
    from skyla_kernel_b200.parts import build_part, declare_part
    spec = PartSpec("rmsnorm", {"width": 80, "eps": 3e-5}, {"weight": "n.weight"})
    rt = _rt(dtype)
    part = build_part("norm", spec, rt)
    w = _tensors(declare_part("norm", spec), 1)
    part.load(dict(w))  # a part may take out of the table what it fuses
    x = torch.randn(6, 80, device=DEV) * 2
    out = torch.empty(6, 80, dtype=rt.act_dtype, device=DEV)
    part.forward(None, x, out)
    torch.testing.assert_close(out.float().cpu(), plain.rmsnorm(x.cpu(), w["n.weight"], 3e-5), **_tol(dtype))


@pytest.mark.parametrize("scaling", [None, {"factor": 8.0, "original_max_position_embeddings": 32, "attn_factor": 0.9}])
def test_rotary_tables(scaling):
    from skyla_kernel_b200.config import PartSpec
    from skyla_kernel_b200.parts import build_part
    rt = _rt("float32")
    spec = PartSpec("rotary_neox", {"n_rot": 48, "theta": 5000.0, "max_positions": 16, "scaling": scaling})
    part = build_part("position", spec, rt)
    assert build_part("position", spec, rt) is part  # one table per parameter set
    cos, sin, n_rot = part.tables(300)  # beyond the first size: the table grows
    assert n_rot == 48 and cos.shape[0] >= 300
    freqs, m = plain.rope_frequencies(48, 5000.0, scaling)
    ang = (torch.arange(cos.shape[0], dtype=torch.float32)[:, None] * freqs[None, :]).double()
    torch.testing.assert_close(cos.cpu(), (torch.cos(ang) * m).float(), rtol=0, atol=1e-6)
    torch.testing.assert_close(sin.cpu(), (torch.sin(ang) * m).float(), rtol=0, atol=1e-6)


def _attention_spec(hidden, nq, nkv, hd, n_rot=None, window=None, qk_norm=True, scale=None, cache_dtype=None):
    from skyla_kernel_b200.config import PartSpec
    rope = PartSpec("rotary_neox", {"n_rot": n_rot or hd, "theta": 10000.0, "max_positions": 64, "scaling": None})
    return PartSpec("gqa_attention", {"hidden_size": hidden, "num_heads": nq, "num_kv_heads": nkv, "head_dim": hd,
                                      "qk_norm": qk_norm, "qk_norm_eps": 1e-5, "scale": scale, "window": window,
                                      "position": rope, "cache_dtype": cache_dtype},
                    {k: f"a.{k}" for k in ("q_proj", "k_proj", "v_proj", "o_proj", "q_norm", "k_norm")})


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("hidden,nq,nkv,hd,n_rot,window,qk_norm,scale,cache_dtype", [
    (80, 5, 5, 16, 16, None, True, None, None),
    (96, 6, 2, 48, 24, None, True, 0.3, None),     # partial rotation, own scale
    (64, 4, 1, 32, 32, 40, False, None, None),      # a window, no q/k norm
    (96, 6, 2, 32, 32, None, True, None, "float32"),  # keys and values kept in 32-bit whatever the activations are
])
def test_attention_part_whole_then_one_by_one(dtype, hidden, nq, nkv, hd, n_rot, window, qk_norm, scale, cache_dtype):
    from skyla_kernel_b200.engine.batch import StepItem
    from skyla_kernel_b200.parts import EntryBinding, build_part, declare_part
    rt = _rt(dtype)
    spec = _attention_spec(hidden, nq, nkv, hd, n_rot, window, qk_norm, scale, cache_dtype)
    part = build_part("mixer", spec, rt)
    w = _tensors(declare_part("mixer", spec), 3, sharp=2.0)
    part.load(dict(w))  # a part may take out of the table what it fuses
    T = 150
    h_all = torch.randn(T, hidden, generator=torch.Generator().manual_seed(4))
    freqs, m = plain.rope_frequencies(n_rot, 10000.0)
    ref = plain.attention(h_all, w["a.q_proj"], w["a.k_proj"], w["a.v_proj"], w["a.o_proj"],
                          w["a.q_norm"] if qk_norm else None, w["a.k_norm"] if qk_norm else None,
                          nq, nkv, hd, 1e-5, freqs, m, n_rot, scale=scale, window=window)
    cache, batcher = _ctx(rt, [part.cache_need()], [None], None, plans=part.step_plans)
    assert cache.groups[0].k.dtype == (torch.float32 if cache_dtype == "float32" else rt.cache_dtype)
    slot = cache.alloc_slot()
    got = []
    for a, b in [(0, 100)] + [(i, i + 1) for i in range(100, T)]:
        cache.reserve([(slot, b - a)])
        ctx = batcher.build([StepItem(slot, [0] * (b - a), [])])
        x = torch.zeros(b - a, hidden, device=DEV)
        part.forward(ctx, h_all[a:b].to(DEV).to(rt.act_dtype), x, EntryBinding(0, True))
        cache.advance([(slot, b - a)])
        got.append(x.cpu())
    from helpers import assert_close
    assert_close(torch.cat(got), ref, dtype, "attention part")
    if window:  # pages wholly outside the window went back to the pool
        assert cache.groups[0].pages.n_held < -(-T // 64) + 1 and cache.groups[0].slot_pages[slot][0] == -1


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_swiglu_part(dtype):
    from skyla_kernel_b200.config import PartSpec
    from skyla_kernel_b200.engine.batch import StepItem
    from skyla_kernel_b200.parts import build_part, declare_part
    rt = _rt(dtype)
    spec = PartSpec("swiglu", {"hidden_size": 80, "intermediate_size": 112},
                    {k: f"f.{k}" for k in ("gate_proj", "up_proj", "down_proj")})
    part = build_part("feed_forward", spec, rt)
    w = _tensors(declare_part("feed_forward", spec), 5, std=0.15)
    part.load(dict(w))  # a part may take out of the table what it fuses
    cache, batcher = _ctx(rt, [], [], None)
    slot = cache.alloc_slot()
    ctx = batcher.build([StepItem(slot, [0] * 9, [])])
    h = torch.randn(9, 80, generator=torch.Generator().manual_seed(6))
    x0 = torch.randn(9, 80, generator=torch.Generator().manual_seed(7))
    x = x0.clone().to(DEV)
    part.forward(ctx, h.to(DEV).to(rt.act_dtype), x)
    ref = x0 + plain.swiglu(h, w["f.gate_proj"], w["f.up_proj"], w["f.down_proj"])
    torch.testing.assert_close(x.cpu(), ref, **_tol(dtype))


def _two_layer_engine(schedule, dtype="float32"):
    """A Qwen3-shaped model whose run order is given: exercises the schedule as data."""
    from skyla_kernel_b200.config import Qwen3Config, ScheduleEntry
    from skyla_kernel_b200.engine import Engine, declared_tensors
    import dataclasses
    from helpers import TINY_A

    class Scheduled(Qwen3Config):
        def to_spec(self):
            spec = super().to_spec()
            return dataclasses.replace(spec, schedule=[ScheduleEntry(*e) for e in schedule])

    cfg = Scheduled(**TINY_A)
    w = _tensors(declared_tensors(cfg.to_spec()), 9, std=0.05, sharp=2.0)
    return Engine(cfg, dict(w), dtype, max_tokens=512), cfg, w  # the engine consumes the table it is given


def _plain_scheduled(cfg, w, tokens, schedule):
    """The plain model with an explicit run order; a run that shares a cache reuses k and v."""
    H, nq, nkv, hd, eps = cfg.hidden_size, cfg.num_attention_heads, cfg.num_key_value_heads, cfg.head_dim, cfg.rms_norm_eps
    freqs, m = plain.rope_frequencies(hd, cfg.rope_theta)
    x = w["model.embed_tokens.weight"][torch.tensor(tokens)]
    kv_of = {}
    for i, (layer, shared) in enumerate(schedule):
        p = f"model.layers.{layer}."
        n = plain.rmsnorm(x, w[p + "input_layernorm.weight"], eps)
        wk, wv = w[p + "self_attn.k_proj.weight"], w[p + "self_attn.v_proj.weight"]
        kn = w[p + "self_attn.k_norm.weight"]
        n_kv = n
        if shared is not None:  # keys and values come from what run `shared` saw and its layer's weights
            n_kv, wk, wv, kn = kv_of[shared]
        else:
            kv_of[i] = (n, wk, wv, kn)
        x = x + _attn_split(n, n_kv, w[p + "self_attn.q_proj.weight"], wk, wv, w[p + "self_attn.o_proj.weight"],
                            w[p + "self_attn.q_norm.weight"], kn, nq, nkv, hd, eps, freqs, m)
        n = plain.rmsnorm(x, w[p + "post_attention_layernorm.weight"], eps)
        x = x + plain.swiglu(n, w[p + "mlp.gate_proj.weight"], w[p + "mlp.up_proj.weight"], w[p + "mlp.down_proj.weight"])
    x = plain.rmsnorm(x, w["model.norm.weight"], eps)
    return x @ w["model.embed_tokens.weight"].T


def _attn_split(n_q, n_kv, wq, wk, wv, wo, qn, kn, nq, nkv, hd, eps, freqs, m):
    T = n_q.shape[0]
    pos = torch.arange(T)
    q = plain.rope_neox(plain.rmsnorm((n_q @ wq.T).view(T, nq, hd), qn, eps), pos, freqs, m, hd)
    k = plain.rope_neox(plain.rmsnorm((n_kv @ wk.T).view(T, nkv, hd), kn, eps), pos, freqs, m, hd)
    v = (n_kv @ wv.T).view(T, nkv, hd)
    out = torch.zeros(T, nq, hd)
    mask = pos[None, :] > pos[:, None]
    for h in range(nq):
        s = (q[:, h] @ k[:, h // (nq // nkv)].T) / math.sqrt(hd)
        out[:, h] = plain.softmax(s.masked_fill(mask, float("-inf"))) @ v[:, h // (nq // nkv)]
    return out.reshape(T, nq * hd) @ wo.T


@pytest.mark.parametrize("schedule", [
    [(0, None), (1, None), (0, None)],            # a layer named twice: two caches of its own
    [(0, None), (1, None), (1, 1), (0, 0)],       # runs that read another run's cache
])
def test_schedule_is_data(schedule):
    from skyla_kernel_b200.engine import StepItem
    eng, cfg, w = _two_layer_engine(schedule)
    assert len(eng.cache.entry_group) == sum(1 for _, s in schedule if s is None)
    toks = torch.randint(0, cfg.vocab_size, (90,), generator=torch.Generator().manual_seed(1)).tolist()
    ref = _plain_scheduled(cfg, w, toks, schedule)
    s = eng.alloc_slot()
    got = [eng.step([StepItem(s, toks[:70], list(range(70)))])]
    got += [eng.step([StepItem(s, [t], [0])]) for t in toks[70:]]
    torch.testing.assert_close(torch.cat(got).cpu(), ref, rtol=1e-4, atol=1e-4)


def test_bad_schedules_are_refused():
    from skyla_kernel_b200.config import ConfigError
    with pytest.raises(ConfigError, match="earlier entry"):
        _two_layer_engine([(0, None), (1, 2), (0, None)])
    with pytest.raises(ConfigError, match="names layer"):
        _two_layer_engine([(0, None), (5, None)])


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_embedding_and_head_parts(dtype):
    from skyla_kernel_b200.config import PartSpec
    from skyla_kernel_b200.parts import build_part, declare_part
    rt = _rt(dtype)
    emb_spec = PartSpec("token_embedding", {"vocab_size": 131, "hidden_size": 80}, {"weight": "e.weight"})
    head_spec = PartSpec("linear_head", {"vocab_size": 131, "hidden_size": 80}, {"weight": "e.weight"})
    w = _tensors(declare_part("embedding", emb_spec), 11, std=0.3)
    assert declare_part("head", head_spec).keys() == w.keys()  # tied: one tensor, declared by both
    emb, head = build_part("embedding", emb_spec, rt), build_part("head", head_spec, rt)
    emb.load(w); head.load(w)
    assert head.proj.weight.data_ptr() == emb.weight.data_ptr()  # and placed on the device once
    toks = torch.tensor([130, 0, 7, 7], dtype=torch.int32, device=DEV)
    x = torch.empty(4, 80, device=DEV)
    emb.forward(None, toks, x)
    assert torch.equal(x.cpu(), w["e.weight"].to(rt.act_dtype if dtype == "bfloat16" else torch.float32).float()[toks.long().cpu()]) \
        or torch.allclose(x.cpu(), w["e.weight"][toks.long().cpu()])
    h = torch.randn(4, 80, generator=torch.Generator().manual_seed(1)).to(DEV).to(rt.act_dtype)
    logits = torch.empty(4, 131, device=DEV)
    head.forward(None, h, logits)
    torch.testing.assert_close(logits.cpu(), h.float().cpu() @ w["e.weight"].T, **_tol(dtype))


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_block_alone(dtype):
    """One pre-norm block from a layer spec: whole, then the same tokens in three steps."""
    from helpers import assert_close
    from skyla_kernel_b200.config import LayerSpec, PartSpec
    from skyla_kernel_b200.engine.batch import StepItem
    from skyla_kernel_b200.parts import EntryBinding, part_class
    rt = _rt(dtype)
    H, nq, nkv, hd, I = 96, 6, 2, 32, 256
    norm = lambda n: PartSpec("rmsnorm", {"width": H, "eps": 2e-5}, {"weight": n})
    spec = LayerSpec("l", "prenorm_residual", {
        "mixer_norm": norm("l.n1"), "mixer": _attention_spec(H, nq, nkv, hd), "ffn_norm": norm("l.n2"),
        "feed_forward": PartSpec("swiglu", {"hidden_size": H, "intermediate_size": I},
                                 {k: f"l.{k}" for k in ("gate_proj", "up_proj", "down_proj")})})
    cls = part_class("block", spec.block)
    w = _tensors(cls.declare(spec), 21, std=0.08, sharp=2.0)
    if dtype == "bfloat16":  # stored in 16 bits, as a served model would be: the tensor-core kernels run
        w = {k: v.to(torch.bfloat16) for k, v in w.items()}
    block = cls(spec, rt)
    block.load(dict(w))
    wf = {k: v.float() for k, v in w.items()}
    T = 90
    x0 = torch.randn(T, H, generator=torch.Generator().manual_seed(3)) * 0.5
    freqs, m = plain.rope_frequencies(hd, 10000.0)
    ref = x0 + plain.attention(plain.rmsnorm(x0, wf["l.n1"], 2e-5), wf["a.q_proj"], wf["a.k_proj"], wf["a.v_proj"],
                               wf["a.o_proj"], wf["a.q_norm"], wf["a.k_norm"], nq, nkv, hd, 1e-5, freqs, m, hd)
    ref = ref + plain.swiglu(plain.rmsnorm(ref, wf["l.n2"], 2e-5), wf["l.gate_proj"], wf["l.up_proj"], wf["l.down_proj"])
    cache, batcher = _ctx(rt, [block.cache_need()], [None], None, plans=block.mixer.step_plans)
    slot = cache.alloc_slot()
    got = []
    for a, b in ((0, 70), (70, 71), (71, 90)):  # a prompt, one token (the few-token kernels), a second chunk
        cache.reserve([(slot, b - a)])
        ctx = batcher.build([StepItem(slot, [0] * (b - a), [])])
        x = x0[a:b].clone().to(DEV)
        block.forward(ctx, x, EntryBinding(0, True))
        cache.advance([(slot, b - a)])
        got.append(x.cpu())
    assert_close(torch.cat(got), ref, dtype, f"block alone {dtype}")


def test_wide_groups_decode_through_the_prompt_kernel():
    """More than 16 query heads per key/value head: the decode kernel's 16-row tile is too small,
    the part must route single tokens through the prompt kernel (and get the same numbers)."""
    from helpers import assert_close
    from skyla_kernel_b200.engine.batch import StepItem
    from skyla_kernel_b200.parts import EntryBinding, build_part, declare_part
    rt = _rt("bfloat16")
    hidden, nq, nkv, hd = 64, 34, 2, 16
    spec = _attention_spec(hidden, nq, nkv, hd)
    part = build_part("mixer", spec, rt)
    assert part._fast == 1
    w = {k: v.to(torch.bfloat16) for k, v in _tensors(declare_part("mixer", spec), 5, sharp=2.0).items()}
    part.load(dict(w))  # a part may take out of the table what it fuses
    wf = {k: v.float() for k, v in w.items()}
    T = 80
    h_all = torch.randn(T, hidden, generator=torch.Generator().manual_seed(6))
    freqs, m = plain.rope_frequencies(hd, 10000.0)
    ref = plain.attention(plain.bf16_round(h_all), wf["a.q_proj"], wf["a.k_proj"], wf["a.v_proj"], wf["a.o_proj"],
                          wf["a.q_norm"], wf["a.k_norm"], nq, nkv, hd, 1e-5, freqs, m, hd)
    cache, batcher = _ctx(rt, [part.cache_need()], [None], None, plans=part.step_plans)
    slot = cache.alloc_slot()
    got = []
    for a, b in [(0, 66)] + [(i, i + 1) for i in range(66, T)]:
        cache.reserve([(slot, b - a)])
        ctx = batcher.build([StepItem(slot, [0] * (b - a), [])])
        x = torch.zeros(b - a, hidden, device=DEV)
        part.forward(ctx, h_all[a:b].to(DEV).to(torch.bfloat16), x, EntryBinding(0, True))
        cache.advance([(slot, b - a)])
        got.append(x.cpu())
    assert_close(torch.cat(got), ref, "bfloat16", "34 query heads over 2 key/value heads")
