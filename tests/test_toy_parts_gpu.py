"""Parts and arrangements that the library does not have, defined HERE and registered from here: a
block with four norms, a block without a feed-forward, a feed-forward that routes every token to one
of several experts, a position encoding other than the library's.  They are toys that no model uses;
what is tested is that the framework's files need no change to take them, layer by layer in one model,
through the loader, the cache, the step function and the generation loop.
"""
import dataclasses

import pytest
import torch

import plain_qwen3 as plain

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def _register():
    from skyla_kernel_b200.config import LayerSpec, ModelSpec, PartSpec, ScheduleEntry, register_architecture
    from skyla_kernel_b200.parts import (Block, Part, register_block, register_feed_forward, register_position)
    from skyla_kernel_b200.weights.loader import TensorDecl

    class ScaledRotary(Part):
        """Rotation by the position divided by ``factor`` (tables in the form the attention part reads)."""
        graph_safe = True

        def __init__(self, spec, rt):
            super().__init__(spec, rt)
            self.n_rot, self.theta, self.factor = int(spec.params["n_rot"]), float(spec.params["theta"]), float(spec.params["factor"])
            self._tables = None

        def tables(self, n_positions):
            if self._tables is None or self._tables[0].shape[0] < n_positions:
                n = max(64, 1 << (n_positions - 1).bit_length())
                i = torch.arange(self.n_rot // 2, dtype=torch.float32)
                freqs = torch.tensor(self.theta, dtype=torch.float32) ** (-2.0 * i / torch.tensor(float(self.n_rot)))
                ang = ((torch.arange(n, dtype=torch.float32) / self.factor)[:, None] * freqs[None, :]).double()
                self._tables = (torch.cos(ang).float().to(self.rt.device), torch.sin(ang).float().to(self.rt.device))
            return self._tables[0], self._tables[1], self.n_rot

    register_position("toy_scaled_rotary", ScaledRotary)

    class RoutedFeedForward(Part):
        """Every token goes to the one expert its router rates highest (the lowest index among equals);
        the expert's gated output is weighted by the router's softmax probability of that expert."""

        def __init__(self, spec, rt):
            super().__init__(spec, rt)
            self.E = int(spec.params["experts"])

        @classmethod
        def declare(cls, spec):
            h, i, e = (int(spec.params[k]) for k in ("hidden_size", "intermediate_size", "experts"))
            t = spec.tensors
            return {t["router"]: TensorDecl((e, h)), t["gate"]: TensorDecl((e, i, h)), t["up"]: TensorDecl((e, i, h)),
                    t["down"]: TensorDecl((e, h, i))}

        def load(self, tensors):
            t = self.spec.tensors
            self.router, self.gate, self.up, self.down = (tensors[t[k]].float().to(self.rt.device)
                                                          for k in ("router", "gate", "up", "down"))

        def forward(self, ctx, h, x):
            n = h.float()
            logits = n @ self.router.T
            choice = logits.argmax(-1)
            p = torch.softmax(logits, -1).gather(1, choice[:, None])
            for e in range(self.E):   # the packed tokens of the step, grouped by expert
                idx = (choice == e).nonzero().flatten()
                if idx.numel():
                    ne = n[idx]
                    x[idx] += p[idx] * ((plain.silu(ne @ self.gate[e].T) * (ne @ self.up[e].T)) @ self.down[e].T)

    register_feed_forward("toy_routed", RoutedFeedForward)

    class SandwichBlock(Block):
        """``x += norm_b(mixer(norm_a(x))); x += norm_d(feed_forward(norm_c(x)))``: four norms."""
        PARTS = (("norm_a", "norm"), ("mixer", "mixer"), ("norm_b", "norm"), ("norm_c", "norm"),
                 ("feed_forward", "feed_forward"), ("norm_d", "norm"))

        def _sub(self, ctx, x, pre, post, run):
            h = ctx.buffer("toy.h", x.shape, ctx.rt.act_dtype)
            pre.forward(ctx, x, h)
            y = ctx.buffer("toy.y", x.shape, torch.float32)
            y.zero_()
            run(h, y)            # a mixer or feed-forward adds its output to what it is given
            out = ctx.buffer("toy.out", x.shape, torch.float32)
            post.forward(ctx, y, out)
            x += out

        def forward(self, ctx, x, entry):
            self._sub(ctx, x, self.norm_a, self.norm_b, lambda h, y: self.mixer.forward(ctx, h, y, entry))
            self._sub(ctx, x, self.norm_c, self.norm_d, lambda h, y: self.feed_forward.forward(ctx, h, y))

    register_block("toy_sandwich", SandwichBlock)

    class MixerOnlyBlock(Block):
        """``x += mixer(norm(x))`` and nothing else."""
        PARTS = (("norm", "norm"), ("mixer", "mixer"))

        def forward(self, ctx, x, entry):
            h = ctx.buffer("toy.h", x.shape, ctx.rt.act_dtype)
            self.norm.forward(ctx, x, h)
            self.mixer.forward(ctx, h, x, entry)

    register_block("toy_mixer_only", MixerOnlyBlock)

    @dataclasses.dataclass(frozen=True)
    class ToyConfig:
        hidden_size: int = 64
        vocab_size: int = 101
        heads: int = 4
        kv_heads: int = 2
        head_dim: int = 32
        experts: int = 4
        expert_size: int = 48
        window: int = 20
        factor: float = 3.0

        @classmethod
        def from_dict(cls, d):
            return cls(**{f.name: d[f.name] for f in dataclasses.fields(cls)})

        def to_dict(self):
            return dict(dataclasses.asdict(self), architectures=["ToyPartsLM"])

        def to_spec(self):
            H = self.hidden_size

            def norm(n, eps=1e-5):
                return PartSpec("rmsnorm", {"width": H, "eps": eps}, {"weight": n})

            def attn(p, position, window, qk_norm):
                t = {k: f"{p}.{k}" for k in ("q_proj", "k_proj", "v_proj", "o_proj")}
                if qk_norm:
                    t.update(q_norm=f"{p}.q_norm", k_norm=f"{p}.k_norm")
                return PartSpec("gqa_attention", {"hidden_size": H, "num_heads": self.heads, "num_kv_heads": self.kv_heads,
                                                  "head_dim": self.head_dim, "qk_norm": qk_norm, "qk_norm_eps": 1e-6,
                                                  "window": window, "position": position}, t)
            scaled = PartSpec("toy_scaled_rotary", {"n_rot": self.head_dim, "theta": 500.0, "factor": self.factor})
            usual = PartSpec("rotary_neox", {"n_rot": self.head_dim // 2, "theta": 10000.0, "max_positions": 64})
            layers = [
                LayerSpec("l0", "toy_sandwich", {
                    "norm_a": norm("l0.a"), "mixer": attn("l0", scaled, None, True), "norm_b": norm("l0.b", 1e-6),
                    "norm_c": norm("l0.c"),
                    "feed_forward": PartSpec("toy_routed", {"hidden_size": H, "intermediate_size": self.expert_size,
                                                            "experts": self.experts},
                                             {k: f"l0.moe.{k}" for k in ("router", "gate", "up", "down")}),
                    "norm_d": norm("l0.d")}),
                LayerSpec("l1", "toy_mixer_only", {"norm": norm("l1.n"), "mixer": attn("l1", usual, self.window, False)}),
                LayerSpec("l2", "prenorm_residual", {
                    "mixer_norm": norm("l2.a"), "mixer": attn("l2", usual, None, True), "ffn_norm": norm("l2.b"),
                    "feed_forward": PartSpec("swiglu", {"hidden_size": H, "intermediate_size": 2 * H},
                                             {k: f"l2.{k}" for k in ("gate_proj", "up_proj", "down_proj")})}),
            ]
            return ModelSpec("ToyPartsLM", self.vocab_size, H, 1 << 20,
                             PartSpec("token_embedding", {"vocab_size": self.vocab_size, "hidden_size": H}, {"weight": "embed"}),
                             layers, [ScheduleEntry(i) for i in range(3)], norm("final"),
                             PartSpec("linear_head", {"vocab_size": self.vocab_size, "hidden_size": H}, {"weight": "embed"}))

    register_architecture("ToyPartsLM", ToyConfig)
    return ToyConfig


def _plain(cfg, w, toks):
    """The toy model restated with the plain implementation's functions, whole sequence at once."""
    H, nq, nkv, hd = cfg.hidden_size, cfg.heads, cfg.kv_heads, cfg.head_dim
    T = len(toks)
    x = w["embed"][torch.tensor(toks)]

    def attn(p, n, freqs, n_rot, positions, window, qk_norm):
        return plain.attention(n, w[f"{p}.q_proj"], w[f"{p}.k_proj"], w[f"{p}.v_proj"], w[f"{p}.o_proj"],
                               w[f"{p}.q_norm"] if qk_norm else None, w[f"{p}.k_norm"] if qk_norm else None,
                               nq, nkv, hd, 1e-6, freqs, 1.0, n_rot, window=window, positions=positions)
    f_scaled, _ = plain.rope_frequencies(hd, 500.0)
    f_usual, _ = plain.rope_frequencies(hd // 2, 10000.0)
    pos = torch.arange(T)
    # l0: four norms, scaled positions, routed experts
    y = attn("l0", plain.rmsnorm(x, w["l0.a"], 1e-5), f_scaled, hd, pos.to(torch.float32) / cfg.factor, None, True)
    x = x + plain.rmsnorm(y, w["l0.b"], 1e-6)
    n = plain.rmsnorm(x, w["l0.c"], 1e-5)
    logits = n @ w["l0.moe.router"].T
    y = torch.zeros_like(x)
    for t in range(T):
        e = int(torch.argmax(logits[t]))
        p = plain.softmax(logits[t])[e]
        y[t] = p * (w["l0.moe.down"][e] @ (plain.silu(w["l0.moe.gate"][e] @ n[t]) * (w["l0.moe.up"][e] @ n[t])))
    x = x + plain.rmsnorm(y, w["l0.d"], 1e-5)
    # l1: a mixer and nothing else, partial rotation, a window, no q/k norm
    x = x + attn("l1", plain.rmsnorm(x, w["l1.n"], 1e-5), f_usual, hd // 2, pos, cfg.window, False)
    # l2: the usual arrangement
    x = x + attn("l2", plain.rmsnorm(x, w["l2.a"], 1e-5), f_usual, hd // 2, pos, None, True)
    x = x + plain.swiglu(plain.rmsnorm(x, w["l2.b"], 1e-5), w["l2.gate_proj"], w["l2.up_proj"], w["l2.down_proj"])
    return plain.rmsnorm(x, w["final"], 1e-5) @ w["embed"].T


def test_toy_blocks_routing_and_positions_in_one_model(tmp_path):
    import skyla_kernel_b200 as skyla
    from skyla_kernel_b200 import write_model_folder
    from skyla_kernel_b200.engine import StepItem
    ToyConfig = _register()
    cfg = ToyConfig()
    folder = write_model_folder(str(tmp_path / "toy"), cfg, seed=5, dtype="float32", linear_std=0.15, norm_std=0.1)
    _, w = plain.read_folder(folder)
    model = skyla.load(folder, dtype="float32", max_tokens=1024)
    eng = model.engine
    # two groups of layers in the cache: all positions (l0, l2) and a window of 20 (l1), which gives pages back
    assert sorted(g.need.window or 0 for g in eng.cache.groups) == [0, 20]
    assert [g.n_layers for g in eng.cache.groups if not g.need.window] == [2]
    g = torch.Generator().manual_seed(1)
    seqs = [torch.randint(0, cfg.vocab_size, (n,), generator=g).tolist() for n in (150, 9, 70)]
    refs = [_plain(cfg, w, q) for q in seqs]
    for round_ in range(2):
        slots = [eng.alloc_slot() for _ in seqs]
        cut = [100, 9, 1]
        out = eng.step([StepItem(s, q[:c], list(range(c))) for s, q, c in zip(slots, seqs, cut)])
        got, o = [[] for _ in seqs], 0
        for i, c in enumerate(cut):
            got[i].append(out[o:o + c]); o += c
        out = eng.step([StepItem(slots[0], seqs[0][100:130], list(range(30))), StepItem(slots[2], seqs[2][1:2], [0])])
        got[0].append(out[:30]); got[2].append(out[30:])
        at = [130, 9, 2]
        while any(at[i] < len(seqs[i]) for i in range(3)):
            live = [i for i in range(3) if at[i] < len(seqs[i])]
            out = eng.step([StepItem(slots[i], [seqs[i][at[i]]], [0]) for i in live])
            for j, i in enumerate(live):
                got[i].append(out[j:j + 1]); at[i] += 1
        for i in range(3):
            torch.testing.assert_close(torch.cat(got[i]).cpu(), refs[i], rtol=2e-4, atol=2e-4)
        held = [g.pages.n_held for g in eng.cache.groups if g.need.window]
        assert held[0] < sum(-(-len(q) // 64) for q in seqs)   # the windowed group gave pages back
        for s in slots:
            eng.free_slot(s)
        eng.cache.check()
    # and through the generation loop
    toks = model.generate([q[:5] for q in seqs], max_new_tokens=4, stop_ids=[])
    for q, t in zip(seqs, toks):
        seq = list(q[:5])
        for tok in t:
            assert tok == int(torch.argmax(_plain(cfg, w, seq)[-1]))
            seq.append(tok)


def test_a_layer_that_lacks_a_part_of_its_arrangement_is_a_configuration_error():
    from skyla_kernel_b200.config import ConfigError, LayerSpec, PartSpec
    from skyla_kernel_b200.parts import part_class
    spec = LayerSpec("l", "prenorm_residual", {"mixer_norm": PartSpec("rmsnorm", {"width": 8, "eps": 1e-5}, {"weight": "n"})})
    with pytest.raises(ConfigError, match="needs a part named 'mixer'.*the layer has mixer_norm"):
        part_class("block", "prenorm_residual").declare(spec)
