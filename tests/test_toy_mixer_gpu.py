"""A toy mixer with fixed-size state of its own, defined here, is registered, built
and stepped without a change to the library's files."""
import dataclasses

import pytest
import torch

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def _register():
    from skyla_kernel_b200.cache import StateNeed
    from skyla_kernel_b200.config import LayerSpec, ModelSpec, PartSpec, ScheduleEntry, register_architecture
    from skyla_kernel_b200.parts import Part, register_mixer
    from skyla_kernel_b200.weights import TensorDecl

    class DecayMixer(Part):
        """state <- a * state + W_in h, token after token; x += W_out state."""

        def __init__(self, spec, rt):
            super().__init__(spec, rt)
            self.hidden, self.width, self.decay = spec.params["hidden_size"], spec.params["state_size"], spec.params["decay"]

        @classmethod
        def declare(cls, spec):
            h, s = spec.params["hidden_size"], spec.params["state_size"]
            return {spec.tensors["w_in"]: TensorDecl((s, h)), spec.tensors["w_out"]: TensorDecl((h, s))}

        def load(self, tensors):
            self.w_in = tensors[self.spec.tensors["w_in"]].to(self.rt.device, torch.float32)
            self.w_out = tensors[self.spec.tensors["w_out"]].to(self.rt.device, torch.float32)

        def cache_need(self):
            return None

        def state_need(self):
            return StateNeed((self.width,), torch.float32)

        def forward(self, ctx, h, x, entry):
            state = ctx.cache.state_of_entry(entry.cache_entry)
            u = h.float() @ self.w_in.T
            slots, cu = ctx.seq_slot.tolist(), ctx.cu.tolist()
            for b, slot in enumerate(slots):
                s = state[slot]
                for t in range(cu[b], cu[b + 1]):
                    s = self.decay * s + u[t]
                    x[t] += self.w_out @ s
                state[slot] = s

    register_mixer("toy_decay", DecayMixer)

    @dataclasses.dataclass(frozen=True)
    class ToyConfig:
        hidden_size: int
        state_size: int
        vocab_size: int
        num_layers: int
        decay: float

        @classmethod
        def from_dict(cls, d):
            return cls(d["hidden_size"], d["state_size"], d["vocab_size"], d["num_layers"], d["decay"])

        def to_dict(self):
            return dict(dataclasses.asdict(self), architectures=["ToyDecayLM"])

        def to_spec(self):
            def norm(n):
                return PartSpec("rmsnorm", {"width": self.hidden_size, "eps": 1e-5}, {"weight": n})
            layers = []
            for i in range(self.num_layers):
                p = f"layers.{i}"
                layers.append(LayerSpec(p, "prenorm_residual", {
                    "mixer_norm": norm(f"{p}.n1"),
                    "mixer": PartSpec("toy_decay", {"hidden_size": self.hidden_size, "state_size": self.state_size,
                                                    "decay": self.decay}, {"w_in": f"{p}.w_in", "w_out": f"{p}.w_out"}),
                    "ffn_norm": norm(f"{p}.n2"),
                    "feed_forward": PartSpec("swiglu", {"hidden_size": self.hidden_size, "intermediate_size": 2 * self.hidden_size},
                                             {k: f"{p}.{k}" for k in ("gate_proj", "up_proj", "down_proj")})}))
            return ModelSpec("ToyDecayLM", self.vocab_size, self.hidden_size, 1 << 20,
                             PartSpec("token_embedding", {"vocab_size": self.vocab_size, "hidden_size": self.hidden_size}, {"weight": "embed"}),
                             layers, [ScheduleEntry(i) for i in range(self.num_layers)], norm("final"),
                             PartSpec("linear_head", {"vocab_size": self.vocab_size, "hidden_size": self.hidden_size}, {"weight": "embed"}))

    register_architecture("ToyDecayLM", ToyConfig)
    return ToyConfig


def _plain(cfg, w, toks):
    import plain_qwen3 as plain
    x = w["embed"][torch.tensor(toks)]
    for i in range(cfg.num_layers):
        p = f"layers.{i}"
        u = plain.rmsnorm(x, w[f"{p}.n1"], 1e-5) @ w[f"{p}.w_in"].T
        s = torch.zeros(cfg.state_size)
        outs = []
        for t in range(len(toks)):
            s = cfg.decay * s + u[t]
            outs.append(w[f"{p}.w_out"] @ s)
        x = x + torch.stack(outs)
        x = x + plain.swiglu(plain.rmsnorm(x, w[f"{p}.n2"], 1e-5), w[f"{p}.gate_proj"], w[f"{p}.up_proj"], w[f"{p}.down_proj"])
    return plain.rmsnorm(x, w["final"], 1e-5) @ w["embed"].T


def test_toy_mixer_with_state(tmp_path):
    from skyla_kernel_b200 import write_model_folder
    from skyla_kernel_b200.config import config_from_folder
    from skyla_kernel_b200.engine import Engine, StepItem
    import plain_qwen3 as plain
    ToyConfig = _register()
    cfg = ToyConfig(hidden_size=48, state_size=20, vocab_size=97, num_layers=2, decay=0.9)
    folder = write_model_folder(str(tmp_path / "toy"), cfg, seed=3, dtype="float32", linear_std=0.1, norm_std=0.1)
    assert isinstance(config_from_folder(folder), ToyConfig)  # the registry finds it by config.json
    _, w = plain.read_folder(folder)
    eng = Engine.from_folder(folder, dtype="float32", max_tokens=256)
    assert eng.cache.groups == [] and eng.cache.state_of_entry(0).shape[1:] == (20,)
    g = torch.Generator().manual_seed(0)
    seqs = [torch.randint(0, 97, (n,), generator=g).tolist() for n in (30, 7, 19)]
    for round_ in range(2):  # the second round reuses slots whose state must start from zero again
        slots = [eng.alloc_slot() for _ in seqs]
        cut = [12, 7, 1]
        first = eng.step([StepItem(s, q[:c], list(range(c))) for s, q, c in zip(slots, seqs, cut)])
        got = [[] for _ in seqs]
        o = 0
        for i, c in enumerate(cut):
            got[i].append(first[o:o + c]); o += c
        t = 0
        while True:
            live = [i for i in range(len(seqs)) if cut[i] + t < len(seqs[i])]
            if not live:
                break
            out = eng.step([StepItem(slots[i], [seqs[i][cut[i] + t]], [0]) for i in live])
            for j, i in enumerate(live):
                got[i].append(out[j:j + 1])
            t += 1
        for i, q in enumerate(seqs):
            torch.testing.assert_close(torch.cat(got[i]).cpu(), _plain(cfg, w, q), rtol=1e-4, atol=1e-4)
        for s in slots:
            eng.free_slot(s)
