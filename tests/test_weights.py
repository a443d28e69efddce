"""Safetensors container, loader errors and the random-weights mode (no GPU)."""
import json
import os
import struct

import pytest
import torch

from helpers import TINY_A, TINY_B, config_dict
from skyla_kernel_b200.config import config_from_dict, config_from_folder
from skyla_kernel_b200.engine.model import declared_tensors
from skyla_kernel_b200.weights import (SafetensorsFile, WeightError, load_weights, write_model_folder,
                                       write_safetensors)


def _folder(tmp_path, base=TINY_A, dtype="float32", seed=0):
    cfg = config_from_dict(config_dict(base))
    return write_model_folder(str(tmp_path / "m"), cfg, seed, dtype), cfg


def test_writer_matches_the_safetensors_package(tmp_path):
    from safetensors.torch import load_file, save_file
    t = {"a": torch.randn(3, 5), "b": torch.randn(7).to(torch.bfloat16), "c": torch.arange(6, dtype=torch.int32)}
    write_safetensors(str(tmp_path / "x.safetensors"), t)
    back = load_file(str(tmp_path / "x.safetensors"))
    for k in t:
        assert back[k].dtype == t[k].dtype and torch.equal(back[k], t[k])
    save_file(t, str(tmp_path / "y.safetensors"))
    f = SafetensorsFile(str(tmp_path / "y.safetensors"))
    for k in t:
        assert torch.equal(f.tensor(k), t[k])


def test_random_folder_loads_and_keeps_storage_types(tmp_path):
    folder, cfg = _folder(tmp_path, TINY_B, "bfloat16", 1)
    assert config_from_folder(folder) == cfg
    w = load_weights(folder, declared_tensors(cfg.to_spec()))
    assert all(v.dtype == torch.bfloat16 for v in w.values())
    assert w["lm_head.weight"].shape == (509, 96)
    folder32, cfg32 = _folder(tmp_path / "f32", TINY_A, "float32", 0)
    w32 = load_weights(folder32, declared_tensors(cfg32.to_spec()))
    assert all(v.dtype == torch.float32 for v in w32.values())  # stored 32-bit stays 32-bit
    assert "lm_head.weight" not in w32  # tied: the embedding is the head


def test_random_weights_depend_on_seed_only(tmp_path):
    a, cfg = _folder(tmp_path / "a", seed=3)
    b, _ = _folder(tmp_path / "b", seed=3)
    c, _ = _folder(tmp_path / "c", seed=4)
    decl = declared_tensors(cfg.to_spec())
    wa, wb, wc = (load_weights(f, decl) for f in (a, b, c))
    assert all(torch.equal(wa[k], wb[k]) for k in wa)
    assert not torch.equal(wa["model.embed_tokens.weight"], wc["model.embed_tokens.weight"])
    n = wa["model.layers.0.input_layernorm.weight"]
    assert abs(n.mean().item() - 1.0) < 0.05
    assert abs(wa["model.embed_tokens.weight"].std().item() - 0.02) < 0.005


def test_one_error_lists_missing_unexpected_and_wrong_shapes(tmp_path):
    from safetensors.torch import load_file, save_file
    folder, cfg = _folder(tmp_path)
    path = os.path.join(folder, "model.safetensors")
    w = load_file(path)
    del w["model.layers.1.mlp.up_proj.weight"]
    del w["model.norm.weight"]
    w["model.layers.0.self_attn.q_proj.weight"] = torch.zeros(64, 63)
    w["stray.weight"] = torch.zeros(2)
    save_file(w, path)
    with pytest.raises(WeightError) as e:
        load_weights(folder, declared_tensors(cfg.to_spec()))
    msg = str(e.value)
    assert "missing tensors (2)" in msg and "model.layers.1.mlp.up_proj.weight" in msg and "model.norm.weight" in msg
    assert "unexpected tensors (1)" in msg and "stray.weight" in msg
    assert "wrong shape" in msg and "[64, 63]" in msg and "[64, 64]" in msg


def test_tied_checkpoint_may_carry_a_head_copy(tmp_path):
    from safetensors.torch import load_file, save_file
    folder, cfg = _folder(tmp_path)
    path = os.path.join(folder, "model.safetensors")
    w = load_file(path)
    w["lm_head.weight"] = w["model.embed_tokens.weight"].clone()
    save_file(w, path)
    spec = cfg.to_spec()
    load_weights(folder, declared_tensors(spec), spec.optional_tensors)
    with pytest.raises(WeightError, match="unexpected"):
        load_weights(folder, declared_tensors(spec))


def test_broken_files(tmp_path):
    folder, cfg = _folder(tmp_path)
    decl = declared_tensors(cfg.to_spec())
    path = os.path.join(folder, "model.safetensors")
    raw = open(path, "rb").read()
    open(path, "wb").write(raw[: len(raw) // 2])
    with pytest.raises(WeightError, match="past end of file"):
        load_weights(folder, decl)
    open(path, "wb").write(struct.pack("<Q", 10 ** 9) + b"{}")
    with pytest.raises(WeightError, match="header"):
        load_weights(folder, decl)
    open(path, "wb").write(b"abc")
    with pytest.raises(WeightError, match="end of file"):
        load_weights(folder, decl)
    os.remove(path)
    with pytest.raises(WeightError, match="no model.safetensors"):
        load_weights(folder, decl)


def test_integer_tables_and_float_kinds(tmp_path):
    from skyla_kernel_b200.weights import TensorDecl
    write_safetensors(str(tmp_path / "model.safetensors"),
                      {"t": torch.arange(4, dtype=torch.int64), "h": torch.ones(2, dtype=torch.float16)})
    w = load_weights(str(tmp_path), {"t": TensorDecl((4,), "int"), "h": TensorDecl((2,), "norm")})
    assert w["t"].dtype == torch.int32 and w["h"].dtype == torch.bfloat16
    with pytest.raises(WeightError, match="integer table"):
        load_weights(str(tmp_path), {"h": TensorDecl((2,), "int"), "t": TensorDecl((4,), "int")})


def test_sharded_folder_with_an_index(tmp_path):
    """A checkpoint in several files: ``model.safetensors.index.json`` names, for every tensor, the
    file that holds it; the loader reads the files the index lists and checks the union."""
    folder, cfg = _folder(tmp_path, TINY_B, "bfloat16", 2)
    decl = declared_tensors(cfg.to_spec())
    whole = load_weights(folder, decl)
    names = sorted(whole)
    shards = {"model-00001-of-00003.safetensors": names[0::3], "model-00002-of-00003.safetensors": names[1::3],
              "model-00003-of-00003.safetensors": names[2::3]}
    sharded = tmp_path / "sharded"
    os.makedirs(sharded)
    with open(os.path.join(folder, "config.json")) as f, open(sharded / "config.json", "w") as g:
        g.write(f.read())
    weight_map = {}
    for fname, ns in shards.items():
        write_safetensors(str(sharded / fname), {n: whole[n] for n in ns})
        weight_map.update({n: fname for n in ns})
    with open(sharded / "model.safetensors.index.json", "w") as f:
        json.dump({"metadata": {}, "weight_map": weight_map}, f)
    # a stray file that the index does not list is not read
    write_safetensors(str(sharded / "stray.safetensors"), {"not.a.weight": torch.zeros(2)})
    got = load_weights(str(sharded), decl)
    assert sorted(got) == names and all(torch.equal(got[n], whole[n]) for n in names)
    # a tensor lost with its shard is reported by name, among all the missing ones
    os.remove(sharded / "model-00002-of-00003.safetensors")
    write_safetensors(str(sharded / "model-00002-of-00003.safetensors"), {n: whole[n] for n in names[1::3][1:]})
    with pytest.raises(WeightError) as e:
        load_weights(str(sharded), decl)
    assert names[1] in str(e.value) and "missing tensors (1)" in str(e.value)
