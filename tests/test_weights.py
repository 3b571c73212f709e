"""Safetensors container, binding by name, the one error, the random-weights mode (no GPU)."""
import json
import os
import struct

import pytest
import torch

from helpers import TINY_A, TINY_B, random_weights, write_folder
from titan_b200.config import config_from_dict, load_config
from titan_b200.parts import declare_weights
from titan_b200.weights import (FolderWeights, SafetensorsError, SafetensorsFile, WeightError,
                                write_model_folder, write_safetensors)


def test_round_trip_against_the_safetensors_package(tmp_path):
    w = random_weights(TINY_A, 0)
    write_folder(str(tmp_path), TINY_A, w)
    f = SafetensorsFile(str(tmp_path / "model.safetensors"))
    assert sorted(f.names()) == sorted(w)
    for n in w:
        assert f.dtype(n) == torch.bfloat16 and torch.equal(f.tensor(n), w[n])
    from safetensors import safe_open            # the independent reader of the format
    with safe_open(str(tmp_path / "model.safetensors"), "pt") as g:
        for n in w:
            assert torch.equal(g.get_tensor(n), w[n])


def test_reads_a_file_written_by_the_safetensors_package(tmp_path):
    from safetensors.torch import save_file
    t = {"a": torch.arange(6, dtype=torch.float32).reshape(2, 3), "b": torch.ones(4, dtype=torch.int32)}
    save_file(t, str(tmp_path / "x.safetensors"))
    f = SafetensorsFile(str(tmp_path / "x.safetensors"))
    assert torch.equal(f.tensor("a"), t["a"]) and f.dtype("b") == torch.int32


@pytest.mark.parametrize("damage", ["short", "header_len", "not_json", "offsets", "size"])
def test_malformed_files(tmp_path, damage):
    p = str(tmp_path / "m.safetensors")
    write_safetensors(p, [("a", (2, 2), torch.float32)], lambda n: torch.zeros(2, 2))
    raw = bytearray(open(p, "rb").read())
    n = struct.unpack("<Q", raw[:8])[0]
    if damage == "short":
        raw = raw[:4]
    elif damage == "header_len":
        raw[:8] = struct.pack("<Q", 1 << 40)
    elif damage == "not_json":
        raw[8:10] = b"!!"
    else:
        h = json.loads(raw[8:8 + n])
        h["a"]["data_offsets"] = [0, 64] if damage == "offsets" else [0, 8]
        blob = json.dumps(h).encode()
        raw = bytearray(struct.pack("<Q", len(blob)) + blob + bytes(raw[8 + n:]))
    open(p, "wb").write(raw)
    with pytest.raises(SafetensorsError):
        SafetensorsFile(p)


def test_one_error_lists_missing_unexpected_and_wrong_shapes(tmp_path):
    w = random_weights(TINY_B, 1)
    del w["model.layers.1.mlp.up_proj.weight"], w["model.norm.weight"]
    w["model.layers.0.self_attn.rotary.inv_freq"] = torch.zeros(4, dtype=torch.bfloat16)
    w["model.layers.2.self_attn.k_proj.weight"] = torch.zeros(96, 95, dtype=torch.bfloat16)
    w["lm_head.weight"] = w["lm_head.weight"].to(torch.int32)
    write_folder(str(tmp_path), TINY_B, w)
    declared = declare_weights(load_config(str(tmp_path)).to_model_spec())
    with pytest.raises(WeightError) as e:
        FolderWeights(str(tmp_path), declared, torch.bfloat16, "cpu")
    err = e.value
    assert err.missing == ["model.layers.1.mlp.up_proj.weight", "model.norm.weight"]
    assert err.unexpected == ["model.layers.0.self_attn.rotary.inv_freq"]
    assert err.wrong_shape == [("model.layers.2.self_attn.k_proj.weight", (96, 95), (96, 96))]
    assert err.wrong_dtype == [("lm_head.weight", "int32")]
    for word in ("missing (2)", "unexpected (1)", "wrong shape", "wrong dtype", "up_proj", "inv_freq"):
        assert word in str(err)


def test_held_dtypes(tmp_path):
    w = random_weights(TINY_A, 0)
    w["model.norm.weight"] = w["model.norm.weight"].float() + 1e-4      # a tensor stored in 32-bit
    write_folder(str(tmp_path), TINY_A, w)
    declared = declare_weights(config_from_dict(TINY_A).to_model_spec())
    by = {d.name: d for d in declared}
    for dt in (torch.bfloat16, torch.float32):
        src = FolderWeights(str(tmp_path), declared, dt, "cpu")
        m = src.get(by["model.layers.0.mlp.down_proj.weight"])
        assert m.dtype == dt and torch.equal(m.float(), w["model.layers.0.mlp.down_proj.weight"].float())
        v = src.get(by["model.norm.weight"])
        assert v.dtype == torch.float32 and torch.equal(v, w["model.norm.weight"])     # stays 32-bit, exactly
        assert src.get(by["model.layers.0.input_layernorm.weight"]).dtype == torch.float32


def test_tied_head_in_the_file_is_tolerated(tmp_path):
    w = random_weights(TINY_A, 0)
    w["lm_head.weight"] = w["model.embed_tokens.weight"].clone()
    write_folder(str(tmp_path), TINY_A, w)
    declared = declare_weights(config_from_dict(TINY_A).to_model_spec())
    with pytest.raises(WeightError):
        FolderWeights(str(tmp_path), declared, torch.bfloat16, "cpu")
    FolderWeights(str(tmp_path), declared, torch.bfloat16, "cpu", ignorable=["lm_head.weight"])


def test_random_weights_mode_writes_a_loadable_folder(tmp_path):
    cfg = config_from_dict(TINY_B)
    a, b, c = (str(tmp_path / x) for x in "abc")
    write_model_folder(a, cfg, seed=5)
    write_model_folder(b, cfg, seed=5)
    write_model_folder(c, cfg, seed=6)
    assert load_config(a) == cfg
    fa, fb, fc = (SafetensorsFile(os.path.join(d, "model.safetensors")) for d in (a, b, c))
    declared = declare_weights(cfg.to_model_spec())
    assert sorted(fa.names()) == sorted(d.name for d in declared)
    n = "model.layers.2.self_attn.q_proj.weight"
    assert torch.equal(fa.tensor(n), fb.tensor(n)) and not torch.equal(fa.tensor(n), fc.tensor(n))
    assert abs(float(fa.tensor(n).float().std()) - 0.02) < 0.004
    assert abs(float(fa.tensor("model.norm.weight").float().mean()) - 1.0) < 0.1
    FolderWeights(a, declared, torch.bfloat16, "cpu")


def test_random_values_are_a_function_of_seed_name_and_index():
    """Counter based: any slice of a tensor can be made alone, a tensor does not depend on its neighbours, and
    the stream is standard normal (the device kernel gives the same bits; that is checked on a GPU)."""
    import numpy as np
    from titan_b200.weights.random_init import standard_normal, tensor_key, values
    key = tensor_key(5, "model.layers.1.mlp.up_proj.weight")
    whole = values(key, 0, 5000, 0.02, 0.0)
    assert np.array_equal(whole[1234:1300], values(key, 1234, 66, 0.02, 0.0))
    assert not np.array_equal(whole[:50], values(tensor_key(5, "model.layers.2.mlp.up_proj.weight"), 0, 50, 0.02, 0.0))
    assert not np.array_equal(whole[:50], values(tensor_key(6, "model.layers.1.mlp.up_proj.weight"), 0, 50, 0.02, 0.0))
    x = standard_normal(key, 0, 400000)
    assert abs(x.mean()) < 0.005 and abs(x.std() - 1) < 0.005 and abs((x ** 4).mean() - 3) < 0.05 and 4 < np.abs(x).max() < 6
    assert abs(np.mean(x[:-1] * x[1:])) < 0.005                       # neighbours are uncorrelated
