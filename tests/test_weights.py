"""Safetensors by tensor name, the one error that lists everything, random weights (no GPU)."""
import json
import os
import struct

import numpy as np
import pytest
import torch

import helpers
import cajeta_llm_b200  # noqa: F401
from cajeta_llm_b200.config import parse_config_dict
from cajeta_llm_b200.engine.model import build_model
from cajeta_llm_b200.parts.base import Runtime
from cajeta_llm_b200.weights.safetensors_io import Checkpoint, SafetensorsFile, WeightFileError, write_safetensors
from cajeta_llm_b200.weights.sources import RandomWeights, SafetensorsWeights, WeightError


def _model(raw, dtype="float32"):
    return build_model(parse_config_dict(raw), Runtime(dtype, device="cpu"))


def test_round_trip_keeps_dtypes(tmp_path):
    t = {"a": torch.randn(3, 5), "b": torch.randn(4).to(torch.bfloat16), "c": torch.arange(6, dtype=torch.int64).reshape(2, 3),
         "d": torch.randn(2, 2).to(torch.float16)}
    p = str(tmp_path / "x.safetensors")
    write_safetensors(p, t)
    f = SafetensorsFile(p)
    assert f.load("a").dtype == torch.float32 and torch.equal(f.load("a"), t["a"])
    assert f.load("b").dtype == torch.bfloat16 and torch.equal(f.load("b"), t["b"])
    assert f.load("c").dtype == torch.int32 and torch.equal(f.load("c"), t["c"].to(torch.int32))   # integer tables as int32
    assert f.load("d").dtype == torch.float16
    f.close()


def test_file_errors_name_the_tensor(tmp_path):
    p = str(tmp_path / "bad.safetensors")
    header = json.dumps({"w": {"dtype": "F32", "shape": [2, 2], "data_offsets": [0, 12]}}).encode()
    with open(p, "wb") as f:
        f.write(struct.pack("<Q", len(header)) + header + b"\0" * 12)
    with pytest.raises(WeightFileError, match="'w'.*needs 16 bytes"):
        SafetensorsFile(p)
    header = json.dumps({"w": {"dtype": "F32", "shape": [2, 2], "data_offsets": [0, 16]}}).encode()
    with open(p, "wb") as f:
        f.write(struct.pack("<Q", len(header)) + header + b"\0" * 8)
    with pytest.raises(WeightFileError, match="outside the payload"):
        SafetensorsFile(p)
    with pytest.raises(WeightFileError, match="neither"):
        Checkpoint(str(tmp_path))


def test_model_folder_written_and_read_by_name(tmp_path, model_dirs):
    m = _model(helpers.TINY_B)
    schema = m.params()
    src = SafetensorsWeights(model_dirs["B"])
    src.check(schema)
    assert "lm_head.weight" not in schema                       # tied
    assert src.checkpoint.dtype_of("model.layers.1.mlp.experts.5.down_proj.weight") == "BF16"
    assert src.checkpoint.shape_of("model.layers.1.mlp.experts.5.down_proj.weight") == (96, 48)
    assert src.checkpoint.shape_of("model.layers.0.mlp.gate_proj.weight") == (160, 96)       # layer 0 is dense
    assert src.checkpoint.shape_of("model.layers.1.mlp.shared_expert_gate.weight") == (1, 96)
    assert torch.all(src.get("model.norm.weight", schema["model.norm.weight"]) == 1)
    w = src.get("model.layers.2.self_attn.q_proj.bias", schema["model.layers.2.self_attn.q_proj.bias"])
    assert abs(float(w.float().std()) - 0.02) < 0.01
    src.close()


def test_one_error_lists_missing_unexpected_and_wrong_shapes(tmp_path, model_dirs):
    ck = Checkpoint(model_dirs["A"])
    tensors = {n: ck.load(n) for n in ck.names()}
    ck.close()
    del tensors["model.layers.1.self_attn.k_proj.bias"]
    del tensors["model.layers.0.mlp.experts.3.up_proj.weight"]
    tensors["model.layers.0.rogue.weight"] = torch.zeros(3)
    tensors["lm_head.weight"] = torch.zeros(255, 64)
    tensors["model.layers.1.mlp.gate.weight"] = torch.zeros(64, 4)
    d = tmp_path / "broken"
    d.mkdir()
    (d / "config.json").write_text(json.dumps(helpers.TINY_A))
    write_safetensors(str(d / "model.safetensors"), tensors)
    with pytest.raises(WeightError) as e:
        _model(helpers.TINY_A).load(SafetensorsWeights(str(d)))
    msg = str(e.value)
    for needle in ("missing (2)", "model.layers.1.self_attn.k_proj.bias", "model.layers.0.mlp.experts.3.up_proj.weight",
                   "unexpected (1)", "model.layers.0.rogue.weight", "wrong shape (2)",
                   "lm_head.weight: expected [256, 64], found [255, 64]",
                   "model.layers.1.mlp.gate.weight: expected [4, 64], found [64, 4]"):
        assert needle in msg, needle


def test_untied_model_refuses_a_missing_head(tmp_path, model_dirs):
    ck = Checkpoint(model_dirs["A"])
    tensors = {n: ck.load(n) for n in ck.names() if n != "lm_head.weight"}
    ck.close()
    d = tmp_path / "nohead"
    d.mkdir()
    write_safetensors(str(d / "model.safetensors"), tensors)
    with pytest.raises(WeightError, match="lm_head.weight"):
        _model(helpers.TINY_A).load(SafetensorsWeights(str(d)))


def test_dtypes_the_engine_holds(model_dirs):
    for dtype, want in (("float32", torch.float32), ("bfloat16", torch.bfloat16)):
        m = _model(helpers.TINY_A, dtype)
        m.load(SafetensorsWeights(model_dirs["A"]))
        att = m.blocks[0].mixer
        moe = m.blocks[0].feed_forward
        assert m.embedding.dtype == want and att.w_qkv.dtype == want and moe.w_gate.dtype == want
        # 4 experts of width 32, then the shared expert (width 64) as 2 chunks of that width
        assert att.w_qkv.shape == (64 + 2 * 32, 64) and moe.w_gate.shape == (6, 32, 64) and moe.w_down.shape == (6, 64, 32)
        ck = Checkpoint(model_dirs["A"])
        sg = ck.load("model.layers.0.mlp.shared_expert.gate_proj.weight").to(want)
        sd = ck.load("model.layers.0.mlp.shared_expert.down_proj.weight").to(want)
        e3 = ck.load("model.layers.0.mlp.experts.3.up_proj.weight").to(want)
        ck.close()
        assert torch.equal(moe.w_gate[4], sg[:32]) and torch.equal(moe.w_gate[5], sg[32:])
        assert torch.equal(moe.w_down[4], sd[:, :32]) and torch.equal(moe.w_down[5], sd[:, 32:])
        assert torch.equal(moe.w_up[3], e3)
        # small tensors used in 32-bit arithmetic are held in float32 (exact for a bfloat16 file)
        assert att.b_qkv.dtype == torch.float32 and moe.router.dtype == torch.float32
        assert m.final_norm.weight.dtype == torch.float32


def test_a_tensor_stored_in_32_bit_stays_so(tmp_path):
    helpers.write_model(str(tmp_path), helpers.TINY_A, seed=5, store_dtype=torch.float32)
    ck = Checkpoint(str(tmp_path))
    assert ck.dtype_of("model.embed_tokens.weight") == "F32"
    w = ck.load("model.layers.0.self_attn.q_proj.weight")
    ck.close()
    assert w.dtype == torch.float32 and not torch.equal(w, w.to(torch.bfloat16).float())     # not rounded on the way
    m = _model(helpers.TINY_A, "float32")
    m.load(SafetensorsWeights(str(tmp_path)))
    assert torch.equal(m.blocks[0].mixer.w_qkv[:64], w)


def test_random_weights_depend_on_seed_and_name_only():
    m = _model(helpers.TINY_A)
    schema = m.params()
    a, b, c = RandomWeights(1), RandomWeights(1), RandomWeights(2)
    names = list(schema)
    for n in (names[3], names[10]):
        assert torch.equal(a.get(n, schema[n]), b.get(n, schema[n]))
        if schema[n].init == "normal":
            assert not torch.equal(a.get(n, schema[n]), c.get(n, schema[n]))
    assert not torch.equal(a.get(names[3], schema[names[3]]).flatten()[:8], a.get(names[10], schema[names[10]]).flatten()[:8])


def test_random_values_follow_the_plain_generator_element_by_element():
    """The numpy generator against its restatement with Python integers: single elements far
    apart (also beyond a chunk of the numpy loop and beyond 2^32), float32 and bfloat16."""
    import plain_random as PR
    from cajeta_llm_b200.parts.plan import ParamSpec
    from cajeta_llm_b200.weights import random_fill as R
    seed, name, std = 7, "model.layers.3.mlp.experts.5.up_proj.weight", 0.02
    key = R.tensor_key(seed, name)
    assert key == PR.key_of(seed, name)
    n = R.CHUNK + 1000
    x = R.fill(n, key, std)
    for i in (0, 1, 2, 4097, R.CHUNK - 1, R.CHUNK, R.CHUNK + 999):
        assert float(x[i]) == PR.value(seed, name, i, std), i
    far = (1 << 33) + 12345
    assert float(R.fill(3, key, std, start=far)[2]) == PR.value(seed, name, far + 2, std)
    assert abs(float(x.mean())) < 3 * std / np.sqrt(n) and abs(float(x.std()) / std - 1.0) < 0.01
    assert float(np.abs(x).max()) <= 4.9 * std
    spec = ParamSpec((40, 50), std=std)
    got = RandomWeights(seed, torch.bfloat16).get(name, spec)
    assert got.dtype == torch.bfloat16 and tuple(got.shape) == (40, 50)
    for i in (0, 7, 1999):
        assert float(got.flatten()[i]) == PR.to_bfloat16(PR.value(seed, name, i, std)), i
    got32 = RandomWeights(seed, torch.float32).get(name, spec)
    assert float(got32.flatten()[1234]) == PR.value(seed, name, 1234, std)
