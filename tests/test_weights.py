"""The safetensors file, binding by name with one collected error, and the random-weights writer (CPU)."""
import json
import struct

import numpy as np
import pytest
import torch

import plain_llama as P
from conftest import TINY_A, TINY_B
from llmi_b200 import WeightBindingError, write_random_model
from llmi_b200.config import parse_config
from llmi_b200.parts.build import expected_tensors
from llmi_b200.weights import SafetensorsError, SafetensorsFile, check_tensors, load_tensors, write_safetensors
from llmi_b200.weights.binding import storage_form


def expected_shapes(cfg):
    arch, c = parse_config(cfg)
    return {n: d.shape for n, d in expected_tensors(arch.model_spec(c)).items()}, arch


def test_expected_tensor_table_matches_reference_names():
    shapes, _ = expected_shapes(TINY_B)
    assert shapes["model.embed_tokens.weight"] == (384, 120)
    assert shapes["model.layers.2.self_attn.q_proj.weight"] == (120, 120)
    assert shapes["model.layers.0.self_attn.k_proj.weight"] == (24, 120)
    assert shapes["model.layers.0.self_attn.v_proj.bias"] == (24,)
    assert shapes["model.layers.1.mlp.down_proj.weight"] == (120, 320)
    assert shapes["lm_head.weight"] == (384, 120) and shapes["model.norm.weight"] == (120,)
    assert len(shapes) == 1 + 3 * 12 + 2
    a, _ = expected_shapes(TINY_A)
    assert "lm_head.weight" not in a and "model.layers.0.self_attn.q_proj.bias" not in a
    assert len(a) == 1 + 2 * 9 + 1


def test_random_folder_roundtrip_and_statistics(tmp_path):
    d = write_random_model(str(tmp_path / "m"), TINY_B, 99)
    f = SafetensorsFile(d + "/model.safetensors")
    shapes, arch = expected_shapes(TINY_B)
    tensors = load_tensors(f, shapes, "cpu", arch.tolerated_extra_tensors)
    assert set(tensors) == set(shapes)
    assert f.parameter_count() == sum(int(np.prod(s)) for s in shapes.values())
    w = tensors["model.layers.0.mlp.gate_proj.weight"]
    assert w.dtype == torch.float32 and abs(float(w.std()) - 0.02) < 0.002 and abs(float(w.mean())) < 0.002
    n = tensors["model.norm.weight"]
    assert abs(float(n.mean()) - 1.0) < 0.05 and 0.05 < float(n.std()) < 0.15
    # same seed, same values; another seed, other values; a tensor does not depend on the others
    d2 = write_random_model(str(tmp_path / "m2"), TINY_B, 99)
    d3 = write_random_model(str(tmp_path / "m3"), TINY_B, 100)
    g = SafetensorsFile(d2 + "/model.safetensors").tensor("model.layers.1.self_attn.o_proj.weight")
    h = SafetensorsFile(d3 + "/model.safetensors").tensor("model.layers.1.self_attn.o_proj.weight")
    assert torch.equal(g, tensors["model.layers.1.self_attn.o_proj.weight"]) and not torch.equal(g, h)
    fewer = dict(TINY_B, num_hidden_layers=2)
    d4 = write_random_model(str(tmp_path / "m4"), fewer, 99)
    assert torch.equal(SafetensorsFile(d4 + "/model.safetensors").tensor("lm_head.weight"), tensors["lm_head.weight"])
    # the plain implementation's own reader sees the same numbers, and config.json is the dict given
    cfg, pw = P.read_model(d)
    assert cfg == TINY_B
    assert np.array_equal(pw["lm_head.weight"], tensors["lm_head.weight"].double().numpy())


def test_bf16_folder_is_the_rounded_fp32_folder(tmp_path):
    a = SafetensorsFile(write_random_model(str(tmp_path / "a"), TINY_A, 5) + "/model.safetensors")
    b = SafetensorsFile(write_random_model(str(tmp_path / "b"), TINY_A, 5, torch.bfloat16) + "/model.safetensors")
    name = "model.layers.1.mlp.up_proj.weight"
    assert b.tensors[name].dtype == "BF16"
    assert torch.equal(b.tensor(name), a.tensor(name).to(torch.bfloat16))
    _, pw = P.read_model(str(tmp_path / "b"))
    assert np.array_equal(pw[name], b.tensor(name).double().numpy())


def test_one_error_lists_everything_wrong(tmp_path):
    d = write_random_model(str(tmp_path / "m"), TINY_A, 1)
    f = SafetensorsFile(d + "/model.safetensors")
    t = {n: f.tensor(n).clone() for n in f.names()}
    del t["model.norm.weight"]
    del t["model.layers.1.mlp.up_proj.weight"]
    t["model.layers.0.self_attn.q_proj.weight"] = torch.zeros(64, 32)
    t["extra.thing"] = torch.zeros(3)
    t["model.layers.0.self_attn.rotary_emb.inv_freq"] = torch.zeros(8)       # tolerated, as the reference does
    t["lm_head.weight"] = torch.zeros(256, 64)                                # tolerated with tied embeddings
    bad = tmp_path / "bad"
    bad.mkdir()
    (bad / "config.json").write_text(json.dumps(TINY_A))
    t["model.layers.0.input_layernorm.weight"] = torch.zeros(64, dtype=torch.int32)   # stands for a U8 tensor below
    write_safetensors(str(bad / "model.safetensors"), t)
    shapes, arch = expected_shapes(TINY_A)
    g = SafetensorsFile(str(bad / "model.safetensors"))
    found = {n: (i.dtype, i.shape) for n, i in g.tensors.items()}
    found["model.layers.0.input_layernorm.weight"] = ("U8", (64,))
    with pytest.raises(WeightBindingError) as e:
        check_tensors(shapes, found, arch.tolerated_extra_tensors, "bad")
    err = e.value
    assert err.missing == ["model.layers.1.mlp.up_proj.weight", "model.norm.weight"] or set(err.missing) == {
        "model.layers.1.mlp.up_proj.weight", "model.norm.weight"}
    assert err.unexpected == ["extra.thing"]
    assert err.wrong_shape == [("model.layers.0.self_attn.q_proj.weight", (64, 32), (64, 64))]
    assert err.wrong_dtype == [("model.layers.0.input_layernorm.weight", "U8")]
    text = str(err)
    for piece in ("missing tensor model.norm.weight", "has shape [64, 32], expected [64, 64]", "has dtype U8",
                  "unexpected tensor extra.thing"):
        assert piece in text
    with pytest.raises(WeightBindingError, match="missing tensor model.norm.weight"):
        load_tensors(g, shapes, "cpu", arch.tolerated_extra_tensors)


def test_storage_rules():
    assert storage_form(torch.zeros(2, dtype=torch.bfloat16)).dtype == torch.bfloat16
    # F16 stays F16 until a part converts it: widening to fp32 is exact (src/model/safetensors.cpp:290-299), so the
    # 32-bit path computes with the file's values, and the bf16 path rounds them once
    assert storage_form(torch.zeros(2, dtype=torch.float16)).dtype == torch.float16
    assert storage_form(torch.zeros(2, dtype=torch.float32)).dtype == torch.float32      # 32-bit stays 32-bit
    assert storage_form(torch.zeros(2, dtype=torch.int64)).dtype == torch.int32          # integer tables
    assert storage_form(torch.zeros(2, dtype=torch.int32)).dtype == torch.int32


def test_integer_storage_is_refused_for_what_a_model_multiplies_with(tmp_path):
    """src/model/model.cpp:185-187: a weight is F32, F16 or BF16; tests/model_test.cpp:111-151."""
    arch, c = parse_config(TINY_A)
    decls = expected_tensors(arch.model_spec(c))
    found = {n: ("F32", d.shape) for n, d in decls.items()}
    check_tensors(decls, found)
    for storage in ("I32", "I64"):
        for name in ("model.layers.0.self_attn.q_proj.weight", "model.norm.weight", "model.embed_tokens.weight"):
            bad = dict(found)
            bad[name] = (storage, decls[name].shape)
            with pytest.raises(WeightBindingError, match=f"{name} has dtype {storage}, expected F32, F16 or BF16"):
                check_tensors(decls, bad)
    # the one role a file may store as integers
    from llmi_b200.parts.registry import TensorDecl
    table = {"ids": TensorDecl((4,), "int_table")}
    check_tensors(table, {"ids": ("I64", (4,))})
    with pytest.raises(WeightBindingError, match="ids has dtype F32, expected I32 or I64"):
        check_tensors(table, {"ids": ("F32", (4,))})


def test_f16_folder_is_read_exactly(tmp_path):
    """An F16 file's values reach the loader's output unrounded (the plain reader widens them the same way)."""
    d = write_random_model(str(tmp_path / "h"), TINY_A, 5, torch.float16)
    f = SafetensorsFile(d + "/model.safetensors")
    arch, c = parse_config(TINY_A)
    decls = expected_tensors(arch.model_spec(c))
    name = "model.layers.1.mlp.up_proj.weight"
    assert f.tensors[name].dtype == "F16"
    got = load_tensors(f, decls, "cpu")
    _, pw = P.read_model(d)
    for n in decls:
        assert got[n].dtype == torch.float16
        assert np.array_equal(got[n].double().numpy(), pw[n])
    assert not torch.equal(got[name].to(torch.bfloat16).float(), got[name].float())     # bf16 would have lost bits


def raw_file(path, header: dict, data: bytes, pad=True):
    blob = json.dumps(header).encode()
    with open(path, "wb") as f:
        f.write(struct.pack("<Q", len(blob)))
        f.write(blob)
        f.write(data)
    return str(path)


def test_malformed_files(tmp_path):
    p = tmp_path / "x.safetensors"
    ok = {"a": {"dtype": "F32", "shape": [2], "data_offsets": [0, 8]}}
    f = SafetensorsFile(raw_file(p, ok, b"\0" * 8))
    assert f.tensor("a").shape == (2,)
    cases = [
        (ok, b"\0" * 9, "trailing"),
        (ok, b"\0" * 7, "bad data_offsets"),
        ({"a": {"dtype": "F32", "shape": [3], "data_offsets": [0, 8]}}, b"\0" * 8, "do not match"),
        ({"a": {"dtype": "Q4", "shape": [2], "data_offsets": [0, 8]}}, b"\0" * 8, "unknown dtype"),
        ({"a": {"dtype": "F32", "shape": [2], "data_offsets": [0, 8], "more": 1}}, b"\0" * 8, "exactly dtype"),
        ({"a": {"dtype": "F32", "shape": [2], "data_offsets": [0, 8]},
          "b": {"dtype": "F32", "shape": [2], "data_offsets": [4, 12]}}, b"\0" * 12, "overlaps"),
        ({"a": {"dtype": "F32", "shape": [2], "data_offsets": [0, 8]},
          "b": {"dtype": "F32", "shape": [1], "data_offsets": [12, 16]}}, b"\0" * 16, "hole"),
        ({"a": {"dtype": "F32", "shape": [-1], "data_offsets": [0, 8]}}, b"\0" * 8, "bad shape"),
    ]
    for header, data, message in cases:
        with pytest.raises(SafetensorsError, match=message):
            SafetensorsFile(raw_file(p, header, data))
    p.write_bytes(b"\x01\x02")
    with pytest.raises(SafetensorsError, match="too short"):
        SafetensorsFile(str(p))
    p.write_bytes(struct.pack("<Q", 1 << 40) + b"{}")
    with pytest.raises(SafetensorsError, match="larger than"):
        SafetensorsFile(str(p))
    p.write_bytes(struct.pack("<Q", 100) + b"{}")
    with pytest.raises(SafetensorsError, match="past the end"):
        SafetensorsFile(str(p))
    p.write_bytes(struct.pack("<Q", 2) + b"[]")
    with pytest.raises(SafetensorsError, match="not a JSON object"):
        SafetensorsFile(str(p))
    with pytest.raises(SafetensorsError, match="cannot open"):
        SafetensorsFile(str(tmp_path / "nothing"))
