"""Weights: the container, names and shapes, the random-weights mode."""
import json
import struct

import numpy as np
import pytest
import torch

import plain_llama as plain
import tiny
from alpacca_b200.engine.loading import build_model, load_model_dir, write_random_model_dir
from alpacca_b200.weights import (FolderSource, RandomSource, SafetensorsError, SafetensorsFile, WeightError,
                                  check_names, write_safetensors)


def test_writer_and_reader_round_trip(tmp_path):
    a = torch.arange(12, dtype=torch.float32).reshape(3, 4)
    b = torch.tensor([1.5, -2.25], dtype=torch.bfloat16)
    c = torch.tensor([[7, -1]], dtype=torch.int32)
    p = tmp_path / "x.safetensors"
    write_safetensors(p, [("a", "F32", (3, 4), lambda: a), ("b", "BF16", (2,), lambda: b),
                          ("c", "I32", (1, 2), lambda: c)], metadata={"k": 1})
    f = SafetensorsFile(p)
    assert set(f.tensors) == {"a", "b", "c"} and f.metadata == {"k": "1"}
    assert torch.equal(f.get("a"), a) and torch.equal(f.get("b"), b) and torch.equal(f.get("c"), c)
    # the test-side reader (own code) reads the same bytes
    other = plain.read_safetensors(p)
    assert np.array_equal(other["a"], a.numpy()) and np.array_equal(other["b"], [1.5, -2.25])


def _raw(tmp_path, header: bytes, data: bytes = b"", hlen=None):
    p = tmp_path / "bad.safetensors"
    p.write_bytes(struct.pack("<Q", len(header) if hlen is None else hlen) + header + data)
    return p


def test_broken_files_are_refused(tmp_path):
    (tmp_path / "short").write_bytes(b"abc")
    with pytest.raises(SafetensorsError, match="too short"):
        SafetensorsFile(tmp_path / "short")
    with pytest.raises(SafetensorsError, match="header length"):
        SafetensorsFile(_raw(tmp_path, b"{}", hlen=10 ** 9))
    with pytest.raises(SafetensorsError, match="not JSON"):
        SafetensorsFile(_raw(tmp_path, b"{nope"))
    h = json.dumps({"w": {"dtype": "F32", "shape": [2, 2], "data_offsets": [0, 16]}}).encode()
    with pytest.raises(SafetensorsError, match="outside the file"):
        SafetensorsFile(_raw(tmp_path, h, b"\0" * 8))
    h = json.dumps({"w": {"dtype": "F32", "shape": [2, 2], "data_offsets": [0, 8]}}).encode()
    with pytest.raises(SafetensorsError, match="needs 16 bytes"):
        SafetensorsFile(_raw(tmp_path, h, b"\0" * 16))
    h = json.dumps({"w": {"dtype": "F8_E4M3", "shape": [2], "data_offsets": [0, 2]}}).encode()
    with pytest.raises(SafetensorsError, match="unsupported dtype"):
        SafetensorsFile(_raw(tmp_path, h, b"\0" * 2))
    # a shape whose byte count wraps around 2^64 to exactly the bytes that are there
    h = json.dumps({"w": {"dtype": "F32", "shape": [2 ** 31, 2 ** 31, 4], "data_offsets": [0, 0]}}).encode()
    with pytest.raises(SafetensorsError, match="does not fit 63 bits"):
        SafetensorsFile(_raw(tmp_path, h, b""))
    # an unknown key whose value is nested a hundred thousand levels deep
    deep = b'{"__metadata__":{},"x":{"dtype":"F32","shape":[],"data_offsets":[0,4],"extra":' + b"[" * 100000 + b"]" * 100000 + b"}}"
    with pytest.raises(SafetensorsError, match="nested deeper"):
        SafetensorsFile(_raw(tmp_path, deep, b"\0" * 4))
    with pytest.raises(SafetensorsError, match="no model.safetensors"):
        FolderSource(tmp_path / "nowhere")


def test_one_error_lists_missing_unexpected_and_wrong_shapes(tmp_path):
    cfg = tiny.TINY_A
    w = tiny.make_weights(cfg, 0)
    del w["model.layers.1.mlp.up_proj.weight"]
    del w["model.norm.weight"]
    w["model.layers.0.self_attn.rotary_emb.inv_freq"] = np.zeros(8, np.float32)
    w["model.layers.0.self_attn.k_proj.weight"] = np.zeros((64, 32), np.float32)
    tiny.write_model_dir(tmp_path, cfg, w)
    with pytest.raises(WeightError) as e:
        load_model_dir(tmp_path, dtype="float32", device="cpu")
    msg = str(e.value)
    assert "2 missing" in msg and "model.layers.1.mlp.up_proj.weight [160, 64]" in msg and "model.norm.weight" in msg
    assert "1 unexpected" in msg and "rotary_emb.inv_freq" in msg
    assert "1 of wrong shape" in msg and "expected [64, 64], found [64, 32]" in msg


def test_tied_head_must_not_be_stored_and_untied_must(tmp_path):
    cfg = tiny.TINY_B            # tied
    w = tiny.make_weights(cfg, 1)
    w["lm_head.weight"] = np.zeros((384, 192), np.float32)
    tiny.write_model_dir(tmp_path / "t", cfg, w)
    with pytest.raises(WeightError, match="unexpected: lm_head.weight"):
        load_model_dir(tmp_path / "t", dtype="float32", device="cpu")
    cfg = tiny.TINY_A            # untied
    w = tiny.make_weights(cfg, 0)
    del w["lm_head.weight"]
    tiny.write_model_dir(tmp_path / "u", cfg, w)
    with pytest.raises(WeightError, match="missing: lm_head.weight"):
        load_model_dir(tmp_path / "u", dtype="float32", device="cpu")


def test_dtypes_in_memory(tmp_path):
    """Matrices are kept in the compute dtype (bfloat16 stays bfloat16), small vectors in float32."""
    d = write_random_model_dir(tmp_path / "m", tiny.TINY_C, 3, dtype=torch.bfloat16)
    assert SafetensorsFile(d / "model.safetensors").tensors["model.embed_tokens.weight"].dtype == "BF16"
    m = load_model_dir(d, dtype="bfloat16", device="cpu")
    blk = m.spec.layers[0]
    assert blk.mixer.qkv.weight.dtype == torch.bfloat16 and blk.mixer.qkv.weight.shape == ((10 + 2 * 5) * 48, 120)
    assert blk.norm1.weight.dtype == torch.float32 and blk.mixer.qkv.bias.dtype == torch.float32
    assert m.spec.embedding.weight.dtype == torch.bfloat16
    m32 = load_model_dir(d, dtype="float32", device="cpu")
    assert m32.spec.layers[0].mixer.qkv.weight.dtype == torch.float32
    assert torch.equal(m32.spec.layers[0].mixer.qkv.weight, blk.mixer.qkv.weight.float())   # widened exactly


def test_fused_layouts(tmp_path):
    d = write_random_model_dir(tmp_path / "m", tiny.TINY_B, 1, dtype=torch.float32)
    m = load_model_dir(d, dtype="float32", device="cpu")
    raw = plain.read_safetensors(d / "model.safetensors")
    p = "model.layers.2."
    qkv = m.spec.layers[2].mixer.qkv.weight.numpy()
    assert np.array_equal(qkv, np.concatenate([raw[p + f"self_attn.{n}_proj.weight"] for n in "qkv"]))
    gu = m.spec.layers[2].ffn.gate_up.weight.numpy().reshape(512 // 8, 2, 8, 192)
    assert np.array_equal(gu[:, 0].reshape(512, 192), raw[p + "mlp.gate_proj.weight"])
    assert np.array_equal(gu[:, 1].reshape(512, 192), raw[p + "mlp.up_proj.weight"])
    # tied: the head's matrix is the embedding's storage
    assert m.spec.head.tied_to is m.spec.embedding


def test_random_mode_writes_a_loadable_folder_and_is_deterministic(tmp_path):
    d1 = write_random_model_dir(tmp_path / "1", tiny.TINY_A, 5, dtype=torch.float32)
    d2 = write_random_model_dir(tmp_path / "2", tiny.TINY_A, 5, dtype=torch.float32)
    d3 = write_random_model_dir(tmp_path / "3", tiny.TINY_A, 6, dtype=torch.float32)
    a, b, c = (plain.read_safetensors(d / "model.safetensors") for d in (d1, d2, d3))
    assert set(a) == set(tiny.tensor_shapes(tiny.TINY_A))
    assert all(a[n].shape == s for n, s in tiny.tensor_shapes(tiny.TINY_A).items())
    assert all(np.array_equal(a[n], b[n]) for n in a) and not np.array_equal(a["lm_head.weight"], c["lm_head.weight"])
    assert json.loads((d1 / "config.json").read_text())["hidden_size"] == 64
    # distributions: matrices N(0, 0.02), norm weights 1 + N(0, 0.02)
    assert abs(a["model.embed_tokens.weight"].std() - 0.02) < 2e-3 and abs(a["model.embed_tokens.weight"].mean()) < 2e-3
    assert abs(a["model.norm.weight"].mean() - 1.0) < 2e-2
    # a tensor's values depend on (seed, name) only, not on the rest of the model
    model = build_model(tiny.TINY_A, "float32", "cpu")
    specs = model.param_specs()
    one = RandomSource([s for s in specs if s.name == "model.norm.weight"], 5, torch.float32).get("model.norm.weight")
    assert np.array_equal(one.numpy(), a["model.norm.weight"])


def test_check_names_accepts_a_fitting_table():
    model = build_model(tiny.TINY_C, "float32", "cpu")
    table = {n: ("F32", s) for n, s in tiny.tensor_shapes(tiny.TINY_C).items()}
    check_names(model.param_specs(), table)
    assert model.n_params() == sum(int(np.prod(s)) for s in tiny.tensor_shapes(tiny.TINY_C).values())
