"""Safetensors reading and writing, the checkpoint check with its one error, and random-weights mode."""
import json
import struct

import pytest
import torch

from conftest import tiny_config
from vllm_cpp_b200 import expected_tensors, load_config, write_random_model
from vllm_cpp_b200.weights import (SafetensorsError, WeightError, WeightStore, open_model_weights,
                                   read_safetensors, write_safetensors)


def test_round_trip_all_types(tmp_path):
    t = {"a": torch.randn(3, 5).to(torch.bfloat16), "b": torch.randn(7).to(torch.float16), "c": torch.randn(2, 2, 2),
         "d": torch.arange(6, dtype=torch.int32).view(2, 3), "e": torch.zeros(0, 4)}
    write_safetensors(tmp_path / "m.safetensors", t, {"k": "v"})
    back = read_safetensors(tmp_path / "m.safetensors")
    assert set(back) == set(t)
    for k in t:
        assert back[k].dtype == t[k].dtype and torch.equal(back[k], t[k])
    # the same bytes mean the same to the independent reader of the plain implementation
    import plain_qwen3
    other = plain_qwen3.read_safetensors(tmp_path / "m.safetensors")
    assert torch.equal(other["a"].float(), t["a"].float()) and torch.equal(other["c"].float(), t["c"])


def test_header_errors(tmp_path):
    p = tmp_path / "bad.safetensors"
    p.write_bytes(b"\x01")
    with pytest.raises(SafetensorsError, match="too short"):
        read_safetensors(p)
    p.write_bytes(struct.pack("<Q", 1 << 40) + b"{}")
    with pytest.raises(SafetensorsError, match="implausible"):
        read_safetensors(p)
    p.write_bytes(struct.pack("<Q", 5) + b"{nope")
    with pytest.raises(SafetensorsError, match="not valid JSON"):
        read_safetensors(p)

    def with_header(h, data=b"\0" * 8):
        blob = json.dumps(h).encode()
        p.write_bytes(struct.pack("<Q", len(blob)) + blob + data)

    with_header({"w": {"dtype": "F8_E4M3", "shape": [8], "data_offsets": [0, 8]}})
    with pytest.raises(SafetensorsError, match="'w'.*F8_E4M3"):
        read_safetensors(p)
    with_header({"w": {"dtype": "F32", "shape": [3], "data_offsets": [0, 8]}})
    with pytest.raises(SafetensorsError, match="'w'.*needs 12"):
        read_safetensors(p)
    with_header({"w": {"dtype": "F32", "shape": [4], "data_offsets": [0, 16]}})
    with pytest.raises(SafetensorsError, match="'w'"):
        read_safetensors(p)      # data runs past the end of the file
    with_header({"w": {"shape": [2]}})
    with pytest.raises(SafetensorsError, match="malformed"):
        read_safetensors(p)


def test_one_error_lists_missing_unexpected_and_wrong_shapes(tmp_path):
    cfg = tiny_config("B")
    folder = write_random_model(cfg, 1, tmp_path / "m")
    tensors = dict(read_safetensors(folder / "model.safetensors"))
    del tensors["model.layers.1.self_attn.k_norm.weight"], tensors["lm_head.weight"]
    tensors["model.layers.0.self_attn.q_proj.bias"] = torch.zeros(192)
    tensors["model.layers.2.mlp.down_proj.weight"] = torch.zeros(96, 201)
    store = WeightStore(tensors, torch.float32, "cpu")
    with pytest.raises(WeightError) as err:
        store.check(expected_tensors(cfg))
    msg = str(err.value)
    assert "missing tensors (2)" in msg and "model.layers.1.self_attn.k_norm.weight" in msg and "lm_head.weight" in msg
    assert "unexpected tensors (1)" in msg and "q_proj.bias" in msg
    assert "wrong shapes (1)" in msg and "expected (96, 200), found (96, 201)" in msg
    with pytest.raises(WeightError, match="no .safetensors"):
        open_model_weights(tmp_path, torch.float32, "cpu")


def test_what_is_stored_is_kept():
    t = {"g16": torch.ones(4).to(torch.bfloat16), "g32": torch.ones(4), "gh": torch.ones(4).to(torch.float16),
         "m": torch.randn(4, 4), "ids": torch.arange(4, dtype=torch.int64)}
    bf = WeightStore(t, torch.bfloat16, "cpu")
    assert bf.vector("g16").dtype == torch.bfloat16 and bf.vector("g32").dtype == torch.float32   # 32-bit stays 32-bit
    assert bf.vector("gh").dtype == torch.float32 and bf.matrix("m").dtype == torch.bfloat16
    assert bf.table("ids").dtype == torch.int32
    f32 = WeightStore(t, torch.float32, "cpu")
    assert f32.vector("g16").dtype == torch.float32 and f32.matrix("m").dtype == torch.float32
    assert torch.equal(bf.matrices(["m", "m"])[4:], t["m"].to(torch.bfloat16))
    both = bf.matrices(["m", "m"], interleave=True)
    assert torch.equal(both[0::2], t["m"].to(torch.bfloat16)) and torch.equal(both[1::2], both[0::2])
    with pytest.raises(WeightError, match="integer table"):
        bf.table("m")
    with pytest.raises(WeightError, match="not in the checkpoint"):
        bf.matrix("nope")


def test_random_weights_mode(tmp_path):
    cfg = tiny_config("A")
    a = write_random_model(cfg, 5, tmp_path / "a")
    b = write_random_model(cfg, 5, tmp_path / "b")
    c = write_random_model(cfg, 6, tmp_path / "c", dtype="float32")
    assert load_config(a) == cfg
    ta, tb, tc = (read_safetensors(d / "model.safetensors") for d in (a, b, c))
    names = {s.name for s in expected_tensors(cfg)}
    assert set(ta) == names and "lm_head.weight" not in names            # tied: the embedding is the head
    assert all(torch.equal(ta[k], tb[k]) for k in ta)                    # a function of (configuration, seed)
    assert not torch.equal(ta["model.embed_tokens.weight"].float(), tc["model.embed_tokens.weight"])
    assert ta["model.norm.weight"].dtype == torch.bfloat16 and tc["model.norm.weight"].dtype == torch.float32
    w = tc["model.layers.0.mlp.up_proj.weight"]
    assert abs(w.std().item() - 0.02) < 0.002 and abs(tc["model.norm.weight"].mean().item() - 1) < 0.05
    assert {s.name: s.shape for s in expected_tensors(tiny_config("B"))}["model.layers.2.self_attn.o_proj.weight"] == (96, 192)


def test_shard_index_is_checked(tmp_path):
    import json
    cfg = tiny_config("A")
    d = write_random_model(cfg, 1, tmp_path / "m")
    (d / "model.safetensors.index.json").write_text(json.dumps({"weight_map": {"x": "model.safetensors", "y": "model-00002.safetensors"}}))
    with pytest.raises(WeightError, match="model-00002.safetensors"):
        open_model_weights(d, torch.float32, "cpu")
    (d / "model.safetensors.index.json").write_text(json.dumps({"weight_map": {"x": "model.safetensors"}}))
    assert "model.norm.weight" in open_model_weights(d, torch.float32, "cpu")
