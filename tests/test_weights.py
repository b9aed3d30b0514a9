"""Weights: the safetensors reader and writer, binding by name with one error for
everything that does not fit, dtype rules, and random-weights mode."""
import json
import os
import struct

import numpy as np
import pytest
import torch

import kllm_b200.models  # noqa: F401
from kllm_b200.config import build_model_spec, parse_config
from kllm_b200.parts.model import DecoderModel
from kllm_b200.parts.spec import TensorSpec
from kllm_b200.weights import (ModelFiles, SafetensorsError, SafetensorsFile, WeightError, load_weights,
                               save_tensors, write_random_model)
from helpers import TINY_A, TINY_B, make_weights, write_model_dir


def raw_file(path, header: str, data: bytes):
    with open(path, "wb") as f:
        f.write(struct.pack("<Q", len(header)))
        f.write(header.encode())
        f.write(data)


# the five corrupt files of the reference's loader test (engine/loader/safetensors_test.go:112-159)
@pytest.mark.parametrize("case", ["short", "huge_header", "past_end", "bytes_disagree", "unknown_dtype",
                                  "negative_dim", "not_json"])
def test_corrupt_files_are_refused(tmp_path, case):
    p = str(tmp_path / "bad.safetensors")
    if case == "short":
        open(p, "wb").write(b"\x01\x02\x03")
    elif case == "huge_header":
        open(p, "wb").write(struct.pack("<Q", 1 << 40) + b"{}")
    elif case == "past_end":
        raw_file(p, '{"t":{"dtype":"F32","shape":[8],"data_offsets":[0,32]}}', bytes(16))
    elif case == "bytes_disagree":
        raw_file(p, '{"t":{"dtype":"F32","shape":[3],"data_offsets":[0,16]}}', bytes(16))
    elif case == "unknown_dtype":
        raw_file(p, '{"t":{"dtype":"F8_E4M3","shape":[4],"data_offsets":[0,4]}}', bytes(4))
    elif case == "negative_dim":
        raw_file(p, '{"t":{"dtype":"F32","shape":[-1],"data_offsets":[0,4]}}', bytes(4))
    elif case == "not_json":
        raw_file(p, '{"t":', bytes(4))
    with pytest.raises(SafetensorsError):
        SafetensorsFile(p)


def test_round_trip_and_library_compatibility(tmp_path):
    from safetensors.torch import load_file, save_file
    t = {"a": torch.randn(3, 5), "b": torch.randn(7).to(torch.bfloat16), "c": torch.arange(6, dtype=torch.int32)}
    p = str(tmp_path / "x.safetensors")
    save_tensors(p, t)
    back = load_file(p)                       # the library reads what we write
    for k in t:
        assert torch.equal(back[k], t[k])
    save_file(t, str(tmp_path / "y.safetensors"))
    f = SafetensorsFile(str(tmp_path / "y.safetensors"))   # we read what the library writes
    assert f.names() == ["a", "b", "c"]
    for k in t:
        assert torch.equal(f.read(k), t[k])
    f.close()


def test_shards_index_and_duplicates(tmp_path):
    d = tmp_path / "m"
    d.mkdir()
    save_tensors(str(d / "part-1.safetensors"), {"a": torch.ones(2)})
    save_tensors(str(d / "part-2.safetensors"), {"b": torch.zeros(3)})
    with ModelFiles(str(d)) as m:                  # every *.safetensors, sorted
        assert m.names() == ["a", "b"]
    (d / "model.safetensors.index.json").write_text(json.dumps(
        {"weight_map": {"a": "part-1.safetensors", "b": "part-2.safetensors"}}))
    with ModelFiles(str(d)) as m:
        assert torch.equal(m.read("b"), torch.zeros(3))
    save_tensors(str(d / "part-3.safetensors"), {"a": torch.ones(2)})
    os.unlink(str(d / "model.safetensors.index.json"))
    with pytest.raises(SafetensorsError, match="both"):
        ModelFiles(str(d))
    with pytest.raises(SafetensorsError):
        ModelFiles(str(tmp_path / "empty-or-missing"))


def model_specs(cfg):
    return DecoderModel(build_model_spec(parse_config(cfg)), torch.float32, "cpu").tensor_specs()


def test_one_error_lists_missing_unexpected_and_wrong_shapes(tmp_path):
    cfg, w = make_weights("A")
    w = dict(w)
    del w["model.layers.1.mlp.up_proj.weight"]
    del w["model.norm.weight"]
    w["model.layers.0.self_attn.q_norm.weight"] = np.ones(16, dtype=np.float32)
    w["extra.bias"] = np.ones(3, dtype=np.float32)
    w["model.layers.0.self_attn.k_proj.weight"] = np.zeros((64, 64), dtype=np.float32)
    w["lm_head.weight"] = np.zeros((256, 60), dtype=np.float32)
    d = write_model_dir(str(tmp_path / "m"), cfg, w)
    with pytest.raises(WeightError) as e:
        load_weights(d, model_specs(cfg), torch.float32, "cpu")
    err = e.value
    assert err.missing == ["model.layers.1.mlp.up_proj.weight", "model.norm.weight"]
    assert err.unexpected == ["extra.bias", "model.layers.0.self_attn.q_norm.weight"]
    assert [(n, got, want) for n, got, want in err.wrong_shape] == [
        ("lm_head.weight", (256, 60), (256, 64)),
        ("model.layers.0.self_attn.k_proj.weight", (64, 64), (32, 64))]
    msg = str(err)
    for needle in ("missing (2)", "unexpected (2)", "wrong shape (2)", "up_proj", "extra.bias", "[256, 60]"):
        assert needle in msg


def test_extra_tensors_are_left_unread_counted_and_named(tmp_path):
    """A folder that holds more than the model asks for (an older checkpoint's
    ``rotary_emb.inv_freq``, a tensor of another head) still loads: the reference uploads
    everything and uses what it needs (backend/model.cu:747-765).  The extras are named in
    a warning with their count; ``strict=True`` refuses them."""
    cfg, w = make_weights("A")
    w = dict(w)
    w["model.layers.0.self_attn.rotary_emb.inv_freq"] = np.ones(8, dtype=np.float32)
    w["score.weight"] = np.ones((2, 64), dtype=np.float32)
    d = write_model_dir(str(tmp_path / "m"), cfg, w)
    with pytest.warns(UserWarning, match=r"2 tensor\(s\).*inv_freq.*score\.weight"):
        t = load_weights(d, model_specs(cfg), torch.float32, "cpu")
    assert "score.weight" not in t and len(t) == len(w) - 2
    with pytest.raises(WeightError) as e:
        load_weights(d, model_specs(cfg), torch.float32, "cpu", strict=True)
    assert e.value.unexpected == ["model.layers.0.self_attn.rotary_emb.inv_freq", "score.weight"]
    assert not e.value.missing and not e.value.wrong_shape


def test_dtype_rules(tmp_path):
    cfg, w = make_weights("A")
    d = write_model_dir(str(tmp_path / "f32"), cfg, w)
    specs = model_specs(cfg)
    t = load_weights(d, specs, torch.bfloat16, "cpu")
    assert t["model.layers.0.mlp.down_proj.weight"].dtype == torch.bfloat16     # matrices in the model dtype
    assert t["model.norm.weight"].dtype == torch.float32                         # 32-bit stays 32-bit
    t = load_weights(d, specs, torch.float32, "cpu")
    assert all(v.dtype == torch.float32 for v in t.values())
    assert np.array_equal(t["lm_head.weight"].numpy(), w["lm_head.weight"])
    d2 = write_model_dir(str(tmp_path / "bf16"), cfg, w, bf16=True)              # a bfloat16 file, widened
    t2 = load_weights(d2, specs, torch.float32, "cpu")
    assert torch.equal(t2["lm_head.weight"], torch.from_numpy(w["lm_head.weight"]).to(torch.bfloat16).float())
    # integer tables become int32; a float where an integer table is expected is refused
    (tmp_path / "i").mkdir()
    save_tensors(str(tmp_path / "i" / "model.safetensors"), {"table": torch.arange(5, dtype=torch.int64)})
    got = load_weights(str(tmp_path / "i"), [TensorSpec("table", (5,), store="int32")], torch.bfloat16, "cpu")
    assert got["table"].dtype == torch.int32 and got["table"].tolist() == [0, 1, 2, 3, 4]
    with pytest.raises(WeightError, match="wrong dtype"):
        load_weights(str(tmp_path / "i"), [TensorSpec("table", (5,))], torch.bfloat16, "cpu")


def test_tied_head_needs_no_tensor_and_ignores_a_copy(tmp_path):
    cfg, w = make_weights("B")
    assert "lm_head.weight" not in w
    specs = model_specs(cfg)
    d = write_model_dir(str(tmp_path / "tied"), cfg, w)
    assert "lm_head.weight" not in load_weights(d, specs, torch.float32, "cpu")
    w2 = dict(w, **{"lm_head.weight": w["model.embed_tokens.weight"].copy()})
    load_weights(write_model_dir(str(tmp_path / "copy"), cfg, w2), specs, torch.float32, "cpu")
    cfg_untied = dict(cfg, tie_word_embeddings=False)
    with pytest.raises(WeightError) as e:
        load_weights(d, model_specs(cfg_untied), torch.float32, "cpu")
    assert e.value.missing == ["lm_head.weight"]


def test_random_weights_mode(tmp_path):
    a = write_random_model(str(tmp_path / "a"), TINY_A, seed=0)
    b = write_random_model(str(tmp_path / "b"), TINY_A, seed=0)
    c = write_random_model(str(tmp_path / "c"), TINY_A, seed=1)
    specs = model_specs(TINY_A)
    ta, tb, tc = (load_weights(x, specs, torch.float32, "cpu") for x in (a, b, c))
    assert set(ta) == {s.name for s in specs}
    assert all(torch.equal(ta[k], tb[k]) for k in ta)
    assert not torch.equal(ta["lm_head.weight"], tc["lm_head.weight"])
    assert abs(float(ta["model.embed_tokens.weight"].std()) - 0.02) < 2e-3
    assert torch.equal(ta["model.norm.weight"], torch.ones(64))
    assert json.load(open(os.path.join(a, "config.json")))["hidden_size"] == 64
    # the same tensor does not depend on what else the model holds: more layers, same layer 0
    more = write_random_model(str(tmp_path / "more"), dict(TINY_A, num_hidden_layers=3), seed=0)
    tm = load_weights(more, model_specs(dict(TINY_A, num_hidden_layers=3)), torch.float32, "cpu")
    assert torch.equal(tm["model.layers.0.mlp.up_proj.weight"], ta["model.layers.0.mlp.up_proj.weight"])
    # tied, spread gains, bfloat16 file
    t = write_random_model(str(tmp_path / "t"), TINY_B, seed=2, dtype=torch.bfloat16, gain_std=0.1)
    with ModelFiles(t) as m:
        assert "lm_head.weight" not in m.names()
        assert m.entry("model.embed_tokens.weight").dtype == torch.bfloat16
        assert m.entry("model.norm.weight").dtype == torch.float32
        assert 0.05 < float(m.read("model.norm.weight").std()) < 0.15
