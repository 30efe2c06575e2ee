"""Safetensors container, binding by name and the random-weights mode (no GPU)."""
import json
import os
import struct

import pytest
import torch

from helpers import CONFIG_A, CONFIG_B, make_model_folder
from inferloop_b200.config import read_model_config
from inferloop_b200.models.decoder import declare_weights
from inferloop_b200.weights import (SafetensorsError, SafetensorsFile, TensorSource, WeightError, load_weights,
                                    random_tensor, write_safetensors)
from inferloop_b200.weights.decl import WeightDecl


def _spec(cfg):
    return read_model_config(json.dumps(cfg))[2]


def test_round_trip_and_agreement_with_safetensors_package(tmp_path):
    tensors = {"a": torch.randn(3, 5), "b": torch.randn(7).to(torch.bfloat16), "c": torch.arange(6, dtype=torch.int32)}
    p = str(tmp_path / "x.safetensors")
    write_safetensors(p, tensors)
    f = SafetensorsFile(p)
    for k, v in tensors.items():
        assert torch.equal(f.tensor(k), v)
    from safetensors import safe_open      # an independent reader agrees
    with safe_open(p, framework="pt") as g:
        for k, v in tensors.items():
            assert torch.equal(g.get_tensor(k), v)


def _raw_file(path, header: dict, payload: bytes, pad_header=True):
    blob = json.dumps(header).encode()
    with open(path, "wb") as fh:
        fh.write(struct.pack("<Q", len(blob)))
        fh.write(blob)
        fh.write(payload)


def test_container_checks(tmp_path):
    p = str(tmp_path / "bad.safetensors")
    ok = {"a": {"dtype": "F32", "shape": [2], "data_offsets": [0, 8]}}
    _raw_file(p, ok, b"\0" * 8)
    SafetensorsFile(p)
    _raw_file(p, ok, b"\0" * 12)
    with pytest.raises(SafetensorsError, match="trailing"):
        SafetensorsFile(p)
    _raw_file(p, {"a": {"dtype": "F32", "shape": [3], "data_offsets": [0, 8]}}, b"\0" * 8)
    with pytest.raises(SafetensorsError, match="needs 12 bytes"):
        SafetensorsFile(p)
    _raw_file(p, {"a": {"dtype": "F32", "shape": [2], "data_offsets": [0, 8]},
                  "b": {"dtype": "F32", "shape": [2], "data_offsets": [4, 12]}}, b"\0" * 12)
    with pytest.raises(SafetensorsError, match="overlaps"):
        SafetensorsFile(p)
    _raw_file(p, {"a": {"dtype": "F32", "shape": [1], "data_offsets": [0, 4]},
                  "b": {"dtype": "F32", "shape": [1], "data_offsets": [8, 12]}}, b"\0" * 12)
    with pytest.raises(SafetensorsError, match="gap"):
        SafetensorsFile(p)
    with open(p, "wb") as fh:
        fh.write(struct.pack("<Q", 40) + b'{"a":1,')
    with pytest.raises(SafetensorsError):
        SafetensorsFile(p)
    with open(p, "wb") as fh:       # duplicate names
        blob = b'{"a":{"dtype":"F32","shape":[1],"data_offsets":[0,4]},"a":{"dtype":"F32","shape":[1],"data_offsets":[0,4]}}'
        fh.write(struct.pack("<Q", len(blob)) + blob + b"\0" * 4)
    with pytest.raises(SafetensorsError, match="duplicate"):
        SafetensorsFile(p)
    with open(p, "wb") as fh:
        fh.write(struct.pack("<Q", 1 << 40))
    with pytest.raises(SafetensorsError, match="exceeds"):
        SafetensorsFile(p)
    with open(p, "wb") as fh:       # a name that is not UTF-8 (found by mutating headers at random)
        blob = b'{"a\xd9\x20":{"dtype":"F32","shape":[1],"data_offsets":[0,4]}}'
        fh.write(struct.pack("<Q", len(blob)) + blob + b"\0" * 4)
    with pytest.raises(SafetensorsError, match="UTF-8"):
        SafetensorsFile(p)
    # an empty tensor whose other dimensions no strides can span
    _raw_file(p, {"a": {"dtype": "F32", "shape": [0, 1 << 62, 8], "data_offsets": [0, 0]}}, b"")
    with pytest.raises(SafetensorsError, match="needs"):
        SafetensorsFile(p)
    _raw_file(p, {"a": {"dtype": "F32", "shape": [0, 1 << 40], "data_offsets": [0, 0]}}, b"")
    assert SafetensorsFile(p).tensor("a").shape == (0, 1 << 40)


def test_index_and_shard_path_escape(tmp_path):
    d = str(tmp_path)
    write_safetensors(os.path.join(d, "s1.safetensors"), {"a": torch.zeros(2)})
    write_safetensors(os.path.join(d, "s2.safetensors"), {"b": torch.ones(2)})
    with open(os.path.join(d, "model.safetensors.index.json"), "w") as fh:
        json.dump({"weight_map": {"a": "s1.safetensors", "b": "s2.safetensors"}}, fh)
    src = TensorSource(d)
    assert sorted(src.names()) == ["a", "b"] and torch.equal(src.tensor("b"), torch.ones(2))
    with open(os.path.join(d, "model.safetensors.index.json"), "w") as fh:
        json.dump({"weight_map": {"a": "../s1.safetensors"}}, fh)
    with pytest.raises(SafetensorsError, match="leaves the folder"):
        TensorSource(d)
    with open(os.path.join(d, "model.safetensors.index.json"), "w") as fh:
        json.dump({"weight_map": {"a": "s1.safetensors"}}, fh)
    TensorSource(d)   # s2 is not named: fine, it is not a shard of this model
    # what a damaged or hostile index can hold, each refused with the reader's own error
    for text, why in (('{"weight_map": {"a": "s1.safetensors\\u0000"}}', "leaves the folder"),
                      ('{"weight_map": {"a": "s2.safetensors", "a": "s1.safetensors"}}', "duplicate"),
                      ("[" * 100000, "malformed index"),
                      ('{"weight_map": [1, 2]}', "malformed index"),
                      ('{"weight_map": {"a": 7}}', "leaves the folder")):
        with open(os.path.join(d, "model.safetensors.index.json"), "w") as fh:
            fh.write(text)
        with pytest.raises(SafetensorsError, match=why):
            TensorSource(d)


def test_index_total_size_must_agree_with_the_shards(tmp_path):
    """metadata.total_size is accepted as the tensors' bytes, or as those plus the shards'
    headers, as an integer or a whole float; anything else is refused
    (crates/model/package/src/storage/source.rs:160-181)."""
    d = str(tmp_path)
    write_safetensors(os.path.join(d, "s1.safetensors"), {"a": torch.zeros(2)})
    write_safetensors(os.path.join(d, "s2.safetensors"), {"b": torch.ones(3, dtype=torch.bfloat16)})
    wm = {"a": "s1.safetensors", "b": "s2.safetensors"}
    payload = 2 * 4 + 3 * 2
    headers = sum(SafetensorsFile(os.path.join(d, f)).data_start for f in ("s1.safetensors", "s2.safetensors"))

    def index(meta):
        with open(os.path.join(d, "model.safetensors.index.json"), "w") as fh:
            json.dump({"metadata": meta, "weight_map": wm}, fh)

    for good in (payload, float(payload), payload + headers):
        index({"total_size": good})
        assert sorted(TensorSource(d).names()) == ["a", "b"]
    index({})                                            # some exporters omit it
    TensorSource(d)
    for bad, why in ((payload + 2, "disagrees"), (payload - 1, "disagrees"), (0, "empty"), (payload + 0.5, "invalid"),
                     ("14", "invalid"), (True, "invalid")):
        index({"total_size": bad})
        with pytest.raises(SafetensorsError, match=why):
            TensorSource(d)


def test_random_weights_in_memory_equal_the_written_folder(tmp_path):
    """One seed, one model: the tensors made directly (the path `--random-weights S` takes,
    there on the device) are the ones a folder written with the same seed loads as."""
    from inferloop_b200.config.registry import read_model_config
    from inferloop_b200.models.decoder import declare_weights
    from inferloop_b200.weights.loader import load_weights
    from inferloop_b200.weights.random_init import random_weights, standard_normal
    d = make_model_folder(str(tmp_path / "m"), CONFIG_B, 11)
    _, _, spec = read_model_config(json.dumps(CONFIG_B))
    decls = declare_weights(spec)
    for dtype in (torch.float32, torch.bfloat16):
        made = random_weights(decls, 11, dtype, "cpu")
        loaded, _ = load_weights(d, decls, spec.weight_prefixes, spec.embedding_name, dtype, "cpu")
        assert set(made) == set(loaded)
        for name in made:
            assert made[name].dtype == loaded[name].dtype and torch.equal(made[name], loaded[name]), name
    # the stream: element i depends on (key, i) alone, and looks like a standard normal
    x = standard_normal(99, 400_000, "cpu")
    assert torch.equal(x[1000:2000], standard_normal(99, 2000, "cpu")[1000:])
    assert abs(float(x.mean())) < 0.01 and abs(float(x.std()) - 1.0) < 0.01
    assert abs(float((x.abs() > 2).float().mean()) - 0.0455) < 0.003 and float(x.abs().max()) < 4.7


def test_random_model_is_seeded_by_name(tmp_path):
    d1 = make_model_folder(str(tmp_path / "m1"), CONFIG_B, 1)
    d2 = make_model_folder(str(tmp_path / "m2"), CONFIG_B, 1)
    d3 = make_model_folder(str(tmp_path / "m3"), CONFIG_B, 2)
    s1, s2, s3 = TensorSource(d1), TensorSource(d2), TensorSource(d3)
    names = s1.names()
    assert "lm_head.weight" in names and "model.layers.2.self_attn.q_proj.bias" in names
    for n in names:
        assert torch.equal(s1.tensor(n), s2.tensor(n))
    assert not torch.equal(s1.tensor("model.embed_tokens.weight"), s3.tensor("model.embed_tokens.weight"))
    w = s1.tensor("model.layers.0.mlp.down_proj.weight")
    assert abs(w.std().item() - 0.02) < 0.002 and abs(w.mean().item()) < 0.002
    n = s1.tensor("model.norm.weight")
    assert abs(n.mean().item() - 1.0) < 0.05 and 0.05 < n.std().item() < 0.15
    # one tensor's values do not depend on which other tensors exist
    decl = WeightDecl("layers.0.mlp.down_proj.weight", (96, 224))
    assert torch.equal(random_tensor(decl, 1, torch.float32), w)
    tied = TensorSource(make_model_folder(str(tmp_path / "a"), CONFIG_A, 0))
    assert "lm_head.weight" not in tied.names()


def _rewrite(folder, edit):
    src = TensorSource(folder)
    tensors = {n: src.tensor(n).clone() for n in src.names()}
    src.close()
    edit(tensors)
    write_safetensors(os.path.join(folder, "model.safetensors"), tensors)


def test_one_error_lists_missing_unexpected_and_wrong_shapes(tmp_path):
    d = make_model_folder(str(tmp_path / "m"), CONFIG_B, 1)
    spec = _spec(CONFIG_B)
    decls = declare_weights(spec)
    load_weights(d, decls, spec.weight_prefixes, spec.embedding_name, torch.float32, "cpu")

    def edit(t):
        del t["model.layers.1.mlp.up_proj.weight"]
        del t["model.norm.weight"]
        t["model.layers.9.extra.weight"] = torch.zeros(2)
        t["model.layers.0.self_attn.q_proj.weight"] = torch.zeros(10, 96)
        t["model.layers.0.self_attn.k_norm.weight"] = torch.zeros(32, dtype=torch.int32)
    _rewrite(d, edit)
    with pytest.raises(WeightError) as e:
        load_weights(d, decls, spec.weight_prefixes, spec.embedding_name, torch.float32, "cpu")
    err = e.value
    assert sorted(err.missing) == ["model.layers.1.mlp.up_proj.weight", "model.norm.weight"]
    assert err.unexpected == ["model.layers.9.extra.weight"]
    assert err.wrong_shape == [("model.layers.0.self_attn.q_proj.weight", (192, 96), (10, 96))]
    assert err.wrong_dtype and err.wrong_dtype[0][0] == "model.layers.0.self_attn.k_norm.weight"
    text = str(err)
    for piece in ("missing (2)", "unexpected (1)", "wrong shape (1)", "expected [192, 96], found [10, 96]"):
        assert piece in text


def test_unexpected_alone_and_prefixes_and_nonfinite(tmp_path):
    d = make_model_folder(str(tmp_path / "m"), CONFIG_A, 0)
    spec = _spec(CONFIG_A)
    decls = declare_weights(spec)
    _rewrite(d, lambda t: t.__setitem__("model.rotary.inv_freq", torch.zeros(4)))
    with pytest.raises(WeightError, match="unexpected"):
        load_weights(d, decls, spec.weight_prefixes, spec.embedding_name, torch.float32, "cpu")
    w, ignored = load_weights(d, decls, spec.weight_prefixes, spec.embedding_name, torch.float32, "cpu",
                              allow_unexpected=True)
    assert ignored == ["model.rotary.inv_freq"] and "embed_tokens.weight" in w

    def to_nested(t):
        t.pop("model.rotary.inv_freq")
        for k in list(t):
            t["model.language_model." + k[len("model."):]] = t.pop(k)
    _rewrite(d, to_nested)
    w, _ = load_weights(d, decls, spec.weight_prefixes, spec.embedding_name, torch.bfloat16, "cpu")
    assert w["embed_tokens.weight"].dtype == torch.bfloat16          # matrices follow the compute dtype
    assert w["norm.weight"].dtype == torch.float32                   # a 32-bit vector stays 32-bit
    _rewrite(d, lambda t: t["model.language_model.norm.weight"].__setitem__(0, float("nan")))
    with pytest.raises(WeightError, match="non-finite"):
        load_weights(d, decls, spec.weight_prefixes, spec.embedding_name, torch.float32, "cpu")
    _rewrite(d, lambda t: [t.pop(k) for k in list(t) if k.endswith("embed_tokens.weight")])
    with pytest.raises(WeightError, match="anchor"):
        load_weights(d, decls, spec.weight_prefixes, spec.embedding_name, torch.float32, "cpu")
