import json
import os

import numpy as np
import pytest
import torch

from garuda_b200.config import build_model
from garuda_b200.weights import (write_random_model, load_model, WeightError, SafetensorsFolder,
                                 write_safetensors, random_weights, SafetensorsError)
from garuda_b200.weights.safetensors_io import SafetensorsFile
from tests.helpers import TINY_A, TINY_B, model_dir
from tests.plain.cpu_ops import CpuOps


def test_safetensors_round_trip(tmp_path):
    t = {"a": torch.randn(3, 5), "b": torch.randn(7).bfloat16(), "c": torch.arange(6, dtype=torch.int32).view(2, 3)}
    p = str(tmp_path / "x.safetensors")
    write_safetensors(p, t)
    f = SafetensorsFile(p)
    for k, v in t.items():
        assert f.entries[k].shape == tuple(v.shape)
        assert torch.equal(f.tensor(k), v)


def test_safetensors_agrees_with_the_reference_reader(tmp_path):
    st = pytest.importorskip("safetensors.torch")
    t = {"w": torch.randn(4, 4), "v": torch.randn(9).bfloat16()}
    p = str(tmp_path / "y.safetensors")
    write_safetensors(p, t)
    back = st.load_file(p)
    assert all(torch.equal(back[k], t[k]) for k in t)


def test_truncated_file_is_refused(tmp_path):
    p = str(tmp_path / "z.safetensors")
    write_safetensors(p, {"w": torch.randn(8, 8)})
    data = open(p, "rb").read()
    open(p, "wb").write(data[:-16])
    with pytest.raises(SafetensorsError, match="outside the file"):
        SafetensorsFile(p)


def test_random_weights_are_seeded_per_tensor():
    a = random_weights(TINY_A, 0)
    b = random_weights(TINY_A, 0)
    c = random_weights(TINY_A, 1)
    assert all(torch.equal(a[k], b[k]) for k in a)
    assert not torch.equal(a["model.layers.0.mlp.up_proj.weight"], c["model.layers.0.mlp.up_proj.weight"])
    # a tensor's values do not depend on which other tensors exist
    bigger = random_weights(dict(TINY_A, num_hidden_layers=3), 0)
    assert torch.equal(a["model.layers.1.self_attn.q_proj.weight"],
                       bigger["model.layers.1.self_attn.q_proj.weight"])
    assert abs(float(a["model.embed_tokens.weight"].std()) - 0.02) < 2e-3
    assert torch.equal(a["model.norm.weight"], torch.ones(64))
    n = random_weights(TINY_B, 1, norm_init=("normal_about_one", 0.1))["model.norm.weight"]
    assert abs(float(n.mean()) - 1) < 0.05 and 0.05 < float(n.std()) < 0.15
    assert "lm_head.weight" not in random_weights(TINY_B, 1)           # tied


def test_folder_has_config_and_weights(tmp_path):
    d = write_random_model(str(tmp_path / "m"), TINY_A, 0)
    assert sorted(os.listdir(d)) == ["config.json", "model.safetensors"]
    assert json.load(open(os.path.join(d, "config.json")))["hidden_size"] == 64


def test_dtypes_after_loading(tmp_path):
    ops = CpuOps()
    d = write_random_model(str(tmp_path / "m"), TINY_A, 0, store_dtype=torch.float32)
    _, model = load_model(d, ops, torch.bfloat16, "cpu")
    assert model.embedding.dtype == torch.bfloat16
    assert model.blocks[0].mixer.w_qkv.dtype == torch.bfloat16
    assert model.blocks[0].mixer_norm.weight.dtype == torch.float32      # stored in 32-bit: stays so
    d2 = write_random_model(str(tmp_path / "m2"), TINY_A, 0, store_dtype=torch.bfloat16)
    _, model = load_model(d2, ops, torch.bfloat16, "cpu")
    assert model.blocks[0].mixer_norm.weight.dtype == torch.bfloat16
    _, model = load_model(d2, ops, torch.float32, "cpu")
    assert model.embedding.dtype == torch.float32 and model.final_norm.weight.dtype == torch.float32


def test_tied_head_is_the_embedding_table(tmp_path):
    d = write_random_model(str(tmp_path / "m"), TINY_B, 1)
    _, model = load_model(d, CpuOps(), torch.float32, "cpu")
    assert model.head.data_ptr() == model.embedding.data_ptr()     # garuda/src/llama/mod.rs:2035-2060


def test_one_error_lists_missing_unexpected_and_wrong_shapes(tmp_path):
    d = str(tmp_path / "m")
    os.makedirs(d)
    t = random_weights(TINY_A, 0)
    del t["model.layers.1.mlp.down_proj.weight"]
    del t["model.norm.weight"]
    t["model.layers.0.self_attn.rotary_emb.inv_freq"] = torch.zeros(8)
    t["model.layers.0.self_attn.k_proj.weight"] = torch.zeros(16, 64)     # should be [32, 64]
    json.dump(TINY_A, open(os.path.join(d, "config.json"), "w"))
    write_safetensors(os.path.join(d, "model.safetensors"), t)
    with pytest.raises(WeightError) as e:
        load_model(d, CpuOps(), torch.float32, "cpu")
    msg = str(e.value)
    assert "model.layers.1.mlp.down_proj.weight" in msg and "model.norm.weight" in msg
    assert "rotary_emb.inv_freq" in msg
    assert "k_proj.weight: file has [16, 64], model needs [32, 64]" in msg
    assert e.value.missing and e.value.unexpected and e.value.wrong_shape


def test_missing_head_only_allowed_when_tied(tmp_path):
    d = str(tmp_path / "m")
    os.makedirs(d)
    t = random_weights(TINY_A, 0)
    del t["lm_head.weight"]
    json.dump(TINY_A, open(os.path.join(d, "config.json"), "w"))
    write_safetensors(os.path.join(d, "model.safetensors"), t)
    with pytest.raises(WeightError, match="lm_head.weight"):
        load_model(d, CpuOps(), torch.float32, "cpu")


def test_non_finite_values_are_refused(tmp_path):
    d = str(tmp_path / "m")
    os.makedirs(d)
    t = random_weights(TINY_A, 0)
    t["model.norm.weight"][3] = float("nan")
    json.dump(TINY_A, open(os.path.join(d, "config.json"), "w"))
    write_safetensors(os.path.join(d, "model.safetensors"), t)
    with pytest.raises(WeightError, match="not finite"):
        load_model(d, CpuOps(), torch.float32, "cpu")


def test_sharded_folder(tmp_path):
    d = str(tmp_path / "m")
    os.makedirs(d)
    t = random_weights(TINY_A, 0)
    names = list(t)
    half = len(names) // 2
    write_safetensors(os.path.join(d, "model-00001-of-00002.safetensors"), {n: t[n] for n in names[:half]})
    write_safetensors(os.path.join(d, "model-00002-of-00002.safetensors"), {n: t[n] for n in names[half:]})
    wm = {n: ("model-00001-of-00002.safetensors" if i < half else "model-00002-of-00002.safetensors")
          for i, n in enumerate(names)}
    json.dump({"weight_map": wm}, open(os.path.join(d, "model.safetensors.index.json"), "w"))
    json.dump(TINY_A, open(os.path.join(d, "config.json"), "w"))
    _, model = load_model(d, CpuOps(), torch.float32, "cpu")
    assert torch.equal(model.embedding, t["model.embed_tokens.weight"])
