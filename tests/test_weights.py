"""Safetensors reading/writing, strict loading and the random-weights mode (no GPU)."""
import json

import pytest
import torch

import qwen_inference_lab_b200.models  # noqa: F401
from qwen_inference_lab_b200.config import Qwen3Config, registry
from qwen_inference_lab_b200.weights import (SafetensorsError, SafetensorsFile, WeightError, load_weights,
                                             write_model_folder, write_safetensors)
from tests.tiny_configs import TINY_A, TINY_B, TINY_C, tiny_weights


def folder_with(tmp_path, cfg, weights, shards=1):
    (tmp_path / "config.json").write_text(json.dumps(cfg))
    names = sorted(weights)
    for i in range(shards):
        part = {n: weights[n] for n in names[i::shards]}
        write_safetensors(tmp_path / f"model-{i:05d}-of-{shards:05d}.safetensors", part)
    return tmp_path


def build(cfg):
    return registry.lookup(cfg).build(Qwen3Config.from_dict(cfg))


def test_safetensors_round_trip_and_compatibility(tmp_path):
    tensors = {"a": torch.randn(3, 5), "b": torch.randn(7).to(torch.bfloat16), "c": torch.arange(6, dtype=torch.int64).reshape(2, 3),
               "empty": torch.zeros(0, 4)}
    write_safetensors(tmp_path / "x.safetensors", tensors, metadata={"format": "pt"})
    with SafetensorsFile(tmp_path / "x.safetensors") as f:
        assert sorted(f.keys()) == sorted(tensors) and f.metadata == {"format": "pt"}
        for name, value in tensors.items():
            assert f.dtype(name) == value.dtype and torch.equal(f.tensor(name).clone(), value)
    safetensors = pytest.importorskip("safetensors.torch")
    loaded = safetensors.load_file(str(tmp_path / "x.safetensors"))      # files we write are standard
    assert all(torch.equal(loaded[n], v) for n, v in tensors.items())
    safetensors.save_file({k: v for k, v in tensors.items()}, str(tmp_path / "y.safetensors"))
    with SafetensorsFile(tmp_path / "y.safetensors") as f:              # and we read standard files
        assert all(torch.equal(f.tensor(n).clone(), v) for n, v in tensors.items())


def test_truncated_and_garbled_files(tmp_path):
    write_safetensors(tmp_path / "x.safetensors", {"a": torch.randn(64, 64)})
    data = (tmp_path / "x.safetensors").read_bytes()
    (tmp_path / "short.safetensors").write_bytes(data[:len(data) // 2])
    with pytest.raises(SafetensorsError, match="truncated|beyond"):
        SafetensorsFile(tmp_path / "short.safetensors")
    (tmp_path / "junk.safetensors").write_bytes(b"\xff" * 64)
    with pytest.raises(SafetensorsError):
        SafetensorsFile(tmp_path / "junk.safetensors")
    (tmp_path / "tiny.safetensors").write_bytes(b"abc")
    with pytest.raises(SafetensorsError):
        SafetensorsFile(tmp_path / "tiny.safetensors")


@pytest.mark.parametrize("cfg,seed,shards", [(TINY_A, 0, 1), (TINY_B, 1, 3), (TINY_C, 2, 2)])
def test_strict_loading_of_single_and_sharded_folders(tmp_path, cfg, seed, shards):
    weights = tiny_weights(cfg, seed, torch.bfloat16)
    model = build(cfg)
    load_weights(model, folder_with(tmp_path, cfg, weights, shards), device="cpu", dtype=torch.bfloat16)
    attention = model.layers[0].mixer
    stacked = torch.cat([weights[f"model.layers.0.self_attn.{n}_proj.weight"] for n in "qkv"])
    assert torch.equal(attention.qkv._weight(), stacked) and attention.qkv._weight().dtype == torch.bfloat16
    assert torch.equal(model.final_norm.weight.data, weights["model.norm.weight"])
    if cfg["attention_bias"]:
        assert torch.equal(attention.out._bias(), weights["model.layers.0.self_attn.o_proj.bias"])
    model32 = build(cfg)
    load_weights(model32, tmp_path, device="cpu", dtype=torch.float32)
    assert all(p.data is None or p.data.dtype == torch.float32 for p in model32.all_named_params().values())
    assert model32.layers[0].mixer.qkv._weight().dtype == torch.float32


def test_tensors_are_cast_to_the_run_dtype_unless_32_bits_are_asked_for(tmp_path):
    """The reference casts every tensor as it loads it (qil/model.py:197); a folder stored in float32 must not
    send a bfloat16 run to the 32-bit kernels behind the user's back."""
    weights = tiny_weights(TINY_A, 0, torch.bfloat16)
    exact = weights["model.norm.weight"].float() + 1e-4                                  # not representable in bfloat16
    weights["model.norm.weight"] = exact
    weights["model.layers.0.mlp.down_proj.weight"] = weights["model.layers.0.mlp.down_proj.weight"].float()
    weights["model.layers.1.input_layernorm.weight"] = weights["model.layers.1.input_layernorm.weight"].half()
    folder = folder_with(tmp_path, TINY_A, weights)
    model = build(TINY_A)
    load_weights(model, folder, device="cpu", dtype=torch.bfloat16)
    params = model.all_named_params()
    assert all(p.data is None or p.data.dtype == torch.bfloat16 for p in params.values())
    assert torch.equal(params["model.norm.weight"].data, exact.to(torch.bfloat16))
    assert model.layers[0].feed_forward.down._weight().dtype == torch.bfloat16
    # asked for by a parameter ...
    model = build(TINY_A)
    model.final_norm.weight.keep_32bit = True
    load_weights(model, folder, device="cpu", dtype=torch.bfloat16)
    params = model.all_named_params()
    assert params["model.norm.weight"].data.dtype == torch.float32 and torch.equal(params["model.norm.weight"].data, exact)
    assert params["model.layers.1.input_layernorm.weight"].data.dtype == torch.bfloat16
    assert model.layers[0].feed_forward.down._weight().dtype == torch.bfloat16
    # ... or for the whole folder
    model = build(TINY_A)
    load_weights(model, folder, device="cpu", dtype=torch.bfloat16, keep_stored_32bit=True)
    params = model.all_named_params()
    assert params["model.norm.weight"].data.dtype == torch.float32
    assert model.layers[0].feed_forward.down._weight().dtype == torch.float32
    assert params["model.layers.1.input_layernorm.weight"].data.dtype == torch.bfloat16       # float16 in the file
    assert params["model.embed_tokens.weight"].data.dtype == torch.bfloat16


def test_tied_tensors_are_compared_after_the_cast(tmp_path):
    weights = tiny_weights(TINY_A, 0, torch.bfloat16)
    embedding = weights["model.embed_tokens.weight"].float()
    weights["model.embed_tokens.weight"] = embedding * (1 + 1e-4)   # differs in float32, the same once cast to bfloat16
    weights["lm_head.weight"] = embedding
    folder = folder_with(tmp_path, TINY_A, weights)
    load_weights(build(TINY_A), folder, device="cpu", dtype=torch.bfloat16)
    with pytest.raises(WeightError, match="tied tensors with different values"):
        load_weights(build(TINY_A), folder, device="cpu", dtype=torch.float32)


def test_tied_weights_either_name_or_both_if_equal(tmp_path):
    weights = tiny_weights(TINY_A, 0, torch.bfloat16)
    assert "lm_head.weight" not in weights
    for variant in ("embed", "head", "both"):
        w = dict(weights)
        if variant in ("head", "both"):
            w["lm_head.weight"] = w["model.embed_tokens.weight"].clone()
        if variant == "head":
            del w["model.embed_tokens.weight"]
        folder = tmp_path / variant
        folder.mkdir()
        model = build(TINY_A)
        load_weights(model, folder_with(folder, TINY_A, w), device="cpu", dtype=torch.bfloat16)
        assert model.head.weight is model.embedding.weight
        assert torch.equal(model.embedding.weight.data, weights["model.embed_tokens.weight"])


def test_one_error_lists_everything_that_is_wrong(tmp_path):
    weights = tiny_weights(TINY_B, 1, torch.bfloat16)
    del weights["model.norm.weight"]
    del weights["model.layers.2.mlp.up_proj.weight"]
    weights["model.layers.0.self_attn.q_norm.weight"] = torch.ones(5, dtype=torch.bfloat16)
    weights["model.layers.0.self_attn.rotary.inv_freq"] = torch.ones(4)
    weights["unknown.weight"] = torch.ones(1)
    with pytest.raises(WeightError) as caught:
        load_weights(build(TINY_B), folder_with(tmp_path, TINY_B, weights), device="cpu", dtype=torch.bfloat16)
    message = str(caught.value)
    for fragment in ("model.norm.weight", "model.layers.2.mlp.up_proj.weight", "unknown.weight", "inv_freq",
                     "model.layers.0.self_attn.q_norm.weight: file has [5], model needs [32]"):
        assert fragment in message
    assert message.count("missing tensors (2)") == 1


@pytest.mark.parametrize("corruption", ["missing", "shape", "extra", "tied", "duplicate", "none", "truncated"])
def test_corrupt_folders_fail_loudly(tmp_path, corruption):
    weights = tiny_weights(TINY_A, 0, torch.bfloat16)
    shards = 1
    if corruption == "missing":
        del weights["model.layers.1.self_attn.k_norm.weight"]
    elif corruption == "shape":
        weights["model.norm.weight"] = torch.ones(1, dtype=torch.bfloat16)
    elif corruption == "extra":
        weights["unknown.weight"] = torch.ones(1)
    elif corruption == "tied":
        weights["lm_head.weight"] = weights["model.embed_tokens.weight"] + 1
    folder = folder_with(tmp_path, TINY_A, weights, shards)
    if corruption == "duplicate":
        write_safetensors(folder / "zz-extra.safetensors", {"model.norm.weight": weights["model.norm.weight"]})
    elif corruption == "none":
        for f in folder.glob("*.safetensors"):
            f.unlink()
    elif corruption == "truncated":
        path = next(folder.glob("*.safetensors"))
        path.write_bytes(path.read_bytes()[:-100])
    with pytest.raises(WeightError):
        load_weights(build(TINY_A), folder, device="cpu", dtype=torch.bfloat16)


def test_random_weights_mode_writes_a_loadable_folder(tmp_path):
    config = Qwen3Config.from_dict(TINY_B)
    write_model_folder(config, 5, tmp_path / "m")
    again = write_model_folder(config, 5, tmp_path / "n")
    other = write_model_folder(config, 6, tmp_path / "o")
    assert (tmp_path / "m" / "model.safetensors").read_bytes() == (again / "model.safetensors").read_bytes()
    assert (tmp_path / "m" / "model.safetensors").read_bytes() != (other / "model.safetensors").read_bytes()
    entry, read_back = registry.read_model_config(tmp_path / "m")
    assert read_back == config
    model = entry.build(read_back)
    load_weights(model, tmp_path / "m", device="cpu", dtype=torch.bfloat16)
    with SafetensorsFile(tmp_path / "m" / "model.safetensors") as f:
        matrix = f.tensor("model.layers.1.mlp.gate_proj.weight").float()
        norm = f.tensor("model.layers.1.input_layernorm.weight").float()
        assert f.dtype("model.embed_tokens.weight") == torch.bfloat16
    assert abs(matrix.std().item() - 0.02) < 0.002 and abs(matrix.mean().item()) < 0.002
    assert abs(norm.mean().item() - 1.0) < 0.03 and 0.02 < norm.std().item() < 0.08
    tied = write_model_folder(Qwen3Config.from_dict(TINY_A), 1, tmp_path / "t")
    with SafetensorsFile(tied / "model.safetensors") as f:
        assert "lm_head.weight" not in f.keys()
