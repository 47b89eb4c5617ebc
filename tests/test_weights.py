"""Weights: the container, loading by name with one error for everything wrong, and the
random-weights mode (CPU)."""
import json
import os

import pytest
import torch

from braidinfer_b200.models import architecture_for
from braidinfer_b200.weights import (RoundedWeightsWarning, UnexpectedTensorsWarning, WeightsError, load_tensors, open_model_folder, save_file, tensor_specs_of,
                                     write_random_model, SafetensorsError)
from tiny import TINY_A, TINY_B, TINY_C, make_folder, read_weights


def specs_for(d):
    arch = architecture_for(d)
    return tensor_specs_of(arch.build_spec(arch.config_from_dict(d)))


def test_random_model_folder_has_config_and_every_tensor(tmp_path):
    folder = make_folder(tmp_path, "B")
    assert json.load(open(os.path.join(folder, "config.json")))["hidden_size"] == 96
    found = open_model_folder(folder)
    specs = specs_for(TINY_B)
    assert set(found) == set(specs)
    f, _ = found["model.layers.2.mlp.down_proj.weight"]
    dt, shape = f.info("model.layers.2.mlp.down_proj.weight")
    assert dt == torch.bfloat16 and shape == (96, 256)
    assert f.info("model.layers.0.self_attn.k_proj.weight")[1] == (2 * 32, 96)


def test_random_weights_depend_on_seed_only(tmp_path):
    a = write_random_model(TINY_A, str(tmp_path / "x"), 5)
    b = write_random_model(TINY_A, str(tmp_path / "y"), 5)
    c = write_random_model(TINY_A, str(tmp_path / "z"), 6)
    ra = open(os.path.join(a, "model.safetensors"), "rb").read()
    assert ra == open(os.path.join(b, "model.safetensors"), "rb").read()
    assert ra != open(os.path.join(c, "model.safetensors"), "rb").read()
    w = read_weights(a)
    assert abs(w["model.norm.weight"].mean().item() - 1.0) < 0.02        # 1 + N(0, 0.02)
    assert abs(w["model.embed_tokens.weight"].std().item() - 0.02) < 0.003


def test_loader_agrees_with_the_tests_own_reader(tmp_path):
    folder = make_folder(tmp_path, "A")
    mine = read_weights(folder)
    got = load_tensors(folder, specs_for(TINY_A), torch.bfloat16, "cpu")
    assert set(got) == set(mine)
    for n in mine:
        assert got[n].dtype == torch.bfloat16
        assert torch.equal(got[n].double(), mine[n])
    got32 = load_tensors(folder, specs_for(TINY_A), torch.float32, "cpu")
    assert all(t.dtype == torch.float32 for t in got32.values())
    assert torch.equal(got32["lm_head.weight"].double(), mine["lm_head.weight"])


def test_a_tensor_stored_in_32_bits_stays_so(tmp_path):
    folder = make_folder(tmp_path, "A")
    tensors = {n: f.tensor(k).clone() for n, (f, k) in open_model_folder(folder).items()}
    tensors["model.norm.weight"] = tensors["model.norm.weight"].float() + 1e-4     # not a bfloat16 value
    save_file(tensors, os.path.join(folder, "model.safetensors"))
    got = load_tensors(folder, specs_for(TINY_A), torch.bfloat16, "cpu")
    assert got["model.norm.weight"].dtype == torch.float32
    assert torch.equal(got["model.norm.weight"], tensors["model.norm.weight"])
    assert got["model.layers.0.input_layernorm.weight"].dtype == torch.bfloat16


def test_one_error_lists_missing_unexpected_and_wrong_shapes(tmp_path):
    folder = make_folder(tmp_path, "B")
    tensors = {n: f.tensor(k).clone() for n, (f, k) in open_model_folder(folder).items()}
    del tensors["model.layers.1.mlp.up_proj.weight"]
    del tensors["model.norm.weight"]
    tensors["model.layers.9.extra.weight"] = torch.zeros(3, dtype=torch.bfloat16)
    tensors["model.layers.0.self_attn.q_proj.weight"] = torch.zeros(10, 96, dtype=torch.bfloat16)
    save_file(tensors, os.path.join(folder, "model.safetensors"))
    with pytest.raises(WeightsError) as e:
        load_tensors(folder, specs_for(TINY_B), torch.bfloat16, "cpu")
    err = e.value                                      # what stops the load and what does not, in one message
    assert sorted(err.missing) == ["model.layers.1.mlp.up_proj.weight", "model.norm.weight"]
    assert err.unexpected == ["model.layers.9.extra.weight"]
    assert err.wrong_shape == [("model.layers.0.self_attn.q_proj.weight", (10, 96), (192, 96))]
    text = str(err)
    for word in ("missing", "unexpected", "wrong shape", "model.norm.weight", "model.layers.9.extra.weight",
                 "[10, 96]", "[192, 96]"):
        assert word in text


def test_a_tensor_nobody_asks_for_is_a_warning_that_lists_it(tmp_path):
    # older exports of this family store a table of rotary frequencies beside every attention layer
    folder = make_folder(tmp_path, "A")
    tensors = {n: f.tensor(k).clone() for n, (f, k) in open_model_folder(folder).items()}
    extra = ["model.layers.0.self_attn.rotary_emb.inv_freq", "model.layers.1.self_attn.rotary_emb.inv_freq"]
    for n in extra:
        tensors[n] = torch.ones(8, dtype=torch.float32)
    save_file(tensors, os.path.join(folder, "model.safetensors"))
    with pytest.warns(UnexpectedTensorsWarning) as rec:
        got = load_tensors(folder, specs_for(TINY_A), torch.bfloat16, "cpu")
    mine = [r for r in rec if r.category is UnexpectedTensorsWarning]
    assert len(mine) == 1 and all(n in str(mine[0].message) for n in extra)
    assert set(got) == set(specs_for(TINY_A))
    with pytest.raises(WeightsError) as e:
        load_tensors(folder, specs_for(TINY_A), torch.bfloat16, "cpu", strict=True)
    assert sorted(e.value.unexpected) == extra and not e.value.missing


def test_float16_weights_are_rounded_with_a_word_and_kept_whole_in_float32(tmp_path):
    import warnings
    folder = make_folder(tmp_path, "A")
    tensors = {n: f.tensor(k).clone() for n, (f, k) in open_model_folder(folder).items()}
    name = "model.layers.0.mlp.up_proj.weight"
    half = (tensors[name].float() * 1.001).to(torch.float16)          # values with more than 8 mantissa bits
    tensors[name] = half
    save_file(tensors, os.path.join(folder, "model.safetensors"))
    with pytest.warns(RoundedWeightsWarning) as rec:
        got = load_tensors(folder, specs_for(TINY_A), torch.bfloat16, "cpu")
    mine = [r for r in rec if r.category is RoundedWeightsWarning]
    assert len(mine) == 1 and name in str(mine[0].message)
    assert got[name].dtype == torch.bfloat16 and torch.equal(got[name], half.to(torch.bfloat16))
    with warnings.catch_warnings():
        warnings.simplefilter("error", RoundedWeightsWarning)
        got32 = load_tensors(folder, specs_for(TINY_A), torch.float32, "cpu")
    assert torch.equal(got32[name], half.float())


def test_tensors_under_one_more_prefix_are_found(tmp_path):
    # a model wrapped into a larger one stores "language_model.model.layers.0..." and so on; a draft head beside it
    # ("mtp.") must not be taken for the model
    folder = make_folder(tmp_path, "A")
    mine = read_weights(folder)
    tensors = {"language_model." + n: f.tensor(k).clone() for n, (f, k) in open_model_folder(folder).items()}
    tensors["mtp.model.layers.0.input_layernorm.weight"] = torch.zeros(64, dtype=torch.bfloat16)
    save_file(tensors, os.path.join(folder, "model.safetensors"))
    with pytest.warns(UnexpectedTensorsWarning):
        got = load_tensors(folder, specs_for(TINY_A), torch.bfloat16, "cpu")
    assert set(got) == set(mine) and all(torch.equal(got[n].double(), mine[n]) for n in mine)
    # one tensor missing under the prefix: the error names it by the name that was asked for
    del tensors["language_model.model.norm.weight"]
    save_file(tensors, os.path.join(folder, "model.safetensors"))
    with pytest.raises(WeightsError) as e:
        load_tensors(folder, specs_for(TINY_A), torch.bfloat16, "cpu")
    assert e.value.missing == ["model.norm.weight"]


def test_tied_head_needs_no_head_tensor(tmp_path):
    folder = make_folder(tmp_path, "C")
    assert "lm_head.weight" not in open_model_folder(folder)
    load_tensors(folder, specs_for(TINY_C), torch.bfloat16, "cpu")
    # with the key absent from config.json, the head is tied exactly when no tensor is stored
    d = dict(TINY_C)
    del d["tie_word_embeddings"]
    specs = specs_for(d)
    assert specs["lm_head.weight"].optional
    load_tensors(folder, specs, torch.bfloat16, "cpu")


def test_sharded_folder_and_bad_files(tmp_path):
    folder = make_folder(tmp_path, "A")
    tensors = {n: f.tensor(k).clone() for n, (f, k) in open_model_folder(folder).items()}
    names = list(tensors)
    os.remove(os.path.join(folder, "model.safetensors"))
    half = len(names) // 2
    save_file({n: tensors[n] for n in names[:half]}, os.path.join(folder, "model-00001-of-00002.safetensors"))
    save_file({n: tensors[n] for n in names[half:]}, os.path.join(folder, "model-00002-of-00002.safetensors"))
    wm = {n: ("model-00001-of-00002.safetensors" if i < half else "model-00002-of-00002.safetensors")
          for i, n in enumerate(names)}
    json.dump({"weight_map": wm}, open(os.path.join(folder, "model.safetensors.index.json"), "w"))
    got = load_tensors(folder, specs_for(TINY_A), torch.bfloat16, "cpu")
    assert torch.equal(got[names[-1]], tensors[names[-1]])
    with pytest.raises(FileNotFoundError):
        open_model_folder(str(tmp_path / "empty"))
    bad = tmp_path / "bad"
    bad.mkdir()
    (bad / "model.safetensors").write_bytes(b"\xff" * 4)
    with pytest.raises(SafetensorsError):
        open_model_folder(str(bad))
