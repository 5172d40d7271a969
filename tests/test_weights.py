"""Weights: safetensors reading and writing, binding by name, the one error, random-weights folders."""
import json

import pytest
import torch

import plain_llama
import tiny
from cuca_b200.config.registry import build_spec
from cuca_b200.models.model import Model
from cuca_b200.weights import safetensors_io as st
from cuca_b200.weights.loader import FolderSource, WeightsError
from cuca_b200.weights.random_init import write_random_model


def test_round_trip_keeps_dtypes(tmp_path):
    tensors = {"a": torch.randn(3, 5).to(torch.bfloat16), "b": torch.randn(7), "ids": torch.arange(6).view(2, 3)}
    st.write_safetensors(tmp_path / "model.safetensors", tensors)
    idx = st.folder_index(tmp_path)
    a, b, ids = (st.read_tensor(idx[k]) for k in ("a", "b", "ids"))
    assert a.dtype == torch.bfloat16 and torch.equal(a, tensors["a"])      # bfloat16 stays bfloat16
    assert b.dtype == torch.float32 and torch.equal(b, tensors["b"])       # 32-bit stays 32-bit
    assert ids.dtype == torch.int32 and torch.equal(ids.long(), tensors["ids"])  # integer tables as int32
    # the oracle's own reader sees the same bytes
    theirs = plain_llama.read_safetensors(tmp_path / "model.safetensors")
    assert torch.equal(theirs["a"], tensors["a"])


def test_random_folder_is_reproducible_and_complete(tmp_path):
    d1 = write_random_model(tmp_path / "m1", tiny.TINY_B, seed=2)
    d2 = write_random_model(tmp_path / "m2", tiny.TINY_B, seed=2)
    d3 = write_random_model(tmp_path / "m3", tiny.TINY_B, seed=3)
    assert (d1 / "model.safetensors").read_bytes() == (d2 / "model.safetensors").read_bytes()
    assert (d1 / "model.safetensors").read_bytes() != (d3 / "model.safetensors").read_bytes()
    assert json.loads((d1 / "config.json").read_text())["num_hidden_layers"] == 3
    cfg, w = plain_llama.load_model_dir(d1)
    assert "lm_head.weight" not in w                      # tied
    assert sum(t.numel() for t in w.values()) == 400032
    assert torch.all(w["model.norm.weight"].float() == 1.0)             # the default: norm weights 1.0
    q = w["model.layers.0.self_attn.q_proj.weight"].float()
    assert q.shape == (96, 96) and abs(float(q.std()) - 0.02) < 2e-3 and abs(float(q.mean())) < 2e-3
    Model(build_spec(cfg)).check_weights(FolderSource(d1))


def test_one_error_lists_missing_unexpected_and_wrong_shapes(tmp_path):
    d = write_random_model(tmp_path / "m", tiny.TINY_A, seed=0)
    w = plain_llama.read_safetensors(d / "model.safetensors")
    del w["model.layers.1.mlp.up_proj.weight"]
    del w["model.norm.weight"]
    w["model.layers.0.self_attn.k_proj.weight"] = torch.zeros(16, 64, dtype=torch.bfloat16)
    w["model.layers.0.mlp.extra.weight"] = torch.zeros(2, 2)
    w["model.layers.0.self_attn.rotary_emb.inv_freq"] = torch.zeros(8)  # skipped, as the reference does
    st.write_safetensors(d / "model.safetensors", w)
    with pytest.raises(WeightsError) as e:
        Model(build_spec(tiny.TINY_A)).check_weights(FolderSource(d))
    err = e.value
    assert err.missing == ["model.layers.1.mlp.up_proj.weight", "model.norm.weight"]
    assert err.unexpected == ["model.layers.0.mlp.extra.weight"]
    assert err.wrong_shape == [("model.layers.0.self_attn.k_proj.weight", (32, 64), (16, 64))]
    text = str(err)
    for piece in ("missing tensors (2)", "unexpected tensors (1)", "wrong shapes (1)", "expected [32, 64] found [16, 64]"):
        assert piece in text


def test_tied_checkpoint_may_carry_lm_head_and_wrapper_prefixes(tmp_path):
    d = write_random_model(tmp_path / "m", tiny.TINY_B, seed=2)
    w = plain_llama.read_safetensors(d / "model.safetensors")
    w["lm_head.weight"] = w["model.embed_tokens.weight"].clone()
    renamed = {("model.language_model." + k[len("model."):] if k.startswith("model.") else k): v for k, v in w.items()}
    st.write_safetensors(d / "model.safetensors", renamed)
    Model(build_spec(tiny.TINY_B)).check_weights(FolderSource(d))


def test_sharded_folder_and_duplicate_names(tmp_path):
    d = write_random_model(tmp_path / "m", tiny.TINY_A, seed=0)
    w = plain_llama.read_safetensors(d / "model.safetensors")
    names = sorted(w)
    (d / "model.safetensors").unlink()
    st.write_safetensors(d / "model-00001-of-00002.safetensors", {n: w[n] for n in names[::2]})
    st.write_safetensors(d / "model-00002-of-00002.safetensors", {n: w[n] for n in names[1::2]})
    Model(build_spec(tiny.TINY_A)).check_weights(FolderSource(d))
    st.write_safetensors(d / "model-00003.safetensors", {names[0]: w[names[0]]})
    with pytest.raises(st.SafetensorsError, match="both"):
        FolderSource(d)


def test_truncated_file_is_refused(tmp_path):
    d = write_random_model(tmp_path / "m", tiny.TINY_A, seed=0)
    raw = (d / "model.safetensors").read_bytes()
    (d / "model.safetensors").write_bytes(raw[: len(raw) // 2])
    with pytest.raises(st.SafetensorsError):
        FolderSource(d)


def test_no_gpu_means_a_loud_error_not_a_fallback():
    if torch.cuda.is_available():
        pytest.skip("a CUDA device is present")
    from cuca_b200.kernels.library import KernelLibraryError
    from cuca_b200.runtime import Runtime
    with pytest.raises(KernelLibraryError, match="no CPU path"):
        Runtime("cuda:0", torch.float32)


def test_random_values_hang_on_seed_name_and_element_only():
    from cuca_b200.weights.loader import host_normal, tensor_key
    key = tensor_key(7, "model.layers.0.mlp.up_proj.weight")
    whole = host_normal(key, 0, 200_000, 0.0, 0.02)
    piece = host_normal(key, 123_457, 1000, 0.0, 0.02)
    assert (piece == whole[123_457:124_457]).all()                       # a piece equals that part of the whole
    assert abs(float(whole.mean())) < 2e-4 and abs(float(whole.std()) - 0.02) < 2e-4
    assert float(abs(whole).max()) > 3.5 * 0.02                          # tails are there
    other = host_normal(tensor_key(7, "model.layers.1.mlp.up_proj.weight"), 0, 1000, 0.0, 0.02)
    assert not (other == whole[:1000]).any()


def test_switched_on_biases_are_drawn_and_norm_weights_can_differ(tmp_path):
    """A configuration with `attention_bias` gets its eight bias tensors, non-zero; the tests' folders carry norm
    weights that differ from 1 and from one another, so that a swapped or dropped norm weight shows in the logits."""
    d = tiny.write_tiny(tmp_path / "c", "C")
    _, w = plain_llama.load_model_dir(d)
    biases = sorted(n for n in w if n.endswith(".bias"))
    assert len(biases) == 8 and all(float(w[n].float().abs().max()) > 0.01 for n in biases)
    norms = [w[n].float() for n in sorted(w) if "norm" in n]
    assert len(norms) == 5
    for i, a in enumerate(norms):
        assert float((a - 1).abs().mean()) > 0.05
        for b in norms[i + 1:]:
            assert not torch.equal(a, b)
    Model(build_spec(tiny.TINY_C)).check_weights(FolderSource(d))
    a_cfg, a_w = plain_llama.load_model_dir(tiny.write_tiny(tmp_path / "a", "A"))
    assert not any(n.endswith(".bias") for n in a_w)                       # no biases unless switched on
