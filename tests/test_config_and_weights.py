"""Configuration, registry and weight loading (no GPU)."""

from __future__ import annotations

import json

import pytest
import torch
from safetensors.torch import load_file, save_file

import tiny_configs
import vllm_from_scratch_b200 as engine
from vllm_from_scratch_b200.parts import DecoderModel


def test_config_reads_keys_and_defaults():
    config = engine.Qwen3Config.from_dict(tiny_configs.TINY_B)
    assert (config.num_hidden_layers, config.hidden_size, config.num_attention_heads,
            config.num_key_value_heads, config.head_dim) == (3, 96, 6, 2, 32)
    assert config.q_width == 192 != config.hidden_size
    assert config.rms_norm_eps == 1e-5 and config.rope_theta == 1e6 and not config.tie_word_embeddings
    assert config.layer_windows == (None, None, None)
    minimal = {k: v for k, v in tiny_configs.TINY_A.items()
               if k not in ("num_key_value_heads", "head_dim", "rms_norm_eps", "rope_theta", "tie_word_embeddings")}
    config = engine.Qwen3Config.from_dict(minimal)
    assert config.num_key_value_heads == 4 and config.head_dim == 16
    assert config.rms_norm_eps == 1e-6 and config.rope_theta == 10000.0 and not config.tie_word_embeddings
    nested = dict(tiny_configs.TINY_A, rope_parameters={"rope_theta": 5e5, "rope_type": "default"})
    assert engine.Qwen3Config.from_dict(nested).rope_theta == 5e5
    assert engine.Qwen3Config.from_dict(config.to_dict()) == config


def test_config_windows_and_round_trip():
    config = engine.Qwen3Config.from_dict(tiny_configs.TINY_C)
    assert config.layer_windows == (None, 24, 24, None)
    assert engine.Qwen3Config.from_dict(config.to_dict()) == config
    by_count = dict(tiny_configs.TINY_C)
    del by_count["layer_types"]
    by_count["max_window_layers"] = 3
    assert engine.Qwen3Config.from_dict(by_count).layer_windows == (None, None, None, 24)


@pytest.mark.parametrize("change,match", [
    ({"hidden_act": "gelu"}, "silu"), ({"attention_bias": True}, "attention_bias"),
    ({"num_key_value_heads": 3}, "multiple"), ({"head_dim": 15}, "even"),
    ({"rope_parameters": {"rope_type": "yarn"}}, "rope_type"), ({"architectures": ["A", "B"]}, "exactly one"),
    ({"vocab_size": 0}, "positive"), ({"rms_norm_eps": 0.0}, "rms_norm_eps"),
])
def test_config_refuses(change, match):
    with pytest.raises(engine.ConfigError, match=match):
        engine.Qwen3Config.from_dict(dict(tiny_configs.TINY_A, **change))


def test_config_missing_keys_listed_together():
    raw = {k: v for k, v in tiny_configs.TINY_A.items() if k not in ("vocab_size", "intermediate_size")}
    with pytest.raises(engine.ConfigError, match="vocab_size.*intermediate_size|intermediate_size.*vocab_size"):
        engine.Qwen3Config.from_dict(raw)


def test_registry():
    assert "Qwen3ForCausalLM" in engine.registered_architectures()
    with pytest.raises(ValueError, match="Qwen3ForCausalLM"):
        engine.get_architecture("NoSuchModel")
    entry, config = engine.load_model_config(tiny_configs.TINY_A)
    spec = entry.build_spec(config)
    assert len(spec.layers) == 2 and [e.layer for e in spec.schedule] == [0, 1]
    assert spec.layers[1].mixer.params["num_kv_heads"] == 2
    assert spec.layers[0].norms["mixer"].params["eps"] == 1e-6
    assert set(spec.layers[0].norms) == {"mixer", "feed_forward"}


def _model(raw, dtype=torch.float32):
    entry, config = engine.load_model_config(raw)
    return DecoderModel(entry.build_spec(config), dtype, "cpu")


def test_random_weights_folder_loads(tmp_path):
    folder = engine.write_random_model(tiny_configs.TINY_B, 3, tmp_path / "m", dtype=torch.bfloat16)
    assert json.loads((folder / "config.json").read_text())["hidden_size"] == 96
    stored = load_file(str(folder / "model.safetensors"))
    assert stored["model.layers.2.self_attn.q_proj.weight"].shape == (192, 96)
    again = engine.write_random_model(tiny_configs.TINY_B, 3, tmp_path / "n", dtype=torch.bfloat16)
    assert torch.equal(stored["lm_head.weight"], load_file(str(again / "model.safetensors"))["lm_head.weight"])
    for dtype in (torch.bfloat16, torch.float32):
        model = _model(tiny_configs.TINY_B, dtype)
        engine.load_weights(model, folder)
        attention = model.layers[0].mixer
        assert attention.qkv.shape == ((6 + 2 * 2) * 32, 96) and attention.qkv.dtype == dtype
        assert torch.equal(attention.qkv[:192].float(), stored["model.layers.0.self_attn.q_proj.weight"].float())
        assert torch.equal(attention.qkv[192:256].float(), stored["model.layers.0.self_attn.k_proj.weight"].float())
        assert attention.q_norm.dtype == torch.float32            # vectors stay 32-bit
        feed_forward = model.layers[1].feed_forward
        assert torch.equal(feed_forward.gate_up[160:].float(), stored["model.layers.1.mlp.up_proj.weight"].float())
        assert model.output_head.weight is not model.embedding.weight


def test_tied_model_ignores_a_stored_head(tmp_path):
    folder = engine.write_random_model(tiny_configs.TINY_A, 1, tmp_path / "m", dtype=torch.float32)
    tensors = load_file(str(folder / "model.safetensors"))
    assert "lm_head.weight" not in tensors
    tensors["lm_head.weight"] = torch.zeros(256, 64)
    save_file(tensors, str(folder / "model.safetensors"))
    model = _model(tiny_configs.TINY_A)
    engine.load_weights(model, folder)
    assert model.output_head.weight is model.embedding.weight


def test_one_error_lists_every_mismatch(tmp_path):
    folder = engine.write_random_model(tiny_configs.TINY_B, 1, tmp_path / "m", dtype=torch.float32)
    tensors = load_file(str(folder / "model.safetensors"))
    del tensors["model.layers.1.mlp.up_proj.weight"]
    del tensors["model.norm.weight"]
    tensors["model.layers.7.mlp.up_proj.weight"] = torch.zeros(2, 2)
    tensors["model.layers.0.self_attn.k_proj.weight"] = torch.zeros(32, 96)
    tensors["lm_head.weight"] = torch.zeros(512, 96)
    save_file(tensors, str(folder / "model.safetensors"))
    with pytest.raises(engine.WeightLoadError) as caught:
        engine.load_weights(_model(tiny_configs.TINY_B), folder)
    error = caught.value
    assert error.missing == ["model.layers.1.mlp.up_proj.weight", "model.norm.weight"]
    assert error.unexpected == ["model.layers.7.mlp.up_proj.weight"]
    assert [name for name, _, _ in error.wrong_shape] == ["lm_head.weight", "model.layers.0.self_attn.k_proj.weight"]
    text = str(error)
    for needle in ("missing (2)", "unexpected (1)", "wrong shape (2)", "[32, 96], expected [64, 96]"):
        assert needle in text


def test_missing_files_and_other_formats(tmp_path):
    with pytest.raises(FileNotFoundError):
        engine.load_weights(_model(tiny_configs.TINY_A), tmp_path / "nowhere")
    (tmp_path / "empty").mkdir()
    with pytest.raises(FileNotFoundError, match="model.safetensors"):
        engine.load_weights(_model(tiny_configs.TINY_A), tmp_path / "empty")
    (tmp_path / "empty" / "pytorch_model.bin").write_bytes(b"")
    with pytest.raises(NotImplementedError, match="safetensors"):
        engine.load_weights(_model(tiny_configs.TINY_A), tmp_path / "empty")


def test_sharded_checkpoint(tmp_path):
    folder = engine.write_random_model(tiny_configs.TINY_A, 1, tmp_path / "m", dtype=torch.float32)
    tensors = load_file(str(folder / "model.safetensors"))
    names = sorted(tensors)
    half = len(names) // 2
    save_file({n: tensors[n] for n in names[:half]}, str(folder / "model-00001-of-00002.safetensors"))
    save_file({n: tensors[n] for n in names[half:]}, str(folder / "model-00002-of-00002.safetensors"))
    (folder / "model.safetensors").unlink()
    weight_map = {n: ("model-00001-of-00002.safetensors" if i < half else "model-00002-of-00002.safetensors")
                  for i, n in enumerate(names)}
    (folder / "model.safetensors.index.json").write_text(json.dumps({"weight_map": weight_map}))
    model = _model(tiny_configs.TINY_A)
    engine.load_weights(model, folder)
    assert torch.equal(model.embedding.weight, tensors["model.embed_tokens.weight"])


def test_engine_refuses_to_run_without_a_gpu_kernel():
    """No CPU fallback: a tensor that is not on a CUDA device is refused loudly."""
    import vllm_from_scratch_b200.kernels as kernels
    with pytest.raises(kernels.KernelError, match="CUDA device"):
        kernels.silu_mul(torch.zeros(2, 8), torch.zeros(2, 4))
    if not torch.cuda.is_available():
        with pytest.raises(RuntimeError, match="no CUDA device"):
            engine.ModelRunner.from_folder("nowhere", "float32", 16, 4, 2, device="cuda")
