"""Configuration parsing, the registry, safetensors round trip, and the loader's one
error that lists missing tensors, unexpected tensors and wrong shapes."""

import json
import os
import shutil
import tempfile

import pytest
import torch

from tiny_models import TINY_A, TINY_B, model_dir

from kv_cache_optimization_for_llm_b200.config import ConfigError, EngineConfig, LlamaConfig
from kv_cache_optimization_for_llm_b200.models.spec import expected_weights
from kv_cache_optimization_for_llm_b200.registry import known_architectures, resolve_architecture
from kv_cache_optimization_for_llm_b200.weights import (WeightError, check_and_load, read_header, read_tensors,
                                                       write_tensors)
from kv_cache_optimization_for_llm_b200.weights.safetensors_io import SafetensorsError


def test_config_reads_every_key():
    c = LlamaConfig.from_dict(TINY_B)
    assert (c.vocab_size, c.hidden_size, c.intermediate_size, c.num_hidden_layers) == (1000, 192, 512, 3)
    assert (c.num_attention_heads, c.num_key_value_heads, c.head_dim) == (6, 1, 32)
    assert c.rms_norm_eps == 1e-6 and c.rope_theta == 500000.0 and not c.tie_word_embeddings
    assert c.rope_scaling.factor == 8.0 and c.rope_scaling.original_max_position_embeddings == 64
    assert c.eos_token_ids == (998, 999) and c.max_position_embeddings == 256
    assert LlamaConfig.from_dict(c.to_dict()) == c


def test_config_defaults_follow_the_format():
    d = {k: v for k, v in TINY_A.items() if k not in ("num_key_value_heads", "head_dim", "rope_theta")}
    c = LlamaConfig.from_dict(d)
    assert c.num_key_value_heads == 4 and c.head_dim == 16 and c.rope_theta == 10000.0
    assert c.rope_scaling is None and c.eos_token_ids == (255,)


@pytest.mark.parametrize("patch,word", [
    ({"vocab_size": None}, "vocab_size"),
    ({"num_key_value_heads": 3}, "multiple"),
    ({"head_dim": 15}, "even"),
    ({"hidden_act": "gelu"}, "hidden_act"),
    ({"attention_bias": True}, "bias"),
    ({"rope_scaling": {"rope_type": "yarn", "factor": 2.0}}, "yarn"),
    ({"rope_scaling": {"rope_type": "llama3", "factor": 8.0}}, "low_freq_factor"),
    ({"rms_norm_eps": 0.0}, "eps"),
    ({"architectures": []}, "architectures"),
])
def test_config_errors_name_the_key(patch, word):
    d = dict(TINY_A)
    d.update(patch)
    with pytest.raises(ConfigError, match=word):
        LlamaConfig.from_dict(d)


def test_registry_knows_llama_and_rejects_others():
    assert known_architectures() == ["LlamaForCausalLM"]
    arch = resolve_architecture(TINY_A)
    spec = arch.build_spec(arch.parse_config(TINY_A))
    assert len(spec.layers) == 2 and [e.layer for e in spec.schedule] == [0, 1]
    with pytest.raises(ValueError, match="MistralForCausalLM.*known: LlamaForCausalLM"):
        resolve_architecture({"architectures": ["MistralForCausalLM"]})


def test_expected_weights_tied_and_untied():
    for cfg, tied in ((TINY_A, True), (TINY_B, False)):
        arch = resolve_architecture(cfg)
        names = expected_weights(arch.build_spec(arch.parse_config(cfg)))
        assert ("lm_head.weight" in names) == (not tied)
        assert names["model.embed_tokens.weight"].shape == (cfg["vocab_size"], cfg["hidden_size"])
        assert names["model.layers.0.self_attn.k_proj.weight"].shape == (
            cfg["num_key_value_heads"] * cfg["head_dim"], cfg["hidden_size"])
        assert names["model.norm.weight"].kind == "vector"
        assert len(names) == 2 + 9 * cfg["num_hidden_layers"] + (0 if tied else 1)


def test_engine_config_dtype_names():
    assert EngineConfig(dtype="bf16").dtype == "bfloat16" and EngineConfig(dtype="fp32").dtype == "float32"
    with pytest.raises(ValueError):
        EngineConfig(dtype="float16")


def test_safetensors_round_trip_keeps_dtypes():
    d = tempfile.mkdtemp()
    t = {"a": torch.randn(3, 5), "b": torch.randn(7).to(torch.bfloat16), "c": torch.arange(6, dtype=torch.int32).view(2, 3)}
    write_tensors(os.path.join(d, "x.safetensors"), t)
    back = read_tensors(os.path.join(d, "x.safetensors"))
    for k in t:
        assert back[k].dtype == t[k].dtype and torch.equal(back[k], t[k])
    header, _ = read_header(os.path.join(d, "x.safetensors"))
    assert header["b"]["dtype"] == "BF16" and header["c"]["shape"] == [2, 3]


def test_truncated_file_is_reported():
    src = os.path.join(model_dir("tiny_a"), "model.safetensors")
    d = tempfile.mkdtemp()
    data = open(src, "rb").read()
    open(os.path.join(d, "model.safetensors"), "wb").write(data[:len(data) // 2])
    with pytest.raises(SafetensorsError, match="truncated"):
        read_header(os.path.join(d, "model.safetensors"))


def _folder_with(tensors, cfg=TINY_A):
    d = tempfile.mkdtemp()
    json.dump(cfg, open(os.path.join(d, "config.json"), "w"))
    write_tensors(os.path.join(d, "model.safetensors"), tensors)
    return d


def test_loader_lists_missing_unexpected_and_wrong_shapes_in_one_error():
    arch = resolve_architecture(TINY_A)
    want = expected_weights(arch.build_spec(arch.parse_config(TINY_A)))
    good = read_tensors(os.path.join(model_dir("tiny_a"), "model.safetensors"))
    assert set(check_and_load(model_dir("tiny_a"), want)) == set(want)
    bad = dict(good)
    del bad["model.layers.1.mlp.up_proj.weight"]
    del bad["model.norm.weight"]
    bad["lm_head.weight"] = torch.zeros(256, 64)                       # tied model: not wanted
    bad["model.layers.0.self_attn.q_proj.weight"] = torch.zeros(64, 63)  # wrong shape
    with pytest.raises(WeightError) as ei:
        check_and_load(_folder_with(bad), want)
    e = ei.value
    assert e.missing == ["model.layers.1.mlp.up_proj.weight", "model.norm.weight"]
    assert e.unexpected == ["lm_head.weight"]
    assert [w[0] for w in e.wrong_shape] == ["model.layers.0.self_attn.q_proj.weight"]
    msg = str(e)
    for word in ("missing (2)", "unexpected (1)", "wrong shape (1)", "stored (64, 63), wanted (64, 64)"):
        assert word in msg


def test_loader_keeps_stored_dtype_and_rejects_integer_matrices():
    arch = resolve_architecture(TINY_A)
    want = expected_weights(arch.build_spec(arch.parse_config(TINY_A)))
    t16 = check_and_load(model_dir("tiny_a", "bfloat16"), want)
    t32 = check_and_load(model_dir("tiny_a", "float32"), want)
    assert all(v.dtype == torch.bfloat16 for v in t16.values())
    assert all(v.dtype == torch.float32 for v in t32.values())
    bad = dict(t32)
    bad["model.norm.weight"] = torch.ones(64, dtype=torch.int32)
    with pytest.raises(WeightError, match="wrong dtype"):
        check_and_load(_folder_with(bad), want)


def test_random_weights_are_a_function_of_config_and_seed():
    from kv_cache_optimization_for_llm_b200.weights import write_random_model
    a, b, c = tempfile.mkdtemp(), tempfile.mkdtemp(), tempfile.mkdtemp()
    write_random_model(a, TINY_A, 3, 0.02)
    write_random_model(b, TINY_A, 3, 0.02)
    write_random_model(c, TINY_A, 4, 0.02)
    ta, tb, tc = (read_tensors(os.path.join(x, "model.safetensors")) for x in (a, b, c))
    assert all(torch.equal(ta[k], tb[k]) for k in ta)
    assert not torch.equal(ta["model.embed_tokens.weight"], tc["model.embed_tokens.weight"])
    assert abs(float(ta["model.norm.weight"].mean()) - 1.0) < 0.02
    assert abs(float(ta["model.embed_tokens.weight"].std()) - 0.02) < 0.002
    assert json.load(open(os.path.join(a, "config.json")))["hidden_size"] == 64
    for x in (a, b, c):
        shutil.rmtree(x)


def test_no_gpu_means_a_clear_error_not_a_fallback():
    if torch.cuda.is_available():
        pytest.skip("a GPU is visible")
    from kv_cache_optimization_for_llm_b200.engine.runner import ModelRunner
    with pytest.raises(RuntimeError, match="no CPU path"):
        ModelRunner(model_dir("tiny_a"), EngineConfig(dtype="float32", num_pages=4))


def test_checkpoint_in_two_shards_with_an_index():
    """model.safetensors.index.json names the file of every tensor; the loader reads all the
    files it names and reports a tensor that none of them holds like any other missing one."""
    arch = resolve_architecture(TINY_B)
    want = expected_weights(arch.build_spec(arch.parse_config(TINY_B)))
    good = read_tensors(os.path.join(model_dir("tiny_b"), "model.safetensors"))
    names = sorted(good)
    half = len(names) // 2
    shards = {"model-00001-of-00002.safetensors": names[:half], "model-00002-of-00002.safetensors": names[half:]}
    d = tempfile.mkdtemp()
    try:
        json.dump(TINY_B, open(os.path.join(d, "config.json"), "w"))
        for fname, ns in shards.items():
            write_tensors(os.path.join(d, fname), {n: good[n] for n in ns})
        index = {"metadata": {}, "weight_map": {n: f for f, ns in shards.items() for n in ns}}
        json.dump(index, open(os.path.join(d, "model.safetensors.index.json"), "w"))
        got = check_and_load(d, want)
        assert set(got) == set(want) and all(torch.equal(got[n], good[n]) for n in want)
        # the second shard loses a tensor
        lost = names[-1]
        write_tensors(os.path.join(d, "model-00002-of-00002.safetensors"), {n: good[n] for n in names[half:-1]})
        with pytest.raises(WeightError) as ei:
            check_and_load(d, want)
        assert ei.value.missing == [lost]
    finally:
        shutil.rmtree(d)


def test_layer_parts_are_a_mapping_and_nested_parts_are_found():
    """A layer names its parts as the block arrangement calls them; a part nested in another
    part's params, whatever its family and however deep, counts for the expected tensors and
    the kernel modules; a layer that names a part the block does not take is refused."""
    from kv_cache_optimization_for_llm_b200.engine.model import kernel_modules_of
    from kv_cache_optimization_for_llm_b200.models.spec import PartSpec, iter_parts
    arch = resolve_architecture(TINY_A)
    spec = arch.build_spec(arch.parse_config(TINY_A))
    fams = [f for f, _ in iter_parts(spec)]
    assert fams.count("position") == 2 and fams.count("mixer") == 2 and fams.count("norm") == 5
    assert set(spec.layers[0].parts) == {"mixer", "mixer_norm", "feed_forward", "ff_norm"}
    # a norm of its own inside the mixer's params, inside a list, under a key that is no family name
    inner = PartSpec("rmsnorm", {"size": 16, "eps": 1e-6}, {"weight": "model.layers.0.self_attn.q_norm.weight"},
                     family="norm")
    spec.layers[0].parts["mixer"].params["extras"] = [{"q_norm": inner}]
    assert ("norm", inner) in list(iter_parts(spec))
    assert expected_weights(spec)["model.layers.0.self_attn.q_norm.weight"].shape == (16,)
    assert "elementwise" in kernel_modules_of(spec, torch.float32)
    spec.layers[1].parts["post_norm"] = inner
    with pytest.raises(ValueError, match="not taken \\['post_norm'\\]"):
        list(iter_parts(spec))


def test_rotary_part_refuses_a_scaling_it_does_not_know():
    from kv_cache_optimization_for_llm_b200.parts.position import rope_inv_freq
    ok = rope_inv_freq(64, 500000.0, {"rope_type": "llama3", "factor": 8.0, "low_freq_factor": 1.0,
                                      "high_freq_factor": 4.0, "original_max_position_embeddings": 64})
    assert ok.shape == (32,)
    with pytest.raises(ValueError, match="yarn"):
        rope_inv_freq(64, 500000.0, {"rope_type": "yarn", "factor": 8.0})


def test_the_profiling_tool_and_the_bench_name_the_same_shapes():
    """``profiling --shape`` and ``bench.py`` build their random models from the same sizes."""
    import importlib.util
    import os
    from kv_cache_optimization_for_llm_b200.profiling import SHAPES
    spec = importlib.util.spec_from_file_location("bench", os.path.join(os.path.dirname(os.path.dirname(__file__)), "bench.py"))
    bench = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(bench)
    assert SHAPES["1b"] == bench.LLAMA_1B and SHAPES["3b"] == bench.LLAMA_3B and SHAPES["8b"] == bench.LLAMA_8B
    assert bench.WORKLOADS["serve3b"]["model"] == SHAPES["3b"] and bench.WORKLOADS["stress8b"]["model"] == SHAPES["8b"]
