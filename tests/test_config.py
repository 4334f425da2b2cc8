"""Configuration: config.json keys -> typed config -> model description; the registry; refusals."""
import copy

import pytest

from fusezap_core_b200.config import (ARCHITECTURES, DenseDecoderConfig, EngineConfig, ModelSpec, PartSpec, ScheduleEntry,
                                      describe, register_architecture)
from tiny_configs import TINY_LLAMA, TINY_QWEN2, TINY_WINDOW


def test_keys_and_defaults():
    c = DenseDecoderConfig.from_hf({"hidden_size": 64, "intermediate_size": 128, "num_hidden_layers": 2,
                                    "num_attention_heads": 4, "vocab_size": 100})
    assert (c.model_type, c.num_key_value_heads, c.head_dim, c.rms_norm_eps, c.max_position_embeddings, c.rope_theta) == \
        ("llama", 4, 16, 1e-6, 4096, 10000.0)
    assert c.rope_scaling.kind == "default" and not c.tie_word_embeddings and c.layer_windows == ()
    c = DenseDecoderConfig.from_hf(TINY_LLAMA)
    assert c.rope_scaling.kind == "llama3" and c.rope_scaling.original_max_position_embeddings == 32
    assert c.rope_scaling.factor == 8.0 and c.rms_norm_eps == 1e-5
    c = DenseDecoderConfig.from_hf({**TINY_QWEN2, "eos_token_id": [5, 9], "bos_token_id": 1})
    assert c.eos_token_ids == (5, 9) and c.bos_token_id == 1 and c.tie_word_embeddings and c.writes_qkv_bias
    assert DenseDecoderConfig.from_hf({**TINY_QWEN2, "eos_token_id": 7}).eos_token_ids == (7,)


def test_rope_parameters_form():
    c = copy.deepcopy(TINY_LLAMA)
    rs = c.pop("rope_scaling"); theta = c.pop("rope_theta")
    c["rope_parameters"] = {"rope_theta": theta, **rs}
    assert DenseDecoderConfig.from_hf(c) == DenseDecoderConfig.from_hf(TINY_LLAMA)
    c["rope_parameters"] = {"rope_theta": 5.0, "rope_type": "default"}
    assert DenseDecoderConfig.from_hf(c).rope_theta == 5.0 and DenseDecoderConfig.from_hf(c).rope_scaling.kind == "default"


def test_windows():
    c = DenseDecoderConfig.from_hf(TINY_WINDOW)
    assert c.layer_windows == (12, 0, 12)
    w = copy.deepcopy(TINY_WINDOW); del w["layer_types"]
    assert DenseDecoderConfig.from_hf(w).layer_windows == (12, 12, 12)
    w["use_sliding_window"] = False
    assert DenseDecoderConfig.from_hf(w).layer_windows == ()
    assert DenseDecoderConfig.from_hf({**TINY_QWEN2, "sliding_window": 4096}).layer_windows == ()   # key alone does nothing
    spec = c.spec()
    assert [l.mixer.params["window"] for l in spec.layers] == [12, 0, 12]


def test_round_trip_through_config_json():
    for cfg in (TINY_LLAMA, TINY_QWEN2, TINY_WINDOW):
        c = DenseDecoderConfig.from_hf(cfg)
        assert DenseDecoderConfig.from_hf(c.to_hf()) == c


@pytest.mark.parametrize("patch,err,match", [
    ({"num_key_value_heads": 3}, ValueError, "multiple"),
    ({"head_dim": 15}, ValueError, "even"),
    ({"hidden_act": "gelu"}, NotImplementedError, "hidden_act"),
    ({"rope_scaling": {"rope_type": "yarn", "factor": 2}}, NotImplementedError, "yarn"),
    ({"rope_scaling": {"rope_type": "llama3"}}, ValueError, "factor"),
    ({"rope_scaling": {"rope_type": "llama3", "factor": 2.0}}, ValueError, "original_max_position"),
    ({"vocab_size": 0}, ValueError, "vocab_size"),
    ({"rms_norm_eps": 0.0}, ValueError, "rms_norm_eps"),
    ({"use_sliding_window": True, "sliding_window": 8, "layer_types": ["full_attention"]}, ValueError, "layer_types"),
])
def test_bad_configs(patch, err, match):
    with pytest.raises(err, match=match):
        DenseDecoderConfig.from_hf({**TINY_LLAMA, **patch})


def test_missing_key_is_named():
    c = copy.deepcopy(TINY_LLAMA); del c["intermediate_size"]
    with pytest.raises(ValueError, match="intermediate_size"):
        DenseDecoderConfig.from_hf(c)


def test_registry():
    typed, spec = describe(TINY_QWEN2)
    assert isinstance(typed, DenseDecoderConfig) and isinstance(spec, ModelSpec) and spec.tie_embeddings
    assert len(spec.layers) == 3 and [e.layer for e in spec.schedule] == [0, 1, 2]
    assert spec.layers[0].mixer.kind == "gqa_attention" and spec.layers[0].ffn.kind == "swiglu"
    assert spec.layers[1].prefix == "model.layers.1."
    with pytest.raises(NotImplementedError, match="mamba.*llama.*qwen2"):
        describe({**TINY_QWEN2, "model_type": "mamba"})
    assert {"llama", "qwen2"} <= set(ARCHITECTURES)
    register_architecture("unit_test_arch", lambda c: describe({**c, "model_type": "llama"}))
    try:
        assert describe({**TINY_LLAMA, "model_type": "unit_test_arch"})[1].architecture == "llama"
    finally:
        del ARCHITECTURES["unit_test_arch"]


def test_schedule_validation():
    _, spec = describe(TINY_LLAMA)
    import dataclasses
    ok = dataclasses.replace(spec, schedule=(ScheduleEntry(0, 0), ScheduleEntry(1, 1), ScheduleEntry(0, 2), ScheduleEntry(1, 1, write_cache=False)))
    ok.validate()
    for bad, match in (((ScheduleEntry(0, 0), ScheduleEntry(1, 0)), "both write"),
                       ((ScheduleEntry(0, 0, write_cache=False),), "before any entry wrote"),
                       ((ScheduleEntry(5, 0),), "names layer 5"), ((), "empty")):
        with pytest.raises(ValueError, match=match):
            dataclasses.replace(spec, schedule=bad).validate()


def test_engine_config():
    e = EngineConfig(max_num_seqs=8, max_prefill_tokens=64)
    assert e.token_budget == 72 and EngineConfig(max_num_batched_tokens=100).token_budget == 100
    for bad in (dict(dtype="float16"), dict(block_size=0), dict(num_blocks=-1), dict(prefill_first=-1), dict(graph_rows=-1),
                dict(prefill_every=0), dict(max_prefill_seqs=0), dict(mixed_prefill_tokens=-3), dict(max_model_len=0)):
        with pytest.raises(ValueError):
            EngineConfig(**bad)
    assert EngineConfig().graph_rows == 256 and EngineConfig(graph_rows=0).graph_rows == 0
    assert EngineConfig(dtype="auto").dtype == "bfloat16"
    r = EngineConfig(max_num_seqs=4).resolved(model_max_len=512)
    assert (r.max_model_len, r.max_prefill_tokens, r.max_prefill_seqs) == (512, 512, 4)
    assert EngineConfig().resolved(8192).max_prefill_tokens == 2048
    with pytest.raises(ValueError, match="exceeds the length"):
        EngineConfig(max_model_len=1024).resolved(512)


def test_the_command_line_is_generated_from_the_engine_config():
    """One source of defaults: a flag that is not given leaves the field at `EngineConfig`'s own default, every field
    that names a flag has one, and the engine, the scheduler and the command line read the same object."""
    import dataclasses
    from fusezap_core_b200.cli import build_parser
    ap = build_parser()
    a = ap.parse_args(["generate", "--random", "tiny-llama", "--prompt-ids", "1,2"])
    assert EngineConfig.from_arguments(a) == EngineConfig()
    a = ap.parse_args(["generate", "--random", "tiny-llama", "--max-num-seqs", "3", "--prefill-first", "2", "--no-lookahead",
                       "--max-num-batched-tokens", "24", "--mixed-prefill-tokens", "5", "--prefill-every", "2",
                       "--max-prefill-seqs", "1", "--dtype", "float32", "--block-size", "8", "--profile"])
    c = EngineConfig.from_arguments(a)
    assert (c.max_num_seqs, c.prefill_first, c.lookahead, c.max_num_batched_tokens, c.mixed_prefill_tokens, c.prefill_every,
            c.max_prefill_seqs, c.dtype, c.block_size, c.profile, c.cuda_graphs) == (3, 2, False, 24, 5, 2, 1, "float32", 8, True, True)
    flags = {x for act in ap._subparsers._group_actions[0].choices["generate"]._actions for x in act.option_strings}
    for f in dataclasses.fields(EngineConfig):
        assert f.metadata["flag"] in flags, f.name


def test_sampling_params_say_who_picks_the_token():
    """Greedy, temperature, top-k and top-p rows are picked by the device kernels; a repetition penalty needs the
    request's history and goes to the host (fusezap/serve/sampling.py:6-10 gives the order of the filters)."""
    from fusezap_core_b200 import SamplingParams
    greedy, temp = SamplingParams(), SamplingParams(temperature=0.7)
    assert greedy.greedy and greedy.on_device and not greedy.filtered
    assert not temp.greedy and temp.on_device and not temp.filtered
    assert SamplingParams(temperature=0.7, top_k=1).greedy and not SamplingParams(temperature=0.7, top_k=1).filtered
    assert SamplingParams(temperature=0.7, top_k=40).filtered and SamplingParams(temperature=0.7, top_p=0.9).filtered
    assert not SamplingParams(top_k=40).filtered, "temperature 0 is greedy whatever the filters say"
    pen = SamplingParams(temperature=0.7, top_k=40, repetition_penalty=1.2)
    assert pen.filtered and not pen.on_device
    for bad in (dict(max_tokens=0), dict(temperature=-1.0), dict(top_p=0.0), dict(top_p=1.5), dict(top_k=-1), dict(repetition_penalty=0.0)):
        with pytest.raises(ValueError):
            SamplingParams(**bad)


def test_generation_config_adds_stop_ids(tmp_path):
    """The end-of-sequence ids of generation_config.json are merged with config.json's (fusezap/serve/models/llama.py:443-451)."""
    import json
    from fusezap_core_b200.config import describe, read_config_json
    from tiny_configs import TINY_QWEN2
    cfg = dict(TINY_QWEN2, eos_token_id=7)
    (tmp_path / "config.json").write_text(json.dumps(cfg))
    assert describe(read_config_json(str(tmp_path)))[1].eos_token_ids == (7,)
    (tmp_path / "generation_config.json").write_text(json.dumps({"eos_token_id": [9, 7, 3]}))
    assert describe(read_config_json(str(tmp_path)))[1].eos_token_ids == (3, 7, 9)
    (tmp_path / "generation_config.json").write_text(json.dumps({"eos_token_id": 11}))
    assert describe(read_config_json(str(tmp_path)))[1].eos_token_ids == (7, 11)
    (tmp_path / "generation_config.json").write_text(json.dumps({"temperature": 0.7}))
    assert describe(read_config_json(str(tmp_path)))[1].eos_token_ids == (7,)
