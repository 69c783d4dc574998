"""Configuration, registry, safetensors container and weight errors (no GPU)."""
import json
import os
import struct
import tempfile

import pytest
import torch

from llmario_b200.config import (ConfigError, LayerCall, Qwen3Config, load_config, load_spec,
                                 register_architecture, registered_architectures,
                                 resolve_architecture)
from llmario_b200.weights import (SafetensorsError, SafetensorsFolder, WeightError,
                                  expected_tensors, load_weights, write_random_model,
                                  write_safetensors)
from util import TINY, config_json, model_dir


def test_config_reads_every_key():
    raw = config_json("B")
    c = Qwen3Config.from_dict(raw)
    assert (c.num_hidden_layers, c.hidden_size, c.num_attention_heads, c.num_key_value_heads,
            c.head_dim, c.intermediate_size, c.vocab_size) == (3, 96, 6, 3, 32, 160, 384)
    assert c.rope_theta == 1e6 and c.rms_norm_eps == 1e-5 and not c.tie_word_embeddings
    assert c.layer_windows == (None, None, None)
    spec = c.to_spec()
    m = spec.layers[0].mixer
    assert m["num_heads"] * m["head_dim"] == 192 != c.hidden_size
    assert m["scale"] == pytest.approx(32 ** -0.5)
    assert m["q_norm"]["eps"] == 1e-5 and spec.final_norm["eps"] == 1e-5
    assert m["position"]["theta"] == 1e6 and m["position"]["rot_dim"] == 32
    assert [c.layer for c in spec.run_order] == [0, 1, 2]
    assert Qwen3Config.from_dict(c.to_dict()) == c


def test_config_defaults_follow_reference():
    raw = config_json("A")
    for k in ("num_key_value_heads", "head_dim", "rope_theta", "max_position_embeddings"):
        raw.pop(k)
    c = Qwen3Config.from_dict(raw)
    assert c.num_key_value_heads == c.num_attention_heads       # safetensors.rs:593-596
    assert c.head_dim == c.hidden_size // c.num_attention_heads  # safetensors.rs:598-601
    assert c.rope_theta == 10000.0 and c.max_position_embeddings == 4096
    raw["rope_parameters"] = {"rope_theta": 777.0}
    assert Qwen3Config.from_dict(raw).rope_theta == 777.0


def test_config_window_layers():
    c = Qwen3Config.from_dict(config_json("C"))
    assert c.layer_windows == (None, 21, 21, None)
    spec = c.to_spec()
    assert [l.mixer["window"] for l in spec.layers] == [None, 21, 21, None]
    raw = config_json("C")
    raw.pop("layer_types")
    raw["max_window_layers"] = 3
    assert Qwen3Config.from_dict(raw).layer_windows == (None, None, None, 21)
    raw["use_sliding_window"] = False
    assert Qwen3Config.from_dict(raw).layer_windows == (None,) * 4


@pytest.mark.parametrize("change,word", [
    ({"num_attention_heads": 5}, "multiple"), ({"head_dim": 15}, "odd"),
    ({"attention_bias": True}, "attention_bias"), ({"hidden_act": "gelu"}, "hidden_act"),
    ({"rope_scaling": {"type": "yarn", "factor": 4}}, "rope_scaling"),
    ({"hidden_size": None}, "missing key 'hidden_size'"),
    ({"use_sliding_window": True, "sliding_window": None}, "sliding_window"),
])
def test_config_refuses(change, word):
    raw = config_json("A")
    raw.update(change)
    with pytest.raises(ConfigError, match=word):
        Qwen3Config.from_dict(raw)


def test_linear_rope_scaling_is_read():
    raw = config_json("A")
    raw["rope_scaling"] = {"type": "linear", "factor": 4.0}
    assert Qwen3Config.from_dict(raw).rope_freq_scale == 0.25      # arch.rs:319-324


def test_registry():
    assert "Qwen3ForCausalLM" in registered_architectures()
    assert resolve_architecture({"architectures": ["Qwen3ForCausalLM"]}) == "Qwen3ForCausalLM"
    assert resolve_architecture({"model_type": "qwen3"}) == "Qwen3ForCausalLM"
    with pytest.raises(ConfigError, match="unsupported architecture: LlamaForCausalLM.*Qwen3"):
        resolve_architecture({"architectures": ["LlamaForCausalLM"]})
    with pytest.raises(ConfigError, match="already registered"):
        register_architecture("Qwen3ForCausalLM", Qwen3Config)
    assert isinstance(load_config(model_dir("A")), Qwen3Config)


def test_run_order_validation():
    import dataclasses
    spec = Qwen3Config.from_dict(config_json("A")).to_spec()
    bad = dataclasses.replace(spec, run_order=(LayerCall(0), LayerCall(1, reads_cache_of=1)))
    with pytest.raises(ConfigError, match="does not come before"):
        bad.validate()
    bad = dataclasses.replace(spec, run_order=(LayerCall(0), LayerCall(5)))
    with pytest.raises(ConfigError, match="names layer 5"):
        bad.validate()
    ok = dataclasses.replace(spec, run_order=(LayerCall(0), LayerCall(1), LayerCall(1),
                                              LayerCall(0, reads_cache_of=0)))
    ok.validate()


def test_random_model_folder_round_trip():
    d = model_dir("B", "bfloat16")
    spec = load_spec(d)
    w = load_weights(d, spec, torch.bfloat16)
    want = expected_tensors(spec)
    assert set(w) == set(want) and "lm_head.weight" in w
    assert all(tuple(w[n].shape) == s for n, s in want.items())
    assert w["model.layers.0.mlp.up_proj.weight"].dtype == torch.bfloat16
    assert abs(w["model.norm.weight"].float().mean().item() - 1) < 0.01
    assert 0.015 < w["model.embed_tokens.weight"].float().std().item() < 0.025
    # the same seed gives the same file, another seed another
    with tempfile.TemporaryDirectory() as d2:
        write_random_model(d2, Qwen3Config.from_dict(config_json("B", "bfloat16")), TINY["B"]["seed"])
        w2 = load_weights(d2, spec, torch.bfloat16)
        assert all(torch.equal(w[n], w2[n]) for n in w)
        write_random_model(d2, Qwen3Config.from_dict(config_json("B", "bfloat16")), 99)
        w3 = load_weights(d2, spec, torch.bfloat16)
        assert not torch.equal(w["lm_head.weight"], w3["lm_head.weight"])


def test_dtype_rule():
    """bfloat16 mode keeps 16-bit tensors in bfloat16 and leaves 32-bit tensors 32-bit;
    float32 mode makes everything float32."""
    d32, d16 = model_dir("A", "float32"), model_dir("A", "bfloat16")
    spec = load_spec(d32)
    assert all(t.dtype == torch.float32 for t in load_weights(d32, spec, torch.bfloat16).values())
    assert all(t.dtype == torch.bfloat16 for t in load_weights(d16, spec, torch.bfloat16).values())
    assert all(t.dtype == torch.float32 for t in load_weights(d16, spec, torch.float32).values())


def test_weight_error_lists_everything():
    src = model_dir("A", "float32")
    spec = load_spec(src)
    folder = SafetensorsFolder(src)
    tensors = {n: folder.tensor(n).clone() for n in folder.names()}
    del tensors["model.layers.1.self_attn.k_norm.weight"]
    del tensors["model.norm.weight"]
    tensors["model.layers.0.mlp.extra.weight"] = torch.zeros(3)
    tensors["model.layers.0.self_attn.q_proj.weight"] = torch.zeros(64, 63)
    with tempfile.TemporaryDirectory() as d:
        write_safetensors(os.path.join(d, "model.safetensors"), tensors)
        with open(os.path.join(d, "config.json"), "w") as f:
            json.dump(config_json("A"), f)
        with pytest.raises(WeightError) as e:
            load_weights(d, spec, torch.float32)
    err = e.value
    assert set(err.missing) == {"model.layers.1.self_attn.k_norm.weight", "model.norm.weight"}
    assert err.unexpected == ["model.layers.0.mlp.extra.weight"]
    assert err.wrong_shape == [("model.layers.0.self_attn.q_proj.weight", (64, 63), (64, 64))]
    text = str(err)
    for word in ("missing (2)", "unexpected (1)", "wrong shape", "[64, 63]", "[64, 64]"):
        assert word in text


def test_tied_head_ignores_stored_output_matrix():
    src = model_dir("A", "float32")    # tied
    spec = load_spec(src)
    folder = SafetensorsFolder(src)
    tensors = {n: folder.tensor(n).clone() for n in folder.names()}
    tensors["lm_head.weight"] = torch.zeros(256, 64)
    with tempfile.TemporaryDirectory() as d:
        write_safetensors(os.path.join(d, "model.safetensors"), tensors)
        with pytest.warns(UserWarning, match="ignoring lm_head.weight"):
            w = load_weights(d, spec, torch.float32)
        assert "lm_head.weight" not in w


def _write_raw(path, header: dict, data: bytes):
    blob = json.dumps(header).encode()
    with open(path, "wb") as f:
        f.write(struct.pack("<Q", len(blob)) + blob + data)


@pytest.mark.parametrize("header,data,word", [
    ({"a": {"dtype": "F32", "shape": [2], "data_offsets": [0, 12]}}, b"\0" * 12, "need 8"),
    ({"a": {"dtype": "F32", "shape": [2], "data_offsets": [0, 8]}}, b"\0" * 4, "outside"),
    ({"a": {"dtype": "Q4", "shape": [2], "data_offsets": [0, 8]}}, b"\0" * 8, "unknown dtype"),
    ({"a": {"dtype": "F32", "shape": [2], "data_offsets": [0, 8]},
      "b": {"dtype": "F32", "shape": [2], "data_offsets": [4, 12]}}, b"\0" * 12, "overlap"),
    ({"a": {"dtype": "F32", "shape": [2]}}, b"", "malformed"),
])
def test_safetensors_refuses_bad_files(header, data, word):
    with tempfile.TemporaryDirectory() as d:
        _write_raw(os.path.join(d, "model.safetensors"), header, data)
        with pytest.raises(SafetensorsError, match=word):
            SafetensorsFolder(d)


def test_safetensors_header_bounds_and_third_party_reader():
    with tempfile.TemporaryDirectory() as d:
        p = os.path.join(d, "model.safetensors")
        with open(p, "wb") as f:
            f.write(struct.pack("<Q", 1 << 40))
        with pytest.raises(SafetensorsError, match="exceeds"):
            SafetensorsFolder(d)
        with open(p, "wb") as f:
            f.write(struct.pack("<Q", 4) + b"[1] ")
        with pytest.raises(SafetensorsError, match="not a JSON object"):
            SafetensorsFolder(d)
        # what this writer produces is read identically by the safetensors package
        t = {"x": torch.arange(6, dtype=torch.float32).reshape(2, 3),
             "y": torch.randn(5).to(torch.bfloat16), "z": torch.arange(4, dtype=torch.int32)}
        write_safetensors(p, t)
        from safetensors.torch import load_file
        other = load_file(p)
        mine = SafetensorsFolder(d)
        for n in t:
            assert torch.equal(other[n], t[n]) and torch.equal(mine.tensor(n), t[n])
        with pytest.raises(SafetensorsError, match="neither"):
            SafetensorsFolder(os.path.join(d, "nowhere"))


def test_sharded_folder():
    src = SafetensorsFolder(model_dir("A", "float32"))
    names = sorted(src.names())
    with tempfile.TemporaryDirectory() as d:
        half = len(names) // 2
        shards = {"model-00001-of-00002.safetensors": names[:half],
                  "model-00002-of-00002.safetensors": names[half:]}
        weight_map = {}
        for shard, ns in shards.items():
            write_safetensors(os.path.join(d, shard), {n: src.tensor(n) for n in ns})
            weight_map.update({n: shard for n in ns})
        with open(os.path.join(d, "model.safetensors.index.json"), "w") as f:
            json.dump({"weight_map": weight_map}, f)
        f2 = SafetensorsFolder(d)
        assert sorted(f2.names()) == names
        assert torch.equal(f2.tensor(names[3]), src.tensor(names[3]))
        weight_map[names[0]] = "model-00002-of-00002.safetensors"
        with open(os.path.join(d, "model.safetensors.index.json"), "w") as f:
            json.dump({"weight_map": weight_map}, f)
        with pytest.raises(SafetensorsError, match="disagree"):
            SafetensorsFolder(d)


def test_python_bindings_match_the_c_declarations():
    """The argument lists that the ctypes bindings declare are those of the exported C entry
    points: same count, same kinds, in the same order."""
    import ctypes
    import pathlib
    import re
    from llmario_b200 import kernels
    src = ""
    for f in sorted((pathlib.Path(kernels.__file__).parent / "csrc").glob("*.cu")):
        src += f.read_text()
    kinds = {ctypes.c_void_p: "P", ctypes.c_int: "I", ctypes.c_longlong: "L", ctypes.c_float: "F",
             ctypes.c_ulonglong: "U", ctypes.c_double: "D"}

    def kind(param: str) -> str:
        param = param.strip()
        if "*" in param or param.startswith("cudaStream_t"):
            return "P"
        base = re.sub(r"\b(const|unsigned)\b", "", param).split()
        if base[:2] == ["long", "long"]:
            return "U" if re.search(r"\bunsigned\b", param) else "L"
        return {"int": "I", "float": "F", "double": "D"}[base[0]]

    sigs = kernels._signatures()
    seen = set()
    for m in re.finditer(r"LLM_EXPORT\s+int\s+(\w+)\s*\(([^)]*)\)\s*\{", src):
        name, params = m.group(1), m.group(2)
        if name not in sigs:
            continue
        seen.add(name)
        declared = "".join(kind(p) for p in params.split(",")) if params.strip() else ""
        bound = "".join(kinds[t] for t in sigs[name])
        assert declared == bound, f"{name}: C has {declared}, the binding {bound}"
    assert seen == set(sigs), sorted(set(sigs) - seen)


def test_decode_split_model_choices():
    """The number of key parts of decode attention: never more CTAs than two waves when one part
    already fills the GPU, more parts for few requests, whole tiles per part, and the same answer
    for the same arguments (recorded CUDA graphs are keyed by it)."""
    from llmario_b200.kernels import decode_splits

    for tile in (32, 64):
        assert decode_splits(1, 8, 64, 444, tile) == 1              # one tile: nothing to cut
        few = decode_splits(1, 8, 4096, 444, tile)
        many = decode_splits(64, 8, 4096, 444, tile)
        assert few > many >= 1
        assert 8 * few <= 2 * 444                                    # at most two waves of CTAs
        for n, length in ((1, 1024), (8, 1024), (8, 8192), (64, 1024), (300, 2048)):
            s = decode_splits(n, 8, length, 444, tile)
            assert 1 <= s <= max(1, length // 64)
            assert s == decode_splits(n, 8, length, 444, tile)
    assert decode_splits(512, 8, 1024, 444, 64) == 1                # more requests than CTAs fit


def test_generation_config_adds_end_of_sequence_ids(tmp_path):
    """``eos_token_id`` of config.json (an id or a list) is merged with that of
    generation_config.json, sorted and without doubles (safetensors.rs:635-651)."""
    import json
    from llmario_b200.config import load_config
    from util import config_json

    raw = dict(config_json("A"), eos_token_id=7)
    (tmp_path / "config.json").write_text(json.dumps(raw))
    assert load_config(str(tmp_path)).eos_token_ids == (7,)
    (tmp_path / "generation_config.json").write_text(json.dumps({"eos_token_id": [9, 7, 3], "top_k": 20}))
    cfg = load_config(str(tmp_path))
    assert cfg.eos_token_ids == (3, 7, 9) and cfg.to_spec().eos_token_ids == (3, 7, 9)
    (tmp_path / "generation_config.json").write_text("{not json")
    with pytest.raises(Exception, match="not valid JSON"):
        load_config(str(tmp_path))
