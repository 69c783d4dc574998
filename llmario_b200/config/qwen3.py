"""Typed configuration of the Qwen3 dense decoder, read from the keys of its ``config.json``.

Keys and defaults follow the reference's safetensors accessors
(crates/engine/formats/src/safetensors.rs:583-652) and its architecture description
(crates/engine/model/src/arch.rs:199-486).  Nothing that ``config.json`` gives is repeated as a
constant anywhere else in the package.
"""
from __future__ import annotations

import json
import os
from dataclasses import dataclass
from typing import Any, Dict, List, Optional, Tuple

from .spec import ConfigError, LayerCall, LayerSpec, ModelSpec, PartSpec


def _need(raw: Dict[str, Any], key: str, kind):
    if key not in raw or raw[key] is None:
        raise ConfigError(f"config.json: missing key '{key}'")
    try:
        return kind(raw[key])
    except (TypeError, ValueError):
        raise ConfigError(f"config.json: key '{key}' has value {raw[key]!r}, "
                          f"expected {kind.__name__}") from None


@dataclass(frozen=True)
class Qwen3Config:
    num_hidden_layers: int
    hidden_size: int
    num_attention_heads: int
    num_key_value_heads: int
    head_dim: int
    intermediate_size: int
    vocab_size: int
    rope_theta: float
    rms_norm_eps: float
    tie_word_embeddings: bool
    max_position_embeddings: int
    # one entry per layer: the number of keys a query sees, None = all earlier keys
    layer_windows: Tuple[Optional[int], ...]
    rope_freq_scale: float = 1.0
    eos_token_ids: Tuple[int, ...] = ()
    bos_token_id: Optional[int] = None
    torch_dtype: str = "bfloat16"

    architecture = "Qwen3ForCausalLM"
    model_type = "qwen3"

    # ---------------------------------------------------------------------------------------
    @classmethod
    def from_dict(cls, raw: Dict[str, Any]) -> "Qwen3Config":
        layers = _need(raw, "num_hidden_layers", int)
        hidden = _need(raw, "hidden_size", int)
        heads = _need(raw, "num_attention_heads", int)
        # default: as many KV heads as query heads (safetensors.rs:593-596)
        kv_heads = int(raw["num_key_value_heads"]) if raw.get("num_key_value_heads") else heads
        if heads <= 0 or kv_heads <= 0 or layers <= 0 or hidden <= 0:
            raise ConfigError("config.json: sizes must be positive")
        # default: hidden / heads (safetensors.rs:598-601); independent of it when given
        head_dim = int(raw["head_dim"]) if raw.get("head_dim") else hidden // heads
        ff = _need(raw, "intermediate_size", int)
        vocab = _need(raw, "vocab_size", int)
        eps = _need(raw, "rms_norm_eps", float)
        theta = raw.get("rope_theta")
        params = raw.get("rope_parameters")
        if theta is None and isinstance(params, dict):
            theta = params.get("rope_theta")  # safetensors.rs:615-621
        theta = float(theta) if theta is not None else 10000.0  # arch.rs:301
        max_pos = int(raw.get("max_position_embeddings") or 4096)  # arch.rs:296

        if heads % kv_heads != 0:
            raise ConfigError(f"unsupported option: num_attention_heads {heads} is not a "
                              f"multiple of num_key_value_heads {kv_heads}")
        if head_dim % 2 != 0:
            raise ConfigError(f"unsupported option: head_dim {head_dim} is odd "
                              "(half-split rotation pairs i with i + head_dim/2)")
        if raw.get("attention_bias"):
            raise ConfigError("unsupported option: attention_bias is true "
                              "(this architecture has no projection biases, arch.rs:477)")
        act = raw.get("hidden_act", "silu")
        if act != "silu":
            raise ConfigError(f"unsupported option: hidden_act '{act}' (forward.rs:511-518 "
                              "uses SiLU gating)")

        # rope scaling: only the linear kind is read (arch.rs:319-324); Qwen3 ships null
        freq_scale = 1.0
        scaling = raw.get("rope_scaling")
        if scaling is None and isinstance(params, dict) and \
                params.get("rope_type", "default") not in ("default", None):
            scaling = params
        if isinstance(scaling, dict):
            kind = scaling.get("type", scaling.get("rope_type"))
            if kind == "linear":
                freq_scale = 1.0 / float(scaling["factor"])
            elif kind not in (None, "default"):
                raise ConfigError(f"unsupported option: rope_scaling type '{kind}'")

        # sliding window: the keys are config.json's own.  With use_sliding_window the layers
        # listed as "sliding_attention" in layer_types (or, without that list, the layers from
        # max_window_layers on) see only the last `sliding_window` keys.
        windows: List[Optional[int]] = [None] * layers
        if raw.get("use_sliding_window"):
            w = raw.get("sliding_window")
            if not w or int(w) <= 0:
                raise ConfigError("config.json: use_sliding_window is true but sliding_window "
                                  f"is {w!r}")
            kinds = raw.get("layer_types")
            if kinds is not None and len(kinds) != layers:
                raise ConfigError(f"config.json: layer_types has {len(kinds)} entries for "
                                  f"{layers} layers")
            first = int(raw.get("max_window_layers", 0) or 0)
            for i in range(layers):
                if kinds is not None:
                    if kinds[i] not in ("full_attention", "sliding_attention"):
                        raise ConfigError(f"unsupported option: layer_types[{i}] = "
                                          f"'{kinds[i]}'")
                    slides = kinds[i] == "sliding_attention"
                else:
                    slides = i >= first
                if slides:
                    windows[i] = int(w)

        eos = raw.get("eos_token_id")
        eos_ids: Tuple[int, ...] = ()
        if isinstance(eos, int):
            eos_ids = (eos,)
        elif isinstance(eos, list):
            eos_ids = tuple(sorted({int(e) for e in eos}))
        bos = raw.get("bos_token_id")
        dtype = raw.get("torch_dtype") or raw.get("dtype") or "bfloat16"
        return cls(layers, hidden, heads, kv_heads, head_dim, ff, vocab, theta, eps,
                   bool(raw.get("tie_word_embeddings", False)), max_pos, tuple(windows),
                   freq_scale, eos_ids, int(bos) if isinstance(bos, int) else None, str(dtype))

    @classmethod
    def from_model_dir(cls, model_dir: str) -> "Qwen3Config":
        path = os.path.join(model_dir, "config.json")
        if not os.path.isfile(path):
            raise ConfigError(f"{path}: no such file")
        with open(path) as f:
            return cls.from_dict(json.load(f))

    def to_dict(self) -> Dict[str, Any]:
        """The ``config.json`` that reads back as this configuration."""
        out: Dict[str, Any] = {
            "architectures": [self.architecture], "model_type": self.model_type,
            "num_hidden_layers": self.num_hidden_layers, "hidden_size": self.hidden_size,
            "num_attention_heads": self.num_attention_heads,
            "num_key_value_heads": self.num_key_value_heads, "head_dim": self.head_dim,
            "intermediate_size": self.intermediate_size, "vocab_size": self.vocab_size,
            "rope_theta": self.rope_theta, "rms_norm_eps": self.rms_norm_eps,
            "tie_word_embeddings": self.tie_word_embeddings,
            "max_position_embeddings": self.max_position_embeddings,
            "hidden_act": "silu", "attention_bias": False, "torch_dtype": self.torch_dtype,
            "rope_scaling": None if self.rope_freq_scale == 1.0 else
            {"type": "linear", "factor": 1.0 / self.rope_freq_scale},
        }
        ws = [w for w in self.layer_windows if w is not None]
        if ws:
            out["use_sliding_window"] = True
            out["sliding_window"] = ws[0]
            out["layer_types"] = ["sliding_attention" if w is not None else "full_attention"
                                  for w in self.layer_windows]
        else:
            out["use_sliding_window"] = False
            out["sliding_window"] = None
        if self.eos_token_ids:
            out["eos_token_id"] = list(self.eos_token_ids)
        if self.bos_token_id is not None:
            out["bos_token_id"] = self.bos_token_id
        return out

    # ---------------------------------------------------------------------------------------
    def to_spec(self) -> ModelSpec:
        """Lay the model out as parts.  Tensor names are the safetensors names of this
        architecture (crates/engine/formats/README.md:116-137)."""
        c = self
        q_width = c.num_attention_heads * c.head_dim
        kv_width = c.num_key_value_heads * c.head_dim
        rope = PartSpec("rope_neox", {
            "rot_dim": c.head_dim,              # full rotary (arch.rs:300)
            "theta": c.rope_theta, "freq_scale": c.rope_freq_scale,
            "attn_factor": 1.0,                 # arch.rs:474
        })

        def norm(width: int, name: str) -> PartSpec:
            return PartSpec("rms_norm", {"width": width, "eps": c.rms_norm_eps,
                                         "tensors": {"weight": (name, (width,))}})

        layers = []
        for i in range(c.num_hidden_layers):
            p = f"model.layers.{i}."
            a = p + "self_attn."
            mixer = PartSpec("attention", {
                "hidden_size": c.hidden_size, "num_heads": c.num_attention_heads,
                "num_kv_heads": c.num_key_value_heads, "head_dim": c.head_dim,
                "scale": c.head_dim ** -0.5,    # forward.rs:466
                "window": c.layer_windows[i],
                "position": rope,
                # per-head norms use the model's eps (forward.rs:442-445)
                "q_norm": norm(c.head_dim, a + "q_norm.weight"),
                "k_norm": norm(c.head_dim, a + "k_norm.weight"),
                "tensors": {
                    "q": (a + "q_proj.weight", (q_width, c.hidden_size)),
                    "k": (a + "k_proj.weight", (kv_width, c.hidden_size)),
                    "v": (a + "v_proj.weight", (kv_width, c.hidden_size)),
                    "o": (a + "o_proj.weight", (c.hidden_size, q_width)),
                },
            })
            m = p + "mlp."
            ffn = PartSpec("swiglu", {
                "hidden_size": c.hidden_size, "intermediate_size": c.intermediate_size,
                "tensors": {
                    "gate": (m + "gate_proj.weight", (c.intermediate_size, c.hidden_size)),
                    "up": (m + "up_proj.weight", (c.intermediate_size, c.hidden_size)),
                    "down": (m + "down_proj.weight", (c.hidden_size, c.intermediate_size)),
                },
            })
            block = PartSpec("pre_norm_residual", {
                "mixer_norm": norm(c.hidden_size, p + "input_layernorm.weight"),
                "feed_forward_norm": norm(c.hidden_size, p + "post_attention_layernorm.weight"),
            })
            layers.append(LayerSpec(block, mixer, ffn, p))

        embedding = PartSpec("token_embedding", {
            "vocab_size": c.vocab_size, "hidden_size": c.hidden_size,
            "tensors": {"table": ("model.embed_tokens.weight", (c.vocab_size, c.hidden_size))},
        })
        head_tensor = "model.embed_tokens.weight" if c.tie_word_embeddings else "lm_head.weight"
        head = PartSpec("linear_head", {
            "vocab_size": c.vocab_size, "hidden_size": c.hidden_size,
            "tied": c.tie_word_embeddings,
            "ignored_when_tied": ("lm_head.weight",),
            "tensors": {"weight": (head_tensor, (c.vocab_size, c.hidden_size))},
        })
        spec = ModelSpec(
            architecture=c.architecture, vocab_size=c.vocab_size, hidden_size=c.hidden_size,
            max_positions=c.max_position_embeddings, embedding=embedding,
            layers=tuple(layers),
            run_order=tuple(LayerCall(i) for i in range(c.num_hidden_layers)),
            final_norm=norm(c.hidden_size, "model.norm.weight"), head=head,
            eos_token_ids=c.eos_token_ids, bos_token_id=c.bos_token_id,
            stored_dtype=c.torch_dtype)
        spec.validate()
        return spec
