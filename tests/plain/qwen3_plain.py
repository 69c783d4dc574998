"""Plain, slow implementation of the Qwen3 dense decoder: whole sequences, no cache.

This file is the oracle of the test-suite.  It shares no code with the package: it parses
``config.json`` itself, reads tensors by their safetensors names through the third-party
``safetensors`` reader, and evaluates every formula with ordinary torch tensor arithmetic on the
CPU (float64 unless asked otherwise).  One function per part of the layer.

The Rust toolchain is not available where these tests are written, so the reference engine cannot
be compiled and run beside it: this implementation rests on the reference's formulas, each cited
below by ``file:line`` inside the reference project.
"""
from __future__ import annotations

import json
import math
import os
from typing import Dict, List, Optional, Sequence, Tuple

import torch


# --------------------------------------------------------------------------------------------
# configuration (own reading of config.json; crates/engine/formats/src/safetensors.rs:583-629)
# --------------------------------------------------------------------------------------------
def read_config(model_dir: str) -> dict:
    with open(os.path.join(model_dir, "config.json")) as f:
        raw = json.load(f)
    cfg = {}
    cfg["layers"] = int(raw["num_hidden_layers"])
    cfg["hidden"] = int(raw["hidden_size"])
    cfg["heads"] = int(raw["num_attention_heads"])
    # default: no grouping (safetensors.rs:593-596)
    cfg["kv_heads"] = int(raw.get("num_key_value_heads") or cfg["heads"])
    # default: hidden / heads (safetensors.rs:598-601)
    cfg["head_dim"] = int(raw.get("head_dim") or cfg["hidden"] // cfg["heads"])
    cfg["ff"] = int(raw["intermediate_size"])
    cfg["vocab"] = int(raw["vocab_size"])
    cfg["eps"] = float(raw["rms_norm_eps"])
    theta = raw.get("rope_theta")
    if theta is None and isinstance(raw.get("rope_parameters"), dict):
        theta = raw["rope_parameters"].get("rope_theta")  # safetensors.rs:615-621
    cfg["theta"] = float(theta if theta is not None else 10000.0)  # arch.rs:301
    cfg["tied"] = bool(raw.get("tie_word_embeddings", False))
    # per-layer window (None = every earlier key); the reference keeps the window off for this
    # family (arch.rs:538-544), the key names below are config.json's own.
    windows: List[Optional[int]] = [None] * cfg["layers"]
    if raw.get("use_sliding_window") and raw.get("sliding_window"):
        w = int(raw["sliding_window"])
        kinds = raw.get("layer_types")
        first = int(raw.get("max_window_layers", 0))
        for i in range(cfg["layers"]):
            slides = (kinds[i] == "sliding_attention") if kinds else (i >= first)
            if slides:
                windows[i] = w
    cfg["windows"] = windows
    scaling = raw.get("rope_scaling")
    cfg["freq_scale"] = 1.0
    if isinstance(scaling, dict) and scaling.get("type", scaling.get("rope_type")) == "linear":
        cfg["freq_scale"] = 1.0 / float(scaling["factor"])  # arch.rs:319-324
    return cfg


def read_tensors(model_dir: str, dtype=torch.float64) -> Dict[str, torch.Tensor]:
    from safetensors.torch import load_file

    tensors = load_file(os.path.join(model_dir, "model.safetensors"))
    return {k: v.to(dtype) for k, v in tensors.items()}


# --------------------------------------------------------------------------------------------
# parts
# --------------------------------------------------------------------------------------------
def embed(table: torch.Tensor, tokens: Sequence[int]) -> torch.Tensor:
    """Row gather, no scaling (crates/engine/model/src/forward.rs:343-349)."""
    return table[torch.tensor(list(tokens), dtype=torch.long)]


def rms_norm(x: torch.Tensor, w: torch.Tensor, eps: float) -> torch.Tensor:
    """y = x * (1/sqrt(mean(x^2)+eps)) * w over the last axis; the weight is the plain gain
    (crates/engine/cpu/src/ops.rs:18-29)."""
    ss = (x * x).sum(dim=-1, keepdim=True)
    scale = 1.0 / torch.sqrt(ss / x.shape[-1] + eps)
    return x * scale * w


def linear(x: torch.Tensor, w: torch.Tensor, b: Optional[torch.Tensor] = None) -> torch.Tensor:
    """y = W x (+ b) with W stored [out][in] (forward.rs:810-830; this architecture has no
    biases, a layer that has them adds them after the product: forward.rs:399-425)."""
    y = x @ w.t()
    return y if b is None else y + b


def per_head_norm(x: torch.Tensor, w: torch.Tensor, eps: float, n_heads: int) -> torch.Tensor:
    """RMS norm of every head slice with one weight shared by the heads and the model's own
    eps (forward.rs:437-446, 832-838)."""
    t = x.shape[0]
    hd = w.shape[0]
    return rms_norm(x.reshape(t, n_heads, hd), w, eps).reshape(t, n_heads * hd)


def rope_neox(x: torch.Tensor, positions: torch.Tensor, n_heads: int, head_dim: int,
              theta: float, freq_scale: float = 1.0) -> torch.Tensor:
    """Half-split rotation: pair (i, i+half), freq = theta^(-2i/rot_dim), angle = pos*freq
    (ops.rs:46-66 with RopeKind::Neox, rot_dim = head_dim: arch.rs:300, 315)."""
    t = x.shape[0]
    half = head_dim // 2
    i = torch.arange(half, dtype=x.dtype)
    freq = torch.tensor(theta, dtype=x.dtype) ** (-(2.0 * i) / head_dim)
    angle = positions.to(x.dtype)[:, None] * freq_scale * freq[None, :]  # [t, half]
    cos, sin = torch.cos(angle)[:, None, :], torch.sin(angle)[:, None, :]
    xh = x.reshape(t, n_heads, head_dim)
    a, b = xh[..., :half], xh[..., half:]
    out = torch.cat([a * cos - b * sin, a * sin + b * cos], dim=-1)
    return out.reshape(t, n_heads * head_dim)


def rope_normal(x: torch.Tensor, positions: torch.Tensor, n_heads: int, head_dim: int,
                rot_dim: int, theta: float, freq_scale: float = 1.0,
                attn_factor: float = 1.0) -> torch.Tensor:
    """Adjacent-pair rotation: angle i turns the pair (2i, 2i+1) of the first ``rot_dim`` values
    of a head; freq = theta^(-2i/rot_dim), angle = pos * freq_scale * freq, cosine and sine
    times ``attn_factor`` (ops.rs:46-66 with RopeKind::Normal, :57-60).  Not used by this
    architecture: it checks the position part of that kind."""
    t = x.shape[0]
    out = x.reshape(t, n_heads, head_dim).clone()
    for i in range(rot_dim // 2):
        freq = theta ** (-(2.0 * i) / rot_dim)
        angle = positions.to(x.dtype) * freq_scale * freq
        cos, sin = torch.cos(angle)[:, None] * attn_factor, torch.sin(angle)[:, None] * attn_factor
        x0, x1 = out[:, :, 2 * i].clone(), out[:, :, 2 * i + 1].clone()
        out[:, :, 2 * i] = x0 * cos - x1 * sin
        out[:, :, 2 * i + 1] = x0 * sin + x1 * cos
    return out.reshape(t, n_heads * head_dim)


def attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, n_heads: int, n_kv: int,
              head_dim: int, window: Optional[int] = None,
              q_positions: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Causal grouped-query attention of one sequence.  Query head h reads KV head h // group;
    score = dot * 1/sqrt(head_dim) (scale after the dot); keys p <= t, and with a window only
    p >= t + 1 - window; softmax with the maximum subtracted; output = sum_p w_p V[p]
    (forward.rs:585-678; group :606; range :643-645; scale :650; ops.rs:69-80).
    ``k``/``v`` hold positions 0..S-1; ``q_positions`` gives the position of each query row
    (default: 0..T-1 with T == S)."""
    tq, s = q.shape[0], k.shape[0]
    if q_positions is None:
        q_positions = torch.arange(tq)
    group = n_heads // n_kv
    scale = 1.0 / math.sqrt(head_dim)
    qh = q.reshape(tq, n_heads, head_dim)
    kh = k.reshape(s, n_kv, head_dim)
    vh = v.reshape(s, n_kv, head_dim)
    out = torch.zeros(tq, n_heads, head_dim, dtype=q.dtype)
    key_pos = torch.arange(s)
    for h in range(n_heads):
        kvh = h // group
        scores = (qh[:, h, :] @ kh[:, kvh, :].t()) * scale  # [tq, s]
        visible = key_pos[None, :] <= q_positions[:, None]
        if window is not None:
            visible &= key_pos[None, :] >= (q_positions[:, None] + 1 - window)
        scores = scores.masked_fill(~visible, float("-inf"))
        m = scores.max(dim=-1, keepdim=True).values
        e = torch.exp(scores - m)
        w = e * (1.0 / e.sum(dim=-1, keepdim=True))
        out[:, h, :] = w @ vh[:, kvh, :]
    return out.reshape(tq, n_heads * head_dim)


def silu(z: torch.Tensor) -> torch.Tensor:
    """z / (1 + exp(-z)) (ops.rs:83-85)."""
    return z / (1.0 + torch.exp(-z))


def swiglu_ffn(h: torch.Tensor, w_gate: torch.Tensor, w_up: torch.Tensor,
               w_down: torch.Tensor) -> torch.Tensor:
    """down(silu(gate h) * (up h)), no biases (forward.rs:500-530; ops.rs:95-99)."""
    return linear(silu(linear(h, w_gate)) * linear(h, w_up), w_down)


def attention_mixer(h: torch.Tensor, positions: torch.Tensor, tensors: Dict[str, torch.Tensor],
                    prefix: str, cfg: dict, window: Optional[int],
                    shared_kv: Optional[Tuple[torch.Tensor, torch.Tensor]] = None):
    """Projections, per-head q/k norm, rotation, attention, output projection, in the
    reference's order norm -> rotation -> (cache) -> attend (forward.rs:399-485).  V is neither
    normed nor rotated.  Returns (output, (k, v)); with ``shared_kv`` the layer makes no keys
    of its own and reads the given ones."""
    hq, hkv, hd = cfg["heads"], cfg["kv_heads"], cfg["head_dim"]
    q = linear(h, tensors[prefix + "q_proj.weight"])
    q = per_head_norm(q, tensors[prefix + "q_norm.weight"], cfg["eps"], hq)
    q = rope_neox(q, positions, hq, hd, cfg["theta"], cfg["freq_scale"])
    if shared_kv is None:
        k = linear(h, tensors[prefix + "k_proj.weight"])
        v = linear(h, tensors[prefix + "v_proj.weight"])
        k = per_head_norm(k, tensors[prefix + "k_norm.weight"], cfg["eps"], hkv)
        k = rope_neox(k, positions, hkv, hd, cfg["theta"], cfg["freq_scale"])
    else:
        k, v = shared_kv
    a = attention(q, k, v, hq, hkv, hd, window, positions)
    return linear(a, tensors[prefix + "o_proj.weight"]), (k, v)


def decoder_layer(x: torch.Tensor, positions: torch.Tensor, tensors: Dict[str, torch.Tensor],
                  layer: int, cfg: dict, kv_round: Optional[str] = None,
                  shared_kv=None):
    """x <- x + Attn(RMSNorm(x)); x <- x + FFN(RMSNorm(x)) (forward.rs:356-362, 390-397,
    473-499, 531-533).  ``kv_round`` names a dtype through which keys and values are rounded
    before they are read back, as a 16-bit cache does (kv.rs:112-126)."""
    p = f"model.layers.{layer}."
    h = rms_norm(x, tensors[p + "input_layernorm.weight"], cfg["eps"])
    mix_in = shared_kv
    a, kv = _mixer_with_round(h, positions, tensors, p + "self_attn.", cfg,
                              cfg["windows"][layer], mix_in, kv_round)
    x = x + a
    h = rms_norm(x, tensors[p + "post_attention_layernorm.weight"], cfg["eps"])
    y = swiglu_ffn(h, tensors[p + "mlp.gate_proj.weight"], tensors[p + "mlp.up_proj.weight"],
                   tensors[p + "mlp.down_proj.weight"])
    return x + y, kv


def _mixer_with_round(h, positions, tensors, prefix, cfg, window, shared_kv, kv_round):
    if kv_round is None or shared_kv is not None:
        return attention_mixer(h, positions, tensors, prefix, cfg, window, shared_kv)
    # make the keys first, round them as the cache would, then attend over the rounded ones
    hq, hkv, hd = cfg["heads"], cfg["kv_heads"], cfg["head_dim"]
    k = linear(h, tensors[prefix + "k_proj.weight"])
    v = linear(h, tensors[prefix + "v_proj.weight"])
    k = per_head_norm(k, tensors[prefix + "k_norm.weight"], cfg["eps"], hkv)
    k = rope_neox(k, positions, hkv, hd, cfg["theta"], cfg["freq_scale"])
    rt = getattr(torch, kv_round)
    k, v = k.to(rt).to(h.dtype), v.to(rt).to(h.dtype)
    return attention_mixer(h, positions, tensors, prefix, cfg, window, (k, v))


def forward_logits(tensors: Dict[str, torch.Tensor], cfg: dict, tokens: Sequence[int],
                   schedule: Optional[List[Tuple[int, Optional[int]]]] = None,
                   kv_round: Optional[str] = None) -> torch.Tensor:
    """Logits [T, vocab] at every position of one whole sequence.

    ``schedule`` is the order in which layers run: a list of (layer, reads_cache_of) where the
    second item, when not None, is the index *in the list* of an earlier entry whose keys and
    values this entry reads instead of making its own.  Default: every layer once, in order."""
    x = embed(tensors["model.embed_tokens.weight"], tokens)
    positions = torch.arange(len(tokens))
    if schedule is None:
        schedule = [(i, None) for i in range(cfg["layers"])]
    made = []
    for layer, reads in schedule:
        shared = made[reads] if reads is not None else None
        x, kv = decoder_layer(x, positions, tensors, layer, cfg, kv_round, shared)
        made.append(kv)
    h = rms_norm(x, tensors["model.norm.weight"], cfg["eps"])  # forward.rs:294-302
    head = tensors["model.embed_tokens.weight"] if cfg["tied"] else tensors["lm_head.weight"]
    return linear(h, head)  # forward.rs:303-316; tied: arch.rs:479


def load(model_dir: str, dtype=torch.float64):
    return read_tensors(model_dir, dtype), read_config(model_dir)


# --------------------------------------------------------------------------------------------
# sampling (crates/engine/decode/src/sampler.rs:234-362, 486-507; rng.rs:14-52)
# --------------------------------------------------------------------------------------------
_M64 = (1 << 64) - 1


def _splitmix64(state: int) -> Tuple[int, int]:
    state = (state + 0x9E3779B97F4A7C15) & _M64
    z = state
    z = ((z ^ (z >> 30)) * 0xBF58476D1CE4E5B9) & _M64
    z = ((z ^ (z >> 27)) * 0x94D049BB133111EB) & _M64
    return state, z ^ (z >> 31)


class PlainRng:
    """xoshiro256** seeded through splitmix64 (rng.rs:25-52)."""

    def __init__(self, seed: int):
        s = []
        st = seed & _M64
        for _ in range(4):
            st, out = _splitmix64(st)
            s.append(out)
        self.s = s

    @staticmethod
    def _rotl(x: int, k: int) -> int:
        return ((x << k) | (x >> (64 - k))) & _M64

    def next_u64(self) -> int:
        s = self.s
        result = (self._rotl((s[1] * 5) & _M64, 7) * 9) & _M64
        t = (s[1] << 17) & _M64
        s[2] ^= s[0]
        s[3] ^= s[1]
        s[1] ^= s[2]
        s[0] ^= s[3]
        s[2] ^= t
        s[3] = self._rotl(s[3], 45)
        return result

    def next_f64(self) -> float:
        return (self.next_u64() >> 11) * (1.0 / (1 << 53))


def plain_sample(logits: Sequence[float], *, temperature: float = 1.0, top_k: int = 0,
                 top_p: float = 1.0, min_p: float = 0.0, repeat_penalty: float = 1.0,
                 presence_penalty: float = 0.0, frequency_penalty: float = 0.0,
                 window_tokens: Sequence[int] = (), u: float = 0.0) -> int:
    """The chain penalties -> (greedy) -> top-k -> top-p -> min-p -> temperature -> softmax ->
    inverse-CDF draw with the uniform ``u`` (sampler.rs:234-362).  Ties go to the lower id."""
    import numpy as np

    l = np.array(logits, dtype=np.float32).copy()
    counts: Dict[int, int] = {}
    for t in window_tokens:
        counts[t] = counts.get(t, 0) + 1
    if counts and (repeat_penalty != 1.0 or presence_penalty != 0.0 or frequency_penalty != 0.0):
        for t, c in counts.items():  # sampler.rs:486-507
            if l[t] <= 0:
                l[t] = np.float32(l[t] * np.float32(repeat_penalty))
            else:
                l[t] = np.float32(l[t] / np.float32(repeat_penalty))
            l[t] = np.float32(l[t] - np.float32(c * frequency_penalty + presence_penalty))
    if temperature <= 0:
        return int(np.argmax(l))  # first maximum wins (sampler.rs:37-45)
    # candidates stay in id order until a filter that needs sorting runs (sampler.rs:247-301)
    by_rank = lambda ids: sorted(ids, key=lambda i: (-float(l[i]), i))
    order = list(range(len(l)))
    is_sorted = False
    if 0 < top_k < len(l):
        order = by_rank(order)[:top_k]
        is_sorted = True

    def soft(ids):
        z = np.array([l[i] for i in ids], dtype=np.float32)
        e = np.exp(z - z.max()).astype(np.float32)
        return e / e.sum(dtype=np.float32)

    if top_p < 1.0 and len(order) > 1:
        if not is_sorted:
            order = by_rank(order)
            is_sorted = True
        p = soft(order)
        cum = np.float32(0)
        last = len(order)
        for i, pi in enumerate(p):
            cum = np.float32(cum + pi)
            if cum >= np.float32(top_p):
                last = i + 1
                break
        order = order[:last]
    if min_p > 0 and len(order) > 1:
        top = max(float(l[i]) for i in order)
        floor = np.float32(np.float32(top) + np.float32(math.log(min_p)))
        order = [i for i in order if l[i] >= floor]
    if temperature != 1.0:
        for i in order:
            l[i] = np.float32(l[i] / np.float32(temperature))
    p = soft(order)
    cum = 0.0
    for i, pi in zip(order, p):
        cum += float(pi)
        if u < cum:
            return int(i)
    return int(order[-1])
