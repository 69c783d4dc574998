"""The plain implementation itself, and the host-side pieces it is compared with (no GPU)."""
import math

import pytest
import torch

from plain import qwen3_plain as P
from llmario_b200.sampling import Xoshiro256StarStar
from util import model_dir, random_tokens


def test_rms_norm_values():
    # the reference's own unit test values: rows of (3, 4), unit weight (ops.rs:153-165)
    x = torch.tensor([[3.0, 4.0]], dtype=torch.float64)
    y = P.rms_norm(x, torch.ones(2, dtype=torch.float64), 0.0)
    assert torch.allclose(y, x / math.sqrt(12.5))
    y = P.rms_norm(x, torch.tensor([2.0, 0.5], dtype=torch.float64), 1e-6)
    assert torch.allclose(y, x / math.sqrt(12.5 + 1e-6) * torch.tensor([2.0, 0.5]))


def test_rope_identity_at_zero_and_norm_kept():
    x = torch.randn(3, 4 * 16, dtype=torch.float64)
    assert torch.equal(P.rope_neox(x, torch.zeros(3), 4, 16, 1e4), x)
    y = P.rope_neox(x, torch.tensor([1, 50, 999]), 4, 16, 1e4)
    assert torch.allclose(y.reshape(3, 4, 16).norm(dim=-1), x.reshape(3, 4, 16).norm(dim=-1))
    # pairs are (i, i + half): rotating by pos p then reading dim 0 mixes dims 0 and 8 only
    e = torch.zeros(1, 16, dtype=torch.float64)
    e[0, 0] = 1
    r = P.rope_neox(e, torch.tensor([1]), 1, 16, 1e4)[0]
    assert r[0] == pytest.approx(math.cos(1)) and r[8] == pytest.approx(math.sin(1))
    assert r[[1, 2, 3, 4, 5, 6, 7, 9]].abs().max() == 0


def test_adjacent_pairs_are_half_split_pairs_of_a_permuted_head():
    """The position part for adjacent pairs gives the order in which a head's values must stand
    for the half-split rotation to turn its pairs: rotating the permuted head and undoing the
    permutation is the adjacent-pair rotation (ops.rs:57-60), also with part of a head rotated."""
    from llmario_b200.config import PartSpec
    from llmario_b200.parts.position import RotaryAdjacentPairs
    heads, hd, theta = 3, 16, 500.0
    x = torch.randn(5, heads * hd, dtype=torch.float64, generator=torch.Generator().manual_seed(1))
    pos = torch.tensor([0, 1, 7, 30, 31])
    for rot in (hd, 8):
        part = RotaryAdjacentPairs(PartSpec("rope_normal", {"rot_dim": rot, "theta": theta}), {},
                                   torch.float32, "cpu")
        perm = part.head_permutation(hd)
        assert sorted(perm.tolist()) == list(range(hd))
        xp = x.reshape(5, heads, hd)[:, :, perm]
        turned = xp.clone()
        turned[:, :, :rot] = P.rope_neox(xp[:, :, :rot].reshape(5, heads * rot), pos, heads, rot,
                                         theta).reshape(5, heads, rot)
        back = torch.empty_like(turned)
        back[:, :, perm] = turned
        want = P.rope_normal(x, pos, heads, hd, rot, theta)
        assert (back.reshape(5, heads * hd) - want).abs().max() < 1e-12
        # the frequencies the kernels get are the formula's, in 32-bit
        i = torch.arange(rot // 2, dtype=torch.float64)
        assert torch.allclose(part.inv_freq.double(), theta ** (-(2.0 * i) / rot), rtol=1e-6)


def test_attention_is_causal_grouped_and_windowed():
    T, Hq, Hkv, hd = 9, 4, 2, 8
    q, k, v = (torch.randn(T, n * hd, dtype=torch.float64) for n in (Hq, Hkv, Hkv))
    full = P.attention(q, k, v, Hq, Hkv, hd)
    k2, v2 = k.clone(), v.clone()
    k2[5:], v2[5:] = 0, 7
    assert torch.allclose(P.attention(q, k2, v2, Hq, Hkv, hd)[:5], full[:5])   # no look ahead
    assert torch.allclose(full[0].reshape(Hq, hd), v[0].reshape(Hkv, hd).repeat_interleave(2, 0))
    win = P.attention(q, k, v, Hq, Hkv, hd, window=3)
    assert torch.allclose(win[:3], full[:3]) and not torch.allclose(win[5], full[5])
    k3, v3 = k.clone(), v.clone()
    k3[:6], v3[:6] = 5, -5          # keys 0..5 are outside the window of row 8 (sees 6, 7, 8)
    assert torch.allclose(P.attention(q, k3, v3, Hq, Hkv, hd, window=3)[8], win[8])
    # one-row-at-a-time with explicit positions equals the whole
    row = P.attention(q[6:7], k[:7], v[:7], Hq, Hkv, hd, None, torch.tensor([6]))
    assert torch.allclose(row[0], full[6])


def test_silu_and_ffn():
    z = torch.tensor([-2.0, 0.0, 3.0], dtype=torch.float64)
    assert torch.allclose(P.silu(z), z * torch.sigmoid(z))
    h = torch.randn(2, 6, dtype=torch.float64)
    wg, wu, wd = torch.randn(5, 6).double(), torch.randn(5, 6).double(), torch.randn(6, 5).double()
    assert torch.allclose(P.swiglu_ffn(h, wg, wu, wd),
                          (torch.nn.functional.silu(h @ wg.T) * (h @ wu.T)) @ wd.T)


def test_whole_equals_prefix_by_prefix():
    """Logits at a position depend on earlier tokens only."""
    tensors, cfg = P.load(model_dir("C", "float32"))
    toks = random_tokens("C", 40, 1)
    whole = P.forward_logits(tensors, cfg, toks)
    for n in (1, 7, 25):
        assert torch.allclose(P.forward_logits(tensors, cfg, toks[:n])[-1], whole[n - 1],
                              atol=1e-12)
    # the window matters: config C with the window switched off gives other logits late on
    cfg2 = dict(cfg, windows=[None] * cfg["layers"])
    other = P.forward_logits(tensors, cfg2, toks)
    assert torch.allclose(other[:20], whole[:20], atol=1e-12)
    assert not torch.allclose(other[30:], whole[30:], atol=1e-6)


def test_run_order_and_shared_cache():
    tensors, cfg = P.load(model_dir("A", "float32"))
    toks = random_tokens("A", 12, 2)
    base = P.forward_logits(tensors, cfg, toks)
    same = P.forward_logits(tensors, cfg, toks, schedule=[(0, None), (1, None)])
    assert torch.equal(base, same)
    twice = P.forward_logits(tensors, cfg, toks, schedule=[(0, None), (1, None), (1, None)])
    shared = P.forward_logits(tensors, cfg, toks, schedule=[(0, None), (1, None), (1, 1)])
    assert not torch.allclose(twice, base) and not torch.allclose(shared, twice)


def test_rng_vectors():
    # published splitmix64 values for seed 0 (rng.rs:57-63)
    st, a = P._splitmix64(0)
    st, b = P._splitmix64(st)
    assert (a, b) == (0xE220A8397B1DCDAF, 0x6E789E6AA1B965F4)
    mine, plain = Xoshiro256StarStar(42), P.PlainRng(42)
    for _ in range(100):
        assert mine.next_u64() == plain.next_u64()
    u = [mine.next_f64() for _ in range(1000)]
    assert all(0 <= x < 1 for x in u) and 0.45 < sum(u) / 1000 < 0.55
    assert Xoshiro256StarStar(43).next_u64() != Xoshiro256StarStar(42).next_u64()


def test_plain_sampler_chain():
    logits = [0.0, 2.0, 2.0, 1.0, -1.0, 0.5]
    assert P.plain_sample(logits, temperature=0) == 1                    # first maximum
    # top-k 2 keeps ids 1, 2 (tie -> lower id first); u walks the sorted order
    assert P.plain_sample(logits, temperature=1, top_k=2, u=0.49) == 1
    assert P.plain_sample(logits, temperature=1, top_k=2, u=0.51) == 2
    # top-p: p(1) = p(2) = 0.32..; 0.6 needs both, 0.3 only the first
    assert P.plain_sample(logits, temperature=1, top_p=0.3, u=0.99) == 1
    assert P.plain_sample(logits, temperature=1, top_p=0.6, u=0.99) == 2
    # min-p 0.5: only logits >= 2 + ln 0.5 = 1.31 survive
    assert P.plain_sample(logits, temperature=1, min_p=0.5, u=0.99) == 2
    # no filter: the walk is in id order
    assert P.plain_sample(logits, temperature=1, u=0.0) == 0
    assert P.plain_sample(logits, temperature=1, u=0.999999) == 5
    # penalties: a positive logit is divided, then count*freq + presence subtracted
    l = P.plain_sample([1.0, 3.0, 2.9], temperature=0, repeat_penalty=2.0, window_tokens=[1])
    assert l == 2
    l = P.plain_sample([1.0, 3.0, 2.9], temperature=0, frequency_penalty=0.06, window_tokens=[1, 1])
    assert l == 2
    # low temperature sharpens
    hits = sum(P.plain_sample(logits, temperature=0.05, u=(i + 0.5) / 200) in (1, 2) for i in range(200))
    assert hits == 200
