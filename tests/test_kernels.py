"""Each kernel alone against a plain float32/float64 torch statement of the same operation, at
sizes other than the engine's tiny configurations."""
import math
import random

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def rnd(*shape, dtype=torch.float32, scale=1.0, seed=0):
    g = torch.Generator().manual_seed(seed + sum(shape))
    return (scale * torch.randn(*shape, generator=g)).to(dtype).to(DEV)


@pytest.mark.parametrize("rows,width", [(1, 40), (7, 1000), (33, 4096), (515, 1024), (2050, 1000),
                                        (600, 2048), (513, 96)])
@pytest.mark.parametrize("out_dtype", [torch.float32, torch.bfloat16])
def test_rms_norm(rows, width, out_dtype):
    from llmario_b200 import kernels
    x, w = rnd(rows, width, scale=3.0), 1 + 0.1 * rnd(width, seed=1)
    out = torch.empty(rows, width, dtype=out_dtype, device=DEV)
    kernels.rms_norm(x, w, out, 1e-5)
    xd = x.double()
    ref = xd * torch.rsqrt((xd * xd).mean(-1, keepdim=True) + 1e-5) * w.double()
    tol = 1e-5 if out_dtype == torch.float32 else 2 ** -8
    assert (out.double() - ref).abs().max() <= tol * ref.abs().max()
    # with a row index: rows in another order
    idx = torch.tensor(list(range(rows))[::-1], dtype=torch.int32, device=DEV)
    out2 = torch.empty_like(out)
    kernels.rms_norm(x, w, out2, 1e-5, idx)
    assert torch.equal(out2, out.flip(0))


@pytest.mark.parametrize("rows,width", [(1, 24), (9, 1000), (700, 4097)])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_add_bias(rows, width, dtype):
    from llmario_b200 import kernels
    out, bias = rnd(rows, width, dtype=dtype, scale=2.0), rnd(width, seed=3)
    want = (out.float() + bias).to(dtype)      # the sum in 32-bit, rounded once
    kernels.add_bias(out, bias)
    assert torch.equal(out, want)


@pytest.mark.parametrize("vocab,width", [(50, 24), (1000, 520)])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_embed(vocab, width, dtype):
    from llmario_b200 import kernels
    table = rnd(vocab, width, dtype=dtype)
    toks = torch.tensor([0, vocab - 1, 3, 3, 17], dtype=torch.int32, device=DEV)
    out = torch.empty(5, width, dtype=torch.float32, device=DEV)
    err = torch.zeros(1, dtype=torch.int32, device=DEV)
    kernels.embed(toks, table, out, err)
    assert torch.equal(out, table[toks.long()].float())
    assert err.item() == 0


@pytest.mark.parametrize("M,N,K", [(1, 50, 24), (5, 130, 100), (70, 300, 257), (130, 64, 512)])
@pytest.mark.parametrize("dt", [(torch.float32, torch.float32), (torch.bfloat16, torch.bfloat16),
                                (torch.bfloat16, torch.float32)])
def test_gemm_simt(M, N, K, dt):
    from llmario_b200 import kernels
    a, w = rnd(M, K, dtype=dt[0]), rnd(N, K, dtype=dt[1], seed=3)
    ref = a.double() @ w.double().t()
    out = torch.empty(M, N, dtype=torch.float32, device=DEV)
    kernels.gemm_simt(a, w, out)
    assert (out.double() - ref).abs().max() <= 1e-5 * ref.abs().max() * math.sqrt(K)
    base = rnd(M, N, seed=9)
    acc = base.clone()
    kernels.gemm_simt(a, w, acc, accumulate=True)
    assert (acc.double() - (base.double() + ref)).abs().max() <= 1e-5 * ref.abs().max() * math.sqrt(K)


@pytest.mark.parametrize("M", [1, 2, 3, 5, 8])
@pytest.mark.parametrize("N,K", [(6, 8), (130, 264), (1000, 4096)])
def test_gemv_bf16(M, N, K):
    from llmario_b200 import kernels
    a, w = rnd(M, K, dtype=torch.bfloat16), rnd(N, K, dtype=torch.bfloat16, seed=3)
    ref = a.double() @ w.double().t()
    tol = 1e-5 * ref.abs().max() * math.sqrt(K)
    out = torch.empty(M, N, dtype=torch.float32, device=DEV)
    kernels.gemv_bf16(a, w, out, 0)
    assert (out.double() - ref).abs().max() <= tol
    base = rnd(M, N, seed=9)
    acc = base.clone()
    kernels.gemv_bf16(a, w, acc, 1)
    assert (acc.double() - (base.double() + ref)).abs().max() <= tol
    if N % 2 == 0:
        half = N // 2
        act = torch.empty(M, half, dtype=torch.float32, device=DEV)
        kernels.gemv_bf16(a, w, act, 2, half)
        g, u = ref[:, :half], ref[:, half:]
        want = g / (1 + torch.exp(-g)) * u
        assert (act.double() - want).abs().max() <= 4 * tol * max(1.0, ref.abs().max().item())


def test_silu_mul():
    from llmario_b200 import kernels
    gu = rnd(9, 2 * 70, scale=4.0)
    out = torch.empty(9, 70, dtype=torch.float32, device=DEV)
    kernels.silu_mul(gu, out)
    g, u = gu[:, :70].double(), gu[:, 70:].double()
    assert (out.double() - g / (1 + torch.exp(-g)) * u).abs().max() <= 1e-5


def paged_setup(lengths, page, Hkv, hd, dtype, seed=0, n_layers_in_page=2, layer=1):
    """A scrambled paged cache holding random keys/values for requests of the given lengths."""
    n_pages = sum(-(-n // page) for n in lengths) + 3
    g = torch.Generator().manual_seed(seed)
    perm = torch.randperm(n_pages, generator=g).tolist()
    storage = torch.zeros(n_pages, n_layers_in_page, 2, Hkv, page, hd, dtype=dtype, device=DEV)
    maxp = max(-(-n // page) for n in lengths) + 1
    table = torch.full((len(lengths), maxp), -1, dtype=torch.int32)
    ks, vs = [], []
    at = 0
    for r, n in enumerate(lengths):
        k = torch.randn(n, Hkv, hd, generator=g).to(dtype)
        v = torch.randn(n, Hkv, hd, generator=g).to(dtype)
        ks.append(k), vs.append(v)
        for j in range(-(-n // page)):
            p = perm[at]
            at += 1
            table[r, j] = p
            m = min(page, n - j * page)
            storage[p, layer, 0, :, :m] = k[j * page:j * page + m].transpose(0, 1).to(DEV)
            storage[p, layer, 1, :, :m] = v[j * page:j * page + m].transpose(0, 1).to(DEV)
    return storage, table.to(DEV), ks, vs


def attention_ref(q, k, v, pos, window, scale):
    """q [Hq, hd], k/v [S, Hkv, hd]: one query at position pos over keys lo..pos."""
    Hq, Hkv = q.shape[0], k.shape[1]
    lo = max(0, pos + 1 - window) if window else 0
    out = torch.zeros_like(q, dtype=torch.float64)
    for h in range(Hq):
        kh = k[lo:pos + 1, h // (Hq // Hkv)].double()
        vh = v[lo:pos + 1, h // (Hq // Hkv)].double()
        s = (kh @ q[h].double()) * scale
        w = torch.softmax(s, 0)
        out[h] = w @ vh
    return out


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("Hq,Hkv,hd,page,window", [(4, 2, 16, 4, None), (6, 1, 48, 16, 37),
                                                   (8, 8, 128, 8, None), (3, 3, 80, 32, 100),
                                                   (10, 2, 256, 16, None)])
def test_attention_generic(dtype, Hq, Hkv, hd, page, window):
    from llmario_b200 import kernels
    lengths = [1, 33, 150, 64, 257]
    storage, table, ks, vs = paged_setup(lengths, page, Hkv, hd, dtype)
    # rows: the last position of every request, plus a run of rows inside request 2
    rows = [(r, n - 1) for r, n in enumerate(lengths)] + [(2, p) for p in range(60, 70)]
    g = torch.Generator().manual_seed(5)
    q = torch.randn(len(rows), Hq, hd, generator=g).to(dtype)
    slot = torch.tensor([r for r, _ in rows], dtype=torch.int32, device=DEV)
    pos = torch.tensor([p for _, p in rows], dtype=torch.int32, device=DEV)
    out = torch.empty(len(rows), Hq * hd, dtype=dtype, device=DEV)
    scale = 1 / math.sqrt(hd)
    kernels.attention_generic(q.reshape(len(rows), -1).to(DEV).contiguous(), out,
                              storage[0, 1, 0], storage[0, 1, 1], storage.stride(0), table, slot,
                              pos, Hq, Hkv, hd, page, scale, window)
    tol = 2e-5 if dtype == torch.float32 else 2e-2
    for i, (r, p) in enumerate(rows):
        ref = attention_ref(q[i], ks[r], vs[r], p, window, scale)
        got = out[i].reshape(Hq, hd).double().cpu()
        assert (got - ref).abs().max() <= tol, (i, r, p)


def test_attention_far_key_stands_out():
    """One key far back among hundreds is made to dominate: the output must be its value."""
    from llmario_b200 import kernels
    Hq, Hkv, hd, page = 4, 2, 32, 8
    n = 700
    storage, table, ks, vs = paged_setup([n], page, Hkv, hd, torch.float32, seed=3,
                                         n_layers_in_page=1, layer=0)
    q = torch.randn(1, Hq, hd)
    far = 13
    for h in range(Hq):
        kvh = h // 2
        ks[0][far, kvh] = 0
    ks[0][far] = 40 * q[0, ::2] / q[0, ::2].norm(dim=-1, keepdim=True)   # aligned with heads 0, 2
    p_idx, s_idx = table[0, far // page].item(), far % page
    storage[p_idx, 0, 0, :, s_idx] = ks[0][far].to(DEV)
    out = torch.empty(1, Hq * hd, dtype=torch.float32, device=DEV)
    kernels.attention_generic(q.reshape(1, -1).to(DEV), out, storage[0, 0, 0], storage[0, 0, 1],
                              storage.stride(0), table, torch.zeros(1, dtype=torch.int32, device=DEV),
                              torch.tensor([n - 1], dtype=torch.int32, device=DEV), Hq, Hkv, hd,
                              page, 1 / math.sqrt(hd), None)
    ref = attention_ref(q[0], ks[0], vs[0], n - 1, None, 1 / math.sqrt(hd))
    got = out.reshape(Hq, hd).double().cpu()
    assert (got - ref).abs().max() <= 2e-5
    for h in (0, 2):   # the heads whose query the far key was aligned with
        assert (got[h] - vs[0][far, h // 2].double()).abs().max() < 1e-3


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("Hq,Hkv,hd,page", [(4, 2, 16, 4), (5, 5, 48, 16), (8, 2, 128, 8)])
def test_qk_norm_rope_store(dtype, Hq, Hkv, hd, page):
    from llmario_b200 import kernels
    rows_pos = [0, 1, 5, 17, 300, 1023]
    if hd == 128:       # enough rows for the kernel that takes four heads per warp
        rows_pos = sorted(set(rows_pos) | set(range(2, 1000, 3)))
    T = len(rows_pos)
    width = (Hq + 2 * Hkv) * hd
    proj = rnd(T, width, scale=2.0)
    qw, kw = 1 + 0.1 * rnd(hd, seed=1), 1 + 0.1 * rnd(hd, seed=2)
    theta, eps = 12345.0, 1e-5
    inv_freq = torch.tensor(np.power(np.float32(theta), -(np.arange(hd // 2, dtype=np.float32) * 2) / hd)
                            .astype(np.float32), device=DEV)
    n_pages = 1024 // page + 1
    storage = torch.zeros(n_pages, 1, 2, Hkv, page, hd, dtype=dtype, device=DEV)
    table = torch.arange(n_pages, dtype=torch.int32, device=DEV).flip(0).reshape(1, -1).contiguous()
    q_out = torch.empty(T, Hq * hd, dtype=dtype, device=DEV)
    slot = torch.zeros(T, dtype=torch.int32, device=DEV)
    pos = torch.tensor(rows_pos, dtype=torch.int32, device=DEV)
    kernels.qk_norm_rope_store(proj, q_out, storage[0, 0, 0], storage[0, 0, 1], storage.stride(0),
                               table, slot, pos, qw, kw, inv_freq, 1.0, Hq, Hkv, hd, hd, page, eps)

    def norm_rope(x, w, p):   # x [H, hd] float64
        x = x * torch.rsqrt((x * x).mean(-1, keepdim=True) + eps) * w.double().cpu()
        half = hd // 2
        ang = p * (theta ** (-(torch.arange(half, dtype=torch.float64) * 2) / hd))
        c, s = torch.cos(ang), torch.sin(ang)
        a, b = x[:, :half], x[:, half:]
        return torch.cat([a * c - b * s, a * s + b * c], -1)

    tol = 3e-4 if dtype == torch.float32 else 3e-2   # 32-bit angle at position 1023: ~1e-4 rad
    pc = proj.double().cpu()
    for i, p in enumerate(rows_pos):
        qr = norm_rope(pc[i, :Hq * hd].reshape(Hq, hd), qw, p)
        kr = norm_rope(pc[i, Hq * hd:(Hq + Hkv) * hd].reshape(Hkv, hd), kw, p)
        vr = pc[i, (Hq + Hkv) * hd:].reshape(Hkv, hd)
        page_id = table[0, p // page].item()
        assert (q_out[i].double().cpu().reshape(Hq, hd) - qr).abs().max() <= tol
        assert (storage[page_id, 0, 0, :, p % page].double().cpu() - kr).abs().max() <= tol
        # values are stored as projected: in bfloat16 half a unit in the last place of the value
        # itself (2^-9 of it) is the bound, which passes the absolute one above 7.7
        vtol = tol if dtype == torch.float32 else tol + 2.0 ** -9 * vr.abs()
        assert ((storage[page_id, 0, 1, :, p % page].double().cpu() - vr).abs() <= vtol).all()
    # the same with the cosines and sines made once for all heads (what the engine does; head
    # size 128 then takes the kernel's vectorised path)
    table_cs = torch.empty(T, hd // 2, 2, dtype=torch.float32, device=DEV)
    kernels.rope_table(pos, inv_freq, table_cs, 1.0)
    q_tab = torch.empty_like(q_out)
    storage2 = torch.zeros_like(storage)
    kernels.qk_norm_rope_store(proj, q_tab, storage2[0, 0, 0], storage2[0, 0, 1], storage2.stride(0),
                               table, slot, pos, qw, kw, inv_freq, 1.0, Hq, Hkv, hd, hd, page, eps,
                               table_cs)
    assert (q_tab.double() - q_out.double()).abs().max() <= tol
    assert (storage2.double() - storage.double()).abs().max() <= tol
    for i, p in enumerate(rows_pos):
        qr = norm_rope(pc[i, :Hq * hd].reshape(Hq, hd), qw, p)
        assert (q_tab[i].double().cpu().reshape(Hq, hd) - qr).abs().max() <= tol
    # on request the consumed projection is cleared, for the split-K product that adds into it
    q_again, used = torch.empty_like(q_out), proj.clone()
    kernels.qk_norm_rope_store(used, q_again, storage[0, 0, 0], storage[0, 0, 1], storage.stride(0),
                               table, slot, pos, qw, kw, inv_freq, 1.0, Hq, Hkv, hd, hd, page, eps,
                               clear_proj=True)
    assert torch.equal(q_again, q_out) and int((used != 0).sum()) == 0
    used = proj.clone()
    kernels.qk_norm_rope_store(used, q_again, storage2[0, 0, 0], storage2[0, 0, 1], storage2.stride(0),
                               table, slot, pos, qw, kw, inv_freq, 1.0, Hq, Hkv, hd, hd, page, eps,
                               table_cs, clear_proj=True)
    # (with many rows the first call took the four-heads-per-warp kernel: not bit for bit the same)
    assert (q_again.double() - q_tab.double()).abs().max() <= tol and int((used != 0).sum()) == 0


@pytest.mark.parametrize("T,N,K", [(1, 128, 64), (16, 256, 128), (5, 200, 72), (40, 384, 4096),
                                   (130, 130, 264), (300, 1000, 512), (64, 4096, 12288),
                                   (700, 384, 520), (1100, 130, 72), (600, 300, 4096),
                                   (1024, 512, 3080)])
def test_gemm_tcgen05(T, N, K):
    from llmario_b200 import kernels
    a, w = rnd(T, K, dtype=torch.bfloat16), rnd(N, K, dtype=torch.bfloat16, seed=3)
    ref = a.double() @ w.double().t()
    tol = 2e-5 * float(ref.abs().max()) * math.sqrt(K) + 1e-6
    out = torch.full((T, N), 7.0, dtype=torch.float32, device=DEV)
    kernels.gemm_tcgen05(a, w, out, 0)
    kernels.check_tc_status(DEV)
    assert (out.double() - ref).abs().max() <= tol
    if T <= 128 and K >= 256:     # split K into a destination the caller keeps at zero
        zeros = torch.zeros(T, N, dtype=torch.float32, device=DEV)
        kernels.gemm_tcgen05(a, w, zeros, 0, splits=2, out_is_zero=True)
        kernels.check_tc_status(DEV)
        assert (zeros.double() - ref).abs().max() <= tol
    outb = torch.empty(T, N, dtype=torch.bfloat16, device=DEV)
    kernels.gemm_tcgen05(a, w, outb, 0)
    assert (outb.double() - ref).abs().max() <= 2 ** -8 * float(ref.abs().max()) + tol
    base = rnd(T, N, seed=9)
    acc = base.clone()
    kernels.gemm_tcgen05(a, w, acc, 1)
    assert (acc.double() - (base.double() + ref)).abs().max() <= tol
    for bn in (16, 64, 256):           # every token tile gives the same product
        o2 = torch.empty(T, N, dtype=torch.float32, device=DEV)
        kernels.gemm_tcgen05(a, w, o2, 0, bn=bn)
        assert (o2.double() - ref).abs().max() <= tol, bn
    try:                               # tiles of 256 tokens on one CTA instead of a CTA pair
        kernels.use_cta_pairs(False)
        o2 = torch.empty(T, N, dtype=torch.bfloat16, device=DEV)
        kernels.gemm_tcgen05(a, w, o2, 0, bn=256)
        assert (o2.double() - ref).abs().max() <= 2 ** -8 * float(ref.abs().max()) + tol
        acc = base.clone()
        kernels.gemm_tcgen05(a, w, acc, 1, bn=256)
        assert (acc.double() - (base.double() + ref)).abs().max() <= tol
    finally:
        kernels.use_cta_pairs(True)
    if K >= 256:                       # K split in three, partial sums added
        acc = base.clone()
        kernels.gemm_tcgen05(a, w, acc, 1, splits=3)
        assert (acc.double() - (base.double() + ref)).abs().max() <= tol
        z = torch.zeros(T, N, dtype=torch.float32, device=DEV)
        kernels.gemm_tcgen05(a, w, z, 0, splits=2)
        assert (z.double() - ref).abs().max() <= tol
    kernels.check_tc_status(DEV)


@pytest.mark.parametrize("T,ff,K", [(3, 64, 64), (20, 200, 136), (150, 1000, 512),
                                    (600, 200, 136), (1030, 72, 64), (40, 208, 72), (700, 1008, 256)])
def test_gemm_tcgen05_gated(T, ff, K):
    from llmario_b200 import kernels
    a, w = rnd(T, K, dtype=torch.bfloat16), rnd(2 * ff, K, dtype=torch.bfloat16, seed=3, scale=0.3)
    ref = a.double() @ w.double().t()
    g, u = ref[:, :ff], ref[:, ff:]
    want = g / (1 + torch.exp(-g)) * u
    act = torch.empty(T, ff, dtype=torch.float32, device=DEV)
    kernels.gemm_tcgen05(a, w, act, 2, ff)
    kernels.check_tc_status(DEV)
    tol = 1e-4 * max(1.0, float(want.abs().max())) * math.sqrt(K)
    assert (act.double() - want).abs().max() <= tol
    actb = torch.empty(T, ff, dtype=torch.bfloat16, device=DEV)
    kernels.gemm_tcgen05(a, w, actb, 2, ff)
    assert (actb.double() - want).abs().max() <= 2 ** -8 * float(want.abs().max()) + tol
    if ff % 16 == 0:      # the same matrices stored as alternating blocks of 16 gate and 16 up rows
        wi = torch.stack([w[:ff].view(ff // 16, 16, K), w[ff:].view(ff // 16, 16, K)], 1).reshape(2 * ff, K)
        act2 = torch.empty(T, ff, dtype=torch.float32, device=DEV)
        kernels.gemm_tcgen05(a, wi.contiguous(), act2, 3, ff)
        kernels.check_tc_status(DEV)
        assert (act2.double() - want).abs().max() <= tol
        try:              # many rows: on one CTA per tile instead of a CTA pair
            kernels.use_cta_pairs(False)
            act3 = torch.empty(T, ff, dtype=torch.bfloat16, device=DEV)
            kernels.gemm_tcgen05(a, wi.contiguous(), act3, 3, ff)
            kernels.check_tc_status(DEV)
            assert (act3.double() - want).abs().max() <= 2 ** -8 * float(want.abs().max()) + tol
        finally:
            kernels.use_cta_pairs(True)


@pytest.mark.parametrize("Hq,Hkv,hd,page,window", [(8, 2, 128, 16, None), (6, 3, 64, 8, 50),
                                                   (4, 4, 32, 4, None), (16, 1, 128, 16, 200),
                                                   (3, 1, 64, 32, None)])
def test_attention_flash(Hq, Hkv, hd, page, window):
    """The tensor-core kernel in its three uses: one-token items with the keys split and
    merged, short portions in one warp, long portions in four warps."""
    from llmario_b200 import kernels
    dtype = torch.bfloat16
    G = Hq // Hkv
    lengths = [1, 33, 150, 64, 700, 385]
    storage, table, ks, vs = paged_setup(lengths, page, Hkv, hd, dtype)
    scale = 1 / math.sqrt(hd)
    g = torch.Generator().manual_seed(5)

    def check(rows, out, q, tol=2e-2):
        for i, (r, p) in enumerate(rows):
            ref = attention_ref(q[i].float(), ks[r].float(), vs[r].float(), p, window, scale)
            got = out[i].reshape(Hq, hd).double().cpu()
            assert (got - ref).abs().max() <= tol, (i, r, p, (got - ref).abs().max())

    # 1. decode rows: the last position of every request, keys split in 1, 3 and 5 parts
    rows = [(r, n - 1) for r, n in enumerate(lengths)]
    q = torch.randn(len(rows), Hq, hd, generator=g).to(dtype)
    qd = q.reshape(len(rows), -1).to(DEV).contiguous()
    slot = torch.tensor([r for r, _ in rows], dtype=torch.int32, device=DEV)
    pos = torch.tensor([p for _, p in rows], dtype=torch.int32, device=DEV)
    for splits in (1, 3, 5):
        out = torch.zeros(len(rows), Hq * hd, dtype=dtype, device=DEV)
        po = torch.empty(len(rows) * Hq * splits * hd, dtype=torch.float32, device=DEV)
        pml = torch.empty(len(rows) * Hq * splits * 2, dtype=torch.float32, device=DEV)
        kernels.attention_flash(qd, out, storage[0, 1, 0], storage[0, 1, 1], storage.stride(0), table,
                                None, len(rows), 16, Hq, Hkv, hd, page, scale, window, splits,
                                po, pml, slot, pos)
        if splits > 1:
            kernels.attention_merge(po, pml, out, None, len(rows), Hq, hd, splits)
        check(rows, out, q)
    # 2. portions: the tail of request 4 as items of changing length, small and large
    small_cap, large_cap = max(1, 16 // G), max(1, 64 // G)
    start = 700 - 150
    sizes, at = [], start
    for n in [1, small_cap, large_cap, 2, large_cap, 3, large_cap]:
        n = min(n, 700 - at)
        if n > 0:
            sizes.append((at, n))
            at += n
    rows = [(4, p) for p in range(start, at)]
    q = torch.randn(len(rows), Hq, hd, generator=g).to(dtype)
    qd = q.reshape(len(rows), -1).to(DEV).contiguous()
    out = torch.zeros(len(rows), Hq * hd, dtype=dtype, device=DEV)
    for cap, rpc in ((small_cap, 16), (large_cap, 64)):
        items = [(p0 - start, n, 4, p0) for p0, n in sizes if (n <= small_cap) == (rpc == 16)]
        if not items:
            continue
        dev = torch.tensor(items, dtype=torch.int32, device=DEV).reshape(-1)
        kernels.attention_flash(qd, out, storage[0, 1, 0], storage[0, 1, 1], storage.stride(0), table,
                                dev, len(items), rpc, Hq, Hkv, hd, page, scale, window)
    check(rows, out, q)


@pytest.mark.parametrize("Hq,Hkv,hd,page,window", [(8, 2, 128, 16, None), (6, 3, 64, 8, 50),
                                                   (4, 4, 32, 4, None), (8, 1, 128, 16, 200),
                                                   (3, 1, 64, 32, None), (32, 8, 128, 16, None),
                                                   (8, 2, 128, 64, None), (4, 4, 64, 128, 100)])
@pytest.mark.parametrize("tma", [False, True])
def test_attention_decode(Hq, Hkv, hd, page, window, tma):
    """The decode kernels (keys on the M side; loads by cp.async or by TMA tiles): one-token
    items with the keys split and merged, and items of a few tokens (at most eight token-head
    pairs)."""
    from llmario_b200 import kernels
    if tma and hd not in (64, 128):
        pytest.skip("the TMA form has head sizes 64 and 128")
    dtype = torch.bfloat16
    G = Hq // Hkv
    lengths = [1, 33, 150, 64, 700, 385]
    storage, table, ks, vs = paged_setup(lengths, page, Hkv, hd, dtype)
    scale = 1 / math.sqrt(hd)
    g = torch.Generator().manual_seed(5)
    common = (storage[0, 1, 0], storage[0, 1, 1], storage.stride(0), table)

    def run(qd, out, items, n, splits=1, po=None, pml=None, slot=None, pos=None):
        if tma:
            kernels.attention_decode_tma(qd, out, storage, 1, table, items, n, Hq, Hkv, hd, page,
                                         scale, window, splits, po, pml, slot, pos)
            kernels.check_tc_status(DEV)
        else:
            kernels.attention_decode(qd, out, *common, items, n, Hq, Hkv, hd, page, scale, window,
                                     splits, po, pml, slot, pos)

    def check(rows, out, q, tol=2e-2):
        for i, (r, p) in enumerate(rows):
            ref = attention_ref(q[i].float(), ks[r].float(), vs[r].float(), p, window, scale)
            got = out[i].reshape(Hq, hd).double().cpu()
            assert (got - ref).abs().max() <= tol, (i, r, p, (got - ref).abs().max())

    rows = [(r, n - 1) for r, n in enumerate(lengths)]
    q = torch.randn(len(rows), Hq, hd, generator=g).to(dtype)
    qd = q.reshape(len(rows), -1).to(DEV).contiguous()
    slot = torch.tensor([r for r, _ in rows], dtype=torch.int32, device=DEV)
    pos = torch.tensor([p for _, p in rows], dtype=torch.int32, device=DEV)
    for splits in (1, 3, 5):
        out = torch.zeros(len(rows), Hq * hd, dtype=dtype, device=DEV)
        po = torch.empty(len(rows) * Hq * splits * hd, dtype=torch.float32, device=DEV)
        pml = torch.empty(len(rows) * Hq * splits * 2, dtype=torch.float32, device=DEV)
        run(qd, out, None, len(rows), splits, po, pml, slot, pos)
        if splits > 1:
            kernels.attention_merge(po, pml, out, None, len(rows), Hq, hd, splits)
        check(rows, out, q)
    cap = 8 // G
    if cap >= 2:       # items of several tokens: every pair has its own causal limit
        start = 700 - 41
        sizes, at = [], start
        for n in [cap, 1, cap, cap - 1 or 1] * 20:
            n = min(n, 700 - at)
            if n <= 0:
                break
            sizes.append((at, n))
            at += n
        rows = [(4, p) for p in range(start, at)]
        q = torch.randn(len(rows), Hq, hd, generator=g).to(dtype)
        qd = q.reshape(len(rows), -1).to(DEV).contiguous()
        out = torch.zeros(len(rows), Hq * hd, dtype=dtype, device=DEV)
        items = torch.tensor([(p0 - start, n, 4, p0) for p0, n in sizes], dtype=torch.int32,
                             device=DEV).reshape(-1)
        run(qd, out, items, len(sizes))
        check(rows, out, q)


@pytest.mark.parametrize("Hq,Hkv,hd,page,window", [(8, 2, 128, 16, None), (6, 3, 64, 8, 50),
                                                   (8, 1, 128, 16, 200), (3, 1, 64, 32, None),
                                                   (32, 8, 128, 64, None), (4, 4, 64, 128, 100)])
@pytest.mark.parametrize("norm", [True, False])
def test_attention_decode_fused(Hq, Hkv, hd, page, window, norm):
    """Norm, rotation, cache write and decode attention in one kernel, against the two kernels
    it stands for (and so, through their tests, against the plain formulas): outputs, the new
    keys and values in the cache, and the cleared projection; keys whole and split; a call that
    reads a cache it does not own."""
    from types import SimpleNamespace
    from llmario_b200 import kernels
    dtype = torch.bfloat16
    lengths = [1, 33, 150, 64, 700, 385, 32, 65]     # new tokens at the start and end of pages too
    rows = len(lengths)
    base, table, _, _ = paged_setup(lengths, page, Hkv, hd, dtype)
    scale, eps = 1 / math.sqrt(hd), 1e-5
    slot = torch.arange(rows, dtype=torch.int32, device=DEV)
    pos = torch.tensor([n - 1 for n in lengths], dtype=torch.int32, device=DEV)
    width = (Hq + 2 * Hkv) * hd
    proj = rnd(rows, width, scale=2.0, seed=3)
    qw = (1 + 0.1 * rnd(hd, seed=1)) if norm else None
    kw = (1 + 0.1 * rnd(hd, seed=2)) if norm else None
    inv_freq = torch.tensor(np.power(np.float32(1e4), -(np.arange(hd // 2, dtype=np.float32) * 2) / hd)
                            .astype(np.float32), device=DEV)
    cs = torch.empty(rows, hd // 2, 2, dtype=torch.float32, device=DEV)
    kernels.rope_table(pos, inv_freq, cs, 1.0)
    bufs = {}

    def buffer(name, shape, dt=torch.bfloat16, zero=False):
        return bufs.setdefault((name, tuple(shape)), torch.empty(*shape, dtype=dt, device=DEV))

    ctx = SimpleNamespace(rows=rows, max_pos=max(lengths) - 1, row_slot=slot, row_pos=pos,
                          buffer=buffer, dtype=dtype,
                          segments=[SimpleNamespace(rows=1) for _ in range(rows)])

    def view_of(storage):
        return SimpleNamespace(storage=storage, slot=1, k=storage[0, 1, 0], v=storage[0, 1, 1],
                               page_stride=storage.stride(0), block_table=table, page_size=page)

    for writes in (True, False):
        w = width if writes else Hq * hd
        for splits in (1, 3, 5):
            # the two kernels
            st_a, used_a = base.clone(), proj[:, :w].clone()
            q = torch.empty(rows, Hq * hd, dtype=dtype, device=DEV)
            kernels.qk_norm_rope_store(used_a, q, st_a[0, 1, 0] if writes else None,
                                       st_a[0, 1, 1] if writes else None, st_a.stride(0), table, slot,
                                       pos, qw, kw, inv_freq, 1.0, Hq, Hkv, hd, hd, page, eps, cs,
                                       clear_proj=True)
            ref = torch.zeros(rows, Hq * hd, dtype=dtype, device=DEV)
            po = torch.empty(rows * Hq * splits * hd, dtype=torch.float32, device=DEV)
            pml = torch.empty(rows * Hq * splits * 2, dtype=torch.float32, device=DEV)
            kernels.attention_decode_tma(q, ref, st_a, 1, table, None, rows, Hq, Hkv, hd, page, scale,
                                         window, splits, po, pml, slot, pos)
            if splits > 1:
                kernels.attention_merge(po, pml, ref, None, rows, Hq, hd, splits)
            # the one kernel
            st_b, used_b = base.clone(), proj[:, :w].clone()
            got = torch.zeros(rows, Hq * hd, dtype=dtype, device=DEV)
            assert kernels.decode_fusion_ok(ctx, view_of(st_b), Hq, Hkv, hd, hd, cs, window)
            kernels.attention_decode_fused(ctx, used_b, got, view_of(st_b), writes, qw, kw, cs, eps,
                                           True, Hq, Hkv, hd, scale, window, splits=splits)
            kernels.check_tc_status(DEV)
            assert int((used_b != 0).sum()) == 0 and int((used_a != 0).sum()) == 0
            # the cache: bit for bit what the rotation kernel wrote, or the neighbouring bfloat16
            # value where the two kernels' sums rounded differently
            diff = (st_b.float() - st_a.float()).abs()
            assert (diff <= 2.0 ** -7 * st_a.float().abs() + 1e-6).all()
            if writes:
                assert not torch.equal(st_a, base)
            else:
                assert torch.equal(st_b, base)
            assert (got.float() - ref.float()).abs().max() <= 2e-2, (writes, splits)

@pytest.mark.parametrize("page,window", [(16, None), (64, None), (16, 200), (64, 130)])
@pytest.mark.parametrize("kernel", ["decode", "decode_tma", "tcgen05", "tcgen05_x2"])
def test_tensor_core_attention_finds_the_key_that_stands_out(kernel, page, window):
    """Random keys would hide a tile, a page or a window's edge read wrongly.  Here single keys
    are made to dominate single query rows: far back among hundreds, on the last and the first
    slot of a page, on both sides of the edge between key tiles, on the first key a window still
    sees and (it must have no weight) on the last one it no longer sees.  The row's output must
    be that key's value."""
    from llmario_b200 import kernels
    Hq, Hkv, hd, n = 8, 2, 128, 700
    G = Hq // Hkv
    dtype = torch.bfloat16
    storage, table, ks, vs = paged_setup([n], page, Hkv, hd, dtype, seed=4)
    scale = 1 / math.sqrt(hd)
    last = n - 1
    lo = max(0, last + 1 - window) if window else 0
    targets = [t for t in (13, page - 1, page, 127, 128, 511, 512, 639, 640, last - 1, last) if t >= lo]
    if window:
        targets += [lo, lo + 1, lo - 1]          # lo - 1 is outside the window of the last position
    if kernel == "tcgen05_x2" and page < 32:
        pytest.skip("two query tiles per CTA need pages of 32 positions or more")
    cap = {"tcgen05": 128 // G, "tcgen05_x2": 256 // G}.get(kernel, 1)
    # rows: for the decode kernels one row per target, all at the last position; for the prompt
    # kernel one item of `cap` tokens that ends at the last position, a target for each of its
    # last rows (a row sees a target only if it lies at or before its own position)
    g = torch.Generator().manual_seed(9)
    if kernel.startswith("tcgen05"):
        rows = [(0, last - cap + 1 + i) for i in range(cap)]
        aim = {cap - 1 - j: t for j, t in enumerate(targets) if t <= last - j and
               (not window or t >= last - j + 1 - window or t == lo - 1)}
    else:
        rows = [(0, last)] * len(targets)
        aim = dict(enumerate(targets))
    q = torch.randn(len(rows), Hq, hd, generator=g)
    k = ks[0].float()
    for i, t in aim.items():      # head 0 of row i points at key t of KV head 0
        u = q[i, 0] / q[i, 0].norm()
        k[t, 0] = 60 * u
    ks[0] = k.to(dtype)
    for t in set(aim.values()):
        pg, sl = table[0, t // page].item(), t % page
        storage[pg, 1, 0, 0, sl] = ks[0][t, 0].to(DEV)
    q = q.to(dtype)
    qd = q.reshape(len(rows), -1).to(DEV).contiguous()
    out = torch.zeros(len(rows), Hq * hd, dtype=dtype, device=DEV)
    common = (storage[0, 1, 0], storage[0, 1, 1], storage.stride(0), table)
    if kernel.startswith("tcgen05"):
        items = torch.tensor([[0, cap, 0, rows[0][1]]], dtype=torch.int32, device=DEV).reshape(-1)
        fn = kernels.attention_tcgen05 if kernel == "tcgen05" else kernels.attention_tcgen05_x2
        fn(qd, out, *common, items, 1, Hq, Hkv, hd, page, scale, window, storage.shape[0])
    else:
        slot = torch.zeros(len(rows), dtype=torch.int32, device=DEV)
        pos = torch.tensor([p for _, p in rows], dtype=torch.int32, device=DEV)
        splits = 3
        po = torch.empty(len(rows) * Hq * splits * hd, dtype=torch.float32, device=DEV)
        pml = torch.empty(len(rows) * Hq * splits * 2, dtype=torch.float32, device=DEV)
        if kernel == "decode_tma":
            kernels.attention_decode_tma(qd, out, storage, 1, table, None, len(rows), Hq, Hkv, hd,
                                         page, scale, window, splits, po, pml, slot, pos)
        else:
            kernels.attention_decode(qd, out, *common, None, len(rows), Hq, Hkv, hd, page, scale,
                                     window, splits, po, pml, slot, pos)
        kernels.attention_merge(po, pml, out, None, len(rows), Hq, hd, splits)
    kernels.check_tc_status(DEV)
    seen = 0
    for i, (r, p) in enumerate(rows):
        ref = attention_ref(q[i].float(), ks[0].float(), vs[0].float(), p, window, scale)
        got = out[i].reshape(Hq, hd).double().cpu()
        assert (got - ref).abs().max() <= 2e-2, (i, p, aim.get(i), (got - ref).abs().max())
        t = aim.get(i)
        if t is None:
            continue
        row_lo = max(0, p + 1 - window) if window else 0
        if row_lo <= t <= p:      # visible: the output of head 0 is the value at the target
            assert (got[0] - vs[0][t, 0].double()).abs().max() < 2e-2, (i, p, t)
            seen += 1
        else:                     # outside the window: it has no weight at all
            assert (got[0] - vs[0][t, 0].double()).abs().max() > 0.5, (i, p, t)
    assert seen >= 5


@pytest.mark.parametrize("Hq,Hkv,hd,page,window", [(8, 2, 128, 16, None), (4, 4, 64, 8, 70),
                                                   (16, 2, 128, 32, None), (2, 2, 64, 64, None),
                                                   (32, 8, 128, 16, 300), (8, 4, 128, 4, None),
                                                   (8, 2, 128, 64, 200), (4, 2, 64, 128, None),
                                                   (8, 8, 128, 256, None)])
def test_attention_tcgen05(Hq, Hkv, hd, page, window):
    """The tcgen05 kernel for prompt portions: items of up to 128 / G tokens at the end of a long
    request (several key tiles, the diagonal tile, a window's edge), short items, and an item at
    the very start of a request."""
    from llmario_b200 import kernels
    dtype = torch.bfloat16
    G = Hq // Hkv
    cap = 128 // G
    lengths = [700, 40, 129]
    storage, table, ks, vs = paged_setup(lengths, page, Hkv, hd, dtype)
    scale = 1 / math.sqrt(hd)
    g = torch.Generator().manual_seed(7)
    # rows: the last 2.5 items of request 0, all of request 1 (from position 0), a 3-token tail
    spans = [(0, 700 - int(2.5 * cap), 700), (1, 0, 40), (2, 126, 129)]
    rows, items = [], []
    for r, a, b in spans:
        at = a
        while at < b:
            n = min(cap, b - at)
            items.append((len(rows), n, r, at))
            rows += [(r, p) for p in range(at, at + n)]
            at += n
    q = torch.randn(len(rows), Hq, hd, generator=g).to(dtype)
    qd = q.reshape(len(rows), -1).to(DEV).contiguous()
    out = torch.zeros(len(rows), Hq * hd, dtype=dtype, device=DEV)
    dev_items = torch.tensor(items, dtype=torch.int32, device=DEV).reshape(-1)
    if page >= 32:
        # two query tiles per CTA: the same rows as items of up to twice as many tokens
        rows2, items2 = [], []
        for r, a, b in spans:
            at = a
            while at < b:
                n = min(2 * cap, b - at)
                items2.append((len(rows2), n, r, at))
                rows2 += [(r, p) for p in range(at, at + n)]
                at += n
        assert rows2 == rows
        out2 = torch.zeros_like(out)
        kernels.attention_tcgen05_x2(qd, out2, storage[0, 1, 0], storage[0, 1, 1], storage.stride(0),
                                     table, torch.tensor(items2, dtype=torch.int32, device=DEV)
                                     .reshape(-1), len(items2), Hq, Hkv, hd, page, scale, window,
                                     storage.shape[0])
        kernels.check_tc_status(DEV)
        for i, (r, p) in enumerate(rows):
            ref = attention_ref(q[i].float(), ks[r].float(), vs[r].float(), p, window, scale)
            got = out2[i].reshape(Hq, hd).double().cpu()
            assert torch.isfinite(got).all(), (i, r, p)
            assert (got - ref).abs().max() <= 2e-2, ("x2", i, r, p, (got - ref).abs().max())
    # with the number of pages given, pages of 32 positions or more come by TMA; without, by copies
    for n_pages in (storage.shape[0], 0):
        out.zero_()
        kernels.attention_tcgen05(qd, out, storage[0, 1, 0], storage[0, 1, 1], storage.stride(0), table,
                                  dev_items, len(items), Hq, Hkv, hd, page, scale, window, n_pages)
        kernels.check_tc_status(DEV)
        for i, (r, p) in enumerate(rows):
            ref = attention_ref(q[i].float(), ks[r].float(), vs[r].float(), p, window, scale)
            got = out[i].reshape(Hq, hd).double().cpu()
            assert torch.isfinite(got).all(), (i, r, p)
            assert (got - ref).abs().max() <= 2e-2, (i, r, p, (got - ref).abs().max())


@pytest.mark.parametrize("Hq,Hkv,hd,page,window", [(32, 4, 128, 64, None), (32, 8, 64, 32, 200),
                                                   (16, 8, 128, 128, 150)])
def test_attention_tcgen05_persistent(Hq, Hkv, hd, page, window):
    """More (item, KV head) pairs than the GPU has SMs: the kernel then runs as one persistent
    CTA per SM that walks several pairs, its rings of tiles running on from one to the next.
    Whole prompts from their first position; against the plain formula on a sample of rows and,
    bit for bit, against the same kernel with one CTA per pair."""
    from llmario_b200 import kernels
    dtype = torch.bfloat16
    G = Hq // Hkv
    cap = 128 // G
    lengths = [900, 333, 64]
    storage, table, ks, vs = paged_setup(lengths, page, Hkv, hd, dtype)
    scale = 1 / math.sqrt(hd)
    g = torch.Generator().manual_seed(17)
    rows, items = [], []
    for r, n in enumerate(lengths):
        for at in range(0, n, cap):
            m = min(cap, n - at)
            items.append((len(rows), m, r, at))
            rows += [(r, p) for p in range(at, at + m)]
    assert len(items) * Hkv > kernels.sm_count()
    q = torch.randn(len(rows), Hq, hd, generator=g).to(dtype)
    qd = q.reshape(len(rows), -1).to(DEV).contiguous()
    dev_items = torch.tensor(items, dtype=torch.int32, device=DEV).reshape(-1)
    outs = []
    for persistent in (True, False):
        out = torch.zeros(len(rows), Hq * hd, dtype=dtype, device=DEV)
        kernels.attention_tcgen05(qd, out, storage[0, 1, 0], storage[0, 1, 1], storage.stride(0),
                                  table, dev_items, len(items), Hq, Hkv, hd, page, scale, window,
                                  storage.shape[0], persistent=persistent)
        kernels.check_tc_status(DEV)
        outs.append(out)
    assert torch.isfinite(outs[0].float()).all()
    assert torch.equal(outs[0], outs[1])
    rng = random.Random(3)
    sample = sorted(set([0, 1, cap - 1, cap, len(rows) - 1, 899, 900, 901] +
                        [rng.randrange(len(rows)) for _ in range(40)]))
    for i in sample:
        r, p = rows[i]
        ref = attention_ref(q[i].float(), ks[r].float(), vs[r].float(), p, window, scale)
        got = outs[0][i].reshape(Hq, hd).double().cpu()
        assert (got - ref).abs().max() <= 2e-2, (i, r, p, (got - ref).abs().max())


@pytest.mark.parametrize("Hq,Hkv,hd,page,window", [(32, 8, 128, 32, None), (16, 4, 64, 64, 900)])
def test_attention_tcgen05_x2_long_prompt_against_the_formulas(Hq, Hkv, hd, page, window):
    """Two query tiles per CTA on a prompt of 2,700 tokens (the length at which the engine
    chooses this kernel) and a portion that continues a request at position 2,700, directly
    against the float64 formula on a sample of rows: the first and last rows of items and of
    the two tiles of an item, rows whose keys end inside a page, and random ones."""
    from llmario_b200 import kernels
    dtype = torch.bfloat16
    G = Hq // Hkv
    cap = 2 * (128 // G)
    lengths = [2700, 2700 + 300]
    storage, table, ks, vs = paged_setup(lengths, page, Hkv, hd, dtype, seed=12)
    scale = 1 / math.sqrt(hd)
    spans = [(0, 0, 2700), (1, 2700, 3000)]
    rows, items = [], []
    for r, a, b in spans:
        for at in range(a, b, cap):
            n = min(cap, b - at)
            items.append((len(rows), n, r, at))
            rows += [(r, p) for p in range(at, at + n)]
    q = torch.randn(len(rows), Hq, hd, generator=torch.Generator().manual_seed(21)).to(dtype)
    out = torch.zeros(len(rows), Hq * hd, dtype=dtype, device=DEV)
    kernels.attention_tcgen05_x2(q.reshape(len(rows), -1).to(DEV).contiguous(), out,
                                 storage[0, 1, 0], storage[0, 1, 1], storage.stride(0), table,
                                 torch.tensor(items, dtype=torch.int32, device=DEV).reshape(-1),
                                 len(items), Hq, Hkv, hd, page, scale, window, storage.shape[0])
    kernels.check_tc_status(DEV)
    assert torch.isfinite(out.float()).all()
    rng = random.Random(5)
    sample = {0, 1, cap // 2 - 1, cap // 2, cap - 1, cap, 2699, 2700, 2700 + cap // 2, len(rows) - 1}
    sample |= {rng.randrange(len(rows)) for _ in range(30)}
    for i in sorted(sample):
        r, p = rows[i]
        ref = attention_ref(q[i].float(), ks[r].float(), vs[r].float(), p, window, scale)
        got = out[i].reshape(Hq, hd).double().cpu()
        assert (got - ref).abs().max() <= 2e-2, (i, r, p, float((got - ref).abs().max()))


@pytest.mark.parametrize("Hq,Hkv,hd,page,window", [(8, 2, 128, 16, None), (6, 3, 64, 8, 50),
                                                   (32, 8, 128, 64, None)])
@pytest.mark.parametrize("splits", [1, 4])
def test_attention_decode_fused_against_the_formulas(Hq, Hkv, hd, page, window, splits):
    """The fused decode kernel directly against float64: per-head norm of the new query and
    key, half-split rotation by the position's angles, the new key and value stored (as
    bfloat16) at the request's last position, attention over the cache."""
    from types import SimpleNamespace
    from llmario_b200 import kernels
    dtype = torch.bfloat16
    lengths = [1, 33, 150, 64, 700, 385, 32, 65]
    rows = len(lengths)
    storage, table, ks, vs = paged_setup(lengths, page, Hkv, hd, dtype, seed=2)
    scale, eps = 1 / math.sqrt(hd), 1e-5
    slot = torch.arange(rows, dtype=torch.int32, device=DEV)
    pos = torch.tensor([n - 1 for n in lengths], dtype=torch.int32, device=DEV)
    width = (Hq + 2 * Hkv) * hd
    proj = rnd(rows, width, scale=2.0, seed=3)
    qw, kw = 1 + 0.1 * rnd(hd, seed=1), 1 + 0.1 * rnd(hd, seed=2)
    inv = np.power(np.float32(1e4), -(np.arange(hd // 2, dtype=np.float32) * 2) / hd).astype(np.float32)
    cs = torch.empty(rows, hd // 2, 2, dtype=torch.float32, device=DEV)
    kernels.rope_table(pos, torch.tensor(inv, device=DEV), cs, 1.0)
    bufs = {}
    ctx = SimpleNamespace(rows=rows, max_pos=max(lengths) - 1, row_slot=slot, row_pos=pos, dtype=dtype,
                          buffer=lambda name, shape, dt=torch.bfloat16, zero=False: bufs.setdefault(
                              (name, tuple(shape)), torch.empty(*shape, dtype=dt, device=DEV)),
                          segments=[SimpleNamespace(rows=1) for _ in range(rows)])
    view = SimpleNamespace(storage=storage, slot=1, k=storage[0, 1, 0], v=storage[0, 1, 1],
                           page_stride=storage.stride(0), block_table=table, page_size=page)
    used = proj.clone()
    got = torch.zeros(rows, Hq * hd, dtype=dtype, device=DEV)
    kernels.attention_decode_fused(ctx, used, got, view, True, qw, kw, cs, eps, True, Hq, Hkv, hd,
                                   scale, window, splits=splits)
    kernels.check_tc_status(DEV)
    assert int((used != 0).sum()) == 0          # what was consumed of the projection is cleared

    def head_norm_rope(x, w, p):       # x [heads, hd] float64
        x = x * (1.0 / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)) * w
        ang = p * torch.tensor(inv, dtype=torch.float64)
        a, b = x[:, :hd // 2], x[:, hd // 2:]
        return torch.cat([a * torch.cos(ang) - b * torch.sin(ang),
                          a * torch.sin(ang) + b * torch.cos(ang)], -1)

    pr = proj.double().cpu()
    qwd, kwd = qw.double().cpu(), kw.double().cpu()
    for r, n in enumerate(lengths):
        p = n - 1
        q = head_norm_rope(pr[r, :Hq * hd].reshape(Hq, hd), qwd, p)
        k_new = head_norm_rope(pr[r, Hq * hd:(Hq + Hkv) * hd].reshape(Hkv, hd), kwd, p)
        v_new = pr[r, (Hq + Hkv) * hd:].reshape(Hkv, hd)
        k, v = ks[r].double().clone(), vs[r].double().clone()
        k[p], v[p] = k_new.bfloat16().double(), v_new.bfloat16().double()
        ref = attention_ref(q.bfloat16().double(), k, v, p, window, scale)
        err = (got[r].reshape(Hq, hd).double().cpu() - ref).abs().max()
        assert err <= 2e-2, (r, n, float(err))
        # the cache holds the new key and value at the request's last position
        pg, s = table[r, p // page].item(), p % page
        assert (storage[pg, 1, 0, :, s].double().cpu() - k_new).abs().max() <= 2e-2 * k_new.abs().max()
        assert (storage[pg, 1, 1, :, s].double().cpu() - v_new).abs().max() <= 2e-2 * v_new.abs().max()


@pytest.mark.parametrize("Hq,Hkv,hd,page,window", [(32, 8, 128, 16, None), (8, 2, 128, 64, None),
                                                   (6, 3, 64, 8, 50), (8, 1, 128, 16, 200),
                                                   (4, 4, 64, 128, 100), (16, 2, 128, 32, None)])
@pytest.mark.parametrize("ctas", [1, 7, 60, 444])
def test_attention_decode_persistent(Hq, Hkv, hd, page, window, ctas):
    """The persistent decode kernel: all (row, KV head) units' tiles shared evenly by a given
    number of one-warp CTAs, so that CTAs begin and end in the middle of units; with one CTA a
    single warp walks everything, with 444 most CTAs have one tile or none and units are cut as
    finely as the number of parts allows.  The parts buffers start as NaNs: a part nobody
    computes must be marked empty, and an empty part must not be read.  Against float64."""
    from llmario_b200 import kernels
    dtype = torch.bfloat16
    lengths = [1, 33, 150, 64, 700, 385, 65, 128, 129, 1000, 2, 447]
    storage, table, ks, vs = paged_setup(lengths, page, Hkv, hd, dtype, seed=9)
    scale = 1 / math.sqrt(hd)
    rows = [(r, n - 1) for r, n in enumerate(lengths)]
    q = torch.randn(len(rows), Hq, hd, generator=torch.Generator().manual_seed(6)).to(dtype)
    # one key stands out for head 0 of the longest request: far back, at a tile's edge
    far = 63 if not window else lengths[9] - window
    ks[9][far, 0] = (6 * math.sqrt(hd) * q[9, 0].float() / q[9, 0].float().norm()).to(dtype)
    storage[table[9, far // page].item(), 1, 0, 0, far % page] = ks[9][far, 0].to(DEV)
    qd = q.reshape(len(rows), -1).to(DEV).contiguous()
    slot = torch.arange(len(rows), dtype=torch.int32, device=DEV)
    pos = torch.tensor([p for _, p in rows], dtype=torch.int32, device=DEV)
    for parts in (2, 4):
        po = torch.full((len(rows) * Hq * parts * hd,), float("nan"), dtype=torch.float32, device=DEV)
        pml = torch.full((len(rows) * Hq * parts * 2,), float("nan"), dtype=torch.float32, device=DEV)
        out = torch.zeros(len(rows), Hq * hd, dtype=dtype, device=DEV)
        kernels.attention_decode_persistent(qd, po, pml, storage, 1, table, slot, pos, Hq, Hkv, hd,
                                            page, scale, window, parts, ctas)
        kernels.attention_merge(po, pml, out, None, len(rows), Hq, hd, parts)
        kernels.check_tc_status(DEV)
        assert torch.isfinite(out.float()).all(), (parts, ctas)
        for i, (r, p) in enumerate(rows):
            ref = attention_ref(q[i].float(), ks[r].float(), vs[r].float(), p, window, scale)
            got = out[i].reshape(Hq, hd).double().cpu()
            assert (got - ref).abs().max() <= 2e-2, (parts, ctas, i, r, p, float((got - ref).abs().max()))
        got = out[9].reshape(Hq, hd).float().cpu()[0]
        assert (got - vs[9][far, 0].float()).abs().max() < 0.1     # the key that stands out


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
@pytest.mark.parametrize("page,D,hd,Hkv", [(16, 128, 128, 2), (4, 64, 32, 3), (8, 128, 64, 1)])
def test_kv_gather(dtype, page, D, hd, Hkv):
    """Requests' keys and values copied from small pages into large scratch pages: every
    position in [lowest, highest] lands at its place, everything else of the scratch pages that
    the items name is zero (the tail behind the last position, positions below the lowest one,
    a page the request gave back), and nothing outside them is touched."""
    from llmario_b200 import kernels
    lengths = [300, 41, 130]
    storage, table, ks, vs = paged_setup(lengths, page, Hkv, hd, dtype, seed=5)
    table = table.clone()
    table[0, 0] = -1                      # request 0 has given its first page back to a window
    lows = [page + 3, 0, 70]              # lowest positions read (request 0: past the page it lost)
    items, tab = [], []
    pages = chunks = 0
    for r, n in enumerate(lengths):
        first_page = lows[r] // D
        n_pages = (n - 1) // D - first_page + 1
        items += [r, first_page * D, n_pages * (D // page), pages, lows[r], n - 1, chunks, 0]
        pages += n_pages
        chunks += n_pages * (D // page)
    scratch = torch.full((pages + 1, 1, 2, Hkv, D, hd), 7.0, dtype=dtype, device=DEV)
    kernels.kv_gather(storage[0, 1, 0], storage[0, 1, 1], storage.stride(0), table, page,
                      scratch[0, 0, 0], scratch[0, 0, 1], scratch.stride(0), D, Hkv, hd,
                      torch.tensor(items, dtype=torch.int32, device=DEV), len(lengths), chunks)
    got = scratch.float().cpu()
    assert bool((got[pages] == 7.0).all())            # the page behind the last one: untouched
    at = 0
    for r, n in enumerate(lengths):
        first_page = lows[r] // D
        n_pages = (n - 1) // D - first_page + 1
        for kv, src in ((0, ks[r]), (1, vs[r])):
            want = torch.zeros(n_pages * D, Hkv, hd)
            lo_chunk = (lows[r] // page) * page        # chunks are copied whole
            if r == 0:
                lo_chunk = max(lo_chunk, page)        # its first page is gone
            a, b = max(lo_chunk, first_page * D), n
            want[a - first_page * D:b - first_page * D] = src[a:b].float()
            # a chunk is copied whole: positions of the last source page behind the request's
            # end hold whatever the cache holds there (zeros in this cache)
            have = got[at:at + n_pages, 0, kv].permute(0, 2, 1, 3).reshape(n_pages * D, Hkv, hd)
            assert torch.equal(have, want), (r, kv)
        at += n_pages
