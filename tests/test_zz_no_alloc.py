"""The allocation-free decode attention entry point, called through its exported C symbol.

Some users of the library cannot allocate device memory when they need attention (all memory
planned at start-up, no tolerance for the stall of an allocation, allocation reserved to another
framework's pool).  For them ``llm_attention_decode_no_alloc`` keeps its partial sums in an array
inside the library.  This test checks its output against a float64 statement of attention and
against the ordinary entry points with caller-allocated scratch, on calls in a row that leave the
shared array dirty for one another (more parts than key tiles, one part, a window, other head
sizes), and that it refuses what it cannot do before launching anything.
"""
import ctypes
import math

import pytest
import torch

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def _setup(lengths, page, Hkv, hd, seed):
    """A paged cache with scrambled pages; also the keys and values per request, in order."""
    g = torch.Generator().manual_seed(seed)
    n_pages = sum(-(-n // page) for n in lengths) + 2
    perm = torch.randperm(n_pages, generator=g).tolist()
    storage = torch.zeros(n_pages, 1, 2, Hkv, page, hd, dtype=torch.bfloat16, device=DEV)
    table = torch.full((len(lengths), max(-(-n // page) for n in lengths)), -1, dtype=torch.int32)
    ks, vs = [], []
    at = 0
    for r, n in enumerate(lengths):
        kv = torch.randn(2, Hkv, n, hd, generator=g).to(torch.bfloat16)
        ks.append(kv[0].transpose(0, 1).contiguous())      # [n, Hkv, hd]
        vs.append(kv[1].transpose(0, 1).contiguous())
        for j in range(-(-n // page)):
            table[r, j] = perm[at]
            m = min(page, n - j * page)
            storage[perm[at], 0, :, :, :m] = kv[:, :, j * page:j * page + m].to(DEV)
            at += 1
    return storage, table.to(DEV), ks, vs


def _reference(q, k, v, pos, window, scale):
    """float64: q [Hq, hd], k/v [S, Hkv, hd]; one query at ``pos`` over keys lo..pos."""
    Hq, Hkv = q.shape[0], k.shape[1]
    lo = max(0, pos + 1 - window) if window else 0
    out = torch.zeros(q.shape, dtype=torch.float64)
    for h in range(Hq):
        kh = k[lo:pos + 1, h // (Hq // Hkv)].double()
        vh = v[lo:pos + 1, h // (Hq // Hkv)].double()
        w = torch.softmax((kh @ q[h].double()) * scale, 0)
        out[h] = w @ vh
    return out


def _entry():
    from llmario_b200 import kernels
    fn = kernels.lib().llm_attention_decode_no_alloc
    P, I, L, F = ctypes.c_void_p, ctypes.c_int, ctypes.c_longlong, ctypes.c_float
    fn.argtypes = [P, P, P, P, L, P, I, P, P, I, I, I, I, I, F, I, I, P]
    fn.restype = I
    return fn


# (lengths, heads, KV heads, head size, page, window, parts); the calls run in this order and
# share the library's array, each finding what the one before left in it
CALLS = [
    ([300, 41, 1000, 7], 8, 2, 128, 16, 0, 4),
    ([64, 513, 129], 8, 2, 128, 16, 0, 3),
    ([20, 700, 33], 8, 2, 128, 16, 0, 16),      # more parts than key tiles: parts without keys
    ([300, 41, 1000, 7], 8, 2, 128, 16, 0, 1),  # one part: no merge, the output written directly
    ([500, 90, 260], 8, 2, 128, 16, 100, 4),    # a window: parts wholly below it hold no keys
    ([150, 333], 12, 3, 64, 32, 0, 3),          # another head size, group and page
    ([77, 200], 4, 4, 32, 8, 50, 2),
]


def test_no_alloc_entry_point_matches_attention_and_the_ordinary_entry_point():
    from llmario_b200 import kernels
    fn = _entry()
    stream = torch.cuda.current_stream().cuda_stream
    for call, (lengths, Hq, Hkv, hd, page, window, splits) in enumerate(CALLS):
        scale = 1 / math.sqrt(hd)
        storage, table, ks, vs = _setup(lengths, page, Hkv, hd, seed=call)
        rows = len(lengths)
        q = torch.randn(rows, Hq, hd, generator=torch.Generator().manual_seed(9 + call))
        # one key is made to stand out for the first head of every KV head: in the last part of
        # the keys for even calls, at the lower edge of what the row may see for odd ones
        for r, n in enumerate(lengths):
            lo = max(0, n - window) if window else 0
            at = n - 1 - (r % 3) if call % 2 == 0 else lo
            for kvh in range(Hkv):
                h = kvh * (Hq // Hkv)
                ks[r][at, kvh] = (6 * math.sqrt(hd) * q[r, h] / q[r, h].norm()).to(torch.bfloat16)
            pg, s = table[r, at // page].item(), at % page
            storage[pg, 0, 0, :, s] = ks[r][at].to(DEV)
        q16 = q.reshape(rows, Hq * hd).to(torch.bfloat16).to(DEV)
        slot = torch.arange(rows, dtype=torch.int32, device=DEV)
        pos = torch.tensor([n - 1 for n in lengths], dtype=torch.int32, device=DEV)
        got = torch.zeros(rows, Hq * hd, dtype=torch.bfloat16, device=DEV)
        status = fn(q16.data_ptr(), got.data_ptr(), storage[0, 0, 0].data_ptr(),
                    storage[0, 0, 1].data_ptr(), storage.stride(0), table.data_ptr(),
                    table.stride(0), slot.data_ptr(), pos.data_ptr(), rows, Hq, Hkv, hd, page,
                    scale, window, splits, stream)
        assert status == 0, (call, status)
        torch.cuda.synchronize()
        for r, n in enumerate(lengths):
            ref = _reference(q16[r].float().cpu().reshape(Hq, hd), ks[r].float(), vs[r].float(),
                             n - 1, window, scale)
            err = (got[r].double().cpu().reshape(Hq, hd) - ref).abs().max()
            assert err <= 2e-2, (call, r, float(err))      # the tolerance of the attention tests
            lo = max(0, n - window) if window else 0
            at = n - 1 - (r % 3) if call % 2 == 0 else lo
            head0 = got[r].float().cpu().reshape(Hq, hd)[0]
            # the key that stands out takes nearly all the weight: the output is its value
            assert (head0 - vs[r][at, 0].float()).abs().max() < 0.1, (call, r)
        # the ordinary entry points with scratch the caller allocates give the same bits
        want = torch.zeros_like(got)
        po = torch.empty(rows * Hq * splits * hd, dtype=torch.float32, device=DEV)
        pml = torch.empty(rows * Hq * splits * 2, dtype=torch.float32, device=DEV)
        kernels.attention_flash(q16, want, storage[0, 0, 0], storage[0, 0, 1], storage.stride(0),
                                table, None, rows, 16, Hq, Hkv, hd, page, scale, window or None,
                                splits, po, pml, slot, pos)
        if splits > 1:
            kernels.attention_merge(po, pml, want, None, rows, Hq, hd, splits)
        torch.cuda.synchronize()
        assert torch.equal(got, want), call


def test_no_alloc_entry_point_refuses_before_it_launches():
    fn = _entry()
    stream = torch.cuda.current_stream().cuda_stream
    Hq, Hkv, hd, page = 8, 2, 128, 16
    storage, table, _, _ = _setup([40], page, Hkv, hd, seed=1)
    q = torch.zeros(4096, Hq * hd, dtype=torch.bfloat16, device=DEV)
    out = torch.full_like(q, 7.0)
    slot = torch.zeros(4096, dtype=torch.int32, device=DEV)
    pos = torch.full((4096,), 39, dtype=torch.int32, device=DEV)

    def call(rows=1, heads=Hq, kv=Hkv, size=hd, pg=page, window=0, splits=2):
        return fn(q.data_ptr(), out.data_ptr(), storage[0, 0, 0].data_ptr(),
                  storage[0, 0, 1].data_ptr(), storage.stride(0), table.data_ptr(), table.stride(0),
                  slot.data_ptr(), pos.data_ptr(), rows, heads, kv, size, pg, 1.0, window, splits,
                  stream)

    assert call(rows=4096, splits=32) == -3        # beyond the array
    assert call(heads=34, kv=2) == -1              # 17 query heads on a KV head: one warp holds 16
    assert call(size=96) == -1                     # a head size without a kernel
    assert call(pg=0) == -2 and call(window=-1) == -2
    assert call(splits=0) == -2 and call(splits=70000) == -2
    assert call(heads=7, kv=2) == -2               # heads that cannot be shared evenly
    torch.cuda.synchronize()
    assert bool((out == 7.0).all())                # nothing was launched, nothing written
    assert call(heads=32, kv=2) == 0               # 16 heads on a KV head is the largest group
    torch.cuda.synchronize()
