"""The allocation-free decode attention entry point, called through its exported C symbol.

Some users of the library cannot allocate device memory when they need attention (all memory
planned at start-up, no tolerance for the stall of an allocation, allocation reserved to another
framework's pool).  For them ``llm_attention_decode_no_alloc`` keeps its partial sums in an array
inside the library.  This test checks that it gives what the ordinary entry points give with
caller-allocated scratch, twice in a row (the array keeps the first call's contents), and that it
refuses a request larger than its array.
"""
import ctypes
import math

import pytest
import torch

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def _setup(lengths, page, Hkv, hd, seed):
    g = torch.Generator().manual_seed(seed)
    n_pages = sum(-(-n // page) for n in lengths) + 2
    perm = torch.randperm(n_pages, generator=g).tolist()
    storage = torch.zeros(n_pages, 1, 2, Hkv, page, hd, dtype=torch.bfloat16, device=DEV)
    table = torch.full((len(lengths), max(-(-n // page) for n in lengths)), -1, dtype=torch.int32)
    at = 0
    for r, n in enumerate(lengths):
        for j in range(-(-n // page)):
            table[r, j] = perm[at]
            m = min(page, n - j * page)
            storage[perm[at], 0, :, :, :m] = torch.randn(2, Hkv, m, hd, generator=g).to(torch.bfloat16).to(DEV)
            at += 1
    return storage, table.to(DEV)


def test_no_alloc_entry_point_matches_the_ordinary_one():
    from llmario_b200 import kernels
    lib = kernels.lib()
    fn = lib.llm_attention_decode_no_alloc
    P, I, L, F = ctypes.c_void_p, ctypes.c_int, ctypes.c_longlong, ctypes.c_float
    fn.argtypes = [P, P, P, P, L, P, I, P, P, I, I, I, I, I, F, I, I, P]
    fn.restype = I
    Hq, Hkv, hd, page = 8, 2, 128, 16
    scale = 1 / math.sqrt(hd)
    stream = torch.cuda.current_stream().cuda_stream
    for call, (lengths, splits) in enumerate([([300, 41, 1000, 7], 4), ([64, 513, 129], 3)]):
        storage, table = _setup(lengths, page, Hkv, hd, seed=call)
        rows = len(lengths)
        q = torch.randn(rows, Hq * hd, generator=torch.Generator().manual_seed(9 + call)).to(torch.bfloat16).to(DEV)
        slot = torch.arange(rows, dtype=torch.int32, device=DEV)
        pos = torch.tensor([n - 1 for n in lengths], dtype=torch.int32, device=DEV)
        want = torch.zeros(rows, Hq * hd, dtype=torch.bfloat16, device=DEV)
        po = torch.empty(rows * Hq * splits * hd, dtype=torch.float32, device=DEV)
        pml = torch.empty(rows * Hq * splits * 2, dtype=torch.float32, device=DEV)
        kernels.attention_flash(q, want, storage[0, 0, 0], storage[0, 0, 1], storage.stride(0), table,
                                None, rows, 16, Hq, Hkv, hd, page, scale, None, splits, po, pml,
                                slot, pos)
        kernels.attention_merge(po, pml, want, None, rows, Hq, hd, splits)
        got = torch.zeros_like(want)
        status = fn(q.data_ptr(), got.data_ptr(), storage[0, 0, 0].data_ptr(),
                    storage[0, 0, 1].data_ptr(), storage.stride(0), table.data_ptr(),
                    table.stride(0), slot.data_ptr(), pos.data_ptr(), rows, Hq, Hkv, hd, page,
                    scale, 0, splits, stream)
        assert status == 0
        torch.cuda.synchronize()
        # the same kernels on the same inputs: the tolerance of the attention tests (2e-2 for
        # bfloat16) is far more than needed, the results agree to the last bit
        assert (got.float() - want.float()).abs().max() <= 2e-2
        assert torch.equal(got, want)
    # beyond the array: refused, nothing launched
    too_many = fn(q.data_ptr(), got.data_ptr(), storage[0, 0, 0].data_ptr(),
                  storage[0, 0, 1].data_ptr(), storage.stride(0), table.data_ptr(), table.stride(0),
                  slot.data_ptr(), pos.data_ptr(), 4096, Hq, Hkv, hd, page, scale, 0, 32, stream)
    assert too_many == -3
    torch.cuda.synchronize()
