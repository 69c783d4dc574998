"""Python face of the CUDA kernels: argument checks, pointers, status codes.

Each function launches one hand-written kernel of ``csrc/`` on the current CUDA stream of torch.
There is no other implementation behind these functions: a tensor that is not on a CUDA device,
or a library that cannot be built, is an error.
"""
from __future__ import annotations

import ctypes
from ctypes import c_float, c_int, c_longlong, c_void_p
from typing import Optional

import torch

from .csrc.build import load_library

F32, BF16 = 0, 1
_DT = {torch.float32: F32, torch.bfloat16: BF16}


class KernelError(RuntimeError):
    pass


_lib = None


def lib():
    global _lib
    if _lib is None:
        _lib = load_library()
        _declare(_lib)
    return _lib


def _signatures():
    """Argument types of every exported entry point, as the C sources declare them (a test
    compares the two): P pointer or stream, I int, L long long, F float."""
    P, I, L, F = c_void_p, c_int, c_longlong, c_float
    return {
        "llm_embed": [P, P, I, P, I, I, I, P, P],
        "llm_rms_norm": [P, P, P, I, P, I, I, F, P],
        "llm_patch_tokens": [P, P, P, I, P],
        "llm_silu_mul": [P, P, I, I, I, P],
        "llm_add_bias": [P, I, P, I, I, P],
        "llm_table_update": [P, I, P, I, P],
        "llm_table_update_counted": [P, I, P, P, I, P],
        "llm_zero_slots": [P, L, P, P, I, P],
        "llm_kv_gather": [P, P, L, P, I, I, P, P, L, I, I, I, I, P, I, I, P],
        "llm_gemm_simt": [P, I, P, I, P, I, I, I, I, I, I, I, I, P],
        "llm_qk_norm_rope_store": [P, I, P, P, P, I, L, P, I, P, P, P, P, P, P, F, I, I, I, I, I,
                                   I, F, I, I, I, P],
        "llm_rope_table": [P, P, P, I, I, F, P],
        "llm_attention_generic": [P, P, P, P, I, L, P, I, P, P, I, I, I, I, I, F, I, P],
        "llm_sample": [P, L, I, I, P, P, P, P, P, P, P, P, P],
        "llm_gemv_bf16": [P, P, P, I, I, I, I, I, I, I, I, I, P],
        "llm_gemm_tcgen05": [P, P, P, I, I, I, I, I, I, I, I, I, I, I, I, P, P],
        "llm_attention_flash": [P, P, P, P, P, P, L, P, I, P, P, P, I, I, I, I, I, I, F, I, I, P],
        "llm_attention_merge": [P, P, P, P, I, I, I, I, P],
        "llm_attention_merge_clear": [P, P, P, P, I, I, I, I, P, I, P],
        "llm_attention_decode_fused": [P, I, P, P, P, P, L, I, I, P, P, L, P, I, P, P, I, P, P, P,
                                       F, I, I, I, I, I, F, I, I, P, P],
        "llm_attention_decode": [P, P, P, P, P, P, L, P, I, P, P, P, I, I, I, I, I, F, I, I, P],
        "llm_attention_decode_tma": [P, P, P, P, P, L, I, I, P, I, P, P, P, I, I, I, I, I, F, I,
                                     I, P, P],
        "llm_attention_decode_persistent": [P, P, P, P, L, I, I, P, I, P, P, I, I, I, I, I, F, I, I, I,
                                            P, P],
        "llm_attention_tcgen05": [P, P, I, P, P, L, L, P, I, P, I, I, I, I, I, F, I, I, P, P],
        "llm_attention_tcgen05_x2": [P, P, I, P, P, L, L, P, I, P, I, I, I, I, I, F, I, P, P],
        "llm_apply_penalties": [P, L, I, P, I, P, P, P, P, P, I, P],
        "llm_random_normal": [P, I, L, ctypes.c_ulonglong, ctypes.c_double, ctypes.c_double, L,
                              P],
    }


def _declare(l) -> None:
    sigs = _signatures()
    for name, args in sigs.items():
        if hasattr(l, name):
            fn = getattr(l, name)
            fn.argtypes = args
            fn.restype = c_int


_raw_stream = getattr(torch._C, "_cuda_getCurrentRawStream", None)
_device_index: Optional[int] = None


def _stream() -> int:
    """The CUDA stream that torch regards as current on this process's device.  (The direct
    query takes a fraction of a microsecond where ``torch.cuda.current_stream()`` takes several;
    a step launches a few hundred kernels.)"""
    global _device_index
    if _raw_stream is None:
        return torch.cuda.current_stream().cuda_stream
    if _device_index is None:
        _device_index = torch.cuda.current_device()
    return _raw_stream(_device_index)


def _ptr(t: Optional[torch.Tensor]) -> Optional[int]:
    return None if t is None else t.data_ptr()


def _dt(t: torch.Tensor) -> int:
    try:
        return _DT[t.dtype]
    except KeyError:
        raise KernelError(f"unsupported dtype {t.dtype}") from None


def _cuda(*tensors: Optional[torch.Tensor]) -> None:
    for t in tensors:
        if t is not None and not t.is_cuda:
            raise KernelError("llmario_b200 kernels run on a CUDA device only; got a tensor on "
                              f"{t.device}")


launches = 0   # kernels of this library launched so far (a claim that bench.py reports)


def _check(status: int, what: str) -> None:
    global launches
    if status == 0:
        launches += 1
        return
    if status == -1:
        raise KernelError(f"{what}: size or dtype not supported by this kernel")
    if status == -2:
        raise KernelError(f"{what}: inconsistent arguments")
    raise KernelError(f"{what}: CUDA error {status}")


# ------------------------------------------------------------------------------------------
def embed(tokens: torch.Tensor, table: torch.Tensor, out: torch.Tensor,
          err_flag: torch.Tensor) -> None:
    """out[t] = table[tokens[t]] as float32; a token outside the table sets err_flag to 1 + t."""
    _cuda(tokens, table, out, err_flag)
    assert tokens.dtype == torch.int32 and out.dtype == torch.float32
    assert table.is_contiguous() and out.is_contiguous()
    rows, width = out.shape
    _check(lib().llm_embed(_ptr(tokens), _ptr(table), _dt(table), _ptr(out), rows, width,
                           table.shape[0], _ptr(err_flag), _stream()), "embed")


def rms_norm(x: torch.Tensor, weight: torch.Tensor, out: torch.Tensor, eps: float,
             rows_index: Optional[torch.Tensor] = None) -> None:
    """out[r] = x[rows_index[r] or r] * rsqrt(mean(x^2) + eps) * weight, x and weight float32."""
    _cuda(x, weight, out, rows_index)
    assert x.dtype == torch.float32 and weight.dtype == torch.float32
    assert x.is_contiguous() and out.is_contiguous()
    rows, width = out.shape
    assert x.shape[1] == width and weight.numel() == width
    _check(lib().llm_rms_norm(_ptr(x), _ptr(weight), _ptr(out), _dt(out), _ptr(rows_index), rows,
                              width, float(eps), _stream()), "rms_norm")


def silu_mul(gate_up: torch.Tensor, out: torch.Tensor) -> None:
    """out[t][j] = silu(gate_up[t][j]) * gate_up[t][ff + j]."""
    _cuda(gate_up, out)
    assert gate_up.dtype == torch.float32 and gate_up.is_contiguous() and out.is_contiguous()
    rows, ff = out.shape
    assert gate_up.shape == (rows, 2 * ff)
    _check(lib().llm_silu_mul(_ptr(gate_up), _ptr(out), _dt(out), rows, ff, _stream()),
           "silu_mul")


def add_bias(out: torch.Tensor, bias: torch.Tensor) -> None:
    """out[t][j] += bias[j] (bias float32; the sum is made in 32-bit and rounded once)."""
    _cuda(out, bias)
    rows, width = out.shape
    assert out.is_contiguous() and bias.dtype == torch.float32 and bias.shape == (width,)
    _check(lib().llm_add_bias(_ptr(out), _dt(out), _ptr(bias), rows, width, _stream()), "add_bias")


def table_update(table: torch.Tensor, updates: torch.Tensor, n: int) -> None:
    """table[u[0]][u[1]] = u[2] for the first n int32 triples of ``updates``."""
    _cuda(table, updates)
    assert table.dtype == torch.int32 and updates.dtype == torch.int32
    _check(lib().llm_table_update(_ptr(table), table.stride(0), _ptr(updates), n, _stream()),
           "table_update")


def patch_tokens(tokens: torch.Tensor, source: torch.Tensor, index: torch.Tensor) -> None:
    """tokens[i] = source[index[i]] for every i with index[i] >= 0 (all int32, on the device)."""
    _cuda(tokens, source, index)
    assert tokens.dtype == source.dtype == index.dtype == torch.int32
    assert tokens.numel() == index.numel()
    _check(lib().llm_patch_tokens(_ptr(tokens), _ptr(source), _ptr(index), tokens.numel(),
                                  _stream()), "patch_tokens")


def table_update_counted(table: torch.Tensor, updates: torch.Tensor, count: torch.Tensor,
                         max_n: int) -> None:
    """As :func:`table_update`, the number of triples read from ``count[0]`` on the device."""
    _cuda(table, updates, count)
    assert table.dtype == torch.int32 and updates.dtype == torch.int32
    _check(lib().llm_table_update_counted(_ptr(table), table.stride(0), _ptr(updates),
                                          _ptr(count), max_n, _stream()), "table_update")


def zero_slots(state: torch.Tensor, slots: torch.Tensor, count: torch.Tensor, max_n: int) -> None:
    """state[slots[i]] = 0 for i < count[0] (read on the device; at most ``max_n``)."""
    _cuda(state, slots, count)
    assert state.is_contiguous() and slots.dtype == torch.int32 and count.dtype == torch.int32
    row_bytes = state[0].numel() * state.element_size()
    _check(lib().llm_zero_slots(_ptr(state), row_bytes, _ptr(slots), _ptr(count), max_n,
                                _stream()), "zero_slots")


def kv_gather(k_src: torch.Tensor, v_src: torch.Tensor, src_page_stride: int,
              block_table: torch.Tensor, page_size: int, k_dst: torch.Tensor, v_dst: torch.Tensor,
              dst_page_stride: int, dst_page_size: int, num_kv_heads: int, head_dim: int,
              items: torch.Tensor, n_items: int, total_chunks: int) -> None:
    """Copy requests' keys and values from cache pages of ``page_size`` positions into scratch
    pages of ``dst_page_size`` (a multiple).  ``k_src`` / ``v_src`` / ``k_dst`` / ``v_dst``: the
    K and V planes of page 0 on either side, pages ``*_page_stride`` elements apart.  ``items``:
    int32 octuples (block-table row, first position, chunks, first scratch page, lowest and
    highest position read, chunks of the items before, 0); a chunk is one source page; chunks
    wholly outside [lowest, highest] or whose page the request no longer holds become zeros."""
    _cuda(k_src, v_src, block_table, k_dst, v_dst, items)
    assert k_src.dtype == k_dst.dtype and items.dtype == torch.int32
    _check(lib().llm_kv_gather(_ptr(k_src), _ptr(v_src), src_page_stride, _ptr(block_table),
                               block_table.stride(0), page_size, _ptr(k_dst), _ptr(v_dst),
                               dst_page_stride, dst_page_size, num_kv_heads, head_dim, _dt(k_src),
                               _ptr(items), n_items, total_chunks, _stream()), "kv_gather")


def gemm_simt(a: torch.Tensor, w: torch.Tensor, out: torch.Tensor, accumulate: bool = False
              ) -> None:
    """out (=|+=) a @ w.T on the CUDA cores with 32-bit accumulation; a [M,K], w [N,K]."""
    _cuda(a, w, out)
    M, K = a.shape
    N = w.shape[0]
    assert w.shape[1] == K and out.shape == (M, N)
    assert a.stride(1) == 1 and w.stride(1) == 1 and out.stride(1) == 1
    _check(lib().llm_gemm_simt(_ptr(a), _dt(a), _ptr(w), _dt(w), _ptr(out), _dt(out), M, N, K,
                               a.stride(0), w.stride(0), out.stride(0), int(accumulate),
                               _stream()), "gemm_simt")


def qk_norm_rope_store(proj: torch.Tensor, q_out: torch.Tensor,
                       k_cache: Optional[torch.Tensor], v_cache: Optional[torch.Tensor],
                       page_stride: int, block_table: torch.Tensor, row_slot: torch.Tensor,
                       row_pos: torch.Tensor, q_norm_w: Optional[torch.Tensor],
                       k_norm_w: Optional[torch.Tensor], inv_freq: Optional[torch.Tensor],
                       attn_factor: float, num_heads: int, num_kv_heads: int, head_dim: int,
                       rot_dim: int, page_size: int, eps: float,
                       cos_sin: Optional[torch.Tensor] = None, clear_proj: bool = False) -> None:
    """Per-head norm, rotation and stores for the rows of ``proj`` (float32,
    [rows, (Hq + 2 Hkv) * hd], or [rows, Hq * hd] when no cache is given)."""
    _cuda(proj, q_out, k_cache, v_cache, block_table, row_slot, row_pos, q_norm_w, k_norm_w,
          inv_freq)
    assert proj.dtype == torch.float32 and proj.stride(1) == 1
    rows = proj.shape[0]
    has_kv = k_cache is not None
    use_norm = q_norm_w is not None
    if rot_dim > 0:
        assert inv_freq is not None and inv_freq.dtype == torch.float32
        assert inv_freq.numel() == rot_dim // 2
    _check(lib().llm_qk_norm_rope_store(
        _ptr(proj), proj.stride(0), _ptr(q_out), _ptr(k_cache), _ptr(v_cache), _dt(q_out),
        page_stride, _ptr(block_table), block_table.stride(0), _ptr(row_slot), _ptr(row_pos),
        _ptr(q_norm_w), _ptr(k_norm_w), _ptr(inv_freq), _ptr(cos_sin), float(attn_factor), rows,
        num_heads,
        num_kv_heads, head_dim, rot_dim, page_size, float(eps), int(has_kv), int(use_norm),
        int(clear_proj), _stream()), "qk_norm_rope_store")


def rope_table(row_pos: torch.Tensor, inv_freq: torch.Tensor, out: torch.Tensor,
               attn_factor: float) -> None:
    """out[t][i] = attn_factor * (cos, sin)(row_pos[t] * inv_freq[i]), float32 [rows, half, 2]."""
    _cuda(row_pos, inv_freq, out)
    rows, half = out.shape[0], out.shape[1]
    assert out.dtype == torch.float32 and out.is_contiguous() and inv_freq.numel() == half
    _check(lib().llm_rope_table(_ptr(row_pos), _ptr(inv_freq), _ptr(out), rows, half,
                                float(attn_factor), _stream()), "rope_table")


def attention_generic(q: torch.Tensor, out: torch.Tensor, k_cache: torch.Tensor,
                      v_cache: torch.Tensor, page_stride: int, block_table: torch.Tensor,
                      row_slot: torch.Tensor, row_pos: torch.Tensor, num_heads: int,
                      num_kv_heads: int, head_dim: int, page_size: int, scale: float,
                      window: Optional[int]) -> None:
    _cuda(q, out, k_cache, v_cache, block_table, row_slot, row_pos)
    assert q.dtype == out.dtype == k_cache.dtype and q.is_contiguous() and out.is_contiguous()
    rows = q.shape[0]
    _check(lib().llm_attention_generic(
        _ptr(q), _ptr(out), _ptr(k_cache), _ptr(v_cache), _dt(q), page_stride, _ptr(block_table),
        block_table.stride(0), _ptr(row_slot), _ptr(row_pos), rows, num_heads, num_kv_heads,
        head_dim, page_size, float(scale), int(window or 0), _stream()),
        f"attention (head_dim {head_dim})")


def sample(logits: torch.Tensor, temperature: torch.Tensor, top_k: torch.Tensor,
           top_p: torch.Tensor, min_p: torch.Tensor, uniform: torch.Tensor,
           out: torch.Tensor, status_out: Optional[torch.Tensor] = None) -> None:
    """One token per row of ``logits`` (float32 [rows, vocab]): greedy where temperature <= 0,
    else top-k, top-p, min-p, temperature, softmax and a draw with the row's uniform.
    ``status_out`` (int32 [4]): the kernel also copies the library's status words there (see
    :func:`status_words`), so that they reach the host in the same copy as the tokens."""
    _cuda(logits, temperature, top_k, top_p, min_p, uniform, out, status_out)
    assert logits.dtype == torch.float32 and logits.stride(1) == 1
    assert uniform.dtype == torch.float64 and top_k.dtype == torch.int32
    rows, vocab = logits.shape
    status = status_words(logits.device) if status_out is not None else None
    _check(lib().llm_sample(_ptr(logits), logits.stride(0), rows, vocab, _ptr(temperature),
                            _ptr(top_k), _ptr(top_p), _ptr(min_p), _ptr(uniform), _ptr(out),
                            _ptr(status), _ptr(status_out), _stream()), "sample")


def apply_penalties(logits: torch.Tensor, triples: torch.Tensor, n: int, repeat: torch.Tensor,
                    freq: torch.Tensor, presence: torch.Tensor,
                    inflight_src: Optional[torch.Tensor] = None,
                    drawn: Optional[torch.Tensor] = None) -> None:
    """For the first n (row, token, count) triples adjust logits[row][token] in place.
    ``inflight_src`` (int32 per row, -1: none) names, by its index in ``drawn``, a token that
    enters the row's window but is still being drawn by the step before: it counts once more."""
    _cuda(logits, triples, repeat, freq, presence, inflight_src, drawn)
    assert (inflight_src is None) == (drawn is None)
    _check(lib().llm_apply_penalties(_ptr(logits), logits.stride(0), logits.shape[1], _ptr(triples),
                                     n, _ptr(repeat), _ptr(freq), _ptr(presence),
                                     _ptr(inflight_src), _ptr(drawn), logits.shape[0], _stream()),
           "apply_penalties")


def random_normal(out: torch.Tensor, key: int, mean: float, std: float, first: int = 0) -> None:
    """out.flat[i] = mean + std * z(key, first + i), z a standard normal that is a function of
    the key and the index alone (the same bits as ``weights.random_normal`` gives on a host)."""
    _cuda(out)
    assert out.is_contiguous()
    _check(lib().llm_random_normal(_ptr(out), _dt(out), out.numel(), int(key), float(mean),
                                   float(std), int(first), _stream()), "random_normal")


# ------------------------------------------------------------------------------------------
# dispatch: which kernel serves which dtype and size
# ------------------------------------------------------------------------------------------
GEMV_MAX_ROWS = 8


def _gemv_ok(a: torch.Tensor, w: torch.Tensor) -> bool:
    return (a.dtype == torch.bfloat16 and w.dtype == torch.bfloat16
            and a.shape[0] <= GEMV_MAX_ROWS and a.shape[1] % 8 == 0
            and a.stride(0) % 8 == 0 and w.stride(0) % 8 == 0
            and a.data_ptr() % 16 == 0 and w.data_ptr() % 16 == 0)


def gemv_bf16(a: torch.Tensor, w: torch.Tensor, out: torch.Tensor, mode: int, half: int = 0
              ) -> None:
    """Weight-streaming product for up to 8 rows.  mode 0: out = a w^T; 1: out += a w^T
    (float32); 2: out = silu(a wg^T) * (a wu^T) with w = [wg; wu], ``half`` rows each."""
    _cuda(a, w, out)
    M, K = a.shape
    N = w.shape[0]
    _check(lib().llm_gemv_bf16(_ptr(a), _ptr(w), _ptr(out), _dt(out), M, N, K, a.stride(0),
                               w.stride(0), out.stride(0), mode, half, _stream()), "gemv_bf16")


_tc_status = {}


def tc_status(device) -> torch.Tensor:
    """The device word in which the tensor-core kernels record a wait that gave up."""
    st = _tc_status.get(device)          # (keyed by the device object first: no conversions)
    if st is None:
        key = torch.device(device).index or 0
        if key not in _tc_status:
            _tc_status[key] = torch.zeros(4, dtype=torch.int32, device=device)
        st = _tc_status[device] = _tc_status[key]
    return st


status_words = tc_status       # word 0: a wait that gave up; word 1: 1 + row of a bad token id


def status_message(words) -> Optional[str]:
    """What non-zero status words say, or None when all is well."""
    if words[0]:
        return f"a tcgen05 / TMA kernel gave up waiting on a barrier (role {int(words[0])})"
    if words[1]:
        return f"token id outside the embedding table at row {int(words[1]) - 1} of a step"
    return None


def clear_status(device) -> None:
    st = _tc_status.get(torch.device(device).index or 0)
    if st is not None:
        st.zero_()


def check_tc_status(device) -> None:
    """Raise if a kernel recorded a failure in the status words: a tensor-core kernel that gave
    up waiting, or a token id outside the embedding table (synchronises the device; the words
    are cleared)."""
    st = _tc_status.get(torch.device(device).index or 0)
    if st is not None:
        msg = status_message(st.tolist())
        if msg:
            st.zero_()
            raise KernelError(msg)


def selftest_wait_gives_up(device, limit_cycles: int = 20000) -> None:
    """Launch a one-block kernel that waits on a barrier at which nothing ever arrives, with a
    limit of ``limit_cycles`` clock cycles (microseconds) instead of the two seconds of the real
    kernels.  It gives up, records role 99 in the status words and returns: the way every
    bounded wait of the TMA / tcgen05 kernels ends, made to happen without a fault."""
    l = lib()
    l.llm_selftest_wait_gives_up.argtypes = [c_void_p, c_longlong, c_void_p]
    l.llm_selftest_wait_gives_up.restype = c_int
    _check(l.llm_selftest_wait_gives_up(_ptr(status_words(device)), int(limit_cycles), _stream()),
           "selftest_wait_gives_up")


def token_tile(rows: int) -> int:
    """Tokens per tile of the tensor-core product: the smallest tile that holds the rows, 256
    (the persistent kernel) once there are enough rows to fill the GPU with such tiles."""
    for bn in (16, 32, 64, 128):
        if rows <= bn:
            return bn
    return 256 if rows >= 512 else 128


def _tc_ok(a: torch.Tensor, w: torch.Tensor) -> bool:
    return (a.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and a.shape[1] % 8 == 0
            and a.stride(0) % 8 == 0 and w.stride(0) % 8 == 0 and a.stride(1) == 1
            and w.stride(1) == 1 and a.data_ptr() % 16 == 0 and w.data_ptr() % 16 == 0)


def use_cta_pairs(on: bool) -> None:
    """Whether products of many rows run on CTA pairs (tcgen05 cta_group::2; the default) or on
    the one-CTA persistent kernel.  For comparisons."""
    l = lib()
    l.llm_set_pair.argtypes = [c_int]
    l.llm_set_pair.restype = None
    l.llm_set_pair(int(on))


def force_pair_k_ranges(n: int) -> None:
    """Cut K into ``n`` ranges in the CTA-pair product that adds into its output, whatever its
    own cost model would choose; 0 gives the choice back to the model.  For measurements."""
    l = lib()
    l.llm_set_pair_ksplits.argtypes = [c_int]
    l.llm_set_pair_ksplits.restype = None
    l.llm_set_pair_ksplits(int(n))


def use_dependent_launch(on: bool) -> None:
    """Whether kernels are launched as programmatic dependents of the one before them (the
    default) or wait for its end.  For measurements."""
    l = lib()
    l.llm_set_pdl.argtypes = [c_int]
    l.llm_set_pdl.restype = None
    l.llm_set_pdl(int(on))


def gemm_tcgen05(a: torch.Tensor, w: torch.Tensor, out: torch.Tensor, mode: int, half: int = 0,
                 bn: Optional[int] = None, splits: int = 1, out_is_zero: bool = False) -> None:
    """Tensor-core product of bfloat16 operands.  mode 0: out = a w^T (bfloat16 or float32);
    1: out += a w^T (float32); 2: out = silu(a wg^T) * (a wu^T), w = [wg; wu] of ``half`` rows
    each; 3: the same with w stored as alternating blocks of 16 gate rows and 16 up rows.
    ``bn``: token tile (16..256); ``splits`` > 1 splits K and adds partial sums with atomics
    (mode 0 then needs ``out`` float32, zeroed here unless ``out_is_zero``)."""
    _cuda(a, w, out)
    T, K = a.shape
    N = w.shape[0]
    assert out.stride(1) == 1
    bn = bn or token_tile(T)
    _check(lib().llm_gemm_tcgen05(_ptr(a), _ptr(w), _ptr(out), _dt(out), T, N, K, a.stride(0),
                                  w.stride(0), out.stride(0), mode, half, bn, splits,
                                  int(out_is_zero), _ptr(tc_status(a.device)), _stream()),
           "gemm_tcgen05")


_sm_count: Optional[int] = None


def sm_count() -> int:
    """Streaming multiprocessors of the device in use (148 on a B200; asked once)."""
    global _sm_count
    if _sm_count is None:
        _sm_count = (torch.cuda.get_device_properties(torch.cuda.current_device())
                     .multi_processor_count if torch.cuda.is_available() else 148)
    return _sm_count

# Up to this many rows a caller may keep a split-K destination at zero itself (the kernel that
# consumes it clears it) instead of having it cleared before every product.
SPLIT_K_MAX_ROWS = 256


def k_splits(rows: int, out_features: int, in_features: int) -> int:
    """How many ways to split K so that a product with few output tiles still fills the GPU."""
    tiles = -(-out_features // 128) * -(-rows // token_tile(rows))
    if tiles >= 2 * sm_count() - 40:
        return 1
    # two CTAs fit an SM: aim at one full wave of two CTAs per SM, at least 256 of K each
    return max(1, min(16, round(2 * sm_count() / tiles), in_features // 256))


def linear(a: torch.Tensor, w: torch.Tensor, out: torch.Tensor, accumulate: bool = False,
           out_is_zero: bool = False) -> None:
    """out (=|+=) a @ w.T with the fastest hand-written kernel that takes these operands:
    tensor cores for bfloat16 (they fetch weights ahead of the kernel before them), the
    CUDA-core kernels for everything else (32-bit operands, unaligned sizes).
    ``out_is_zero``: the caller guarantees that ``out`` holds zeros, so a split-K product need
    not clear it first."""
    if _tc_ok(a, w):
        rows, k = a.shape
        n = w.shape[0]
        splits = k_splits(rows, n, k) if out.dtype == torch.float32 else 1
        gemm_tcgen05(a, w, out, 1 if accumulate else 0, splits=splits, out_is_zero=out_is_zero)
    elif _gemv_ok(a, w):
        gemv_bf16(a, w, out, 1 if accumulate else 0)
    else:
        gemm_simt(a, w, out, accumulate)


def gated_interleave_ok(gate: torch.Tensor, up: torch.Tensor) -> bool:
    """Whether the gate and up matrices can be stored interleaved for the tensor-core product."""
    return (gate.dtype == torch.bfloat16 and up.dtype == torch.bfloat16 and gate.is_cuda
            and gate.shape == up.shape and gate.shape[0] % 16 == 0 and gate.shape[1] % 8 == 0)


def gate_up_silu(ctx, h: torch.Tensor, w_gate_up: torch.Tensor, act: torch.Tensor,
                 interleaved: bool = False) -> None:
    """act = silu(h Wg^T) * (h Wu^T) for Wg, Wu stacked in ``w_gate_up`` ([2 ff][hidden]):
    gate rows then up rows, or (``interleaved``) alternating blocks of 16 gate and 16 up rows."""
    rows, ff = act.shape
    if interleaved:
        if not _tc_ok(h, w_gate_up):
            raise KernelError("interleaved gate/up weights need the tensor-core product")
        gemm_tcgen05(h, w_gate_up, act, 3, ff)
        return
    if _tc_ok(h, w_gate_up):
        gemm_tcgen05(h, w_gate_up, act, 2, ff)
        return
    if _gemv_ok(h, w_gate_up):
        gemv_bf16(h, w_gate_up, act, 2, ff)
        return
    gu = ctx.buffer("ffn.gate_up", (rows, 2 * ff), torch.float32)
    linear(h, w_gate_up, gu)
    silu_mul(gu, act)


FLASH_HEAD_DIMS = (32, 64, 128)
ATTENTION_MAX_HEAD_DIM = 256      # MAX_HD of attention_generic.cu, the kernel of last resort


def attention_refusal(num_heads: int, num_kv_heads: int, head_dim: int) -> Optional[str]:
    """Why no attention kernel of this library takes these sizes, or None when one does (the
    generic kernel takes every head size that is a multiple of 8 up to 256 and every group)."""
    if head_dim <= 0 or head_dim % 8 != 0 or head_dim > ATTENTION_MAX_HEAD_DIM:
        return (f"head_dim {head_dim}: the attention kernels take multiples of 8 up to "
                f"{ATTENTION_MAX_HEAD_DIM}")
    if num_kv_heads <= 0 or num_heads % num_kv_heads != 0:
        return f"{num_heads} query heads cannot be shared among {num_kv_heads} KV heads"
    return None


def attention_flash(q: torch.Tensor, out: torch.Tensor, k_cache: torch.Tensor,
                    v_cache: torch.Tensor, page_stride: int, block_table: torch.Tensor,
                    items: Optional[torch.Tensor], n_items: int, rows_per_cta: int,
                    num_heads: int, num_kv_heads: int, head_dim: int, page_size: int,
                    scale: float, window: Optional[int], splits: int = 1,
                    part_o: Optional[torch.Tensor] = None, part_ml: Optional[torch.Tensor] = None,
                    row_slot: Optional[torch.Tensor] = None,
                    row_pos: Optional[torch.Tensor] = None) -> None:
    """Tensor-core attention over the paged cache for ``n_items`` work items (int32 quadruples
    first row, tokens, request slot, first position); without ``items`` every row is an item
    of one token given by ``row_slot`` / ``row_pos``.  With ``splits`` > 1 the result is left
    in ``part_o`` / ``part_ml`` for :func:`attention_merge`."""
    _cuda(q, out, k_cache, v_cache, block_table, items, part_o, part_ml, row_slot, row_pos)
    assert q.dtype == torch.bfloat16 and k_cache.dtype == torch.bfloat16
    _check(lib().llm_attention_flash(
        _ptr(q), _ptr(out), _ptr(part_o), _ptr(part_ml), _ptr(k_cache), _ptr(v_cache),
        page_stride, _ptr(block_table), block_table.stride(0), _ptr(items), _ptr(row_slot),
        _ptr(row_pos), n_items, rows_per_cta, num_heads, num_kv_heads, head_dim, page_size,
        float(scale), int(window or 0), splits, _stream()), f"attention_flash (head_dim {head_dim})")


def attention_decode(q: torch.Tensor, out: torch.Tensor, k_cache: torch.Tensor,
                     v_cache: torch.Tensor, page_stride: int, block_table: torch.Tensor,
                     items: Optional[torch.Tensor], n_items: int, num_heads: int,
                     num_kv_heads: int, head_dim: int, page_size: int, scale: float,
                     window: Optional[int], splits: int = 1,
                     part_o: Optional[torch.Tensor] = None, part_ml: Optional[torch.Tensor] = None,
                     row_slot: Optional[torch.Tensor] = None,
                     row_pos: Optional[torch.Tensor] = None) -> None:
    """Decode form of the tensor-core attention: items of at most eight (token, head of the
    group) pairs, keys on the M side of the tile.  Arguments as :func:`attention_flash`."""
    _cuda(q, out, k_cache, v_cache, block_table, items, part_o, part_ml, row_slot, row_pos)
    assert q.dtype == torch.bfloat16 and k_cache.dtype == torch.bfloat16
    _check(lib().llm_attention_decode(
        _ptr(q), _ptr(out), _ptr(part_o), _ptr(part_ml), _ptr(k_cache), _ptr(v_cache),
        page_stride, _ptr(block_table), block_table.stride(0), _ptr(items), _ptr(row_slot),
        _ptr(row_pos), n_items, num_heads, num_kv_heads, head_dim, page_size, float(scale),
        int(window or 0), splits, _stream()), f"attention_decode (head_dim {head_dim})")


def attention_decode_tma(q: torch.Tensor, out: torch.Tensor, storage: torch.Tensor, slot: int,
                         block_table: torch.Tensor, items: Optional[torch.Tensor], n_items: int,
                         num_heads: int, num_kv_heads: int, head_dim: int, page_size: int,
                         scale: float, window: Optional[int], splits: int = 1,
                         part_o: Optional[torch.Tensor] = None,
                         part_ml: Optional[torch.Tensor] = None,
                         row_slot: Optional[torch.Tensor] = None,
                         row_pos: Optional[torch.Tensor] = None) -> None:
    """As :func:`attention_decode`, with K and V fetched by TMA tile loads from the group's
    whole cache tensor ``storage`` [pages, slots, 2, kv heads, page size, head dim]."""
    _cuda(q, out, storage, block_table, items, part_o, part_ml, row_slot, row_pos)
    assert q.dtype == torch.bfloat16 and storage.dtype == torch.bfloat16
    assert storage.is_contiguous() and storage.dim() == 6
    _check(lib().llm_attention_decode_tma(
        _ptr(q), _ptr(out), _ptr(part_o), _ptr(part_ml), _ptr(storage), storage.shape[0],
        storage.shape[1], slot, _ptr(block_table), block_table.stride(0), _ptr(items),
        _ptr(row_slot), _ptr(row_pos), n_items, num_heads, num_kv_heads, head_dim, page_size,
        float(scale), int(window or 0), splits, _ptr(tc_status(q.device)), _stream()),
        f"attention_decode_tma (head_dim {head_dim})")


def attention_decode_persistent(q: torch.Tensor, part_o: torch.Tensor, part_ml: torch.Tensor,
                                storage: torch.Tensor, slot: int, block_table: torch.Tensor,
                                row_slot: torch.Tensor, row_pos: torch.Tensor, num_heads: int,
                                num_kv_heads: int, head_dim: int, page_size: int, scale: float,
                                window: Optional[int], parts: int, ctas: Optional[int] = None) -> None:
    """Decode attention of one new token per row with the tiles of all (row, KV head) units
    shared evenly by ``ctas`` one-warp CTAs (default: what the GPU holds at once).  Leaves
    ``parts`` parts per (row, head) in ``part_o`` / ``part_ml`` (some marked empty) for
    :func:`attention_merge` with ``splits = parts``."""
    _cuda(q, part_o, part_ml, storage, block_table, row_slot, row_pos)
    assert q.dtype == torch.bfloat16 and storage.dtype == torch.bfloat16
    assert storage.is_contiguous() and storage.dim() == 6
    rows = q.shape[0]
    assert part_o.numel() >= rows * num_heads * parts * head_dim
    _check(lib().llm_attention_decode_persistent(
        _ptr(q), _ptr(part_o), _ptr(part_ml), _ptr(storage), storage.shape[0], storage.shape[1],
        slot, _ptr(block_table), block_table.stride(0), _ptr(row_slot), _ptr(row_pos), rows,
        num_heads, num_kv_heads, head_dim, page_size, float(scale), int(window or 0), parts,
        int(ctas or DECODE_TMA_CTAS_PER_SM * sm_count()), _ptr(tc_status(q.device)), _stream()),
        f"attention_decode_persistent (head_dim {head_dim})")


def attention_tcgen05(q: torch.Tensor, out: torch.Tensor, k_cache: torch.Tensor,
                      v_cache: torch.Tensor, page_stride: int, block_table: torch.Tensor,
                      items: torch.Tensor, n_items: int, num_heads: int, num_kv_heads: int,
                      head_dim: int, page_size: int, scale: float, window: Optional[int],
                      n_pages: int = 0, persistent: bool = True) -> None:
    """Attention of prompt portions on tcgen05: items of at most 128 / (heads per KV head)
    tokens; scores and output accumulate in tensor memory.  ``n_pages``: pages of the cache that
    ``k_cache`` / ``v_cache`` are planes of; given it, pages of 32 positions or more are
    fetched by TMA, and with ``persistent`` and more (item, KV head) pairs than SMs one CTA per
    SM walks its share of the pairs."""
    _cuda(q, out, k_cache, v_cache, block_table, items)
    assert q.dtype == torch.bfloat16 and k_cache.dtype == torch.bfloat16
    assert q.is_contiguous() and out.is_contiguous()
    _check(lib().llm_attention_tcgen05(
        _ptr(q), _ptr(out), q.shape[0], _ptr(k_cache), _ptr(v_cache), page_stride, int(n_pages),
        _ptr(block_table), block_table.stride(0), _ptr(items), n_items, num_heads, num_kv_heads,
        head_dim, page_size, float(scale), int(window or 0), int(persistent),
        _ptr(tc_status(q.device)), _stream()), f"attention_tcgen05 (head_dim {head_dim})")


def attention_tcgen05_x2(q: torch.Tensor, out: torch.Tensor, k_cache: torch.Tensor,
                         v_cache: torch.Tensor, page_stride: int, block_table: torch.Tensor,
                         items: torch.Tensor, n_items: int, num_heads: int, num_kv_heads: int,
                         head_dim: int, page_size: int, scale: float, window: Optional[int],
                         n_pages: int) -> None:
    """As :func:`attention_tcgen05` with two query tiles per CTA: items of at most
    2 * 128 / (heads per KV head) tokens.  Pages of a power of two of at least 32 positions."""
    _cuda(q, out, k_cache, v_cache, block_table, items)
    assert q.dtype == torch.bfloat16 and k_cache.dtype == torch.bfloat16
    assert q.is_contiguous() and out.is_contiguous()
    _check(lib().llm_attention_tcgen05_x2(
        _ptr(q), _ptr(out), q.shape[0], _ptr(k_cache), _ptr(v_cache), page_stride, int(n_pages),
        _ptr(block_table), block_table.stride(0), _ptr(items), n_items, num_heads, num_kv_heads,
        head_dim, page_size, float(scale), int(window or 0), _ptr(tc_status(q.device)),
        _stream()), f"attention_tcgen05_x2 (head_dim {head_dim})")


def decode_tma_ok(view, head_dim: int) -> bool:
    st = getattr(view, "storage", None)
    ps = view.page_size
    return (st is not None and st.is_contiguous() and head_dim in (64, 128)
            and ps & (ps - 1) == 0 and st.shape[0] * st.shape[1] * 2 < (1 << 31))


def attention_merge(part_o: torch.Tensor, part_ml: torch.Tensor, out: torch.Tensor,
                    rows: Optional[torch.Tensor], n_rows: int, num_heads: int, head_dim: int,
                    splits: int, clear: Optional[torch.Tensor] = None) -> None:
    """Merge the parts of split keys.  ``clear`` (float32 [rows, >= heads * head_dim]): the
    first heads * head_dim values of every merged row of it are zeroed as well."""
    _cuda(part_o, part_ml, out, rows, clear)
    _check(lib().llm_attention_merge_clear(
        _ptr(part_o), _ptr(part_ml), _ptr(out), _ptr(rows), n_rows, num_heads, head_dim, splits,
        _ptr(clear), clear.stride(0) if clear is not None else 0, _stream()), "attention_merge")


FUSE_DECODE = "few waves"     # or "always" / "never": for measurements (see fuse_decode)


def fuse_decode(mode: str) -> None:
    """When decode attention runs fused with the rotation and the cache write: "few waves" (the
    default), "always" or "never".  For measurements; sets it for parts driven from Python and
    for the native step driver alike."""
    global FUSE_DECODE
    code = {"few waves": 0, "always": 1, "never": 2}[mode]
    FUSE_DECODE = mode
    l = lib()
    l.llm_set_fuse_decode.argtypes = [c_int]
    l.llm_set_fuse_decode.restype = None
    l.llm_set_fuse_decode(code)


def decode_fusion_ok(ctx, view, num_heads: int, num_kv_heads: int, head_dim: int, rot_dim: int,
                     cos_sin: Optional[torch.Tensor], window: Optional[int] = None) -> bool:
    """Whether the step runs norm, rotation, cache write and attention as one kernel: every
    row a single new token, 16-bit, whole heads rotated by the step's table of cosines and
    sines, a cache the TMA decode kernel takes, and at most two waves of CTAs (every wave pays
    the longer start of the fused kernel; from about four waves on that costs more than the
    separate rotation kernel: Qwen3-8B sizes at batch 64, 5.71 against 5.67 ms a step)."""
    if FUSE_DECODE == "never":
        return False
    ok = (ctx.dtype == torch.bfloat16 and cos_sin is not None and rot_dim == head_dim
          and num_heads // num_kv_heads <= 8 and decode_tma_ok(view, head_dim)
          and all(s.rows == 1 for s in ctx.segments))
    if not ok or FUSE_DECODE == "always":
        return ok
    reach = min(ctx.max_pos + 1, window) if window else ctx.max_pos + 1
    resident = DECODE_TMA_CTAS_PER_SM * sm_count()
    return (ctx.rows * num_kv_heads * decode_splits(ctx.rows, num_kv_heads, reach, resident,
                                                   DECODE_TMA_TILE) <= 2 * resident)


def attention_decode_fused(ctx, proj: torch.Tensor, out: torch.Tensor, view, writes_cache: bool,
                           q_norm_w: Optional[torch.Tensor], k_norm_w: Optional[torch.Tensor],
                           cos_sin: torch.Tensor, eps: float, clear: bool, num_heads: int,
                           num_kv_heads: int, head_dim: int, scale: float,
                           window: Optional[int], splits: Optional[int] = None) -> None:
    """A decode step's attention from the output of the q/k/v product ``proj`` (float32
    [rows, (heads + 2 kv heads) * head_dim], or only the queries when another call owns the
    cache): per-head norm, rotation, write of the new key and value, attention over the cache
    and, with split keys, the merge.  With ``clear`` what was consumed of ``proj`` is zeroed."""
    _cuda(proj, out, view.storage, view.block_table, ctx.row_slot, ctx.row_pos, q_norm_w,
          k_norm_w, cos_sin)
    assert proj.dtype == torch.float32 and proj.stride(1) == 1 and out.dtype == torch.bfloat16
    assert cos_sin.dtype == torch.float32 and cos_sin.is_contiguous()
    rows = ctx.rows
    reach = min(ctx.max_pos + 1, window) if window else ctx.max_pos + 1
    if splits is None:
        splits = decode_splits(rows, num_kv_heads, reach, DECODE_TMA_CTAS_PER_SM * sm_count(),
                               DECODE_TMA_TILE)
    part_o = part_ml = None
    if splits > 1:
        part_o = ctx.buffer("attn.part_o", (rows * num_heads * splits * head_dim,), torch.float32)
        part_ml = ctx.buffer("attn.part_ml", (rows * num_heads * splits * 2,), torch.float32)
    st = view.storage
    _check(lib().llm_attention_decode_fused(
        _ptr(proj), proj.stride(0), _ptr(out), _ptr(part_o), _ptr(part_ml), _ptr(st), st.shape[0],
        st.shape[1], view.slot, _ptr(view.k if writes_cache else None),
        _ptr(view.v if writes_cache else None), view.page_stride, _ptr(view.block_table),
        view.block_table.stride(0), _ptr(ctx.row_slot), _ptr(ctx.row_pos), rows, _ptr(q_norm_w),
        _ptr(k_norm_w), _ptr(cos_sin), float(eps), int(clear), num_heads, num_kv_heads, head_dim,
        view.page_size, float(scale), int(window or 0), splits, _ptr(tc_status(proj.device)),
        _stream()), f"attention_decode_fused (head_dim {head_dim})")
    if splits > 1:
        attention_merge(part_o, part_ml, out, None, rows, num_heads, head_dim, splits,
                        clear=proj if clear else None)


def decode_splits(n_items: int, num_kv_heads: int, max_len: int, resident: int = 592,
                  tile: int = 32) -> int:
    """Parts into which the keys of a one-token item are cut.  ``resident``: how many CTAs of
    the kernel the GPU holds at once; ``tile``: keys of the kernel's tiles (parts are whole
    tiles).  The cost of a choice is modelled as waves of CTAs times the length of one CTA's
    walk (its keys, in units of 32, plus a fixed start-up worth about 96 keys), plus the merge,
    which grows with the number of parts; measured step times at batch 1, 8 and 64 and contexts
    of 1024 and 4096 keys rank the choices the same way."""
    ctas = max(1, n_items * num_kv_heads)
    tiles = max(1, -(-max_len // tile))
    best, best_cost = 1, None
    for s in range(1, min(32, max(1, max_len // 64)) + 1):
        waves = -(-ctas * s // resident)
        cost = waves * (-(-tiles // s) * (tile // 32) + 3) + 0.1 * s
        if best_cost is None or cost < best_cost - 1e-9:
            best, best_cost = s, cost
    return best


DECODE_TMA_TILE = 32      # keys of a tile of attention_decode_tma.cu
DECODE_TMA_CTAS_PER_SM = 4    # its one-warp CTAs that fit an SM at head size 128
PERSISTENT_ATTENTION_MAX_KEYS = 6144
