"""Time one kernel of the library on given sizes with CUDA events.

    python -m llmario_b200.benchmarks.kernels gemm --rows 8 --out 24576 --in 4096 --mode gated
    python -m llmario_b200.benchmarks.kernels attention --batch 8 --context 1024
    python -m llmario_b200.benchmarks.kernels prefill-attention --tokens 2048
    python -m llmario_b200.benchmarks.kernels step --batch 8 --context 1024
    python -m llmario_b200.benchmarks.kernels prompt-step --tokens 2048 --layers 4

Between timed launches a buffer larger than the L2 cache is overwritten unless ``--no-flush`` is
given.  Prints the median time, the bytes or flops it stands for, and the rate.
"""
from __future__ import annotations

import argparse
import sys

import torch

from .. import kernels

DEV = "cuda:0"


def timed(fn, reps: int, flush, chain: int = 1) -> float:
    """Median time of a launch in ms.  ``chain`` > 1: that many launches, recorded as a CUDA
    graph, between the two events (time per launch): the host's own time to issue a launch, tens
    of microseconds from Python, is then out of the picture, as it is inside a recorded step."""
    for _ in range(3):
        fn()
    torch.cuda.synchronize()
    if chain > 1:      # recorded once and replayed: Python cannot issue launches as fast as they run
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            for _ in range(chain):
                fn()
        run = graph.replay
    else:
        run = fn
    times = []
    for _ in range(reps):
        if flush is not None:
            flush.zero_()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        run()
        b.record()
        torch.cuda.synchronize()
        times.append(a.elapsed_time(b) / chain)
    times.sort()
    return times[len(times) // 2]


def cmd_gemm(a) -> None:
    T, N, K = a.rows, a.out, getattr(a, "in")
    kernels.use_cta_pairs(not a.one_cta)
    kernels.force_pair_k_ranges(a.k_ranges)
    x = torch.randn(T, K, device=DEV).bfloat16()
    w = (0.02 * torch.randn(N, K, device=DEV)).bfloat16()
    flush = None if a.no_flush else torch.empty(256 << 20, dtype=torch.uint8, device=DEV)
    if a.mode == "gated":
        out = torch.empty(T, N // 2, dtype=torch.bfloat16, device=DEV)
        fn = lambda: kernels.gemm_tcgen05(x, w, out, 3 if a.interleaved else 2, N // 2, bn=a.tile)
    elif a.mode == "accumulate":
        out = torch.zeros(T, N, dtype=torch.float32, device=DEV)
        fn = lambda: kernels.gemm_tcgen05(x, w, out, 1, bn=a.tile, splits=a.splits)
    elif a.mode == "gemv":
        out = torch.zeros(T, N, dtype=torch.float32, device=DEV)
        fn = lambda: kernels.gemv_bf16(x, w, out, 0)
    elif a.mode == "simt":
        out = torch.zeros(T, N, dtype=torch.float32, device=DEV)
        fn = lambda: kernels.gemm_simt(x, w, out)
    else:
        out = torch.empty(T, N, dtype=torch.float32 if a.f32 else torch.bfloat16, device=DEV)
        fn = lambda: kernels.gemm_tcgen05(x, w, out, 0, bn=a.tile, splits=a.splits)
    ms = timed(fn, a.reps, flush)
    kernels.check_tc_status(DEV)
    print(f"gemm {a.mode} rows={T} out={N} in={K} tile={a.tile} splits={a.splits}: "
          f"{ms * 1e3:.1f} us, weights {N * K * 2 / ms / 1e6:.0f} GB/s, "
          f"{2.0 * T * N * K / ms / 1e9:.1f} TFLOP/s")


def _paged(batch: int, context: int, Hkv: int, hd: int, page: int):
    pages_per = -(-context // page)
    n_pages = batch * pages_per
    storage = torch.randn(n_pages, 1, 2, Hkv, page, hd, device=DEV).bfloat16()
    perm = torch.randperm(n_pages, device=DEV).to(torch.int32)
    return storage, perm.reshape(batch, pages_per).contiguous()


def cmd_attention(a) -> None:
    B, S, Hq, Hkv, hd, page = a.batch, a.context, a.heads, a.kv_heads, a.head_dim, a.page_size
    storage, table = _paged(B, S, Hkv, hd, page)
    q = torch.randn(B, Hq * hd, device=DEV).bfloat16()
    out = torch.empty_like(q)
    slot = torch.arange(B, dtype=torch.int32, device=DEV)
    pos = torch.full((B,), S - 1, dtype=torch.int32, device=DEV)
    tma = not (a.row_major or a.cp_async)
    splits = a.splits or kernels.decode_splits(B, Hkv, S, (kernels.DECODE_TMA_CTAS_PER_SM if tma else 6) * kernels.sm_count(),
                                               kernels.DECODE_TMA_TILE if tma else 32)
    po = torch.empty(B * Hq * splits * hd, dtype=torch.float32, device=DEV)
    pml = torch.empty(B * Hq * splits * 2, dtype=torch.float32, device=DEV)
    flush = None if a.no_flush else torch.empty(256 << 20, dtype=torch.uint8, device=DEV)

    if a.persistent:
        parts = 4
        po = torch.empty(B * Hq * parts * hd, dtype=torch.float32, device=DEV)
        pml = torch.empty(B * Hq * parts * 2, dtype=torch.float32, device=DEV)

    def fn():
        if a.persistent:
            kernels.attention_decode_persistent(q, po, pml, storage, 0, table, slot, pos, Hq, Hkv, hd,
                                                page, hd ** -0.5, None, parts)
            kernels.attention_merge(po, pml, out, None, B, Hq, hd, parts)
            return
        if a.row_major:
            kernels.attention_flash(q, out, storage[0, 0, 0], storage[0, 0, 1], storage.stride(0),
                                    table, None, B, 16, Hq, Hkv, hd, page, hd ** -0.5, None, splits,
                                    po, pml, slot, pos)
        elif a.cp_async:
            kernels.attention_decode(q, out, storage[0, 0, 0], storage[0, 0, 1], storage.stride(0),
                                     table, None, B, Hq, Hkv, hd, page, hd ** -0.5, None, splits,
                                     po, pml, slot, pos)
        else:
            kernels.attention_decode_tma(q, out, storage, 0, table, None, B, Hq, Hkv, hd, page,
                                         hd ** -0.5, None, splits, po, pml, slot, pos)
        if splits > 1:
            kernels.attention_merge(po, pml, out, None, B, Hq, hd, splits)

    ms = timed(fn, a.reps, flush, a.chain)
    nbytes = B * S * Hkv * hd * 2 * 2
    print(f"decode attention batch={B} context={S} heads={Hq}/{Hkv} hd={hd} splits={splits}: "
          f"{ms * 1e3:.1f} us, cache {nbytes / ms / 1e6:.0f} GB/s")


def cmd_prefill_attention(a) -> None:
    T, Hq, Hkv, hd, page = a.tokens, a.heads, a.kv_heads, a.head_dim, a.page_size
    storage, table = _paged(1, T, Hkv, hd, page)
    q = torch.randn(T, Hq * hd, device=DEV).bfloat16()
    out = torch.empty_like(q)
    x2 = not (a.mma_sync or a.cp_async or a.one_tile) and page >= 32
    cap = max(1, (64 if a.mma_sync else 256 if x2 else 128) // (Hq // Hkv))
    items = torch.tensor([[s, min(cap, T - s), 0, s] for s in range(0, T, cap)],
                         dtype=torch.int32, device=DEV).reshape(-1)
    n = items.numel() // 4
    if a.mma_sync:
        fn = lambda: kernels.attention_flash(q, out, storage[0, 0, 0], storage[0, 0, 1],
                                             storage.stride(0), table, items, n, 64, Hq, Hkv, hd,
                                             page, hd ** -0.5, None)
    elif x2:
        fn = lambda: kernels.attention_tcgen05_x2(q, out, storage[0, 0, 0], storage[0, 0, 1],
                                                  storage.stride(0), table, items, n, Hq, Hkv, hd,
                                                  page, hd ** -0.5, a.window, storage.shape[0])
    else:
        fn = lambda: kernels.attention_tcgen05(q, out, storage[0, 0, 0], storage[0, 0, 1],
                                               storage.stride(0), table, items, n, Hq, Hkv, hd,
                                               page, hd ** -0.5, a.window,
                                               0 if a.cp_async else storage.shape[0],
                                               persistent=not a.one_cta_per_item)
    ms = timed(fn, a.reps, None, a.chain)
    kernels.check_tc_status(DEV)
    flops = 2.0 * T * T * Hq * hd          # causal: half of QK^T and PV
    print(f"prefill attention tokens={T} heads={Hq}/{Hkv} hd={hd}: {ms * 1e3:.1f} us, "
          f"{flops / ms / 1e9:.1f} TFLOP/s (causal flops)")


def cmd_step(a) -> None:
    """Decode steps of a whole model, for a list of the kernels a step launches: prompts are
    prefilled, then ``--steps`` decode steps run between cudaProfilerStart and cudaProfilerStop."""
    import random

    from ..cli import preset_config
    from ..engine import Model, ModelRunner, StepEntry

    from .. import driver
    driver.use_persistent_decode(a.persistent)
    kernels.use_dependent_launch(not a.no_dependent_launch)
    kernels.fuse_decode(a.fuse)
    model = Model.random(preset_config(a.model, a.layers), 0, "bfloat16", DEV)
    runner = ModelRunner(model, page_size=a.page_size, cache_tokens=a.batch * (a.context + 256),
                         max_requests=max(a.batch, 8), max_context=8192, use_graphs=not a.eager)
    rng, vocab = random.Random(0), model.vocab_size
    for i in range(a.batch):
        runner.step([StepEntry(i, [rng.randrange(vocab) for _ in range(a.context)], [])])

    def decode():
        runner.step([StepEntry(i, [rng.randrange(vocab)], [0]) for i in range(a.batch)])

    for _ in range(3):
        decode()
    torch.cuda.synchronize()
    start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    torch.cuda.profiler.start()          # for a profiler run with --profile-from-start off
    start.record()
    for _ in range(a.steps):
        decode()
    end.record()
    torch.cuda.synchronize()
    torch.cuda.profiler.stop()
    print(f"decode step {a.model} layers={len(model.blocks)} "
          f"batch={a.batch} context={a.context}: {start.elapsed_time(end) / a.steps * 1e3:.1f} us/step")


def cmd_prompt_step(a) -> None:
    """One prompt of ``--tokens`` tokens in one step, ``--steps`` times, between
    cudaProfilerStart and cudaProfilerStop (for a list of the kernels a prompt step launches)."""
    import random

    from ..cli import preset_config
    from ..engine import Model, ModelRunner, StepEntry

    from .. import driver
    driver.use_gather(not a.no_gather)
    model = Model.random(preset_config(a.model, a.layers), 0, "bfloat16", DEV)
    runner = ModelRunner(model, page_size=a.page_size, cache_tokens=a.tokens + 256, max_requests=2,
                         max_context=max(8192, a.tokens + 256), token_budget=a.tokens)
    rng, vocab = random.Random(0), model.vocab_size

    def prompt(i):
        runner.step([StepEntry(i, [rng.randrange(vocab) for _ in range(a.tokens)], [a.tokens - 1])])
        runner.close(i)

    for i in range(2):
        prompt(i)
    torch.cuda.synchronize()
    start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    torch.cuda.profiler.start()
    start.record()
    for i in range(a.steps):
        prompt(10 + i)
    end.record()
    torch.cuda.synchronize()
    torch.cuda.profiler.stop()
    kernels.check_tc_status(DEV)
    print(f"prompt step {a.model} layers={len(model.blocks)} tokens={a.tokens} "
          f"pages of {a.page_size}: {start.elapsed_time(end) / a.steps * 1e3:.1f} us/step")


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__.split("\n\n")[0])
    sub = ap.add_subparsers(dest="cmd", required=True)
    g = sub.add_parser("gemm")
    g.add_argument("--rows", type=int, default=8)
    g.add_argument("--out", type=int, default=4096)
    g.add_argument("--in", type=int, default=4096)
    g.add_argument("--mode", default="store", choices=["store", "accumulate", "gated", "gemv", "simt"])
    g.add_argument("--tile", type=int, default=None)
    g.add_argument("--splits", type=int, default=1)
    g.add_argument("--one-cta", action="store_true",
                   help="many rows: the one-CTA persistent kernel instead of CTA pairs")
    g.add_argument("--k-ranges", type=int, default=0,
                   help="ranges of K in the CTA-pair product that adds into its output "
                        "(0: its own cost model chooses)")
    g.add_argument("--f32", action="store_true")
    g.add_argument("--interleaved", action="store_true",
                   help="gated mode: the matrix holds alternating blocks of 16 gate and 16 up rows")
    g.set_defaults(fn=cmd_gemm)
    d = sub.add_parser("attention")
    d.add_argument("--batch", type=int, default=8)
    d.add_argument("--context", type=int, default=1024)
    d.add_argument("--splits", type=int, default=0)
    d.add_argument("--cp-async", action="store_true",
                   help="the decode kernel that loads with cp.async instead of TMA tiles")
    d.add_argument("--chain", type=int, default=1,
                   help="launches per timed interval (hides the host's launch time)")
    d.add_argument("--persistent", action="store_true",
                   help="the persistent decode kernel: all tiles shared evenly by resident CTAs")
    d.add_argument("--row-major", action="store_true",
                   help="the 16-row kernel of attention_flash.cu instead of the decode kernel")
    d.set_defaults(fn=cmd_attention)
    p = sub.add_parser("prefill-attention")
    p.add_argument("--tokens", type=int, default=2048)
    p.add_argument("--mma-sync", action="store_true",
                   help="the mma.sync kernel of attention_flash.cu instead of the tcgen05 kernel")
    p.add_argument("--cp-async", action="store_true",
                   help="K and V by cp.async copies even where the pages are large enough for TMA")
    p.add_argument("--one-tile", action="store_true",
                   help="one query tile per CTA even where the pages allow two")
    p.add_argument("--one-cta-per-item", action="store_true",
                   help="with --one-tile: a CTA per (item, KV head) instead of a persistent CTA per SM")
    p.add_argument("--window", type=int, default=None, help="attend to this many last keys only")
    p.add_argument("--chain", type=int, default=1,
                   help="launches per timed interval (hides the host's launch time)")
    p.set_defaults(fn=cmd_prefill_attention)
    st = sub.add_parser("step")
    st.add_argument("--model", default="qwen3-8b")
    st.add_argument("--layers", type=int, default=None)
    st.add_argument("--batch", type=int, default=8)
    st.add_argument("--context", type=int, default=1024)
    st.add_argument("--steps", type=int, default=4)
    st.add_argument("--page-size", type=int, default=16)
    st.add_argument("--eager", action="store_true", help="no CUDA graphs")
    st.add_argument("--fuse", default="few waves", choices=["few waves", "always", "never"],
                    help="when decode attention runs fused with the rotation and the cache write")
    st.add_argument("--no-dependent-launch", action="store_true",
                    help="every kernel waits for the end of the one before it")
    st.add_argument("--persistent", action="store_true",
                    help="decode attention by the persistent kernel where its CTAs make one to five waves")
    st.set_defaults(fn=cmd_step)
    ps = sub.add_parser("prompt-step")
    ps.add_argument("--model", default="qwen3-8b")
    ps.add_argument("--layers", type=int, default=None)
    ps.add_argument("--tokens", type=int, default=2048)
    ps.add_argument("--steps", type=int, default=2)
    ps.add_argument("--page-size", type=int, default=16)
    ps.add_argument("--no-gather", action="store_true",
                    help="attention reads small cache pages as they are (instead of a gathered copy)")
    ps.set_defaults(fn=cmd_prompt_step)
    for s in (g, d, p):
        s.add_argument("--reps", type=int, default=20)
        s.add_argument("--no-flush", action="store_true")
    for s in (d, p):
        s.add_argument("--heads", type=int, default=32)
        s.add_argument("--kv-heads", type=int, default=8)
        s.add_argument("--head-dim", type=int, default=128)
        s.add_argument("--page-size", type=int, default=16)
    a = ap.parse_args(argv)
    a.fn(a)
    return 0


if __name__ == "__main__":
    sys.exit(main())
