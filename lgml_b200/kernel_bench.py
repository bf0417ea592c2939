"""Time one kernel of the engine alone, at sizes given on the command line.

    python -m lgml_b200.kernel_bench gemm --m 8 --n 28672 --k 4096 [--swiglu] [--f32-out]
    python -m lgml_b200.kernel_bench decode_attention --batch 8 --context 2176 --heads 32 --kv-heads 8 --head-dim 128
    python -m lgml_b200.kernel_bench prefill_attention --tokens 2048 --heads 32 --kv-heads 8 --head-dim 128
    python -m lgml_b200.kernel_bench rmsnorm --rows 8 --width 4096 --parts 9

Each case is run over a ring of input buffers larger than the L2 cache, so that weights and
cache pages come from HBM as they do in a decode step; warm-up launches first, then the timed
launches between two CUDA events.  It prints the time per launch and the bytes or flops per
second that the kernel's own inputs and outputs amount to.  The same commands are what the
profiles under ``profiles/`` were captured from.
"""
from __future__ import annotations

import argparse
import sys

import torch

from . import ops

DEV = "cuda:0"
L2_BYTES = 126 << 20


USE_GRAPH = True


def timed(fn, n_buffers: int, warmup: int, iters: int) -> float:
    """Microseconds per call of fn(i), i cycling over the buffers.  The timed calls are
    captured into one CUDA graph and replayed, so that the host's launch cost (tens of
    microseconds from Python) does not sit between kernels that take less than that; launches
    follow one another as they do inside a captured decode step."""
    for i in range(warmup):
        fn(i % n_buffers)
    torch.cuda.synchronize()
    start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    if USE_GRAPH:
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g, capture_error_mode="relaxed"):
            for i in range(iters):
                fn(i % n_buffers)
        g.replay()
        torch.cuda.synchronize()
        start.record()
        g.replay()
        end.record()
    else:
        start.record()
        for i in range(iters):
            fn(i % n_buffers)
        end.record()
    torch.cuda.synchronize()
    return start.elapsed_time(end) * 1e3 / iters


def ring(bytes_per_buffer: int) -> int:
    return max(2, -(-2 * L2_BYTES // max(bytes_per_buffer, 1)))


def case_gemm(a) -> None:
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    M, N, K = a.m, a.n, a.k
    nb = min(ring(N * K * 2), 24)
    ws = [(torch.randn(N, K, device=DEV) * 0.02).to(torch.bfloat16) for _ in range(nb)]
    x = torch.randn(M, K, device=DEV).to(torch.bfloat16)
    n_out = N // 2 if a.swiglu else N
    out = torch.empty(M, n_out, dtype=torch.float32 if a.f32_out else torch.bfloat16, device=DEV)
    splits = None if a.splits < 0 else a.splits
    scratch = torch.empty(max(64 * M * N, 1), dtype=torch.float32, device=DEV) if not a.swiglu else None

    def run(i):
        if a.library:
            torch.mm(x, ws[i].t())
        elif a.swiglu:
            ops.gemm_tcgen05(x, ws[i], out, None, status, swiglu=True)
        else:
            ops.gemm_tcgen05(x, ws[i], out, None, status, n_splits=splits, scratch=scratch, partials_ok=a.partials)

    us = timed(run, nb, a.warmup, a.iters)
    byts = (N * K + M * K) * 2 + M * n_out * out.element_size()
    print(f"gemm M={M} N={N} K={K} swiglu={a.swiglu} library={a.library} splits={ops.tcgen05_splits(M, N, K) if splits is None else splits}: "
          f"{us:.2f} us, {byts / us / 1e3:.0f} GB/s, {2.0 * M * N * K / us / 1e6:.1f} TFLOP/s, status {int(status.item())}")


def case_decode_attention(a) -> None:
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    B, ctx, H, G, D = a.batch, a.context, a.heads, a.kv_heads, a.head_dim
    pages_per_seq = -(-ctx // 64)
    per_set = B * pages_per_seq
    nb = ring(per_set * G * 64 * D * 2 * 2)
    n_pages = per_set * nb
    k = torch.randn(n_pages, G, 64, D, device=DEV).to(torch.bfloat16)
    v = torch.randn(n_pages, G, 64, D, device=DEV).to(torch.bfloat16)
    q = torch.randn(B, H * D, device=DEV).to(torch.bfloat16)
    out = torch.empty_like(q)
    positions = torch.full((B,), ctx - 1, dtype=torch.int32, device=DEV)
    seq_of = torch.arange(B, dtype=torch.int32, device=DEV)
    tables = [(torch.randperm(per_set) + i * per_set).to(torch.int32).reshape(B, pages_per_seq).to(DEV) for i in range(nb)]
    n_splits = a.splits if a.splits > 0 else ops.decode_splits(B, G, H // G, ctx)
    scratch = torch.empty(max(B * H * n_splits * (D + 2), 1), dtype=torch.float32, device=DEV)
    us = timed(lambda i: ops.decode_attention(q, positions, seq_of, tables[i], k, v, out, H, D ** -0.5, 0, status, n_splits, scratch),
               nb, a.warmup, a.iters)
    byts = B * ctx * G * D * 2 * 2
    print(f"decode_attention batch={B} context={ctx} heads={H}/{G} head_dim={D} splits={n_splits}: {us:.2f} us, {byts / us / 1e3:.0f} GB/s, status {int(status.item())}")


def case_prefill_attention(a) -> None:
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    T, H, G, D = a.tokens, a.heads, a.kv_heads, a.head_dim
    n_pages = -(-T // 64)
    k = torch.randn(n_pages, G, 64, D, device=DEV).to(torch.bfloat16)
    v = torch.randn(n_pages, G, 64, D, device=DEV).to(torch.bfloat16)
    q = torch.randn(T, H * D, device=DEV).to(torch.bfloat16)
    out = torch.empty_like(q)
    positions = torch.arange(T, dtype=torch.int32, device=DEV)
    table = torch.randperm(n_pages).to(torch.int32).reshape(1, n_pages).to(DEV)
    tt = ops.prefill_tile_tokens(H, G) if a.mma else (ops.prefill_tc_tile_tokens(H, G) if a.single else ops.prefill_twin_tile_tokens(H, G))
    tiles = torch.tensor([(0, t0, min(tt, T - t0), 0) for t0 in reversed(range(0, T, tt))], dtype=torch.int32, device=DEV)   # longest first
    fn = ops.prefill_attention if a.mma else (ops.prefill_attention_tc if a.single else ops.prefill_attention_twin)
    us = timed(lambda i: fn(q, positions, tiles, table, k, v, out, H, D ** -0.5, 0, status), 1, a.warmup, a.iters)
    flops = 4.0 * H * D * T * (T + 1) / 2
    print(f"prefill_attention ({'mma.sync' if a.mma else 'tcgen05'}) tokens={T} heads={H}/{G} head_dim={D}: {us:.2f} us, {flops / us / 1e6:.1f} TFLOP/s (causal), status {int(status.item())}")


def case_rmsnorm(a) -> None:
    rows, width, parts = a.rows, a.width, a.parts
    nb = min(ring(rows * width * 4), 16)
    xs = [torch.randn(rows, width, device=DEV) for _ in range(nb)]
    w = torch.ones(width, device=DEV)
    out = torch.empty(rows, width, dtype=torch.bfloat16, device=DEV)
    if a.bf16_delta:
        deltas = [torch.randn(rows, width, device=DEV).to(torch.bfloat16) for _ in range(nb)]
    elif parts > 0:
        deltas = [ops.Partials(torch.randn(parts, rows, width, device=DEV)) for _ in range(min(nb, 4))]
    else:
        deltas = [None]
    us = timed(lambda i: ops.rmsnorm(xs[i], w, 1e-5, out, delta=deltas[i % len(deltas)]), nb, a.warmup, a.iters)
    byts = rows * width * (4 + 2) + (rows * width * (4 + (2 if a.bf16_delta else 4 * parts)) if deltas[0] is not None else 0)
    print(f"rmsnorm rows={rows} width={width} parts={parts} bf16_delta={a.bf16_delta}: {us:.2f} us, {byts / us / 1e3:.0f} GB/s")


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="python -m lgml_b200.kernel_bench")
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--iters", type=int, default=50)
    ap.add_argument("--no-graph", action="store_true", help="launch the timed calls one by one from the host")
    sub = ap.add_subparsers(dest="case", required=True)
    g = sub.add_parser("gemm")
    g.add_argument("--m", type=int, default=8)
    g.add_argument("--n", type=int, default=28672)
    g.add_argument("--k", type=int, default=4096)
    g.add_argument("--swiglu", action="store_true")
    g.add_argument("--f32-out", action="store_true")
    g.add_argument("--library", action="store_true", help="time the library product on the same operands instead")
    g.add_argument("--partials", action="store_true", help="leave the K splits' partial sums to the next kernel")
    g.add_argument("--splits", type=int, default=-1)
    d = sub.add_parser("decode_attention")
    d.add_argument("--batch", type=int, default=8)
    d.add_argument("--context", type=int, default=2176)
    d.add_argument("--heads", type=int, default=32)
    d.add_argument("--kv-heads", type=int, default=8)
    d.add_argument("--head-dim", type=int, default=128)
    d.add_argument("--splits", type=int, default=0)
    p = sub.add_parser("prefill_attention")
    p.add_argument("--tokens", type=int, default=2048)
    p.add_argument("--heads", type=int, default=32)
    p.add_argument("--kv-heads", type=int, default=8)
    p.add_argument("--head-dim", type=int, default=128)
    p.add_argument("--mma", action="store_true", help="the mma.sync kernel instead of the tcgen05 one")
    p.add_argument("--single", action="store_true", help="the tcgen05 kernel with one tile per CTA and one page per step")
    r = sub.add_parser("rmsnorm")
    r.add_argument("--rows", type=int, default=8)
    r.add_argument("--width", type=int, default=4096)
    r.add_argument("--parts", type=int, default=9)
    r.add_argument("--bf16-delta", action="store_true", help="add a bfloat16 delta (a product's output) instead of float32 partial sums")
    a = ap.parse_args(argv)
    global USE_GRAPH
    USE_GRAPH = not a.no_graph
    if not torch.cuda.is_available():
        print("kernel_bench needs a CUDA device", file=sys.stderr)
        return 1
    {"gemm": case_gemm, "decode_attention": case_decode_attention, "prefill_attention": case_prefill_attention, "rmsnorm": case_rmsnorm}[a.case](a)
    return 0


if __name__ == "__main__":
    sys.exit(main())
