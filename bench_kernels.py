"""Single-kernel timing at model sizes, for profiling one kernel without the model around it.

    python bench_kernels.py tc_gemm --mode gate_up --rows 2048 --row-tile 128
    python bench_kernels.py tc_gemm --mode down --rows 8
    python bench_kernels.py attention_decode --batch 64 --context 8192
    python bench_kernels.py attention_prefill --tokens 2048
    python bench_kernels.py dense --rows 8 --n 7168 --k 5120 --impl grouped

Each run warms the kernel up, times ``--iters`` launches with CUDA events and prints one line with
the time per launch and the achieved bytes or flops per second.  The inputs are larger than the L2
cache at the default sizes.  Profiler captures name this file so that they run committed code only.  It is a measuring tool beside
``bench.py``, not part of the package.
"""
from __future__ import annotations

import argparse
import math
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))

from sharpinference_b200.kernels import ops  # noqa: E402

DEV = "cuda:0"


USE_GRAPH = False


def _time(fn, iters: int, warmup: int = 3) -> float:
    """Milliseconds per call.  With --graph the calls are captured once and replayed, which takes the
    host's launch cost out of the measurement (short kernels are otherwise timed by it)."""
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    if USE_GRAPH:
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            for _ in range(iters):
                fn()
        graph.replay()
        torch.cuda.synchronize()
        a.record()
        graph.replay()
        b.record()
    else:
        a.record()
        for _ in range(iters):
            fn()
        b.record()
    torch.cuda.synchronize()
    ops.check_status(DEV)
    return a.elapsed_time(b) / iters


def tc_gemm(ns) -> None:
    E, I, H, T = ns.experts, ns.inter, ns.hidden, ns.rows
    g = torch.Generator(device=DEV).manual_seed(0)
    used = min(E, ns.active) if ns.active else E
    counts = torch.zeros(E, dtype=torch.int64)
    if ns.skew > 0:
        share = torch.tensor([(1.0 - ns.skew) ** e for e in range(used)], dtype=torch.float64)
        counts[:used] = torch.floor(share / share.sum() * T).to(torch.int64)
    else:
        counts[:used] = T // used
    counts[: T - int(counts.sum())] += 1
    offsets = torch.cat([torch.zeros(1, dtype=torch.int64), torch.cumsum(counts, 0)]).to(torch.int32).to(DEV)
    if ns.mode == "gate_up":
        w = torch.empty(E, 2 * I, H, dtype=torch.bfloat16, device=DEV).normal_(0, 0.02, generator=g)
        a = torch.empty(T, H, dtype=torch.bfloat16, device=DEV).normal_(0, 1, generator=g)
        scale = torch.rand(T, device=DEV, generator=g)
        fn = lambda: ops.tc_grouped_gemm(a, w, offsets, mode=ops.TC_MODE_SWIGLU, row_scale=scale, row_tile=ns.row_tile,
                                         k_split=ns.k_split, max_ctas=ns.max_ctas)
        weight_bytes, flops = used * 2 * I * H * 2, 2 * T * 2 * I * H
    else:
        w = torch.empty(E, H, I, dtype=torch.bfloat16, device=DEV).normal_(0, 0.02, generator=g)
        a = torch.empty(T, I, dtype=torch.bfloat16, device=DEV).normal_(0, 1, generator=g)
        out = torch.zeros(T, H, device=DEV)
        rows = torch.randperm(T, device=DEV).to(torch.int32)
        fn = lambda: ops.tc_grouped_gemm(a, w, offsets, mode=ops.TC_MODE_STORE, out=out, out_rows=rows, accumulate=True,
                                         row_tile=ns.row_tile, k_split=ns.k_split, max_ctas=ns.max_ctas)
        weight_bytes, flops = used * H * I * 2, 2 * T * H * I
    if ns.beside:
        # the library's dense product (rows x N x K, operands in L2 for the most part) on a second stream beside
        # every launch: what a mixture layer's shared expert does while the routed experts stream their weights
        M2, N2, K2 = (int(v) for v in ns.beside.split(","))
        a2 = torch.randn(M2, K2, device=DEV).to(torch.bfloat16)
        w2 = torch.randn(N2, K2, device=DEV).to(torch.bfloat16)
        o2 = torch.empty(M2, N2, device=DEV)
        side = torch.cuda.Stream()
        dense = lambda: torch.mm(a2, w2.t(), out_dtype=torch.float32, out=o2)
        alone_dense = _time(dense, ns.iters)
        alone = _time(fn, ns.iters)
        inner = fn

        def fn():
            main = torch.cuda.current_stream()
            side.wait_stream(main)
            with torch.cuda.stream(side):
                for _ in range(ns.beside_count):
                    dense()
            inner()
            main.wait_stream(side)
        print(f"alone: grouped {alone * 1e3:.1f} us, dense {M2}x{N2}x{K2} {alone_dense * 1e3:.1f} us x {ns.beside_count} "
              f"({2 * M2 * N2 * K2 / alone_dense / 1e9:.0f} TFLOP/s)")
    ms = _time(fn, ns.iters)
    print(f"tc_gemm {ns.mode} rows={T} experts={used}/{E} row_tile={ops.tc_row_tile(T, ops.TC_MODE_SWIGLU if ns.mode == "gate_up" else ops.TC_MODE_STORE, E) if ns.row_tile is None else ns.row_tile}: {ms * 1e3:.1f} us, "
          f"weights {weight_bytes / ms / 1e6:.0f} GB/s, {flops / ms / 1e9:.0f} TFLOP/s")


def dense(ns) -> None:
    """A dense product of a few rows: the grouped tensor-core kernel with one group, the weight-streaming kernel for up to 16 rows, or the library.  The weights rotate through enough copies to exceed the L2 cache, as in a model of many layers."""
    M, N, K = ns.rows, ns.n, ns.k
    copies = max(2, (300 << 20) // (N * K * 2) + 1)
    ws = [torch.empty(N, K, dtype=torch.bfloat16, device=DEV).normal_(0, 0.02) for _ in range(copies)]
    a = torch.randn(M, K, device=DEV).to(torch.bfloat16)
    out = torch.empty(M, N, device=DEV)
    state = {"i": 0}

    def fn():
        w = ws[state["i"] % copies]
        state["i"] += 1
        if ns.impl == "grouped":
            ops.tc_dense(a, w, out=out)
        elif ns.impl == "rows":
            ops.dense_rows(a, w, swiglu=ns.swiglu, out=None if ns.swiglu else out)
        else:
            y = torch.mm(a, w.t(), out_dtype=torch.float32, out=out)
            if ns.swiglu:
                ops.swiglu(y, torch.bfloat16)
    ms = _time(fn, max(ns.iters, copies))
    print(f"dense {ns.impl} rows={M} N={N} K={K}{' swiglu' if ns.swiglu else ''}: {ms * 1e3:.1f} us, "
          f"weights {N * K * 2 / ms / 1e6:.0f} GB/s")


def router(ns) -> None:
    """Router logits, sigmoid and top-1 for a prompt portion's tokens (fp32), each call on another copy of the
    activations so that they come from memory as after the norm kernel of a long step."""
    T, H, E = ns.tokens, ns.hidden, ns.experts
    copies = max(2, (300 << 20) // (T * H * 4) + 1)
    hs = [torch.randn(T, H, device=DEV) for _ in range(copies)]
    wr = torch.randn(E, H, device=DEV) * 0.05
    state = {"i": 0}

    def fn():
        ops.router_top1(hs[state["i"] % copies], wr)
        state["i"] += 1
    ms = _time(fn, max(ns.iters, copies))
    print(f"router_top1 tokens={T} hidden={H} experts={E}: {ms * 1e3:.1f} us, "
          f"{(T * H * 4 + E * H * 4) / ms / 1e6:.0f} GB/s of activations and router rows read once")


def elementwise(ns) -> None:
    """The memory-bound kernels between the products of a prompt step, each call on another copy of its inputs
    (copies that exceed L2 together), with the bytes each has to move."""
    T, H, I = ns.tokens, ns.hidden, ns.inter
    nq, nkv, d, ps = ns.heads, ns.kv_heads, ns.head_dim, ns.page_size
    state = {"i": 0}

    def rotate(items):
        def pick():
            state["i"] += 1
            return items[state["i"] % len(items)]
        return pick

    if ns.op == "add_rmsnorm":
        copies = max(2, (300 << 20) // (T * H * 8) + 1)
        xs = rotate([(torch.randn(T, H, device=DEV), torch.randn(T, H, device=DEV)) for _ in range(copies)])
        w = torch.ones(H, device=DEV)
        nbytes = T * H * (4 + 4 + 4 + 2 + (4 if ns.fp32_copy else 0))

        def fn():
            x, delta = xs()
            ops.add_rmsnorm(x, delta, w, 1e-5, torch.bfloat16, want_fp32=ns.fp32_copy)
    elif ns.op == "swiglu":
        copies = max(2, (300 << 20) // (T * 2 * I * 4) + 1)
        gus = rotate([torch.randn(T, 2 * I, device=DEV) for _ in range(copies)])
        nbytes = T * I * (8 + 2)
        fn = lambda: ops.swiglu(gus(), torch.bfloat16)
    elif ns.op == "gather":
        copies = max(2, (300 << 20) // (T * H * 2) + 1)
        hs = rotate([torch.randn(T, H, device=DEV).to(torch.bfloat16) for _ in range(copies)])
        rows = torch.randperm(T, device=DEV).to(torch.int32)
        nbytes = T * H * 4
        fn = lambda: ops.gather_rows_bf16(hs(), rows)
    else:   # qkv_post: rotation, L2 norm, q store, keys and values into pages
        width = (nq + 2 * nkv) * d
        copies = max(2, (300 << 20) // (T * width * 4) + 1)
        qkvs = rotate([torch.randn(T, width, device=DEV) for _ in range(copies)])
        pages = (T + ps - 1) // ps
        kv = torch.zeros(pages, 2, nkv, ps, d, dtype=torch.bfloat16, device=DEV)
        table = torch.arange(pages, dtype=torch.int32, device=DEV).view(1, pages)
        positions = torch.arange(T, dtype=torch.int32, device=DEV)
        row_req = torch.zeros(T, dtype=torch.int32, device=DEV)
        inv_freq = (500000.0 ** (-torch.arange(0, d, 2, device=DEV, dtype=torch.float32) / d)).contiguous()
        q = torch.empty(T, nq, d, dtype=torch.bfloat16, device=DEV)
        nbytes = T * width * 4 + T * width * 2
        fn = lambda: ops.qkv_post(qkvs(), positions, row_req, table, inv_freq, q, kv, nq=nq, nkv=nkv, d=d, page_size=ps,
                                  pairing=ops.ROPE_INTERLEAVED, l2_eps=1e-5, temp_attn_scale=0.0, temp_floor_scale=0.0,
                                  write_kv=True)
    ms = _time(fn, max(ns.iters, 8))
    print(f"{ns.op} tokens={T}: {ms * 1e3:.1f} us, {nbytes / 1e6:.0f} MB -> {nbytes / ms / 1e6:.0f} GB/s")


def _cache(batch: int, context: int, nkv: int, d: int, ps: int):
    blocks = (context + ps - 1) // ps
    pages = batch * blocks
    kv = torch.empty(pages, 2, nkv, ps, d, dtype=torch.bfloat16, device=DEV).normal_(0, 1)
    table = torch.randperm(pages, device=DEV).to(torch.int32).view(batch, blocks).contiguous()
    return kv, table


def attention_decode(ns) -> None:
    B, S, nq, nkv, d, ps = ns.batch, ns.context, ns.heads, ns.kv_heads, ns.head_dim, ns.page_size
    kv, table = _cache(B, S, nkv, d, ps)
    q = torch.randn(B, nq, d, device=DEV).to(torch.bfloat16)
    positions = torch.full((B,), S - 1, dtype=torch.int32, device=DEV)
    if ns.others_context:                       # one row at the full context, the others shorter
        positions[1:] = min(ns.others_context, S) - 1
    row_req = torch.arange(B, dtype=torch.int32, device=DEV)
    out = torch.empty(B, nq * d, dtype=torch.bfloat16, device=DEV)
    kind = {"full": ops.MASK_FULL, "chunk": ops.MASK_CHUNK}[ns.mask]
    keys = int((positions.long() + 1).sum())
    fn = lambda: ops.attention_decode(q, kv, table, row_req, positions, out, rows=None, num_rows=B, nq=nq, nkv=nkv, d=d,
                                      page_size=ps, mask_kind=kind, mask_span=ns.span, scale=1 / math.sqrt(d),
                                      max_context=S, max_keys=keys)
    ms = _time(fn, ns.iters)
    nbytes = keys * nkv * d * 2 * 2
    print(f"attention_decode batch={B} context={S}{'/' + str(ns.others_context) if ns.others_context else ''} heads={nq}/{nkv} d={d}: {ms * 1e3:.1f} us, {nbytes / ms / 1e6:.0f} GB/s")


def attention_prefill(ns) -> None:
    T, nq, nkv, d, ps = ns.tokens, ns.heads, ns.kv_heads, ns.head_dim, ns.page_size
    start = ns.start
    kv, table = _cache(1, start + T, nkv, d, ps)
    q = torch.randn(T, nq, d, device=DEV).to(torch.bfloat16)
    rows = 64 if ns.warp_mma else ops.TC_PREFILL_TILE
    tiles = torch.tensor([[t0, min(rows, T - t0), start + t0, 0] for t0 in range(0, T, rows)], dtype=torch.int32, device=DEV)
    out = torch.empty(T, nq * d, dtype=torch.bfloat16, device=DEV)
    kind = {"full": ops.MASK_FULL, "chunk": ops.MASK_CHUNK}[ns.mask]
    kernel = ops.attention_prefill if ns.warp_mma else ops.attention_prefill_tc
    fn = lambda: kernel(q, kv, table, tiles, out, nq=nq, nkv=nkv, d=d, page_size=ps, mask_kind=kind,
                        mask_span=ns.span, scale=1 / math.sqrt(d))
    ms = _time(fn, ns.iters)
    pairs = sum(min(start + t + 1, (start + t) % ns.span + 1 if kind == ops.MASK_CHUNK else start + t + 1) for t in range(T))
    flops = 4 * nq * d * pairs
    print(f"attention_prefill ({'m16n8k16' if ns.warp_mma else 'tcgen05'}) tokens={T} start={start} heads={nq}/{nkv} d={d}: {ms * 1e3:.1f} us, {flops / ms / 1e9:.0f} TFLOP/s")


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    sub = ap.add_subparsers(dest="kernel", required=True)
    p = sub.add_parser("tc_gemm")
    p.add_argument("--mode", choices=["gate_up", "down"], default="gate_up")
    p.add_argument("--rows", type=int, default=2048)
    p.add_argument("--experts", type=int, default=16)
    p.add_argument("--active", type=int, default=0, help="experts that receive rows (0 = all)")
    p.add_argument("--hidden", type=int, default=5120)
    p.add_argument("--inter", type=int, default=8192)
    p.add_argument("--row-tile", type=int, default=None)
    p.add_argument("--k-split", type=int, default=None)
    p.add_argument("--max-ctas", type=int, default=0, help="persistent kernel: at most this many SMs (0 = all)")
    p.add_argument("--beside", default="", help="M,N,K of a library product launched on a second stream beside each call")
    p.add_argument("--beside-count", type=int, default=1)
    p.add_argument("--skew", type=float, default=0.0,
                   help="0: equal groups; else expert e gets rows in proportion to (1 - skew)^e")
    p.set_defaults(fn=tc_gemm)
    p = sub.add_parser("dense")
    p.add_argument("--rows", type=int, default=8)
    p.add_argument("--n", type=int, default=7168)
    p.add_argument("--k", type=int, default=5120)
    p.add_argument("--swiglu", action="store_true", help="SwiGLU after the product (rows: in its epilogue; library: a second kernel)")
    p.add_argument("--impl", choices=["grouped", "rows", "library"], default="grouped")
    p.set_defaults(fn=dense)
    p = sub.add_parser("elementwise")
    p.add_argument("--op", choices=["add_rmsnorm", "swiglu", "gather", "qkv_post"], default="add_rmsnorm")
    p.add_argument("--tokens", type=int, default=2048)
    p.add_argument("--hidden", type=int, default=5120)
    p.add_argument("--inter", type=int, default=8192)
    p.add_argument("--heads", type=int, default=40)
    p.add_argument("--kv-heads", type=int, default=8)
    p.add_argument("--head-dim", type=int, default=128)
    p.add_argument("--page-size", type=int, default=64)
    p.add_argument("--fp32-copy", action="store_true", help="add_rmsnorm: also write the unrounded copy (as before a router)")
    p.set_defaults(fn=elementwise)
    p = sub.add_parser("router")
    p.add_argument("--tokens", type=int, default=2048)
    p.add_argument("--hidden", type=int, default=5120)
    p.add_argument("--experts", type=int, default=16)
    p.set_defaults(fn=router)
    for name, fn in (("attention_decode", attention_decode), ("attention_prefill", attention_prefill)):
        p = sub.add_parser(name)
        p.add_argument("--batch", type=int, default=8)
        p.add_argument("--context", type=int, default=8192)
        p.add_argument("--others-context", type=int, default=0,
                       help="attention_decode: rows after the first have this many keys (a batch of unequal lengths)")
        p.add_argument("--tokens", type=int, default=2048)
        p.add_argument("--start", type=int, default=0)
        p.add_argument("--heads", type=int, default=40)
        p.add_argument("--kv-heads", type=int, default=8)
        p.add_argument("--head-dim", type=int, default=128)
        p.add_argument("--page-size", type=int, default=64)
        p.add_argument("--mask", choices=["full", "chunk"], default="full")
        p.add_argument("--span", type=int, default=8192)
        p.add_argument("--warp-mma", action="store_true", help="attention_prefill: the m16n8k16 kernel with 64-row tiles")
        p.set_defaults(fn=fn)
    for sp in sub.choices.values():
        sp.add_argument("--iters", type=int, default=10)
        sp.add_argument("--graph", action="store_true", help="time replays of a CUDA graph of the calls")
    ns = ap.parse_args(argv)
    global USE_GRAPH
    USE_GRAPH = ns.graph
    if not torch.cuda.is_available():
        print("bench_kernels.py needs a CUDA device", file=sys.stderr)
        return 2
    ns.fn(ns)
    return 0


if __name__ == "__main__":
    sys.exit(main())
