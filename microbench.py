"""Times single kernels at given sizes with CUDA events (inputs larger than L2 are rotated
so that weights come from DRAM), and reports bytes or FLOPs per second.

    python microbench.py attention_decode --batch 64 --context 520
    python microbench.py linear --rows 8 --n 6144 --k 4096 [--kernel skinny|tc64|tc128|tc256]
    python microbench.py attention_prefill --tokens 2048 --seqs 1 [--kernel tc]
    python microbench.py gemm --rows 2048 --n 28672 --k 4096 --tile 256
    python microbench.py sampling --rows 64 --vocab 128256 --temperature 0.7 --top-k 40 --top-p 0.9

One JSON line per run.  It is also the small, self-ending workload that profiler captures
are taken on.
"""
from __future__ import annotations

import argparse
import json
import math
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
from supersonic_b200.csrc import ops  # noqa: E402

DEV = "cuda:0"


def _time(fn, iters, warmup=3):
    """Microseconds per launch: ``iters`` launches captured in one CUDA graph (so that host
    time per launch does not count) and replayed between two events."""
    for i in range(warmup):
        fn(i)
    torch.cuda.synchronize()
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.stream(side):
        with torch.cuda.graph(graph, stream=side):
            for i in range(iters):
                fn(i)
    torch.cuda.current_stream().wait_stream(side)
    graph.replay()
    torch.cuda.synchronize()
    start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    start.record()
    graph.replay()
    end.record()
    torch.cuda.synchronize()
    return start.elapsed_time(end) / iters * 1e3


def attention_decode(args):
    n_q, n_kv, hd, B, ctx = args.heads, args.kv_heads, args.head_dim, args.batch, args.context
    pages_per = (ctx + 63) // 64 + 1
    n_pages = B * pages_per
    k = torch.randn(n_pages, n_kv, 64, hd, device=DEV).bfloat16()
    v = torch.randn(n_pages, n_kv, 64, hd, device=DEV).bfloat16()
    table = torch.randperm(n_pages).to(torch.int32).view(B, pages_per).to(DEV)
    pos = torch.full((B,), ctx - 1, dtype=torch.int32, device=DEV)
    if args.ragged:
        pos = torch.randint(0, ctx, (B,), generator=torch.Generator().manual_seed(0)).to(torch.int32).to(DEV)
    slot = torch.arange(B, dtype=torch.int32, device=DEV)
    q = torch.randn(B, (n_q + 2 * n_kv) * hd, device=DEV).bfloat16()
    out = torch.empty(B, n_q * hd, dtype=torch.bfloat16, device=DEV)
    splits = args.splits
    pages = (ctx + 63) // 64
    chunk = 0 if args.chunk_pages < 0 else (args.chunk_pages or -(-pages // splits))     # negative: the kernel decides
    max_chunks = -(-pages // chunk) if chunk else min(-(-pages // 2), 296 // n_kv + 1)
    if args.kind == 2:
        nf, nc = ops.attention_decode_chunked_scratch(B, n_q, n_kv, hd, max_chunks)
    else:
        nf, nc = ops.attention_decode_scratch(B, n_q, n_kv, hd, splits)
    scratch = torch.empty(max(nf, 1), device=DEV)
    counters = torch.zeros(max(nc, 1), dtype=torch.int32, device=DEV)
    cos = sin = None
    if args.fused:                                   # rotation and append inside, as a decode step runs it
        ang = torch.arange(ctx, device=DEV, dtype=torch.float64)[:, None] * \
            (1.0 / 10000 ** (torch.arange(hd // 2, device=DEV, dtype=torch.float64) * 2 / hd))[None, :]
        cos, sin = ang.cos().float().contiguous(), ang.sin().float().contiguous()
    if args.kind == 2:                               # the tensor-core kernel on its persistent grid
        fn = lambda i: ops.attention_decode_chunked(q, k, v, pos, slot, table, out, n_q, n_kv, hd, 6, None,
                                                    1 / math.sqrt(hd), chunk, max_chunks, scratch, counters,
                                                    cos=cos, sin=sin, pdl=args.pdl, cluster=args.cluster)
    else:
        fn = lambda i: ops.attention_decode(q, k, v, pos, slot, table, out, n_q, n_kv, hd, 6, None,
                                            1 / math.sqrt(hd), splits, scratch, counters, cos=cos, sin=sin, pdl=args.pdl)
    us = _time(fn, args.iters)
    nbytes = int((pos.long() + 1).sum()) * n_kv * hd * 2 * 2
    return {"kernel": "attention_decode", "kind": args.kind, "fused": bool(args.fused), "batch": B, "context": ctx, "splits": splits, "us": round(us, 2),
            "GB/s": round(nbytes / us / 1e3, 1)}


def linear(args):
    B, N, K = args.rows, args.n, args.k
    copies = max(2, int(400e6 // (N * K * 2)) + 1)
    ws = [(torch.randn(N, K, device=DEV) * 0.02).bfloat16() for _ in range(copies)]
    x = torch.randn(B, K, device=DEV).bfloat16()
    out = torch.empty(B, N, dtype=torch.bfloat16, device=DEV)
    if args.kernel == "skinny":                             # the mma.sync skinny GEMM, one block per row tile
        fn = lambda i: ops.skinny_gemm(x, ws[i % copies], out, pdl=args.pdl)
    elif args.kernel.startswith("gv"):                      # gv = automatic splits, gv4 = 4 splits
        splits = int(args.kernel[2:]) if len(args.kernel) > 2 else ops.gemv_tc_splits(N, K)
        nf, nc = ops.gemv_tc_scratch(B, N, splits)
        partials = torch.empty(max(nf, 4), device=DEV)
        counters = torch.zeros(max(nc, 1), dtype=torch.int32, device=DEV)
        if args.accumulate:
            acc = torch.zeros(B, N, device=DEV)
            fn = lambda i: ops.gemv_tc(x, ws[i % copies], acc, mode=ops.TC_ACCUMULATE, splits=splits, pdl=args.pdl)
        else:
            fn = lambda i: ops.gemv_tc(x, ws[i % copies], out, splits=splits, partials=partials, counters=counters,
                                       pdl=args.pdl)
    else:
        tile = int(args.kernel[2:])
        fn = lambda i: ops.gemm_tc(x, ws[i % copies], out, tile_n=tile)
    us = _time(fn, args.iters)
    ops.check_device_errors()
    return {"kernel": args.kernel, "rows": B, "n": N, "k": K, "pdl": bool(args.pdl), "us": round(us, 2),
            "GB/s": round(N * K * 2 / us / 1e3, 1)}


def gemm(args):
    M, N, K = args.rows, args.n, args.k
    copies = max(2, int(300e6 // (N * K * 2)) + 1)
    ws = [(torch.randn(N, K, device=DEV) * 0.02).bfloat16() for _ in range(copies)]
    a = torch.randn(M, K, device=DEV).bfloat16()
    if args.accumulate:                               # add into a float32 output, as the o and down projections do
        out = torch.zeros(M, N, device=DEV)
        us = _time(lambda i: ops.gemm_tc(a, ws[i % copies], out, mode=ops.TC_ACCUMULATE, tile_n=args.tile,
                                         splits=args.k_parts), args.iters)
    else:
        out = torch.empty(M, N, dtype=torch.bfloat16, device=DEV)
        us = _time(lambda i: ops.gemm_tc(a, ws[i % copies], out, tile_n=args.tile), args.iters)
    ops.check_device_errors()
    return {"kernel": f"gemm_tc{args.tile}", "accumulate": bool(args.accumulate), "k_parts": args.k_parts, "m": M, "n": N, "k": K, "us": round(us, 2),
            "TFLOP/s": round(2.0 * M * N * K / us / 1e6, 1)}


def attention_prefill(args):
    n_q, n_kv, hd, S, T = args.heads, args.kv_heads, args.head_dim, args.seqs, args.tokens
    pages_per = (T + 63) // 64
    k = torch.randn(S * pages_per, n_kv, 64, hd, device=DEV).bfloat16()
    v = torch.randn(S * pages_per, n_kv, 64, hd, device=DEV).bfloat16()
    table = torch.randperm(S * pages_per).to(torch.int32).view(S, pages_per).to(DEV)
    q = torch.randn(S * T, (n_q + 2 * n_kv) * hd, device=DEV).bfloat16()
    out = torch.empty(S * T, n_q * hd, dtype=torch.bfloat16, device=DEV)
    cu = torch.arange(S + 1, dtype=torch.int32, device=DEV) * T
    start = torch.zeros(S, dtype=torch.int32, device=DEV)
    slot = torch.arange(S, dtype=torch.int32, device=DEV)
    kernel = ops.attention_prefill_tc if args.kernel == "tc" else ops.attention_prefill   # --kernel tc: tcgen05
    us = _time(lambda i: kernel(q, k, v, cu, start, slot, table, out, T, n_q, n_kv, hd, 6, None,
                                1 / math.sqrt(hd)), args.iters)
    ops.check_device_errors()
    flops = S * 4.0 * n_q * hd * T * (T + 1) / 2
    return {"kernel": "attention_prefill_tc" if args.kernel == "tc" else "attention_prefill", "seqs": S, "tokens": T,
            "us": round(us, 2),
            "TFLOP/s": round(flops / us / 1e6, 1)}


def sampling(args):
    """The pick of a step: argmax at temperature 0, else a draw under the given cuts.  Eight sets of
    logits in turn (64 rows of 128,256 are 33 MB each)."""
    rows, V = args.rows, args.vocab
    g = torch.Generator(device=DEV).manual_seed(3)
    logits = [3 * torch.randn(rows, V, device=DEV, generator=g) for _ in range(8)]
    slots = torch.arange(rows, dtype=torch.int32, device=DEV)
    state = (torch.arange(1, rows + 1, dtype=torch.int64, device=DEV) * 0x9E3779B97F4A7C15) & ((1 << 62) - 1)
    out = torch.empty(rows, dtype=torch.int32, device=DEV)
    if args.temperature <= 0:
        us = _time(lambda i: ops.argmax(logits[i % 8], out), args.iters)
    else:
        us = _time(lambda i: ops.sample(logits[i % 8], args.temperature, args.top_k, args.top_p, slots, state, out), args.iters)
    return {"kernel": "argmax" if args.temperature <= 0 else "sample", "rows": rows, "vocab": V,
            "temperature": args.temperature, "top_k": args.top_k, "top_p": args.top_p, "us": round(us, 2),
            "GB/s": round(rows * V * 4 / us / 1e3, 1)}


def main(argv=None):
    ap = argparse.ArgumentParser(description=__doc__.split("\n\n")[0])
    sub = ap.add_subparsers(dest="what", required=True)
    for name in ("attention_decode", "linear", "gemm", "attention_prefill", "sampling"):
        p = sub.add_parser(name)
        p.add_argument("--iters", type=int, default=20)
        p.add_argument("--heads", type=int, default=32)
        p.add_argument("--kv-heads", type=int, default=8)
        p.add_argument("--head-dim", type=int, default=128)
        p.add_argument("--batch", type=int, default=8)
        p.add_argument("--context", type=int, default=520)
        p.add_argument("--splits", type=int, default=8)
        p.add_argument("--rows", type=int, default=8)
        p.add_argument("--n", type=int, default=6144)
        p.add_argument("--k", type=int, default=4096)
        p.add_argument("--kernel", default="skinny")
        p.add_argument("--tile", type=int, default=256)
        p.add_argument("--k-parts", type=int, default=1, help="gemm --accumulate: parts a tile's K range is cut into")
        p.add_argument("--kind", type=int, default=2, help="attention_decode: 1 CUDA cores, 2 tensor cores (persistent grid)")
        p.add_argument("--chunk-pages", type=int, default=0, help="attention_decode --kind 2: pages per chunk (default: pages / --splits)")
        p.add_argument("--cluster", type=int, default=0,
                       help="attention_decode --kind 2: chunks a sequence as a thread-block cluster (2, 4, 8; 0: the persistent grid)")
        p.add_argument("--ragged", action="store_true", help="attention_decode: lengths uniform in [1, --context]")
        p.add_argument("--accumulate", action="store_true", help="linear gv*, gemm: add into a float32 output")
        p.add_argument("--pdl", action="store_true", help="launch as programmatic dependents")
        p.add_argument("--fused", action="store_true", help="attention_decode: rotate and append inside")
        p.add_argument("--seqs", type=int, default=1)
        p.add_argument("--tokens", type=int, default=2048)
        p.add_argument("--vocab", type=int, default=128256)
        p.add_argument("--temperature", type=float, default=0.0, help="sampling: 0 is the greedy pick")
        p.add_argument("--top-k", type=int, default=0)
        p.add_argument("--top-p", type=float, default=1.0)
    args = ap.parse_args(argv)
    print(json.dumps(globals()[args.what](args)))


if __name__ == "__main__":
    main()
