"""Single-kernel cases: run one kernel of the engine on synthetic operands, time it with CUDA events and
print what it achieved against the roofline.  The same command under `ncu` gives the profiles in profiles/.

    python -m wllm_b200.kernels.cases gemm --m 2048 --n 32768 --k 2048 --epilogue gelu_tanh
    python -m wllm_b200.kernels.cases gemm --m 8 --n 2048 --k 16384 --split
    python -m wllm_b200.kernels.cases attention-decode --requests 16 --context 8192
    python -m wllm_b200.kernels.cases attention-prefill --requests 1 --tokens 2048 --context 2048
    python -m wllm_b200.kernels.cases sampling --rows 8 --vocab 256000 --top-k 50 --top-p 0.9
    python -m wllm_b200.kernels.cases gemm-f32 --m 16 --n 49152 --k 3072
    python -m wllm_b200.kernels.cases attention-f32 --requests 16 --context 6000 --tokens 1 --heads 16 --kv-heads 16

Operands are larger than L2 where the case is bound by memory (several weight copies are cycled), so the
figures are DRAM figures.  Peaks: MEASURED_PEAKS.json at the repository root when present, else the fallback
6.65 TB/s and 1.59 PFLOP/s.
"""
from __future__ import annotations

import argparse
import json
import math
import os
import sys

import torch

from . import ops

DEV = "cuda:0"


def peaks():
    path = os.path.join(os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))), "MEASURED_PEAKS.json")
    try:
        with open(path) as f:
            raw = json.load(f)
        return float(raw["hbm_gbs"]), float(raw["bf16_tflops"]), "measured"
    except (OSError, ValueError, KeyError):
        return 6650.0, 1590.0, "fallback"


def timed(fn, iters: int, warmup: int = 3) -> float:
    """Milliseconds per call, CUDA events around `iters` calls after `warmup`."""
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    start.record()
    for _ in range(iters):
        fn()
    end.record()
    torch.cuda.synchronize()
    return start.elapsed_time(end) / iters


def gemm(args) -> None:
    M, N, K = args.m, args.n, args.k
    a = (torch.randn(M, K, device=DEV) * 0.1).to(torch.bfloat16)
    copies = max(1, min(8, int(300e6 // (N * K * 2)) + 1))       # cycle weights so that they come from DRAM
    ws = [(torch.randn(N, K, device=DEV) * 0.1).to(torch.bfloat16) for _ in range(copies)]
    parts = ops.split_plan(M, N, K) if args.split else 1
    code = args.epilogue
    if parts > 1:
        out = torch.empty((parts, M, N), dtype=torch.float32, device=DEV)
    else:
        cols = N // 2 if code in ("gelu_tanh", "silu") else N
        out = torch.empty((M, cols), dtype=torch.float32 if code == "f32" or args.split else torch.bfloat16, device=DEV)
    i = [0]

    def run():
        i[0] += 1
        w = ws[i[0] % copies]
        if parts > 1:
            ops.gemm_bf16_tc(a, w, out, "f32", k_splits=parts)
        else:
            ops.gemm_bf16_tc(a, w, out, "f32" if args.split else code, half_rows=args.half_rows or None)
    ms = timed(run, args.iters)
    hbm, tf, src = peaks()
    flops, byts = 2.0 * M * N * K, (N * K + M * K) * 2.0 + out.numel() * out.element_size()
    print(f"gemm_bf16_tc M={M} N={N} K={K} epilogue={code} parts={parts}: {ms * 1e3:.1f} us, "
          f"{flops / ms / 1e9:.1f} TFLOP/s ({flops / ms / 1e9 / tf:.3f} of {src} {tf:.0f}), "
          f"{byts / ms / 1e6:.0f} GB/s ({byts / ms / 1e6 / hbm:.3f} of {src} {hbm:.0f}), status {ops.tc_gemm_status(DEV)}")


def gemm_f32(args) -> None:
    """The 32-bit FMA product against a measured loop of fused multiply-adds (no tensor cores)."""
    M, N, K = args.m, args.n, args.k
    a = torch.randn(M, K, device=DEV) * 0.1
    copies = max(1, min(8, int(300e6 // (N * K * 4)) + 1))
    ws = [torch.randn(N, K, device=DEV) * 0.1 for _ in range(copies)]
    out = torch.empty((M, N), device=DEV)
    i = [0]

    def run():
        i[0] += 1
        ops.gemm_f32(a, ws[i[0] % copies], out)
    ms = timed(run, args.iters)
    hbm, _, src = peaks()
    fma_peak = ops.fma_peak_tflops(DEV)
    flops, byts = 2.0 * M * N * K, (N * K + M * K + M * N) * 4.0
    print(f"gemm_f32 M={M} N={N} K={K}: {ms * 1e3:.1f} us, {flops / ms / 1e9:.2f} TFLOP/s "
          f"({flops / ms / 1e9 / fma_peak:.3f} of a measured FMA loop's {fma_peak:.1f}), "
          f"{byts / ms / 1e6:.0f} GB/s ({byts / ms / 1e6 / hbm:.3f} of {src} {hbm:.0f})")


def attention_f32(args) -> None:
    """The 32-bit attention (one warp per row, or per row and chunk of 64 keys) as a step context would call it."""
    nq, nkv, hd, ps = args.heads, args.kv_heads, args.head_dim, args.page_size
    R, ctx, q_len = args.requests, args.context, args.tokens
    pages_each = -(-ctx // ps)
    num_pages = R * pages_each + 1
    k = torch.randn(num_pages, nkv, ps, hd, device=DEV) * 0.5
    v = torch.randn(num_pages, nkv, ps, hd, device=DEV) * 0.5
    table = torch.randperm(num_pages - 1, device=DEV).to(torch.int32).view(R, pages_each).contiguous()
    n = R * q_len
    q = torch.randn(n, nq * hd, device=DEV) * 0.5
    out = torch.empty_like(q)
    treq = torch.arange(R, dtype=torch.int32, device=DEV).repeat_interleave(q_len)
    pos = (torch.arange(ctx - q_len, ctx, dtype=torch.int32, device=DEV)).repeat(R)
    rows, chunks = n * nq, ops.simt_chunks(ctx, 0)
    scratch = None
    if not args.walk and chunks > 1 and rows <= 4096 and rows * chunks <= 65536:
        scratch = torch.empty(rows * chunks * (hd + 2), device=DEV)
    if q_len > 1 and not args.walk:          # portions of prompts: the tiled kernel, as the attention part chooses
        starts = torch.arange(0, n, q_len, dtype=torch.int32, device=DEV)
        qlens = torch.full((R,), q_len, dtype=torch.int32, device=DEV)
        ctxs = torch.full((R,), ctx, dtype=torch.int32, device=DEV)
        ms = timed(lambda: ops.paged_attention_simt_tiled(q, out, k, v, starts, qlens, ctxs, table, q_len, nq, nkv, hd, ps, 0,
                                                          1.0 / math.sqrt(hd)), args.iters)
        how = "tiled"
    else:
        ms = timed(lambda: ops.paged_attention_simt(q, out, k, v, treq, pos, table, nq, nkv, hd, ps, 0, 1.0 / math.sqrt(hd),
                                                    scratch, chunks), args.iters)
        how = "split by chunks" if scratch is not None else "walk"
    hbm, _, src = peaks()
    kv_bytes = 2.0 * R * ctx * nkv * hd * 4
    keys_seen = R * sum(ctx - q_len + i + 1 for i in range(q_len))
    print(f"attention f32 requests={R} context={ctx} tokens={q_len} heads={nq}/{nkv} head_dim={hd} "
          f"{how}: {ms * 1e3:.1f} us, {kv_bytes / ms / 1e6:.0f} GB/s of keys "
          f"and values ({kv_bytes / ms / 1e6 / hbm:.3f} of {src} {hbm:.0f}), {4.0 * nq * hd * keys_seen / ms / 1e9:.2f} TFLOP/s")


def attention(args, decode: bool) -> None:
    nq, nkv, hd, ps = args.heads, args.kv_heads, args.head_dim, args.page_size
    R, ctx = args.requests, args.context
    q_len = 1 if decode else args.tokens
    pages_each = -(-ctx // ps)
    num_pages = R * pages_each + 1
    k = (torch.randn(num_pages, nkv, ps, hd, device=DEV) * 0.5).to(torch.bfloat16)
    v = (torch.randn(num_pages, nkv, ps, hd, device=DEV) * 0.5).to(torch.bfloat16)
    table = torch.randperm(num_pages - 1, device=DEV).to(torch.int32).view(R, pages_each).contiguous()
    n = R * q_len
    q = (torch.randn(n, nq * hd, device=DEV) * 0.5).to(torch.bfloat16)
    out = torch.empty_like(q)
    starts = torch.arange(0, n, q_len, dtype=torch.int32, device=DEV)
    qlens = torch.full((R,), q_len, dtype=torch.int32, device=DEV)
    ctxs = torch.full((R,), ctx, dtype=torch.int32, device=DEV)
    scale = 1.0 / math.sqrt(hd)
    if decode:
        split_keys, max_splits = ops.decode_split_plan(R * nkv, ctx, 32 if hd % 64 == 0 else 64)
        scratch = torch.empty(ops.attention_mma_scratch_floats(R, nq, hd, max_splits), device=DEV)

        def run():
            ops.attention_mma_decode(q, out, k, v, starts, qlens, ctxs, table, nq, nkv, hd, ps, 0, scale, split_keys,
                                     max_splits, scratch)
    else:
        split_above = 0 if args.no_share else ops.prefill_share_plan([q_len] * R, [ctx] * R, nq, nkv, hd, False)
        halves = torch.empty(ops.attention_prefill_halves_floats(R, q_len, nq, nkv, hd), device=DEV) if split_above else None

        def run():
            ops.attention_mma_prefill(q, out, k, v, starts, qlens, ctxs, table, q_len, nq, nkv, hd, ps, 0, scale, False,
                                      split_above=split_above, halves=halves)
    ms = timed(run, args.iters)
    hbm, tf, src = peaks()
    kv_bytes = 2.0 * R * ctx * nkv * hd * 2
    first = ctx - q_len
    keys_seen = R * sum(first + i + 1 for i in range(q_len)) if q_len < 4096 else R * q_len * (first + q_len / 2)
    flops = 4.0 * nq * hd * keys_seen
    what = "attention decode" if decode else "attention prefill"
    print(f"{what} requests={R} context={ctx} tokens={q_len} heads={nq}/{nkv} head_dim={hd} page={ps}: {ms * 1e3:.1f} us, "
          f"{kv_bytes / ms / 1e6:.0f} GB/s of keys and values ({kv_bytes / ms / 1e6 / hbm:.3f} of {src} {hbm:.0f}), "
          f"{flops / ms / 1e9:.1f} TFLOP/s ({flops / ms / 1e9 / tf:.3f} of {src} {tf:.0f}), status {ops.tc_gemm_status(DEV)}")


def sampling(args) -> None:
    """The sampling passes on rows of logits that lie in L2 (as the head's product leaves them), options on the device."""
    from ..sampling import SamplingParams
    from ..sampling.sampler import Sampler
    rows, V = args.rows, args.vocab
    sp = SamplingParams(temperature=args.temperature, top_k=args.top_k, top_p=args.top_p, min_p=args.min_p, seed=1)
    sampler = Sampler(DEV)
    logits = torch.randn(rows, V, device=DEV) * 3.0
    logits[:, 77] += 8.0                                        # a peaked row, as a model's is
    lists = ([sp] * rows, [3] * rows, [7] * rows, [set()] * rows)
    sampler.launch(logits, *lists)                              # sends the options once
    greedy = args.temperature == 0.0
    if greedy:
        ms = timed(lambda: sampler.launch(logits, *lists), args.iters)
    else:
        from ..sampling.sampler import pack_options
        filters = pack_options(*lists)[1]
        ms = timed(lambda: sampler.launch_packed(logits, filters), args.iters)
    passes = 1 if greedy else 2 + (1 if filters & 1 else 0) + (2 if filters & 2 else 0)
    print(f"sampling rows={rows} vocab={V} temperature={args.temperature} top_k={args.top_k} top_p={args.top_p} "
          f"min_p={args.min_p}: {ms * 1e3:.1f} us, {passes} passes over {rows * V * 4 / 1e6:.1f} MB of logits "
          f"({passes * rows * V * 4 / ms / 1e6:.0f} GB/s out of L2)")


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="python -m wllm_b200.kernels.cases", description=__doc__.split("\n\n")[0])
    sub = ap.add_subparsers(dest="case", required=True)
    g = sub.add_parser("gemm")
    g.add_argument("--m", type=int, default=2048)
    g.add_argument("--n", type=int, default=32768)
    g.add_argument("--k", type=int, default=2048)
    g.add_argument("--epilogue", default="bf16", choices=["bf16", "f32", "gelu_tanh", "silu"])
    g.add_argument("--split", action="store_true", help="cut K into parts as a step of few rows does (float32 slabs)")
    g.add_argument("--half-rows", type=int, default=0, help="half the W tile's rows (0: the plan's choice)")
    g32 = sub.add_parser("gemm-f32")
    g32.add_argument("--m", type=int, default=16)
    g32.add_argument("--n", type=int, default=49152)
    g32.add_argument("--k", type=int, default=3072)
    for name in ("attention-decode", "attention-prefill", "attention-f32"):
        a = sub.add_parser(name)
        a.add_argument("--requests", type=int, default=16)
        a.add_argument("--context", type=int, default=8192)
        a.add_argument("--tokens", type=int, default=2048, help="new tokens per request (prefill)")
        a.add_argument("--heads", type=int, default=8)
        a.add_argument("--kv-heads", type=int, default=1)
        a.add_argument("--head-dim", type=int, default=256)
        a.add_argument("--page-size", type=int, default=64)
        a.add_argument("--no-share", action="store_true", help="prefill: never share a heavy tile between two CTAs")
        a.add_argument("--walk", action="store_true", help="attention-f32: one warp per row even where chunks would be split or rows tiled")
    sm = sub.add_parser("sampling")
    sm.add_argument("--rows", type=int, default=8)
    sm.add_argument("--vocab", type=int, default=256000)
    sm.add_argument("--temperature", type=float, default=0.8)
    sm.add_argument("--top-k", type=int, default=0)
    sm.add_argument("--top-p", type=float, default=1.0)
    sm.add_argument("--min-p", type=float, default=0.0)
    for p in sub.choices.values():
        p.add_argument("--iters", type=int, default=10)
    args = ap.parse_args(argv)
    if not torch.cuda.is_available():
        print("a CUDA device is needed", file=sys.stderr)
        return 1
    if args.case == "gemm":
        gemm(args)
    elif args.case == "gemm-f32":
        gemm_f32(args)
    elif args.case == "attention-f32":
        attention_f32(args)
    elif args.case == "sampling":
        sampling(args)
    else:
        attention(args, decode=args.case == "attention-decode")
    return 0


if __name__ == "__main__":
    sys.exit(main())
