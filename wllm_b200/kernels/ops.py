"""Python faces of the CUDA kernels: one function per entry point.

Each function checks what the kernel cannot (device, layout, element type), passes
raw pointers and the current CUDA stream, and turns a non-zero status into an
exception.  Nothing here computes: without a CUDA device or the compiled
extension the functions raise; there is no other implementation to fall back to.
The parts of a model call these through the module (`ops.rmsnorm(...)`), so a test
can put a stand-in in a function's place.

`launches` counts the kernel launches issued through this module (a captured CUDA
graph replays its launches without passing here; the engine adds those itself).
"""
from __future__ import annotations

import functools

import ctypes
from ctypes import c_float, c_void_p

import torch

from .build import KernelBuildError, load_family

launches = 0

_F32, _BF16 = 0, 1
_sms = None


def sm_count() -> int:
    """Multiprocessors of the current CUDA device (148 on a B200); every launch plan below is sized from it.
    Without a device (the plans are also exercised on the host) the B200's number stands in."""
    global _sms
    if _sms is None:
        _sms = torch.cuda.get_device_properties(torch.cuda.current_device()).multi_processor_count \
            if torch.cuda.is_available() else 148
    return _sms
_STATUS = {1: "element type not supported", 2: "size not supported", 3: "pointer or stride not aligned",
           4: "size beyond the entry point's fixed scratch", 5: "device set-up failed"}


class KernelError(RuntimeError):
    pass


def _dt(t: torch.Tensor) -> int:
    if t.dtype == torch.float32:
        return _F32
    if t.dtype == torch.bfloat16:
        return _BF16
    raise KernelError(f"element type {t.dtype} not supported (float32 or bfloat16)")


def _need_cuda(*tensors: torch.Tensor) -> None:
    for t in tensors:
        if t is not None and not t.is_cuda:
            raise KernelError("the engine's kernels run on a CUDA device only; got a tensor on " + str(t.device))


def _ptr(t) -> c_void_p:
    return c_void_p(0 if t is None else t.data_ptr())


_raw_stream = getattr(torch._C, "_cuda_getCurrentRawStream", None)


def _stream() -> c_void_p:
    """The current stream of the current device (it changes under a graph capture, so it is looked up at every
    launch; the raw lookup costs a fraction of a microsecond where the Stream object costs fifteen)."""
    if _raw_stream is not None:
        return c_void_p(_raw_stream(torch.cuda.current_device()))
    return c_void_p(torch.cuda.current_stream().cuda_stream)


def _check(status: int, what: str) -> None:
    global launches
    if status == 0:
        launches += 1
        return
    if status >= 1000:
        raise KernelError(f"{what}: CUDA launch failed with error {status - 1000}")
    raise KernelError(f"{what}: {_STATUS.get(status, 'status ' + str(status))}")


def _int32(t: torch.Tensor, name: str) -> torch.Tensor:
    if t.dtype != torch.int32 or not t.is_contiguous():
        raise KernelError(f"{name} must be a contiguous int32 tensor")
    return t


def embed_gather(ids: torch.Tensor, table: torch.Tensor, scale: float, out: torch.Tensor) -> torch.Tensor:
    """out[n, :] = float(table[ids[n], :]) * scale; `out` is the float32 residual stream."""
    _need_cuda(ids, table, out)
    n, (V, H) = ids.shape[0], table.shape
    assert out.dtype == torch.float32 and out.is_contiguous() and out.shape == (n, H) and table.is_contiguous()
    lib = load_family("embedding")
    _check(lib.wllm_embed_gather(_ptr(_int32(ids, "ids")), _ptr(table), _dt(table), c_float(scale), _ptr(out),
                                 n, H, V, _stream()), "embed_gather")
    return out


def patch_tokens(ids: torch.Tensor, dst: torch.Tensor, sampled: torch.Tensor, src: torch.Tensor) -> None:
    """ids[dst[i]] = sampled[src[i]] on the device: tokens that the previous step sampled and the host has
    not read yet become inputs of this step."""
    _need_cuda(ids, dst, sampled, src)
    n = dst.shape[0]
    assert src.shape[0] == n
    lib = load_family("embedding")
    _check(lib.wllm_patch_tokens(_ptr(_int32(ids, "ids")), _ptr(_int32(dst, "dst")), _ptr(_int32(sampled, "sampled")),
                                 _ptr(_int32(src, "src")), n, _stream()), "patch_tokens")


def rmsnorm(resid: torch.Tensor, delta, weight: torch.Tensor, eps: float, offset: float, out: torch.Tensor,
            rows=None, delta_splits: int = 0) -> torch.Tensor:
    """Fold `delta` into the residual (when given), then norm: see csrc/norm.cu.  With `delta_splits` = S > 0,
    `delta` is [S, n, H] float32 partial sums that are added in order."""
    _need_cuda(resid, delta, weight, out, rows)
    H = resid.shape[1]
    n = rows.shape[0] if rows is not None else resid.shape[0]
    assert resid.dtype == torch.float32 and resid.is_contiguous() and out.is_contiguous() and out.shape == (n, H)
    assert weight.shape == (H,) and weight.is_contiguous()
    split_stride = 0
    if delta is not None:
        assert delta.is_contiguous()
        if delta_splits:
            assert delta.shape == (delta_splits,) + tuple(resid.shape) and delta.dtype == torch.float32
            split_stride = resid.numel()
        else:
            assert delta.shape == resid.shape
    lib = load_family("norm")
    _check(lib.wllm_rmsnorm(_ptr(resid), _ptr(delta), _dt(delta) if delta is not None else _F32, max(1, delta_splits),
                            ctypes.c_longlong(split_stride), _ptr(weight), _dt(weight), c_float(eps), c_float(offset),
                            _ptr(out), _dt(out), _ptr(_int32(rows, "rows") if rows is not None else None), n, H,
                            _stream()), "rmsnorm")
    return out


def rope_kv_write(qkv: torch.Tensor, q_out: torch.Tensor, positions: torch.Tensor, slots, inv_freq: torch.Tensor,
                  k_pages, v_pages, nq: int, nkv: int, hd: int, rot_dim: int, page_size: int, in_splits: int = 0,
                  pairing: str = "half") -> None:
    """Rotate the q and k heads of the fused rows `qkv` [n, (nq+2nkv)*hd] (or [S, n, ...] float32 partial sums
    when in_splits = S > 0); rotated q goes to `q_out` [n, nq*hd], rotated k and v to the pages.
    pairing 'half': element j turns with j + rot_dim/2; 'interleaved': 2j with 2j + 1."""
    if pairing not in ("half", "interleaved"):
        raise KernelError(f"rotary pairing {pairing!r} not supported (half, interleaved)")
    _need_cuda(qkv, q_out, positions, slots, inv_freq, k_pages, v_pages)
    width = (nq + 2 * nkv) * hd
    if in_splits:
        assert qkv.dim() == 3 and qkv.shape[0] == in_splits and qkv.is_contiguous() and qkv.dtype == torch.float32
        n, row_stride, split_stride = qkv.shape[1], qkv.stride(1), qkv.stride(0)
    else:
        assert qkv.dim() == 2 and qkv.stride(1) == 1
        n, row_stride, split_stride = qkv.shape[0], qkv.stride(0), 0
    assert qkv.shape[-1] == width and q_out.shape == (n, nq * hd) and q_out.stride(1) == 1
    assert inv_freq.dtype == torch.float32 and inv_freq.numel() == rot_dim // 2 and inv_freq.is_contiguous()
    if slots is not None:
        assert k_pages.is_contiguous() and v_pages.is_contiguous() and k_pages.dtype == q_out.dtype == v_pages.dtype
    lib = load_family("rope_cache")
    _check(lib.wllm_rope_kv_write(_ptr(qkv), _dt(qkv), row_stride, max(1, in_splits), ctypes.c_longlong(split_stride),
                                  _ptr(q_out), _dt(q_out), q_out.stride(0), _ptr(_int32(positions, "positions")),
                                  _ptr(_int32(slots, "slots") if slots is not None else None), _ptr(inv_freq),
                                  _ptr(k_pages), _ptr(v_pages), n, nq, nkv, hd, rot_dim, page_size,
                                  1 if pairing == "interleaved" else 0, _stream()),
           "rope_kv_write")


SIMT_CHUNK = 64    # keys per chunk of the one-warp-per-row attention (csrc/attention_simt.cu)


def simt_chunks(max_ctx: int, window: int) -> int:
    """Upper bound of the chunks of 64 keys that a row of a step touches, from the longest context of the
    step (and the window, if the layer has one)."""
    most = -(-max(1, max_ctx) // SIMT_CHUNK)
    return min(most, -(-window // SIMT_CHUNK) + 1) if window > 0 else most


def paged_attention_simt(q: torch.Tensor, out: torch.Tensor, k_pages: torch.Tensor, v_pages: torch.Tensor,
                         token_req: torch.Tensor, positions: torch.Tensor, block_table: torch.Tensor,
                         nq: int, nkv: int, hd: int, page_size: int, window: int, scale: float,
                         scratch: torch.Tensor | None = None, max_chunks: int = 0) -> torch.Tensor:
    """q: [n, nq*hd] view (row stride free); pages: [num_pages, nkv, page_size, hd]; out: [n, nq*hd].
    With `scratch` (float32, n * nq * max_chunks * (hd + 2) floats) and max_chunks = simt_chunks(...) > 1 every
    (row, chunk of 64 keys) gets a warp of its own and a second kernel merges them; the result is the same,
    bit for bit, as without."""
    _need_cuda(q, out, k_pages, v_pages, token_req, positions, block_table, scratch)
    n = q.shape[0]
    assert q.stride(1) == 1 and out.stride(1) == 1 and q.dtype == out.dtype == k_pages.dtype == v_pages.dtype
    assert k_pages.is_contiguous() and v_pages.is_contiguous() and block_table.dim() == 2
    if scratch is not None:
        assert scratch.dtype == torch.float32 and scratch.is_contiguous() and max_chunks >= 1
        assert scratch.numel() >= n * nq * max_chunks * (hd + 2)
    lib = load_family("attention_simt")
    _check(lib.wllm_paged_attention_simt(_ptr(q), q.stride(0), _ptr(out), out.stride(0), _ptr(k_pages), _ptr(v_pages),
                                         _dt(q), _ptr(_int32(token_req, "token_req")),
                                         _ptr(_int32(positions, "positions")), _ptr(_int32(block_table, "block_table")),
                                         block_table.shape[1], n, nq, nkv, hd, page_size, window, c_float(scale),
                                         _ptr(scratch), max_chunks if scratch is not None else 0,
                                         _stream()), f"paged_attention_simt(head_dim={hd}, heads={nq}/{nkv})")
    if scratch is not None and max_chunks > 1:
        global launches
        launches += 1    # the merge kernel
    return out


def paged_attention_simt_tiled(q: torch.Tensor, out: torch.Tensor, k_pages: torch.Tensor, v_pages: torch.Tensor,
                               req_q_start: torch.Tensor, req_q_len: torch.Tensor, req_ctx_len: torch.Tensor,
                               block_table: torch.Tensor, max_q_len: int, nq: int, nkv: int, hd: int, page_size: int,
                               window: int, scale: float) -> torch.Tensor:
    """The same attention as `paged_attention_simt`, bit for bit, for steps that bring portions of prompts: a CTA
    takes 32 rows of one (request, key/value head) and reads every tile of keys and values once for all of them
    (csrc/attention_simt.cu, tiled).  Head sizes up to 256; requests are given by their start, length and context."""
    _need_cuda(q, out, k_pages, v_pages, req_q_start, req_q_len, req_ctx_len, block_table)
    assert q.stride(1) == 1 and out.stride(1) == 1 and q.dtype == out.dtype == k_pages.dtype == v_pages.dtype
    assert k_pages.is_contiguous() and v_pages.is_contiguous() and block_table.dim() == 2
    lib = load_family("attention_simt")
    _check(lib.wllm_paged_attention_simt_tiled(_ptr(q), q.stride(0), _ptr(out), out.stride(0), _ptr(k_pages), _ptr(v_pages),
                                               _dt(q), _ptr(_int32(req_q_start, "req_q_start")),
                                               _ptr(_int32(req_q_len, "req_q_len")), _ptr(_int32(req_ctx_len, "req_ctx_len")),
                                               _ptr(_int32(block_table, "block_table")), block_table.shape[1],
                                               req_q_len.shape[0], max_q_len, nq, nkv, hd, page_size, window, c_float(scale),
                                               _stream()), f"paged_attention_simt_tiled(head_dim={hd}, heads={nq}/{nkv})")
    return out


def _indexed(device) -> torch.device:
    device = torch.device(device)
    if device.index is None and device.type == "cuda":
        device = torch.device("cuda", torch.cuda.current_device())
    return device


def _status_word(device) -> torch.Tensor:
    """One int32 per device that stays 0 unless a kernel's bounded wait ran out (see tc_gemm_status)."""
    device = _indexed(device)
    status = _tc_status.get(device)
    if status is None:
        with torch.inference_mode(False):      # whoever asks first: the word is written in place from any mode later
            status = torch.zeros(1, dtype=torch.int32, device=device)
        _tc_status[device] = status
    return status


def mma_head_dim_ok(hd: int) -> bool:
    """Head sizes the tensor-core attention kernels are built for (one build per size)."""
    return hd % 16 == 0 and 16 <= hd <= 256


def attention_mma_scratch_floats(requests: int, nq: int, hd: int, max_splits: int) -> int:
    return requests * nq * max_splits * (hd + 2)


@functools.lru_cache(maxsize=4096)
def decode_split_plan(heads: int, max_ctx: int, tile: int) -> tuple:
    """(split_keys, max_splits) for the decode attention of `heads` (request, key/value head) pairs with up to
    max_ctx keys each.  Every pair is cut into parts of split_keys keys (whole tiles, at least 128) plus a
    shorter rest, one CTA a part, and the CTAs start longest first (the rests last).  Two part sizes are
    weighed by when their last CTA ends on 148 SMs: equal parts, one an SM at most; and parts of the SMs'
    even share of all keys, whose short rests run on the SMs that the whole parts leave free."""
    heads = max(1, heads)
    per_cta = 2 * tile                                          # a CTA costs about two tiles beside its keys

    def up(keys):
        return max(128, -(-keys // tile) * tile)

    def finish(keys):
        splits = -(-max_ctx // keys)
        rest, whole = max_ctx - (splits - 1) * keys, (splits - 1) * heads
        if whole + heads <= sm_count():
            return (keys if splits > 1 else rest) + per_cta
        if whole < sm_count():
            return max(keys + per_cta, -(-heads // (sm_count() - whole)) * (rest + per_cta))
        return -(-(whole + heads) // sm_count()) * (keys + per_cta)
    equal = up(-(-max_ctx // max(1, sm_count() // heads)))
    share = min(up(max_ctx), up(-(-max_ctx * heads // sm_count())))
    keys = min((equal, share), key=lambda k: (finish(k), -k))
    return keys, -(-max_ctx // keys)


def attention_mma_decode(q, out, k_pages, v_pages, req_q_start, req_q_len, req_ctx_len, block_table, nq: int, nkv: int,
                         hd: int, page_size: int, window: int, scale: float, split_keys: int, max_splits: int,
                         scratch: torch.Tensor) -> None:
    """bfloat16 attention of the requests that bring one token (csrc/attention_mma.cu, decode)."""
    _need_cuda(q, out, k_pages, v_pages, req_q_start, req_q_len, req_ctx_len, block_table, scratch)
    assert q.dtype == torch.bfloat16 == out.dtype == k_pages.dtype and q.stride(1) == 1 and out.stride(1) == 1
    assert k_pages.is_contiguous() and v_pages.is_contiguous() and scratch.dtype == torch.float32
    R = req_q_len.shape[0]
    assert scratch.numel() >= attention_mma_scratch_floats(R, nq, hd, max_splits)
    lib = load_family("attention_mma", {"HEAD_DIM": hd})
    _check(lib.wllm_attention_mma_decode(_ptr(q), q.stride(0), _ptr(out), out.stride(0), _ptr(k_pages), _ptr(v_pages),
                                         ctypes.c_longlong(k_pages.shape[0]),
                                         _ptr(_int32(req_q_start, "req_q_start")), _ptr(_int32(req_q_len, "req_q_len")),
                                         _ptr(_int32(req_ctx_len, "req_ctx_len")),
                                         _ptr(_int32(block_table, "block_table")), block_table.shape[1], R, nq, nkv,
                                         page_size, window, c_float(scale), split_keys, max_splits, _ptr(scratch),
                                         _ptr(_status_word(q.device)), _stream()),
           f"attention_mma_decode(head_dim={hd}, heads={nq}/{nkv})")
    global launches
    launches += 1 if max_splits > 1 else 0    # the merge kernel


def attention_prefill_halves_floats(requests: int, max_q_len: int, nq: int, nkv: int, hd: int) -> int:
    """Floats of the `halves` buffer of a prefill launch that shares heavy tiles between two CTAs."""
    tiles = -(-(max_q_len * (nq // nkv)) // 128)
    return tiles * nkv * requests * 2 * 128 * (hd + 4)


def prefill_share_plan(q_lens, ctx_lens, nq: int, nkv: int, hd: int, skip_single: bool) -> int:
    """`split_above` for attention_mma_prefill, from the step's request lengths on the host.  A prompt processed
    from its start gives its 128-row tiles 1, 2, ... tiles of keys to walk, and a grid of at most one CTA an
    SM then ends with its heaviest tile.  Such a grid is launched with two CTAs a tile, and the tiles that are
    heavier than a fair share (a quarter above the mean per SM, at least 8) are halved.  0: no sharing."""
    if hd % 64 != 0:
        return 0
    rep = nq // nkv
    longest = max((n for n in q_lens if not (skip_single and n == 1)), default=0)
    if longest <= 0 or -(-(longest * rep) // 128) * nkv * len(q_lens) > sm_count():
        return 0
    work = heaviest = 0
    for q_len, ctx_len in zip(q_lens, ctx_lens):
        if q_len <= 0 or (skip_single and q_len == 1):
            continue
        pos0, rows = ctx_len - q_len, q_len * rep
        for first in range(0, rows, 128):
            walked = (pos0 + (min(rows, first + 128) - 1) // rep) // 64 + 1
            work += walked * nkv
            heaviest = max(heaviest, walked)
    fair = max(8, -(-5 * work // (4 * sm_count())))
    return fair if heaviest > fair else 0


def attention_mma_prefill(q, out, k_pages, v_pages, req_q_start, req_q_len, req_ctx_len, block_table, max_q_len: int,
                          nq: int, nkv: int, hd: int, page_size: int, window: int, scale: float,
                          skip_single: bool, split_above: int = 0, halves: torch.Tensor | None = None) -> None:
    """bfloat16 attention of the requests that bring several tokens (csrc/attention_mma.cu, prefill).
    split_above > 0 (head sizes in steps of 64): a tile of 128 rows that walks more than that many tiles of 64
    keys is computed by two CTAs, half of the keys each; `halves` (float32) holds their partial results."""
    _need_cuda(q, out, k_pages, v_pages, req_q_start, req_q_len, req_ctx_len, block_table, halves)
    if split_above > 0:
        assert hd % 64 == 0 and halves is not None and halves.dtype == torch.float32 and halves.is_contiguous()
        assert halves.numel() >= attention_prefill_halves_floats(req_q_len.shape[0], max_q_len, nq, nkv, hd)
    assert q.dtype == torch.bfloat16 == out.dtype == k_pages.dtype and q.stride(1) == 1 and out.stride(1) == 1
    assert k_pages.is_contiguous() and v_pages.is_contiguous()
    lib = load_family("attention_mma", {"HEAD_DIM": hd})
    _check(lib.wllm_attention_mma_prefill(_ptr(q), q.stride(0), _ptr(out), out.stride(0), _ptr(k_pages), _ptr(v_pages),
                                          ctypes.c_longlong(k_pages.shape[0]),
                                          _ptr(_int32(req_q_start, "req_q_start")), _ptr(_int32(req_q_len, "req_q_len")),
                                          _ptr(_int32(req_ctx_len, "req_ctx_len")),
                                          _ptr(_int32(block_table, "block_table")), block_table.shape[1],
                                          req_q_len.shape[0], max_q_len, nq, nkv, page_size, window, c_float(scale),
                                          1 if skip_single else 0, split_above, _ptr(halves) if split_above > 0 else None,
                                          _ptr(_status_word(q.device)), _stream()),
           f"attention_mma_prefill(head_dim={hd}, heads={nq}/{nkv})")


def gated_act(gate_up: torch.Tensor, out: torch.Tensor, act: str) -> torch.Tensor:
    """out[n, c] = act(gate_up[n, c]) * gate_up[n, I + c]."""
    _need_cuda(gate_up, out)
    n, two_i = gate_up.shape
    assert gate_up.is_contiguous() and out.is_contiguous() and out.shape == (n, two_i // 2) and out.dtype == gate_up.dtype
    code = {"gelu_tanh": 0, "silu": 1}.get(act)
    if code is None:
        raise KernelError(f"activation {act!r} not supported (gelu_tanh, silu)")
    lib = load_family("activation")
    _check(lib.wllm_gated_act(_ptr(gate_up), _ptr(out), _dt(gate_up), code, n, two_i // 2, _stream()), "gated_act")
    return out


def gemm_f32(a: torch.Tensor, w: torch.Tensor, out: torch.Tensor | None = None) -> torch.Tensor:
    """out[M, N] = a[M, K] @ w[N, K]^T in true 32-bit arithmetic (csrc/gemm_f32.cu)."""
    _need_cuda(a, w, out)
    assert a.dtype == torch.float32 and w.dtype == torch.float32 and a.stride(1) == 1 and w.stride(1) == 1
    M, K = a.shape
    N = w.shape[0]
    assert w.shape[1] == K
    if out is None:
        out = torch.empty((M, N), dtype=torch.float32, device=a.device)
    assert out.stride(1) == 1 and out.shape == (M, N) and out.dtype == torch.float32
    lib = load_family("gemm_f32")
    lib.wllm_gemm_f32_scratch_floats.restype = ctypes.c_longlong
    need = lib.wllm_gemm_f32_scratch_floats(M, N, K)       # partial sums of the few-rows kernel when K has several segments
    scratch = torch.empty(need, dtype=torch.float32, device=a.device) if need else None
    _check(lib.wllm_gemm_f32(_ptr(a), a.stride(0), _ptr(w), w.stride(0), _ptr(out), out.stride(0), M, N, K, _ptr(scratch),
                             ctypes.c_longlong(need), _stream()), "gemm_f32")
    if need:
        global launches
        launches += 1        # the kernel that adds the partial sums
    return out


def fma_peak_tflops(device, iters: int = 20000) -> float:
    """TFLOP/s of a loop of independent 32-bit fused multiply-adds on every SM (csrc/gemm_f32.cu): what the
    32-bit products are measured against, at the clock the device runs such a loop at."""
    sms = torch.cuda.get_device_properties(device).multi_processor_count
    blocks = sms * 8
    out = torch.empty(blocks * 256, dtype=torch.float32, device=device)
    lib = load_family("gemm_f32")
    best = 0.0
    with torch.cuda.device(device):
        for _ in range(4):
            start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            start.record()
            _check(lib.wllm_fma_loop(_ptr(out), blocks, iters, _stream()), "fma_loop")
            end.record()
            torch.cuda.synchronize()
            best = max(best, blocks * 256 * 8 * 2.0 * iters / (start.elapsed_time(end) * 1e-3) / 1e12)
    return best


_TC_EPILOGUES = {"bf16": 0, "f32": 1, "gelu_tanh": 2, "silu": 3}
_tc_status: dict = {}


def tc_gemm_ok(a: torch.Tensor, w: torch.Tensor) -> bool:
    """Shapes the tensor-memory GEMM takes: bfloat16, unit inner strides, K and pitches in steps of 8."""
    return (a.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and a.dim() == 2 and w.dim() == 2
            and a.stride(1) == 1 and w.stride(1) == 1 and a.shape[1] % 8 == 0 and a.stride(0) % 8 == 0
            and w.stride(0) % 8 == 0 and a.data_ptr() % 16 == 0 and w.data_ptr() % 16 == 0)


@functools.lru_cache(maxsize=4096)
def tile_plan(M: int, N: int, K: int, gated: bool = False, may_split: bool = True) -> tuple:
    """(half_rows, parts).  More than 128 rows: see _pair_plan.  At most 128 rows, the product is bound by streaming W: the W tile of a
    stage is two halves of `half_rows` rows, and K is cut into `parts` (at most 16: whoever reads the partial
    sums loads that many at once).  Chosen so that tiles x parts fill the SMs evenly: the cost of a choice is
    the bytes of W that the busiest CTA streams, plus a fixed price per tile and a little per part."""
    if M > 128:
        return _pair_plan(M, N, K, gated), 1
    least = 48 if M <= 32 else (32 if M <= 64 else 16)     # a stage must hold the 128 rows the tensor core reads at A
    kblocks = -(-K // 64)
    cols = N // 2 if gated else N
    best = None
    for half in (128, 112, 96, 80, 64, 48, 32, 16):
        if half < least:
            continue
        tiles = -(-cols // (half if gated else 2 * half))
        wanted = max(1, min(kblocks, sm_count() // tiles, 16)) if may_split else 1
        per = -(-kblocks // wanted)
        parts = -(-kblocks // per)
        waves = -(-(tiles * parts) // sm_count())
        cost = waves * (per * half + 192) * (1.0 + 0.004 * parts)
        if best is None or cost < best[0]:
            best = (cost, half, parts)
    return best[1], best[2]


@functools.lru_cache(maxsize=1)
def resident_pairs() -> int:
    """Pairs of CTAs of the two-CTA product that the device holds at once (74 on 148 SMs)."""
    return max(1, int(load_family("gemm_bf16_tc").wllm_gemm_bf16_tc_resident_pairs()))


def _pair_plan(M: int, N: int, K: int, gated: bool) -> int:
    """half_rows for a product of more than 128 rows, on pairs of CTAs with tiles of 256 rows by 2 * half columns.
    The pairs walk the tiles in rounds; what a round costs was fitted to measurements at 2,048 rows: a block of K
    takes time in proportion to the bytes a CTA loads for it (its 128 rows of A and `half` rows of W: wider tiles
    do more arithmetic per byte from the L2), and a tile's drain is hidden behind the next tile's products except
    with wide tiles (half > 128: one accumulator), where it is paid every round.  Narrower halves than 128 were
    measured too (no faster a block), so they only win where they save a round; with a gate the tile is the two
    halves of 128."""
    if gated:
        return 128
    pairs, kblocks, tiles_m = resident_pairs(), -(-K // 64), -(-M // 256)
    best = None
    for half in (128, 112, 96, 80, 64, 144, 160, 176, 192, 208, 224, 240, 256):
        rounds = -(-(tiles_m * -(-N // (2 * half))) // pairs)
        block_us, drain_us = 0.0017 * (128 + max(half, 128)), 1.0 + 3.0 * max(half, 128) / 128
        cost = rounds * kblocks * block_us + (rounds if half > 128 else 1) * drain_us
        if best is None or cost < best[0] * 0.97:          # another width must pay by 3 %
            best = (cost, half)
    return best[1]


@functools.lru_cache(maxsize=4096)
def product_plan(M: int, N: int, K: int) -> tuple:
    """(half_rows, parts) for a projection whose reader adds partial sums: up to 128 rows tile_plan's choice; above,
    pairs of CTAs, and K is cut into parts as long as the tiles leave at least half of the pairs idle (a prompt of
    256 tokens has 8 tiles of its down projection for 74 pairs): as many parts as fit, of at least 4 blocks of K."""
    if M <= 128:
        return tile_plan(M, N, K)
    half = _pair_plan(M, N, K, False)
    pairs, kblocks = resident_pairs(), -(-K // 64)
    tiles = -(-M // 256) * -(-N // (2 * half))
    wanted = min(pairs // tiles, kblocks // 4, 16)
    if wanted < 2:
        return half, 1
    per = -(-kblocks // wanted)
    return half, -(-kblocks // per)


def split_plan(M: int, N: int, K: int) -> int:
    """Parts to cut K into so that a product of few rows still gives every SM a share of the weights."""
    return product_plan(M, N, K)[1]


def gemm_bf16_tc(a: torch.Tensor, w: torch.Tensor, out: torch.Tensor | None = None, epilogue: str = "bf16",
                 max_ctas: int | None = None, k_splits: int = 1, half_rows: int | None = None, checked: bool = False) -> torch.Tensor:
    """out = a @ w^T on tcgen05 tensor cores (csrc/gemm_bf16_tc.cu).  epilogue 'bf16' | 'f32' (32-bit out) |
    'gelu_tanh' | 'silu' (w = [gate; up] stacked: out[M, N/2] = act(a gate^T) * (a up^T)).
    k_splits > 1 ('f32' only) cuts K into parts; `out` is then [k_splits, M, N] partial sums.
    half_rows: the tile of products of at most 128 rows (see tile_plan, which chooses it when None)."""
    _need_cuda(a, w, out)
    if not checked and not tc_gemm_ok(a, w):        # `checked`: the caller has asked tc_gemm_ok already
        raise KernelError("gemm_bf16_tc: bfloat16 operands with K and row pitches in steps of 8 elements, 16-byte "
                          f"aligned; got a{tuple(a.shape)} stride {a.stride()} w{tuple(w.shape)} stride {w.stride()}")
    M, K = a.shape
    N = w.shape[0]
    assert w.shape[1] == K
    code = _TC_EPILOGUES[epilogue]
    cols = N // 2 if code >= 2 else N
    shape = (M, cols) if k_splits == 1 else (k_splits, M, cols)
    if out is None:
        out = torch.empty(shape, dtype=torch.float32 if code == 1 else torch.bfloat16, device=a.device)
    assert out.shape == shape and out.stride(-1) == 1 and out.dtype == (torch.float32 if code == 1 else torch.bfloat16)
    assert k_splits == 1 or (code == 1 and out.is_contiguous())
    status = _status_word(a.device)
    if max_ctas is None:
        max_ctas = sm_count()
    lib = load_family("gemm_bf16_tc")
    if half_rows is None:
        half_rows = tile_plan(M, N, K, code >= 2, k_splits > 1)[0]
    _check(lib.wllm_gemm_bf16_tc(_ptr(a), a.stride(0), _ptr(w), w.stride(0), _ptr(out), out.stride(-2), M, N, K, code,
                                 k_splits, half_rows, _ptr(status), max_ctas, _stream()),
           f"gemm_bf16_tc({M}x{N}x{K}, {epilogue}, {k_splits} parts)")
    return out


GAVE_UP = {11: "GEMM producer", 12: "GEMM tensor-core issue", 13: "GEMM epilogue", 21: "decode attention",
           22: "prefill attention (mma)", 23: "prefill attention loads", 24: "prefill attention tensor-core issue",
           25: "prefill attention softmax"}


def tc_gemm_status(device) -> int:
    """0, or the code of a role of the tensor-memory GEMM or attention kernels that gave up waiting
    (synchronises; the engine reads the same word with every step's sampled ids instead)."""
    status = _tc_status.get(_indexed(device))
    return 0 if status is None else int(status.item())


def reset_kernel_status(device) -> None:
    status = _tc_status.get(_indexed(device))
    if status is not None:
        status.zero_()


TC_MIN_ROWS = 65   # fewer rows outside project(): the vendor's library (see linear())


def linear(a: torch.Tensor, w: torch.Tensor, out: torch.Tensor | None = None, f32_out: bool = False) -> torch.Tensor:
    """a @ w^T.

    float32 operands: this engine's own FMA kernel (no reduced-precision matrix mode can reach it).
    bfloat16 operands: the tcgen05 / tensor-memory kernel of csrc/gemm_bf16_tc.cu when the shapes allow
    (K and pitches in steps of 8) and the step has more than a handful of rows (steps of few rows go
    through project() instead); otherwise the vendor's matrix library with 32-bit accumulation, which is where the reference engine sends every projection
    (src/wllm/models/llama.py:95-98).  `f32_out` asks for 32-bit results from bfloat16 operands (logits).
    """
    if a.dtype == torch.float32:
        return gemm_f32(a, w, out)
    _need_cuda(a, w)
    if tc_gemm_ok(a, w) and (a.shape[0] >= TC_MIN_ROWS or f32_out):
        return gemm_bf16_tc(a, w, out, "f32" if f32_out else "bf16", checked=True)
    global launches
    launches += 1
    r = torch.matmul(a, w.t(), out=out) if out is not None and not f32_out else torch.matmul(a, w.t())
    return r.float() if f32_out else r


def project(a: torch.Tensor, w: torch.Tensor, buffer) -> tuple:
    """a @ w^T for a layer's projections whose reader can add partial sums itself (the norm and the rotary
    kernels do).  Returns (tensor, parts).  parts = 0: `tensor` is the plain product [n, N] in the operands'
    type.  parts = S > 0 (bfloat16 steps whose tiles alone would leave most SMs idle: up to 128 rows, which are
    bound by streaming the weights, and short prompts): `tensor` is [S, n, N] float32 partial sums over S parts of
    K, left by a split-K run of the tensor-memory GEMM in which every SM takes a share.  `buffer(name, shape, dtype)` supplies the output."""
    n, N = a.shape[0], w.shape[0]
    if a.dtype == torch.bfloat16 and tc_gemm_ok(a, w):
        half, parts = product_plan(n, N, a.shape[1])
        if n <= 128 or parts > 1:
            out = buffer("parts", (parts, n, N), torch.float32)
            gemm_bf16_tc(a, w, out if parts > 1 else out[0], "f32", k_splits=parts, half_rows=half, checked=True)
            return out, parts
    return linear(a, w, buffer("product", (n, N), a.dtype)), 0


def gated_linear(a: torch.Tensor, w_gate_up: torch.Tensor, act: str, out: torch.Tensor, scratch) -> torch.Tensor:
    """out[n, I] = act(a @ gate^T) * (a @ up^T) with w_gate_up = [gate; up].  bfloat16 with enough rows: one
    tensor-memory GEMM whose epilogue applies the activation; otherwise product, then activation kernel
    (`scratch(shape, dtype)` supplies the [n, 2I] intermediate)."""
    if a.dtype == torch.bfloat16 and tc_gemm_ok(a, w_gate_up):
        return gemm_bf16_tc(a, w_gate_up, out, act, checked=True)
    gu = linear(a, w_gate_up, scratch((a.shape[0], w_gate_up.shape[0]), a.dtype))
    return gated_act(gu, out, act)


__all__ = ["KernelError", "KernelBuildError", "embed_gather", "rmsnorm", "rope_kv_write", "paged_attention_simt",
           "paged_attention_simt_tiled",
           "attention_mma_decode", "attention_mma_prefill", "mma_head_dim_ok", "gemm_bf16_tc", "tc_gemm_ok",
           "tc_gemm_status",
           "gated_act", "gemm_f32", "linear", "project", "gated_linear", "split_plan"]
