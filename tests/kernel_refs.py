"""Plain PyTorch statements of what each CUDA entry point computes.

Two uses.  The `-m gpu` kernel tests compare every kernel with the function of the
same name here, in float32 or float64 on the host.  And `install(monkeypatch)` puts
these functions in the kernels' place so that the engine's host logic (batch
building, block tables, page reuse, scheduling) can be exercised without a GPU; that
is a test double, not a path of the product, which has no CPU implementation.
"""
from __future__ import annotations

import math

import torch


def embed_gather(ids, table, scale, out):
    out.copy_(table[ids.long()].float() * scale)
    return out


def rmsnorm(resid, delta, weight, eps, offset, out, rows=None, delta_splits=0):
    if delta is not None and delta_splits:
        r = resid
        for part in delta:           # partial sums, added to the row in order
            r = r + part
    else:
        r = resid if delta is None else resid + delta.float()
    if rows is not None:
        r = r[rows.long()]
    elif delta is not None:
        resid.copy_(r)
    inv = 1.0 / torch.sqrt(r.pow(2).mean(-1, keepdim=True) + eps)
    out.copy_(((r * inv) * (offset + weight.float())).to(out.dtype))
    return out


def rope_kv_write(qkv, q_out, positions, slots, inv_freq, k_pages, v_pages, nq, nkv, hd, rot_dim, page_size, in_splits=0,
                  pairing="half"):
    if in_splits:
        total = torch.zeros_like(qkv[0])
        for part in qkv:
            total = total + part
        qkv = total
    n = qkv.shape[0]
    x = qkv.float().clone().view(n, nq + 2 * nkv, hd)
    ang = positions.float()[:, None] * inv_freq.float()[None, :]
    cos, sin = ang.cos()[:, None, :], ang.sin()[:, None, :]
    half = rot_dim // 2
    qk = x[:, : nq + nkv, :]
    if pairing == "interleaved":      # element 2j turns with 2j + 1
        x1, x2 = qk[..., 0:rot_dim:2].clone(), qk[..., 1:rot_dim:2].clone()
        qk[..., 0:rot_dim:2] = x1 * cos - x2 * sin
        qk[..., 1:rot_dim:2] = x2 * cos + x1 * sin
    else:                             # element j turns with j + rot_dim/2
        x1, x2 = qk[..., :half].clone(), qk[..., half:rot_dim].clone()
        qk[..., :half] = x1 * cos - x2 * sin
        qk[..., half:rot_dim] = x2 * cos + x1 * sin
    rounded = x.to(q_out.dtype)
    q_out.copy_(rounded[:, :nq].reshape(n, -1))
    if slots is None:
        return
    for t in range(n):
        s = int(slots[t])
        if s < 0:
            continue
        page, off = divmod(s, page_size)
        k_pages[page, :, off, :] = rounded[t, nq:nq + nkv]
        v_pages[page, :, off, :] = rounded[t, nq + nkv:]


def paged_attention(q, out, k_pages, v_pages, token_req, positions, block_table, nq, nkv, hd, page_size, window, scale,
                    dtype=torch.float32):
    n = q.shape[0]
    rep = nq // nkv
    for t in range(n):
        pos, table = int(positions[t]), block_table[int(token_req[t])]
        first = max(0, pos - window + 1) if window > 0 else 0
        keys = torch.arange(first, pos + 1, device=k_pages.device)
        pages = table[(keys // page_size).long()].long()
        offs = (keys % page_size).long()
        k = k_pages[pages, :, offs, :].to(dtype)   # [keys, nkv, hd]
        v = v_pages[pages, :, offs, :].to(dtype)
        qt = q[t].to(dtype).view(nq, hd)
        for h in range(nq):
            s = (k[:, h // rep, :] @ qt[h]) * scale
            p = torch.softmax(s, dim=0)
            out[t, h * hd:(h + 1) * hd] = (p @ v[:, h // rep, :]).to(out.dtype)
    return out


def paged_attention_simt(q, out, k_pages, v_pages, token_req, positions, block_table, nq, nkv, hd, page_size, window,
                         scale, scratch=None, max_chunks=0):
    return paged_attention(q, out, k_pages, v_pages, token_req, positions, block_table, nq, nkv, hd, page_size, window,
                           scale)


def paged_attention_simt_tiled(q, out, k_pages, v_pages, req_q_start, req_q_len, req_ctx_len, block_table, max_q_len, nq,
                               nkv, hd, page_size, window, scale):
    token_req, positions = [], []
    for r, (n, c) in enumerate(zip(req_q_len.tolist(), req_ctx_len.tolist())):
        token_req += [r] * n
        positions += list(range(c - n, c))
    return paged_attention(q, out, k_pages, v_pages, torch.tensor(token_req, dtype=torch.int32),
                           torch.tensor(positions, dtype=torch.int32), block_table, nq, nkv, hd, page_size, window, scale)


def gated_act(gate_up, out, act):
    inter = gate_up.shape[1] // 2
    g, u = gate_up[:, :inter].float(), gate_up[:, inter:].float()
    if act == "gelu_tanh":
        a = 0.5 * g * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (g + 0.044715 * g.pow(3))))
    elif act == "silu":
        a = g / (1.0 + torch.exp(-g))
    else:
        raise ValueError(act)
    out.copy_((a * u).to(out.dtype))
    return out


def gemm_f32(a, w, out=None):
    r = a @ w.t()
    if out is None:
        return r
    out.copy_(r)
    return out


def linear(a, w, out=None, f32_out=False):
    r = a.float() @ w.float().t()
    r = r if f32_out else r.to(a.dtype)
    if out is None:
        return r
    out.copy_(r)
    return out


def project(a, w, buffer):
    return linear(a, w), 0


def gated_linear(a, w_gate_up, act, out, scratch):
    return gated_act(linear(a, w_gate_up), out, act)


def install(monkeypatch):
    """Replace the kernels by these functions (host-logic tests only)."""
    from wllm_b200.kernels import ops
    for name in ("embed_gather", "rmsnorm", "rope_kv_write", "paged_attention_simt", "paged_attention_simt_tiled", "gated_act", "gemm_f32", "linear", "project", "gated_linear"):
        monkeypatch.setattr(ops, name, globals()[name])
