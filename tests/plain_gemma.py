"""Plain, slow Gemma 1 written from the reference's formulas.

Whole sequences, no cache, one function per part, float32 (or float64)
throughout, nothing imported from the engine package.  Every function cites
the reference file and lines (paths inside the Sehastrajit-S/wLLM project) whose
formula it restates.  Weights are a dict keyed by checkpoint tensor names
(`model.embed_tokens.weight`, `model.layers.{i}.self_attn.q_proj.weight`, ...).

`tests/golden/make_golden.py` compared this file once with the reference's own
`GemmaForCausalLM` on the CPU; the small outputs of that run are committed in
`tests/golden/`, and `tests/test_plain_gemma.py` re-checks them.
"""
from __future__ import annotations

import math

import torch


def embed(ids: torch.Tensor, table: torch.Tensor, hidden_size: int) -> torch.Tensor:
    """x = E[ids] * sqrt(hidden_size)  (src/wllm/models/llama.py:399-403,
    scale set in src/wllm/models/gemma.py:158)."""
    return table[ids] * (float(hidden_size) ** 0.5)


def rms_norm(x: torch.Tensor, w: torch.Tensor, eps: float) -> torch.Tensor:
    """x * rsqrt(mean(x^2) + eps) * (1 + w)  (src/wllm/models/gemma.py:42-51)."""
    var = x.pow(2).mean(-1, keepdim=True)
    return x * torch.rsqrt(var + eps) * (1.0 + w)


def rope_tables(positions: torch.Tensor, head_dim: int, theta: float):
    """inv_freq[j] = theta^(-2j/head_dim); angle = pos * inv_freq, duplicated
    over both halves (src/wllm/models/llama.py:55, 58-62)."""
    inv_freq = 1.0 / (theta ** (torch.arange(0, head_dim, 2, dtype=torch.float32, device=positions.device) / head_dim))
    ang = positions.to(torch.float32)[:, None] * inv_freq[None, :]
    ang = torch.cat((ang, ang), dim=-1)
    return ang.cos(), ang.sin()


def rotate_half(x: torch.Tensor) -> torch.Tensor:
    """cat(-x[hd/2:], x[:hd/2])  (src/wllm/models/llama.py:47-49)."""
    half = x.shape[-1] // 2
    return torch.cat((-x[..., half:], x[..., :half]), dim=-1)


def apply_rope(x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor) -> torch.Tensor:
    """x*cos + rotate_half(x)*sin, x: [T, heads, hd], cos/sin: [T, hd]
    (src/wllm/models/llama.py:65-71)."""
    return x * cos[:, None, :].to(x.dtype) + rotate_half(x) * sin[:, None, :].to(x.dtype)


def attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, window: int | None = None) -> torch.Tensor:
    """Causal softmax(q k^T / sqrt(hd)) v with grouped heads: query head h uses
    key/value head h // (nq/nkv)  (src/wllm/models/llama.py:74-79, 109-112;
    scale src/wllm/models/llama.py:242).  q: [T,nq,hd], k/v: [T,nkv,hd].
    `window` (not used by Gemma 1) keeps keys p-window+1..p only."""
    T, nq, hd = q.shape
    nkv = k.shape[1]
    rep = nq // nkv
    out = torch.empty_like(q)
    idx = torch.arange(T, device=q.device)
    mask = idx[None, :] <= idx[:, None]
    if window is not None:
        mask &= idx[None, :] > idx[:, None] - window
    for h in range(nq):
        g = h // rep
        s = (q[:, h, :] @ k[:, g, :].T) * (1.0 / math.sqrt(hd))
        s = s.masked_fill(~mask, float("-inf"))
        p = torch.softmax(s, dim=-1)
        out[:, h, :] = p @ v[:, g, :]
    return out


def gelu_tanh(x: torch.Tensor) -> torch.Tensor:
    """0.5 x (1 + tanh(sqrt(2/pi) (x + 0.044715 x^3)))  (F.gelu(approximate=
    "tanh") in src/wllm/models/gemma.py:62)."""
    return 0.5 * x * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (x + 0.044715 * x.pow(3))))


def feed_forward(x: torch.Tensor, wg: torch.Tensor, wu: torch.Tensor, wd: torch.Tensor) -> torch.Tensor:
    """down(gelu_tanh(gate(x)) * up(x))  (src/wllm/models/gemma.py:54-62)."""
    return (gelu_tanh(x @ wg.T) * (x @ wu.T)) @ wd.T


def self_attention(x, w, prefix, positions, cfg):
    """q/k/v projections, rotation, attention, output projection
    (src/wllm/models/llama.py:100-115)."""
    T = x.shape[0]
    nq, nkv, hd = cfg["num_attention_heads"], cfg["num_key_value_heads"], cfg["head_dim"]
    q = (x @ w[prefix + "q_proj.weight"].T).view(T, nq, hd)
    k = (x @ w[prefix + "k_proj.weight"].T).view(T, nkv, hd)
    v = (x @ w[prefix + "v_proj.weight"].T).view(T, nkv, hd)
    cos, sin = rope_tables(positions, hd, cfg["rope_theta"])
    q, k = apply_rope(q, cos, sin), apply_rope(k, cos, sin)
    o = attention(q, k, v).reshape(T, nq * hd)
    return o @ w[prefix + "o_proj.weight"].T


def decoder_layer(x, w, i, positions, cfg):
    """x += attn(norm_in(x)); x += mlp(norm_post(x))  (src/wllm/models/gemma.py:83-93)."""
    p = f"model.layers.{i}."
    h = rms_norm(x, w[p + "input_layernorm.weight"], cfg["rms_norm_eps"])
    x = x + self_attention(h, w, p + "self_attn.", positions, cfg)
    h = rms_norm(x, w[p + "post_attention_layernorm.weight"], cfg["rms_norm_eps"])
    x = x + feed_forward(h, w[p + "mlp.gate_proj.weight"], w[p + "mlp.up_proj.weight"], w[p + "mlp.down_proj.weight"])
    return x


def logits_head(h: torch.Tensor, w: dict, cfg: dict) -> torch.Tensor:
    """Tied: h @ E^T with the unscaled table; untied: lm_head.weight
    (src/wllm/models/llama.py:443-446)."""
    if cfg.get("tie_word_embeddings", True):
        return h @ w["model.embed_tokens.weight"].T
    return h @ w["lm_head.weight"].T


def forward(ids: list[int] | torch.Tensor, w: dict, cfg: dict, dtype=torch.float32) -> torch.Tensor:
    """Logits [T, vocab] of one whole sequence (src/wllm/models/llama.py:405-415,
    432-434).  `cfg` is the raw config.json dictionary with head_dim filled in."""
    where = w["model.embed_tokens.weight"].device     # the host in the tests of the tiny models; any device works
    ids = torch.as_tensor(ids, dtype=torch.long).to(where)
    w = {k: t.to(dtype) for k, t in w.items()}
    positions = torch.arange(ids.shape[0], device=where)
    x = embed(ids, w["model.embed_tokens.weight"], cfg["hidden_size"])
    for i in range(cfg["num_hidden_layers"]):
        x = decoder_layer(x, w, i, positions, cfg)
    x = rms_norm(x, w["model.norm.weight"], cfg["rms_norm_eps"])
    return logits_head(x, w, cfg)


def greedy(ids: list[int], w: dict, cfg: dict, n: int) -> list[int]:
    """Full recompute for each new token (src/wllm/models/llama.py:599-610)."""
    ids = list(ids)
    out = []
    for _ in range(n):
        t = int(forward(ids, w, cfg)[-1].argmax())
        out.append(t)
        ids.append(t)
    return out


def random_weights(cfg: dict, seed: int, std: float = 0.02, norm_std: float = 0.1) -> dict:
    """Seeded weights by checkpoint tensor name, rounded to bfloat16 values so
    that a bfloat16 model folder and this float32 dict hold the same numbers."""
    g = torch.Generator().manual_seed(seed)
    H, I, V = cfg["hidden_size"], cfg["intermediate_size"], cfg["vocab_size"]
    nq, nkv, hd = cfg["num_attention_heads"], cfg["num_key_value_heads"], cfg["head_dim"]

    def mat(*shape, s=std):
        return (torch.randn(*shape, generator=g) * s).to(torch.bfloat16).to(torch.float32)

    w = {"model.embed_tokens.weight": mat(V, H)}
    for i in range(cfg["num_hidden_layers"]):
        p = f"model.layers.{i}."
        w[p + "self_attn.q_proj.weight"] = mat(nq * hd, H)
        w[p + "self_attn.k_proj.weight"] = mat(nkv * hd, H)
        w[p + "self_attn.v_proj.weight"] = mat(nkv * hd, H)
        w[p + "self_attn.o_proj.weight"] = mat(H, nq * hd)
        w[p + "mlp.gate_proj.weight"] = mat(I, H)
        w[p + "mlp.up_proj.weight"] = mat(I, H)
        w[p + "mlp.down_proj.weight"] = mat(H, I)
        w[p + "input_layernorm.weight"] = mat(H, s=norm_std)
        w[p + "post_attention_layernorm.weight"] = mat(H, s=norm_std)
    w["model.norm.weight"] = mat(H, s=norm_std)
    if not cfg.get("tie_word_embeddings", True):
        w["lm_head.weight"] = mat(V, H)
    return w


# ---------------------------------------------------------------------------
# Sampling, restated from src/wllm/engine/sampling.py.
# ---------------------------------------------------------------------------

def penalise_repeats(logits: torch.Tensor, generated: list[int], penalty: float) -> torch.Tensor:
    """Seen tokens: positive logits divided, negative multiplied by `penalty`
    (src/wllm/engine/sampling.py:45-58)."""
    logits = logits.clone()
    if penalty == 1.0 or not generated:
        return logits
    idx = torch.tensor(sorted(set(generated)), dtype=torch.long)
    row = logits[idx]
    logits[idx] = torch.where(row > 0, row / penalty, row * penalty)
    return logits


def kept_mask(scaled: torch.Tensor, top_k: int, top_p: float, min_p: float) -> torch.Tensor:
    """Tokens that survive top-k, top-p and min-p, all three judged on the
    softmax of the whole scaled row sorted downwards; rank 0 always stays
    (src/wllm/engine/sampling.py:61-98)."""
    V = scaled.shape[0]
    sorted_logits, sorted_idx = torch.sort(scaled, descending=True, stable=True)
    keep = torch.ones(V, dtype=torch.bool)
    if top_k > 0:
        keep &= torch.arange(V) < top_k
    probs = torch.softmax(sorted_logits, dim=-1)
    if top_p < 1.0:
        over = probs.cumsum(-1) > top_p
        over[0] = False
        keep &= ~over
    if min_p > 0.0:
        below = probs < min_p * probs[0]
        below[0] = False
        keep &= ~below
    mask = torch.zeros(V, dtype=torch.bool)
    mask[sorted_idx[keep]] = True
    return mask


def sampling_distribution(logits, temperature, top_k=0, top_p=1.0, min_p=0.0,
                          repetition_penalty=1.0, generated=()):
    """(probabilities over the vocabulary, log-probabilities before truncation)
    as the reference's `sample` builds them (src/wllm/engine/sampling.py:115-137).
    For temperature 0 the distribution is one-hot at the arg-max of the penalised
    logits and the log-probabilities are those at temperature 1."""
    logits = penalise_repeats(logits.to(torch.float64), list(generated), repetition_penalty)
    if temperature == 0.0:
        probs = torch.zeros_like(logits)
        probs[int(logits.argmax())] = 1.0
        return probs, torch.log_softmax(logits, dim=-1)
    scaled = logits / max(temperature, 1e-5)
    mask = kept_mask(scaled, top_k, top_p, min_p)
    probs = torch.softmax(scaled.masked_fill(~mask, float("-inf")), dim=-1)
    return probs, torch.log_softmax(scaled, dim=-1)
