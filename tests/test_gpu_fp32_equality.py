"""Gemma-7B's layer widths in the true 32-bit path, prompts from one token to thousands, run four ways
(each prompt whole; token by token with all prompts in one batch; portions of 512 tokens; mixed, up to four
live requests with portions of some beside single tokens of others and so few pages that they are used
again; the token-by-token steps replayed from captured CUDA graphs), logits at ALL positions:

  * the four ways agree bit for bit (every row's digest, a 64-bit sum over the row's bit patterns);
  * the whole-prompt logits stay within a stated bound of the plain implementation, which runs on the same
    device on the same weight tensors (views into the engine's own, no copy) in float32.

Two sizes.  The default (part of every `-m gpu` run) has two layers, a vocabulary of 4,096 and prompts up to
700 tokens.  `WLLM_FP32_EQUALITY=full` is the whole model (28 layers, 256,000-token vocabulary, 34 GB of
weights, 16 prompts of 1 to 6,000 tokens); it takes minutes and prints one JSON line (also appended to the
file `WLLM_FP32_EQUALITY_OUT` names) with the largest difference, the first differing place if any, the time of
each way, the pages' high-water mark and what the 32-bit kernels reached in decode and prefill:

    WLLM_FP32_EQUALITY=full python -m pytest tests/test_gpu_fp32_equality.py -m gpu -x -q -s
"""
import json
import os
import time

import pytest
import torch

import plain_gemma as plain
import traces

pytestmark = pytest.mark.gpu
FULL = os.environ.get("WLLM_FP32_EQUALITY", "") == "full"
WIDTHS = dict(hidden_size=3072, num_attention_heads=16, num_key_value_heads=16, head_dim=256, intermediate_size=24576)
SIZES = {
    "small": dict(layers=2, vocab=4096, lengths=[1, 2, 65, 300, 513, 700], portion=128, page=16, mixed_portion=96,
                  bound=2e-4),
    "full": dict(layers=28, vocab=256000, lengths=[1, 2, 17, 64, 65, 255, 512, 777, 1024, 1500, 2048, 2777, 3500,
                                                   4096, 5000, 6000], portion=512, page=64, mixed_portion=1024,
                 bound=2e-3),
}


def token_by_token(requests: dict) -> list:
    """Step t brings token t of every request that has one: all requests in one batch, ended as they run out."""
    steps, longest = [], max(len(t) for t in requests.values())
    for t in range(longest):
        live = [(rid, toks) for rid, toks in requests.items() if len(toks) > t]
        steps.append({"step": t, "entries": [{"id": rid, "tokens": [toks[t]], "want": [0]} for rid, toks in live],
                      "end": [rid for rid, toks in live if len(toks) == t + 1]})
    return steps


def row_digests(logits: torch.Tensor) -> torch.Tensor:
    """One 64-bit number per row that changes with any bit of the row (-0.0 counted as 0.0)."""
    V = logits.shape[1]
    mult = (torch.arange(V, device=logits.device, dtype=torch.int64) * 2654435761 + 40503) | 1
    out = []
    for r in range(0, logits.shape[0], 256):
        bits = (logits[r:r + 256] + 0.0).contiguous().view(torch.int32).to(torch.int64)
        out.append((bits * mult).sum(dim=1))
    return torch.cat(out)


def plain_weights(model, cfg: dict) -> dict:
    """The engine's weight tensors under their checkpoint names (views: the fused matrices are cut, not copied)."""
    nq, nkv, hd, inter = cfg["num_attention_heads"], cfg["num_key_value_heads"], cfg["head_dim"], cfg["intermediate_size"]
    w = {"model.embed_tokens.weight": model.embedding.table, "model.norm.weight": model.final_norm.weight}
    for i, b in enumerate(model.blocks):
        p = f"model.layers.{i}."
        q, k = nq * hd, nkv * hd
        w[p + "self_attn.q_proj.weight"], w[p + "self_attn.k_proj.weight"] = b.mixer.wqkv[:q], b.mixer.wqkv[q:q + k]
        w[p + "self_attn.v_proj.weight"], w[p + "self_attn.o_proj.weight"] = b.mixer.wqkv[q + k:], b.mixer.wo
        w[p + "mlp.gate_proj.weight"], w[p + "mlp.up_proj.weight"] = b.feed_forward.wgu[:inter], b.feed_forward.wgu[inter:]
        w[p + "mlp.down_proj.weight"] = b.feed_forward.wd
        w[p + "input_layernorm.weight"], w[p + "post_attention_layernorm.weight"] = b.norm_in.weight, b.norm_post.weight
    return w


def run_cut(model, engine_config, steps: list, page: int, on_step=None, graphs: bool = False):
    """Replay a trace on a fresh cache of exactly the pages it needs.  Returns ({(request, position): digest},
    seconds, pages at the high-water mark, pages in the pool, [(live requests, cached tokens, ms)] per step).
    `graphs`: steps in which every request brings one token are replayed from captured CUDA graphs."""
    from wllm_b200.engine import StepEntry, build_runner
    pages = -(-traces.peak_tokens(steps, round_to=page) // page)
    runner = build_runner(model, engine_config, num_pages=pages)
    if graphs:
        runner.enable_graphs()
    live, pos, keys, digests, events, loads = {}, {}, [], [], [], []
    torch.cuda.synchronize()
    start = time.perf_counter()
    for s in steps:
        entries = []
        for e in s["entries"]:
            rid = e["id"]
            if rid not in live:
                live[rid], pos[rid] = runner.cache.open(rid), 0
            entries.append(StepEntry(live[rid], e["tokens"], e["want"]))
            keys.extend((rid, pos[rid] + w) for w in e["want"])
            pos[rid] += len(e["tokens"])
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        logits = runner.step(entries)
        b.record()
        events.append((a, b))
        loads.append((len(entries), sum(pos[e["id"]] for e in s["entries"]), sum(len(e["tokens"]) for e in s["entries"])))
        if on_step is not None:
            on_step(s, logits)
        digests.append(row_digests(logits))
        del logits
        for rid in s["end"]:
            runner.cache.close(live.pop(rid))
    torch.cuda.synchronize()
    seconds = time.perf_counter() - start
    runner.cache.check()
    assert runner.cache.free_pages() == [pages]
    flat = torch.cat(digests).cpu().tolist()
    assert len(flat) == len(keys)
    times = [(n, cached, tokens, a.elapsed_time(b)) for (n, cached, tokens), (a, b) in zip(loads, events)]
    high = list(runner.cache.pages_high_water)
    del runner
    torch.cuda.empty_cache()
    return dict(zip(keys, flat)), seconds, high, pages, times


def test_four_ways_agree_bit_for_bit_and_with_plain():
    from wllm_b200.config import EngineConfig, GemmaConfig
    from wllm_b200.engine import build_model
    from wllm_b200.kernels import ops
    size = SIZES["full" if FULL else "small"]
    raw = dict(architectures=["GemmaForCausalLM"], model_type="gemma", num_hidden_layers=size["layers"],
               vocab_size=size["vocab"], max_position_embeddings=8192, rope_theta=10000.0, rms_norm_eps=1e-6,
               tie_word_embeddings=True, **WIDTHS)
    torch.backends.cuda.matmul.allow_tf32 = False
    torch.set_float32_matmul_precision("highest")
    engine_config = EngineConfig(dtype=torch.float32, block_size=size["page"], max_num_seqs=len(size["lengths"]) + 1)
    model = build_model(None, torch.float32, engine_config.device, config=GemmaConfig.from_dict(raw), random_seed=4)
    weights = plain_weights(model, raw)
    g = torch.Generator().manual_seed(6)
    requests = {f"r{i}": torch.randint(0, size["vocab"], (n,), generator=g).tolist() for i, n in enumerate(size["lengths"])}

    # each prompt whole, against the plain implementation prompt by prompt
    worst = {"diff": 0.0, "where": None, "scale": 0.0, "plain_seconds": 0.0}

    def against_plain(step, logits):
        rid = step["entries"][0]["id"]
        torch.cuda.synchronize()
        began = time.perf_counter()
        want = plain.forward(requests[rid], weights, raw)
        torch.cuda.synchronize()
        worst["plain_seconds"] += time.perf_counter() - began
        worst["scale"] = max(worst["scale"], float(want.abs().max()))
        for r in range(0, want.shape[0], 512):
            per_row = (logits[r:r + 512].double() - want[r:r + 512].double()).abs().max(dim=1).values
            top = float(per_row.max())
            if top > worst["diff"]:
                worst["diff"], worst["where"] = top, (rid, r + int(per_row.argmax()))
    record = {"workload": "fp32 equality", "layers": size["layers"], "vocab": size["vocab"], "prompts": size["lengths"],
              "page_size": size["page"], "weight_bytes": model.weight_bytes()}
    cuts = {"whole": traces.whole(requests), "token_by_token": token_by_token(requests),
            "portions": traces.portions(requests, sizes=(size["portion"],)),
            "mixed": traces.mixed(requests, seed=8, max_live=4, decode_tail=32, max_portion=size["mixed_portion"])}
    first, problems = None, []
    for name, steps in cuts.items():
        rows, seconds, high, pages, times = run_cut(model, engine_config, steps, size["page"],
                                                    against_plain if name == "whole" else None,
                                                    graphs=name == "token_by_token")
        record[name] = {"seconds": round(seconds, 2), "steps": len(steps), "pages": pages, "pages_high_water": high}
        if name == "whole":
            first = rows
            n, cached, tokens, ms = max(times, key=lambda t: t[2])          # the longest prompt's step
            attn = 4.0 * WIDTHS["num_attention_heads"] * WIDTHS["head_dim"] * tokens * (tokens + 1) / 2 * size["layers"]
            per_token = size["layers"] * (3072 * (16 + 32) * 256 + 16 * 256 * 3072 + 3 * 3072 * 24576) + size["vocab"] * 3072
            record[name]["longest"] = {"tokens": tokens, "ms": round(ms, 1),
                                       "tflops": round((2.0 * per_token * tokens + attn) / ms / 1e9, 2)}
        else:
            assert set(rows) == set(first)
            bad = sorted((k for k in first if first[k] != rows[k]), key=lambda k: (int(k[0][1:]), k[1]))
            record[name]["first_differing"] = list(bad[0]) if bad else None
            record[name]["rows_differing"] = len(bad)
            if bad:
                problems.append(f"{name}: {len(bad)} of {len(first)} rows differ from the whole prompts', first at {bad[0]}")
        if name == "token_by_token":
            per_token_cache = 2 * size["layers"] * WIDTHS["num_key_value_heads"] * WIDTHS["head_dim"] * 4
            points = []
            for want_cached in (0.1, 0.5, 0.9):          # steps early, midway and late in the run
                n, cached, tokens, ms = times[int(want_cached * (len(times) - 1))]
                gb = (record["weight_bytes"] + cached * per_token_cache) / 1e9
                points.append({"requests": n, "cached_tokens": cached, "ms": round(ms, 2), "gb_read": round(gb, 2),
                               "gbs": round(gb / ms * 1e3, 0)})
            record[name]["decode_points"] = points
    record["rows"] = len(first)
    record["max_abs_diff_vs_plain"], record["at"], record["logit_scale"] = worst["diff"], worst["where"], worst["scale"]
    record["bound"] = size["bound"]
    record["plain_seconds_inside_whole"] = round(worst["plain_seconds"], 2)
    record["fma_loop_tflops"] = round(ops.fma_peak_tflops(engine_config.device), 1)
    line = json.dumps(record)
    print("\n" + line)
    if os.environ.get("WLLM_FP32_EQUALITY_OUT"):
        with open(os.environ["WLLM_FP32_EQUALITY_OUT"], "a") as f:
            f.write(line + "\n")
    assert not problems, "; ".join(problems)
    assert worst["diff"] < size["bound"], f"largest difference from the plain implementation {worst['diff']:.3e} at {worst['where']}"
