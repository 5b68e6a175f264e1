"""The engine at head sizes between the two tiny configurations' and Gemma's own: 16 (the smallest step), 64 and
192 (tensor-memory prefill on one CTA a tile, TMA decode), 80 (mma.sync with a cp.async ring) and 128 (pairs of
CTAs).  A two-layer model with grouped heads (4 query heads on 2 key/value heads), a width and a vocabulary that are
no powers of two; whole prompts, mixed batches with pages used again and decoded tails against the plain
implementation, in 32-bit (bit-equal across the cuts as well) and in bfloat16."""
import pytest
import torch

import traces
from helpers import max_diff

pytestmark = pytest.mark.gpu


def config(hd):
    return dict(architectures=["GemmaForCausalLM"], model_type="gemma", num_hidden_layers=2, hidden_size=72,
                num_attention_heads=4, num_key_value_heads=2, head_dim=hd, intermediate_size=200, vocab_size=333,
                max_position_embeddings=400, rope_theta=3000.0, rms_norm_eps=1e-5, tie_word_embeddings=True)


@pytest.mark.parametrize("hd", [16, 64, 80, 128, 192])
def test_other_head_sizes_match_plain_under_every_cut(hd, tmp_path):
    import os

    import plain_gemma as plain
    from safetensors.torch import load_file
    from test_gpu_replay import gpu_runner
    from wllm_b200.weights import write_random_model
    cfg = config(hd)
    folder = write_random_model(str(tmp_path / "m"), cfg, seed=hd)
    w = {k: v.float() for k, v in load_file(os.path.join(folder, "model.safetensors")).items()}
    g = torch.Generator().manual_seed(hd)
    reqs = {f"r{i}": torch.randint(0, cfg["vocab_size"], (n,), generator=g).tolist() for i, n in enumerate((150, 3, 66, 260, 31))}
    ref = {}
    for rid, toks in reqs.items():
        ref.update({(rid, p): row for p, row in enumerate(plain.forward(toks, w, cfg))})
    scale = max(float(r.abs().max()) for r in ref.values())
    for dtype, tol in ((torch.float32, 5e-5), (torch.bfloat16, 0.006 * max(1.0, scale))):
        first = None
        for cut, steps in (("whole", traces.whole(reqs)), ("tail", traces.tail_singly(reqs, tail=20)),
                           ("mixed", traces.mixed(reqs, seed=hd, max_portion=70))):
            pages = -(-traces.peak_tokens(steps) // 16)
            runner = gpu_runner(folder, dtype, 16, pages, poison=True)
            rows = traces.run_in_process(runner, steps)
            worst = max_diff(rows, ref)
            assert worst < tol, f"head size {hd}, {dtype}, {cut}: largest difference {worst:.3e} (logits up to {scale:.2f})"
            if dtype == torch.float32:
                if first is None:
                    first = rows
                else:
                    bad = sorted(k for k in first if not torch.equal(first[k], rows[k]))
                    assert not bad, f"head size {hd}, {cut}: first differing (request, position) {bad[0]}"
