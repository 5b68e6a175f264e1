"""Made the files in this folder: the plain implementation (tests/plain_gemma.py)
compared once with the reference project's own GemmaForCausalLM on the CPU.

Run from the repository root with the reference checkout's `src` folder given:

    python tests/golden/make_golden.py /path/to/wLLM/src

For both tiny configurations it loads the same seeded weights into the
reference's model class (strict), runs one whole sequence through both, prints
the largest difference, and stores the reference's logits and greedy tokens:

    golden_<A|B>.safetensors   ids [T] int64, logits [T, vocab] float32,
                               prompt [P] int64, greedy [16] int64
"""
import sys
from pathlib import Path

import torch
from safetensors.torch import save_file

ROOT = Path(__file__).resolve().parents[2]
sys.path.insert(0, str(ROOT / "tests"))
sys.path.insert(0, sys.argv[1])

import plain_gemma as plain  # noqa: E402
from tiny_configs import CONFIGS, SEEDS  # noqa: E402
from wllm.models.config import ModelConfig  # noqa: E402
from wllm.models.gemma import GemmaForCausalLM  # noqa: E402
from wllm.models.llama import generate_greedy_naive  # noqa: E402


def main():
    for name, raw in CONFIGS.items():
        w = plain.random_weights(raw, SEEDS[name])
        mc = ModelConfig(
            vocab_size=raw["vocab_size"], hidden_size=raw["hidden_size"],
            intermediate_size=raw["intermediate_size"], num_hidden_layers=raw["num_hidden_layers"],
            num_attention_heads=raw["num_attention_heads"], num_key_value_heads=raw["num_key_value_heads"],
            rms_norm_eps=raw["rms_norm_eps"], rope_theta=raw["rope_theta"],
            max_position_embeddings=raw["max_position_embeddings"], tie_word_embeddings=True,
            attention_bias=False, explicit_head_dim=raw["head_dim"])
        model = GemmaForCausalLM(mc).to(torch.float32).eval()
        model.load_state_dict(w, strict=True)
        g = torch.Generator().manual_seed(100 + SEEDS[name])
        T = 13 if name == "A" else 21
        ids = torch.randint(0, raw["vocab_size"], (T,), generator=g)
        prompt = ids[:7]
        with torch.inference_mode():
            ref_logits = model(ids[None])[0]
            ref_greedy = generate_greedy_naive(model, prompt[None], 16)[0, 7:]
        mine = plain.forward(ids, w, raw)
        mine_greedy = plain.greedy(prompt.tolist(), w, raw, 16)
        diff = (mine - ref_logits).abs().max().item()
        print(f"tiny {name}: max |plain - reference| = {diff:.3e}, "
              f"argmax equal: {bool((mine.argmax(-1) == ref_logits.argmax(-1)).all())}, "
              f"greedy equal: {mine_greedy == ref_greedy.tolist()}")
        save_file({"ids": ids, "logits": ref_logits.clone(), "prompt": prompt.clone(),
                   "greedy": ref_greedy.clone()},
                  str(Path(__file__).parent / f"golden_{name}.safetensors"))


if __name__ == "__main__":
    main()
