"""The kernel families of the package and the build of all of them at once."""
from __future__ import annotations

from concurrent.futures import ThreadPoolExecutor

from .build import compile_family

# family -> list of define sets to build ahead of time ({} = the family has no variants)
FAMILIES = {
    "embedding": [{}],
    "norm": [{}],
    "rope_cache": [{}],
    "attention_simt": [{}],
    "activation": [{}],
    "gemm_f32": [{}],
    "sampling": [{}],
    "staging": [{}],
    "gemm_bf16_tc": [{}],
    # tensor-core attention is built per head size; others are built when a model first asks
    "attention_mma": [{"HEAD_DIM": 256}, {"HEAD_DIM": 32}, {"HEAD_DIM": 48}],
    "attention_decode_static": [{"HEAD_DIM": 256}],
}


def compile_all(verbose: bool = True) -> list:
    jobs = [(fam, d) for fam, variants in FAMILIES.items() for d in variants]
    with ThreadPoolExecutor(max_workers=8) as pool:
        return list(pool.map(lambda j: compile_family(j[0], j[1] or None, verbose), jobs))
