"""The engine's host logic (batches, block tables, page reuse) with the kernels replaced
by their plain statements (tests/kernel_refs.py): every way of cutting the same
requests gives the plain implementation's logits.  No GPU; the `-m gpu` tests repeat
this with the real kernels."""
import pytest
import torch

import kernel_refs
import traces
from helpers import host_runner, make_folder, max_diff, plain_rows, random_requests
from tiny_configs import PAGE_SIZES

LENGTHS = {"A": (7, 19, 33, 70, 41, 12, 90, 55, 66, 100), "B": (1, 4, 50, 64, 120, 37, 81, 2, 130, 77)}


@pytest.fixture(scope="module")
def setups(tmp_path_factory):
    out = {}
    for name in ("A", "B"):
        folder = make_folder(tmp_path_factory.mktemp("m"), name)
        reqs = random_requests(name, LENGTHS[name], seed=5)
        out[name] = (folder, reqs, plain_rows(folder, name, reqs))
    return out


@pytest.mark.parametrize("name", ["A", "B"])
@pytest.mark.parametrize("mode", ["whole", "tail", "portions", "mixed"])
def test_every_cut_matches_plain(setups, monkeypatch, name, mode):
    kernel_refs.install(monkeypatch)
    folder, reqs, ref = setups[name]
    steps = {"whole": traces.whole, "tail": traces.tail_singly, "portions": traces.portions,
             "mixed": lambda r: traces.mixed(r, seed=3)}[mode](reqs)
    ps = PAGE_SIZES[name]
    pages = -(-traces.peak_tokens(steps) // ps)
    runner = host_runner(folder, torch.float32, ps, pages)
    rows = traces.run_in_process(runner, steps)
    assert max_diff(rows, ref) < 2e-5
    assert runner.cache.free_pages() == [pages]
    if mode == "mixed":
        assert runner.cache.groups[0].pool.takes > pages, "the trace must use pages again"


# ---- launch plans worked out on the host (pure functions of sizes) ----

def test_decode_split_plan_covers_the_context_in_whole_tiles():
    from wllm_b200.kernels import ops
    for heads in (1, 3, 8, 16, 31, 64, 128, 1000):
        for ctx in (1, 64, 129, 300, 4096, 8118, 100000):
            for tile in (32, 64):
                keys, splits = ops.decode_split_plan(heads, ctx, tile)
                assert keys >= 128 and keys % tile == 0 and 1 <= splits <= 256 or ctx > 128 * 256
                assert (splits - 1) * keys < ctx <= splits * keys       # no empty part, every key covered
    # few pairs of many keys: about one part an SM; many pairs: one part each
    assert ops.decode_split_plan(8, 8192, 32) == (448, 19)
    assert ops.decode_split_plan(1000, 4096, 32)[1] == 1


def test_tile_plan_of_products_of_few_rows():
    from wllm_b200.kernels import ops
    for M in (1, 8, 32, 33, 64, 65, 128):
        for N, K, gated in ((2048, 2048, False), (2560, 2048, False), (2048, 16384, False), (32768, 2048, True), (300, 200, False)):
            half, parts = ops.tile_plan(M, N, K, gated, not gated)
            assert half % 16 == 0 and (48 if M <= 32 else 32 if M <= 64 else 16) <= half <= 128
            kblocks = -(-K // 64)
            assert 1 <= parts <= 16 and -(-kblocks // parts) * (parts - 1) < kblocks
    assert ops.tile_plan(300, 2048, 2048) == (128, 1)             # more than 128 rows: pairs of CTAs, full width


def test_prefill_share_plan_only_for_grids_that_fit_the_sms_once():
    from wllm_b200.kernels import ops
    assert ops.prefill_share_plan([2048], [2048], 8, 1, 64, False) == 18       # 128 tiles, the heaviest walks 32
    assert ops.prefill_share_plan([2048], [16384], 8, 1, 64, False) == 0       # every tile walks about the same
    assert ops.prefill_share_plan([2048] * 4, [2048] * 4, 8, 1, 64, False) == 0   # more CTAs than SMs anyway
    assert ops.prefill_share_plan([1, 1], [500, 600], 8, 1, 64, True) == 0     # single tokens are the decode kernel's
    assert ops.prefill_share_plan([2048], [2048], 8, 1, 48, False) == 0        # head sizes without the tcgen05 kernel


def test_sampling_options_are_packed_row_by_row():
    """The one int32 array that carries a step's sampling options to the device, and the bits that say which
    selection passes some row needs."""
    import numpy as np
    from wllm_b200.sampling import SamplingParams
    from wllm_b200.sampling.sampler import pack_options
    params = [SamplingParams(temperature=0.5, top_k=7), SamplingParams(), SamplingParams(temperature=1.5, min_p=0.25, repetition_penalty=1.5)]
    host, filters = pack_options(params, [4, 5, 6], [2 ** 40 + 3, 9, 2 ** 63 + 1], [{8, 2}, {1}, {30, 10, 20}])
    rows, f = 3, host.view(np.float32)
    assert f[0:3].tolist() == [0.5, 0.0, 1.5] and host[3:6].tolist() == [7, 0, 0]
    assert f[6:9].tolist() == [1.0, 1.0, 1.0] and f[9:12].tolist() == [0.0, 0.0, 0.25] and f[12:15].tolist() == [1.0, 1.0, 1.5]
    lo, hi = host[15:18].view(np.uint32).astype(np.uint64), host[18:21].view(np.uint32).astype(np.uint64)
    assert ((hi << np.uint64(32)) | lo).tolist() == [2 ** 40 + 3, 9, 2 ** 63 + 1]
    assert host[21:24].tolist() == [4, 5, 6]
    # generated ids travel only for rows with a penalty, sorted, behind their offsets
    assert host[8 * rows:9 * rows + 1].tolist() == [0, 0, 0, 3] and host[9 * rows + 1:].tolist() == [10, 20, 30]
    assert filters == 3                                   # a row with top-k: all three selection passes
    assert pack_options(params[1:], [0, 0], [0, 0], [set(), set()])[1] == 1        # min-p alone: the first pass only
    assert pack_options([SamplingParams(temperature=0.7)], [0], [0], [set()])[1] == 0
    assert pack_options([SamplingParams(temperature=0.0, top_k=5)], [0], [0], [set()])[1] == 0   # greedy rows ask for none
