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
