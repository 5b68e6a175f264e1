"""The framework takes parts and architectures it has never seen, without a change to its
files: a toy mixer with per-request state of its own (a decaying sum of its inputs), a
rotary encoding over half of each head, a windowed attention layer (a second cache group
whose pages are given back as the window passes them), a run order that names one block
twice and lets one run read another run's cache.  All of it is defined and registered
here, written to a model folder by the random-weights mode, loaded, and stepped under
every way of cutting; the logits are compared with a plain whole-sequence statement of
the same toy model, and in 32-bit with each other bit for bit.  The toy is no model of
anyone's; it exists to exercise the seams."""
from dataclasses import asdict, dataclass

import pytest
import torch

import plain_gemma as plain
import traces
from helpers import folder_weights, max_diff
from wllm_b200.config import register_architecture
from wllm_b200.config.base import ConfigReader
from wllm_b200.kernels import ops
from wllm_b200.parts import MIXERS, LayerRun, ModelPlan, ParamSpec, StateNeed, spec

pytestmark = pytest.mark.gpu


@MIXERS.register("toy_decay")
class ToyDecayMixer:
    """state <- decay * state + x (per request, 32-bit, carried from step to step);  y = state @ W^T."""

    def __init__(self, spec, hidden_size, model_dtype):
        self.decay, self.weight_name = float(spec.decay), spec.weight
        self.hidden_size, self.model_dtype = hidden_size, model_dtype
        self.weight = None

    def cache_need(self):
        return StateNeed((("sum", (self.hidden_size,), torch.float32),))

    def param_specs(self):
        return [ParamSpec(self.weight_name, (self.hidden_size, self.hidden_size))]

    def load(self, fetch):
        self.weight = fetch(self.weight_name).contiguous()

    def __call__(self, x, ctx, cache):
        state = ctx.state(cache.state_names["sum"])
        sums = torch.empty(x.shape, dtype=torch.float32, device=x.device)
        starts, lens, slots = ctx.host["req_q_start"], ctx.host["req_q_len"], ctx.host["req_slot"]
        for start, n, slot in zip(starts.tolist(), lens.tolist(), slots.tolist()):
            s = state[slot]
            for t in range(start, start + n):
                s = self.decay * s + x[t].float()
                sums[t] = s
            state[slot] = s
        return ops.linear(sums.to(self.model_dtype), self.weight)


@dataclass(frozen=True)
class ToyConfig:
    vocab_size: int
    hidden_size: int
    intermediate_size: int
    num_heads: int
    num_kv_heads: int
    head_dim: int
    window: int
    decay: float
    eps: float
    theta: float
    max_positions: int
    architecture = "ToyDecayForCausalLM"

    @classmethod
    def from_dict(cls, raw, where="config.json"):
        r = ConfigReader(raw, where)
        cfg = cls(*(r.integer(k) for k in ("vocab_size", "hidden_size", "intermediate_size", "num_heads", "num_kv_heads",
                                           "head_dim", "window")),
                  r.number("decay"), r.number("eps"), r.number("theta"), r.integer("max_positions"))
        r.finish()
        return cfg

    def to_dict(self):
        return dict(asdict(self), architectures=[self.architecture])


def _norm(name, c):
    return spec("rmsnorm", weight=name, eps=c.eps, unit_offset=False)


def _ffn(p, c):
    return spec("gated_dense", intermediate_size=c.intermediate_size, activation="silu", gate_proj=p + "gate.weight",
                up_proj=p + "up.weight", down_proj=p + "down.weight")


def _attention(p, c, window):
    return spec("attention", num_heads=c.num_heads, num_kv_heads=c.num_kv_heads, head_dim=c.head_dim, window=window,
                position=spec("rope", theta=c.theta, head_dim=c.head_dim, rotary_dim=c.head_dim // 2),
                q_proj=p + "q.weight", k_proj=p + "k.weight", v_proj=p + "v.weight", o_proj=p + "o.weight")


@register_architecture("ToyDecayForCausalLM", ToyConfig)
def toy_plan(c):
    def block(i, mixer):
        p = f"blocks.{i}."
        return spec("pre_norm", norm_in=_norm(p + "norm_in.weight", c), mixer=mixer,
                    norm_post=_norm(p + "norm_post.weight", c), feed_forward=_ffn(p + "ffn.", c))
    blocks = [block(0, spec("toy_decay", decay=c.decay, weight="blocks.0.mix.weight")),
              block(1, _attention("blocks.1.attn.", c, None)),
              block(2, _attention("blocks.2.attn.", c, c.window)),
              block(3, _attention("blocks.3.attn.", c, None))]
    # block 0 runs twice (each run has its own state); run 4 reads the keys and values that run 1 wrote
    runs = [LayerRun(0), LayerRun(1), LayerRun(2), LayerRun(0), LayerRun(3, cache_from=1)]
    return ModelPlan(hidden_size=c.hidden_size, vocab_size=c.vocab_size, max_positions=c.max_positions,
                     embedding=spec("scaled_embedding", weight="embed.weight", vocab_size=c.vocab_size, scale=1.0),
                     blocks=blocks, final_norm=_norm("final_norm.weight", c),
                     head=spec("logits_head", tied=False, weight="head.weight", vocab_size=c.vocab_size), runs=runs)


TOY = dict(architectures=["ToyDecayForCausalLM"], vocab_size=300, hidden_size=48, intermediate_size=80, num_heads=4,
           num_kv_heads=2, head_dim=32, window=20, decay=0.8, eps=1e-5, theta=100.0, max_positions=512)


# -- the same toy model, plainly: whole sequences, no cache -------------------------------------
def _plain_norm(x, w, eps):
    return x * torch.rsqrt(x.pow(2).mean(-1, keepdim=True) + eps) * w


def _plain_rope_half(x, positions, theta):
    rot = x.shape[-1] // 2
    cos, sin = plain.rope_tables(positions, rot, theta)
    return torch.cat([plain.apply_rope(x[..., :rot], cos, sin), x[..., rot:]], dim=-1)


def _plain_attention(h, w, p, c, window, kv=None):
    T = h.shape[0]
    pos = torch.arange(T)
    q = _plain_rope_half((h @ w[p + "q.weight"].T).view(T, c.num_heads, c.head_dim), pos, c.theta)
    if kv is None:
        k = _plain_rope_half((h @ w[p + "k.weight"].T).view(T, c.num_kv_heads, c.head_dim), pos, c.theta)
        v = (h @ w[p + "v.weight"].T).view(T, c.num_kv_heads, c.head_dim)
        kv = (k, v)
    o = plain.attention(q, kv[0], kv[1], window=window).reshape(T, -1)
    return o @ w[p + "o.weight"].T, kv


def plain_toy(ids, w, c):
    x = w["embed.weight"][torch.as_tensor(ids)]
    kv_of_run = {}
    for run, (b, src) in enumerate([(0, None), (1, None), (2, None), (0, None), (3, 1)]):
        p = f"blocks.{b}."
        h = _plain_norm(x, w[p + "norm_in.weight"], c.eps)
        if b == 0:
            s, sums = torch.zeros(c.hidden_size), []
            for t in range(h.shape[0]):
                s = c.decay * s + h[t]
                sums.append(s)
            y = torch.stack(sums) @ w[p + "mix.weight"].T
        else:
            y, kv = _plain_attention(h, w, p + "attn.", c, c.window if b == 2 else None, kv_of_run.get(src))
            kv_of_run[run] = kv
        x = x + y
        h = _plain_norm(x, w[p + "norm_post.weight"], c.eps)
        x = x + (torch.nn.functional.silu(h @ w[p + "ffn.gate.weight"].T) * (h @ w[p + "ffn.up.weight"].T)) @ w[p + "ffn.down.weight"].T
    return _plain_norm(x, w["final_norm.weight"], c.eps) @ w["head.weight"].T


@pytest.fixture(scope="module")
def toy(tmp_path_factory):
    from wllm_b200.weights import write_random_model
    folder = write_random_model(str(tmp_path_factory.mktemp("toy") / "m"), TOY, seed=4, std=0.08, vector_std=0.3)
    c = ToyConfig.from_dict(TOY)
    w = folder_weights(folder)
    g = torch.Generator().manual_seed(6)
    reqs = {f"r{i}": torch.randint(0, c.vocab_size, (n,), generator=g).tolist() for i, n in enumerate((5, 64, 31, 90, 2, 47, 70, 25, 88, 60, 33))}
    ref = {(rid, p): row for rid, toks in reqs.items() for p, row in enumerate(plain_toy(toks, w, c))}
    return folder, reqs, ref


def test_the_model_is_built_from_the_registered_parts(toy):
    from wllm_b200.config import config_from_folder
    from wllm_b200.engine import ComposedModel
    arch, cfg = config_from_folder(toy[0])
    model = ComposedModel(arch.make_plan(cfg), torch.float32)
    assert isinstance(model.blocks[0].mixer, ToyDecayMixer)
    assert [(g.name, g.layers, g.window) for g in model.group_specs] == [("all-2x32", 1, None), ("window20-2x32", 1, 20)]
    assert [s.name for s in model.state_specs] == ["run0.sum", "run3.sum"]         # one state per run of the block
    refs = model.cache_refs
    assert (refs[4].group, refs[4].layer, refs[4].writes) == (refs[1].group, refs[1].layer, False)
    assert "blocks.0.mix.weight" in {p.name for p in model.param_specs()}
    assert len([p for p in model.param_specs() if p.name.startswith("blocks.0.")]) == 6   # shared weights listed once


@pytest.mark.parametrize("dtype,tol", [(torch.float32, 5e-5), (torch.bfloat16, 6e-2)])
def test_every_cut_of_the_toy_model_matches_its_plain_statement(toy, dtype, tol):
    from test_gpu_replay import gpu_runner
    folder, reqs, ref = toy
    first = None
    for name, make in (("whole", traces.whole), ("tail", lambda r: traces.tail_singly(r, 16)),
                       ("portions", traces.portions), ("mixed", lambda r: traces.mixed(r, seed=5))):
        steps = make(reqs)
        pages = -(-traces.peak_tokens(steps) // 16)
        runner = gpu_runner(folder, dtype, 16, pages)
        rows = traces.run_in_process(runner, steps)
        assert max_diff(rows, ref) < tol, name
        assert runner.cache.free_pages() == [pages, pages] and runner.cache.slots.num_free == 8
        if name == "mixed":
            assert all(g.pool.takes > pages for g in runner.cache.groups)
        if dtype == torch.float32:
            if first is None:
                first = rows
            else:
                bad = sorted(k for k in first if not torch.equal(first[k], rows[k]))
                assert not bad, f"{name}: first differing (request, position) {bad[0]}"


def test_a_model_with_state_of_its_own_is_never_replayed_from_a_captured_graph(toy):
    """A captured decode step runs twice when it is captured and replays the launches its parts chose from host
    data at that moment; a mixer that carries state from step to step would count a token twice and keep
    writing to the slots of the capture.  So the runner steps such a model eagerly whatever was asked for, and
    the tail decoded token by token still matches the plain statement."""
    from test_gpu_replay import gpu_runner
    folder, reqs, ref = toy
    steps = traces.tail_singly(reqs, 16)
    runner = gpu_runner(folder, torch.float32, 16, -(-traces.peak_tokens(steps) // 16))
    assert not runner.model.graph_safe
    runner.enable_graphs()
    rows = traces.run_in_process(runner, steps)
    assert runner.graph_launches == 0 and not runner._graphs
    assert max_diff(rows, ref) < 5e-5


def test_the_window_group_holds_fewer_pages_than_the_full_one(toy):
    from test_gpu_replay import gpu_runner
    folder, reqs, _ = toy
    runner = gpu_runner(folder, torch.float32, 16, 16)
    rc = runner.cache.open("long")
    from wllm_b200.engine import StepEntry
    toks = reqs["r3"]
    for i in range(0, len(toks), 10):
        runner.step([StepEntry(rc, toks[i:i + 10], [])])
    full, win = rc.tables
    assert sum(p >= 0 for p in full) == 6 and sum(p >= 0 for p in win) <= 3 and win[0] == -1
