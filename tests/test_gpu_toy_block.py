"""A norm and an arrangement of a block that the framework has never seen, defined and registered here: a layer norm
with mean subtraction and a bias, and a block whose mixer and feed-forward both read ONE norm of the stream and are
added to it together (x = x + mixer(n(x)) + feed_forward(n(x))).  With them every one of the seven registries has
been extended from a test: embedding, head, position, mixer, feed-forward (the other toy tests), norm and block
(this one).  The toy model is written to a folder by the random-weights mode, loaded, stepped under every way of
cutting, with captured graphs for its decode steps, and compared with a plain whole-sequence statement of itself;
in 32-bit the cuts agree bit for bit.  It is no model of anyone's."""
from dataclasses import asdict, dataclass

import pytest
import torch

import plain_gemma as plain
import traces
from helpers import folder_weights, max_diff
from wllm_b200.config import register_architecture
from wllm_b200.config.base import ConfigReader
from wllm_b200.parts import BLOCKS, FEED_FORWARDS, MIXERS, NORMS, ModelPlan, ParamSpec, Partials, spec

pytestmark = pytest.mark.gpu


def _whole(branch) -> torch.Tensor:
    """A branch output as one float32 tensor (a step of few rows leaves a product in partial sums)."""
    if isinstance(branch, Partials):
        return branch.tensor.sum(0)
    return branch.float()


@NORMS.register("toy_layernorm")
class ToyLayerNorm:
    """(x - mean) / sqrt(var + eps) * w + b over the 32-bit stream; the pending branch is folded in first.  Plain
    tensor operations."""
    graph_safe = True

    def __init__(self, spec, hidden_size, model_dtype):
        self.names, self.eps = (spec.weight, spec.bias), float(spec.eps)
        self.hidden_size, self.model_dtype = hidden_size, model_dtype
        self.weight = self.bias = None

    def param_specs(self):
        return [ParamSpec(self.names[0], (self.hidden_size,), "vector"), ParamSpec(self.names[1], (self.hidden_size,), "vector")]

    def load(self, fetch):
        self.weight, self.bias = fetch(self.names[0]).float(), fetch(self.names[1]).float()

    def _norm(self, x):
        # statistics in 64-bit: whatever order a library reduction takes for a given number of rows, the result
        # rounded to 32 bits is the same, so the cuts stay bit-equal
        xd = x.double()
        centred = xd - xd.mean(-1, keepdim=True)
        inv = torch.rsqrt((centred * centred).mean(-1, keepdim=True) + self.eps)
        return (centred * inv).float() * self.weight + self.bias

    def __call__(self, residual, ctx):
        if residual.pending is not None:
            residual.stream += _whole(residual.pending)
            residual.pending = None
        return self._norm(residual.stream).to(self.model_dtype)

    def rows(self, residual, rows, ctx):
        x = residual.stream[rows.long()]
        if residual.pending is not None:
            x = x + _whole(residual.pending)[rows.long()]
        return self._norm(x).to(self.model_dtype)


@BLOCKS.register("toy_parallel")
class ToyParallelBlock:
    """x = x + mixer(n(x)) + feed_forward(n(x)): one norm, both branches from it, one sum left pending."""
    graph_safe = True

    def __init__(self, spec, hidden_size, model_dtype):
        kw = dict(hidden_size=hidden_size, model_dtype=model_dtype)
        self.norm = NORMS.build(spec.norm, **kw)
        self.mixer = MIXERS.build(spec.mixer, **kw)
        self.feed_forward = FEED_FORWARDS.build(spec.feed_forward, **kw)

    def parts(self):
        return [self.norm, self.mixer, self.feed_forward]

    def cache_need(self):
        return self.mixer.cache_need()

    def __call__(self, residual, ctx, cache):
        h = self.norm(residual, ctx)
        # both branches are whole before they are added: a buffer of the step's arena may serve both products
        mixed = _whole(self.mixer(h, ctx, cache)).clone()
        residual.pending = mixed + _whole(self.feed_forward(h, ctx))


@dataclass(frozen=True)
class ToyParallelConfig:
    vocab_size: int
    hidden_size: int
    intermediate_size: int
    num_layers: int
    num_heads: int
    num_kv_heads: int
    head_dim: int
    eps: float
    theta: float
    max_positions: int
    architecture = "ToyParallelForCausalLM"

    @classmethod
    def from_dict(cls, raw, where="config.json"):
        r = ConfigReader(raw, where)
        cfg = cls(*(r.integer(k) for k in ("vocab_size", "hidden_size", "intermediate_size", "num_layers", "num_heads",
                                           "num_kv_heads", "head_dim")),
                  r.number("eps"), r.number("theta"), r.integer("max_positions"))
        r.finish()
        return cfg

    def to_dict(self):
        return dict(asdict(self), architectures=[self.architecture])


def _ln(p, c):
    return spec("toy_layernorm", weight=p + "weight", bias=p + "bias", eps=c.eps)


@register_architecture("ToyParallelForCausalLM", ToyParallelConfig)
def toy_plan(c):
    def block(i):
        p = f"layers.{i}."
        return spec("toy_parallel", norm=_ln(p + "ln.", c),
                    mixer=spec("attention", num_heads=c.num_heads, num_kv_heads=c.num_kv_heads, head_dim=c.head_dim, window=None,
                               position=spec("rope", theta=c.theta, head_dim=c.head_dim, rotary_dim=c.head_dim),
                               q_proj=p + "q.weight", k_proj=p + "k.weight", v_proj=p + "v.weight", o_proj=p + "o.weight"),
                    feed_forward=spec("gated_dense", intermediate_size=c.intermediate_size, activation="gelu_tanh",
                                      gate_proj=p + "gate.weight", up_proj=p + "up.weight", down_proj=p + "down.weight"))
    return ModelPlan(hidden_size=c.hidden_size, vocab_size=c.vocab_size, max_positions=c.max_positions,
                     embedding=spec("scaled_embedding", weight="embed.weight", vocab_size=c.vocab_size, scale=1.0),
                     blocks=[block(i) for i in range(c.num_layers)], final_norm=_ln("final_ln.", c),
                     head=spec("logits_head", tied=True, weight="embed.weight", vocab_size=c.vocab_size))


TOY = dict(architectures=["ToyParallelForCausalLM"], vocab_size=211, hidden_size=72, intermediate_size=104, num_layers=3,
           num_heads=6, num_kv_heads=3, head_dim=16, eps=1e-5, theta=500.0, max_positions=256)


# -- the same toy model, plainly: whole sequences, no cache -------------------------------------
def _plain_ln(x, w, b, eps):
    centred = x - x.mean(-1, keepdim=True)
    return centred * torch.rsqrt((centred * centred).mean(-1, keepdim=True) + eps) * w + b


def plain_toy(ids, w, c):
    x = w["embed.weight"][torch.as_tensor(ids)]
    T = x.shape[0]
    cos, sin = plain.rope_tables(torch.arange(T), c.head_dim, c.theta)
    for i in range(c.num_layers):
        p = f"layers.{i}."
        h = _plain_ln(x, w[p + "ln.weight"], w[p + "ln.bias"], c.eps)
        q = plain.apply_rope((h @ w[p + "q.weight"].T).view(T, c.num_heads, c.head_dim), cos, sin)
        k = plain.apply_rope((h @ w[p + "k.weight"].T).view(T, c.num_kv_heads, c.head_dim), cos, sin)
        v = (h @ w[p + "v.weight"].T).view(T, c.num_kv_heads, c.head_dim)
        attn = plain.attention(q, k, v).reshape(T, -1) @ w[p + "o.weight"].T
        gate = torch.nn.functional.gelu(h @ w[p + "gate.weight"].T, approximate="tanh")
        x = x + attn + (gate * (h @ w[p + "up.weight"].T)) @ w[p + "down.weight"].T
    return _plain_ln(x, w["final_ln.weight"], w["final_ln.bias"], c.eps) @ w["embed.weight"].T


@pytest.fixture(scope="module")
def toy(tmp_path_factory):
    from wllm_b200.weights import write_random_model
    folder = write_random_model(str(tmp_path_factory.mktemp("toy_parallel") / "m"), TOY, seed=8, std=0.08, vector_std=0.3)
    c = ToyParallelConfig.from_dict(TOY)
    w = folder_weights(folder)
    g = torch.Generator().manual_seed(9)
    reqs = {f"r{i}": torch.randint(0, c.vocab_size, (n,), generator=g).tolist() for i, n in enumerate((3, 70, 29, 64, 2, 51, 17))}
    ref = {(rid, p): row for rid, toks in reqs.items() for p, row in enumerate(plain_toy(toks, w, c))}
    return folder, reqs, ref


def test_the_model_is_built_from_the_registered_norm_and_block(toy):
    from wllm_b200.config import config_from_folder
    from wllm_b200.engine import ComposedModel
    arch, cfg = config_from_folder(toy[0])
    model = ComposedModel(arch.make_plan(cfg), torch.float32)
    assert all(isinstance(b, ToyParallelBlock) and isinstance(b.norm, ToyLayerNorm) for b in model.blocks)
    assert isinstance(model.final_norm, ToyLayerNorm) and model.graph_safe
    names = {p.name for p in model.param_specs()}
    assert {"layers.0.ln.bias", "layers.2.down.weight", "final_ln.bias", "embed.weight"} <= names and "head.weight" not in names


@pytest.mark.parametrize("dtype,tol", [(torch.float32, 5e-5), (torch.bfloat16, 6e-2)])
def test_every_cut_of_the_toy_model_matches_its_plain_statement(toy, dtype, tol):
    from test_gpu_replay import gpu_runner
    folder, reqs, ref = toy
    first = None
    for name, make in (("whole", traces.whole), ("tail", lambda r: traces.tail_singly(r, 16)),
                       ("portions", traces.portions), ("mixed", lambda r: traces.mixed(r, seed=3))):
        steps = make(reqs)
        pages = -(-traces.peak_tokens(steps) // 16)
        runner = gpu_runner(folder, dtype, 16, pages)
        if name == "tail":
            runner.enable_graphs()             # the decoded tail replays captured steps: every part says it may
        rows = traces.run_in_process(runner, steps)
        assert max_diff(rows, ref) < tol, name
        assert runner.cache.free_pages() == [pages]
        if name == "tail":
            assert runner.graph_launches > 0
        if dtype == torch.float32:
            if first is None:
                first = rows
            else:
                bad = sorted(k for k in first if not torch.equal(first[k], rows[k]))
                assert not bad, f"{name}: first differing (request, position) {bad[0]}"
