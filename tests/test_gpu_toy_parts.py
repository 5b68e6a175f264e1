"""More kinds of part that the framework has never seen, registered from here: a feed-forward
with routing (each token goes through the one expert its router picks, router logits in 32-bit),
another position encoding (rotary with positions divided by a factor and neighbouring elements
turning together, which the attention mixer takes through the same interface as the built-in
one), an embedding that adds a learned vector per absolute position, and a head that caps its
logits with a tanh.  A toy architecture made of them,
with the two kinds of feed-forward alternating by layer, is written to a folder by the
random-weights mode, loaded and stepped under every way of cutting; the logits are compared with
a plain whole-sequence statement of the same toy, and in 32-bit with each other bit for bit.
The toy is no model of anyone's; it exists to exercise the seams."""
from dataclasses import asdict, dataclass

import pytest
import torch

import plain_gemma as plain
import traces
from helpers import folder_weights, max_diff
from wllm_b200.config import register_architecture
from wllm_b200.config.base import ConfigReader
from wllm_b200.kernels import ops
from wllm_b200.parts import EMBEDDINGS, FEED_FORWARDS, HEADS, POSITIONS, LayerRun, ModelPlan, ParamSpec, spec

pytestmark = pytest.mark.gpu


@POSITIONS.register("rope_stretched")
class StretchedRotary:
    """Rotary angles of position / factor, elements 2j and 2j + 1 turning together: the mixer reads `inv_freq`,
    `rotary_dim` and `pairing`, nothing else."""
    pairing = "interleaved"

    def __init__(self, spec, device=None):
        self.rotary_dim = int(spec.head_dim)
        exponent = torch.arange(0, self.rotary_dim, 2, dtype=torch.float32) / self.rotary_dim
        self.inv_freq = (1.0 / (float(spec.theta) ** exponent) / float(spec.factor)).to(torch.float32)

    def to(self, device):
        self.inv_freq = self.inv_freq.to(device)
        return self


@EMBEDDINGS.register("toy_positioned_embedding")
class PositionedEmbedding:
    """x[t] = E[id[t]] + P[position[t]]: a learned vector per absolute position, beside the token's."""

    def __init__(self, spec, hidden_size, model_dtype):
        self.names, self.vocab, self.places = (spec.weight, spec.position_weight), int(spec.vocab_size), int(spec.max_positions)
        self.hidden_size, self.table, self.places_table = hidden_size, None, None

    def param_specs(self):
        return [ParamSpec(self.names[0], (self.vocab, self.hidden_size), "table"),
                ParamSpec(self.names[1], (self.places, self.hidden_size), "table")]

    def load(self, fetch):
        self.table, self.places_table = fetch(self.names[0]).contiguous(), fetch(self.names[1]).contiguous()

    def __call__(self, token_ids, ctx):
        out = ctx.buffer("residual", (token_ids.shape[0], self.hidden_size), torch.float32)
        ops.embed_gather(token_ids, self.table, 1.0, out)
        return out.add_(self.places_table[ctx.positions.long()].float())


@HEADS.register("toy_capped_head")
class CappedHead:
    """logits = cap * tanh(h E^T / cap), with the embedding's table."""

    def __init__(self, spec, hidden_size, model_dtype, embedding):
        self.cap, self.embedding = float(spec.cap), embedding

    def param_specs(self):
        return []

    def load(self, fetch):
        pass

    def __call__(self, hidden_rows, ctx):
        return self.cap * torch.tanh(ops.linear(hidden_rows, self.embedding.table, f32_out=True) / self.cap)


@FEED_FORWARDS.register("toy_routed")
class ToyRoutedFeedForward:
    """y[t] = weight(t) * down_e(relu(up_e(x[t]))) with e = arg-max of the router's 32-bit logits and
    weight = sigmoid of that logit.  Tokens are grouped by expert on the host; it is a toy."""

    def __init__(self, spec, hidden_size, model_dtype):
        self.experts, self.inter, self.prefix = int(spec.experts), int(spec.intermediate_size), spec.prefix
        self.hidden_size, self.model_dtype = hidden_size, model_dtype
        self.router = self.up = self.down = None

    def param_specs(self):
        H, I, p = self.hidden_size, self.inter, self.prefix
        out = [ParamSpec(p + "router.weight", (self.experts, H), "vector")]       # kept in 32-bit
        for e in range(self.experts):
            out += [ParamSpec(f"{p}experts.{e}.up.weight", (I, H)), ParamSpec(f"{p}experts.{e}.down.weight", (H, I))]
        return out

    def load(self, fetch):
        p = self.prefix
        self.router = fetch(p + "router.weight").float().contiguous()
        self.up = [fetch(f"{p}experts.{e}.up.weight").contiguous() for e in range(self.experts)]
        self.down = [fetch(f"{p}experts.{e}.down.weight").contiguous() for e in range(self.experts)]

    def __call__(self, x, ctx):
        logits = ops.linear(x.float(), self.router)                       # 32-bit router
        top, chosen = logits.max(dim=-1)
        out = torch.zeros(x.shape, dtype=torch.float32, device=x.device)
        for e in range(self.experts):
            rows = (chosen == e).nonzero().flatten()
            if rows.numel():
                h = torch.relu(ops.linear(x[rows].contiguous(), self.up[e]))
                out[rows] = ops.linear(h, self.down[e]).float() * torch.sigmoid(top[rows]).unsqueeze(-1)
        return out.to(self.model_dtype)


@dataclass(frozen=True)
class ToyRoutedConfig:
    vocab_size: int
    hidden_size: int
    intermediate_size: int
    num_layers: int
    num_heads: int
    num_kv_heads: int
    head_dim: int
    experts: int
    eps: float
    theta: float
    stretch: float
    cap: float
    max_positions: int
    architecture = "ToyRoutedForCausalLM"

    @classmethod
    def from_dict(cls, raw, where="config.json"):
        r = ConfigReader(raw, where)
        cfg = cls(*(r.integer(k) for k in ("vocab_size", "hidden_size", "intermediate_size", "num_layers", "num_heads",
                                           "num_kv_heads", "head_dim", "experts")),
                  r.number("eps"), r.number("theta"), r.number("stretch"), r.number("cap"), r.integer("max_positions"))
        r.finish()
        return cfg

    def to_dict(self):
        return dict(asdict(self), architectures=[self.architecture])


@register_architecture("ToyRoutedForCausalLM", ToyRoutedConfig)
def toy_routed_plan(c):
    def norm(name):
        return spec("rmsnorm", weight=name, eps=c.eps, unit_offset=True)

    def block(i):
        p = f"layers.{i}."
        attention = spec("attention", num_heads=c.num_heads, num_kv_heads=c.num_kv_heads, head_dim=c.head_dim, window=None,
                         position=spec("rope_stretched", theta=c.theta, head_dim=c.head_dim, factor=c.stretch),
                         q_proj=p + "q.weight", k_proj=p + "k.weight", v_proj=p + "v.weight", o_proj=p + "o.weight")
        if i % 2 == 0:      # the kind of feed-forward is chosen layer by layer
            ffn = spec("toy_routed", experts=c.experts, intermediate_size=c.intermediate_size, prefix=p + "moe.")
        else:
            ffn = spec("gated_dense", intermediate_size=c.intermediate_size, activation="gelu_tanh",
                       gate_proj=p + "gate.weight", up_proj=p + "up.weight", down_proj=p + "down.weight")
        return spec("pre_norm", norm_in=norm(p + "norm_in.weight"), mixer=attention, norm_post=norm(p + "norm_post.weight"),
                    feed_forward=ffn)
    return ModelPlan(hidden_size=c.hidden_size, vocab_size=c.vocab_size, max_positions=c.max_positions,
                     embedding=spec("toy_positioned_embedding", weight="embed.weight", position_weight="places.weight",
                                    vocab_size=c.vocab_size, max_positions=c.max_positions),
                     blocks=[block(i) for i in range(c.num_layers)], final_norm=norm("final_norm.weight"),
                     head=spec("toy_capped_head", cap=c.cap),
                     runs=[LayerRun(i) for i in range(c.num_layers)])


TOY = dict(architectures=["ToyRoutedForCausalLM"], vocab_size=200, hidden_size=64, intermediate_size=96, num_layers=3,
           num_heads=4, num_kv_heads=4, head_dim=16, experts=3, eps=1e-6, theta=50.0, stretch=4.0, cap=2.0, max_positions=256)


# -- the same toy, plainly: whole sequences, no cache -------------------------------------------
def plain_toy(ids, w, c):
    def norm(x, name):
        return x * torch.rsqrt(x.pow(2).mean(-1, keepdim=True) + c.eps) * (1.0 + w[name])
    def turn(x):        # elements 2j and 2j + 1 of every head turn together
        y = torch.empty_like(x)
        x1, x2 = x[..., 0::2], x[..., 1::2]
        y[..., 0::2] = x1 * cos[:, None, :] - x2 * sin[:, None, :]
        y[..., 1::2] = x2 * cos[:, None, :] + x1 * sin[:, None, :]
        return y
    T = len(ids)
    x = w["embed.weight"][torch.as_tensor(ids)] + w["places.weight"][:T]
    margin = torch.full((T,), float("inf"))          # the closest call any router makes on each token
    cos, sin = (t[:, :c.head_dim // 2] for t in plain.rope_tables(torch.arange(T).float() / c.stretch, c.head_dim, c.theta))
    for i in range(c.num_layers):
        p = f"layers.{i}."
        h = norm(x, p + "norm_in.weight")
        q = turn((h @ w[p + "q.weight"].T).view(T, c.num_heads, c.head_dim))
        k = turn((h @ w[p + "k.weight"].T).view(T, c.num_kv_heads, c.head_dim))
        v = (h @ w[p + "v.weight"].T).view(T, c.num_kv_heads, c.head_dim)
        x = x + plain.attention(q, k, v).reshape(T, -1) @ w[p + "o.weight"].T
        h = norm(x, p + "norm_post.weight")
        if i % 2 == 0:
            logits = h @ w[p + "moe.router.weight"].T
            top, chosen = logits.max(-1)
            two = logits.topk(2, dim=-1).values
            margin = torch.minimum(margin, two[:, 0] - two[:, 1])
            y = torch.zeros_like(h)
            for t in range(T):
                e = int(chosen[t])
                y[t] = torch.relu(h[t] @ w[f"{p}moe.experts.{e}.up.weight"].T) @ w[f"{p}moe.experts.{e}.down.weight"].T
            x = x + y * torch.sigmoid(top).unsqueeze(-1)
        else:
            gate = torch.nn.functional.gelu(h @ w[p + "gate.weight"].T, approximate="tanh")
            x = x + (gate * (h @ w[p + "up.weight"].T)) @ w[p + "down.weight"].T
    return c.cap * torch.tanh(norm(x, "final_norm.weight") @ w["embed.weight"].T / c.cap), margin


@pytest.fixture(scope="module")
def toy(tmp_path_factory):
    from wllm_b200.weights import write_random_model
    folder = write_random_model(str(tmp_path_factory.mktemp("toy_routed") / "m"), TOY, seed=9, std=0.1, vector_std=0.3)
    c = ToyRoutedConfig.from_dict(TOY)
    w = folder_weights(folder)
    g = torch.Generator().manual_seed(2)
    reqs = {f"r{i}": torch.randint(0, c.vocab_size, (n,), generator=g).tolist() for i, n in enumerate((40, 3, 77, 18, 64, 9))}
    ref, clear = {}, {}
    for rid, toks in reqs.items():
        logits, margin = plain_toy(toks, w, c)
        ref.update({(rid, p): row for p, row in enumerate(logits)})
        unclear = (margin < 0.05).nonzero().flatten()
        clear[rid] = int(unclear[0]) if unclear.numel() else len(toks)     # positions before the first close call
    return folder, reqs, ref, w, c, clear


def test_parts_are_chosen_layer_by_layer(toy):
    from wllm_b200.config import config_from_folder
    from wllm_b200.engine import ComposedModel
    from wllm_b200.parts.feed_forward import GatedDense
    arch, cfg = config_from_folder(toy[0])
    model = ComposedModel(arch.make_plan(cfg), torch.float32)
    kinds = [type(b.feed_forward) for b in model.blocks]
    assert kinds == [ToyRoutedFeedForward, GatedDense, ToyRoutedFeedForward]
    assert all(isinstance(b.mixer.position, StretchedRotary) for b in model.blocks)
    assert isinstance(model.embedding, PositionedEmbedding) and isinstance(model.head, CappedHead)
    assert not model.graph_safe          # parts that do not say they may be captured keep the model eager
    names = {p.name for p in model.param_specs()}
    assert "layers.0.moe.experts.2.down.weight" in names and "layers.1.gate.weight" in names


def test_the_router_spreads_the_tokens(toy):
    _, reqs, _, w, c, _ = toy
    x = w["embed.weight"][torch.as_tensor(reqs["r2"])] + w["places.weight"][:len(reqs["r2"])]
    h = x * torch.rsqrt(x.pow(2).mean(-1, keepdim=True) + c.eps) * (1.0 + w["layers.0.norm_in.weight"])
    chosen = (h @ w["layers.0.moe.router.weight"].T).argmax(-1)
    assert len(set(chosen.tolist())) == c.experts        # the toy's weights do send tokens to every expert


@pytest.mark.parametrize("dtype,tol", [(torch.float32, 5e-5), (torch.bfloat16, 6e-2)])
def test_every_cut_of_the_routed_toy_matches_its_plain_statement(toy, dtype, tol):
    from test_gpu_replay import gpu_runner
    folder, reqs, ref, _, _, clear = toy
    # Under bfloat16 a token whose two best router logits nearly tie may go to the other expert, and
    # everything behind it in its request then differs by more than rounding.  That is a property of
    # routing, not of a cut: bfloat16 is compared on each request's positions before its first close call
    # (the plain router's margin below 0.05); 32-bit is compared everywhere.
    if dtype == torch.bfloat16:
        ref = {k: v for k, v in ref.items() if k[1] < clear[k[0]]}
        assert len(ref) >= 60
    first = None
    for name, make in (("whole", traces.whole), ("tail", lambda r: traces.tail_singly(r, 8)),
                       ("portions", traces.portions), ("mixed", lambda r: traces.mixed(r, seed=3))):
        steps = make(reqs)
        pages = -(-traces.peak_tokens(steps) // 16)
        runner = gpu_runner(folder, dtype, 16, pages)
        rows = traces.run_in_process(runner, steps)
        assert max_diff({k: v for k, v in rows.items() if k in ref}, ref) < tol, name
        if dtype == torch.float32:
            if first is None:
                first = rows
            else:
                bad = sorted(k for k in first if not torch.equal(first[k], rows[k]))
                assert not bad, f"{name}: first differing (request, position) {bad[0]}"
        assert runner.cache.free_pages() == [pages]
