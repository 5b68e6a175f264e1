"""The model that every architecture becomes: parts built from a plan, run in the plan's order.

`ComposedModel` knows no architecture.  It builds the blocks of the plan from the
part registries, sorts the layer runs into cache groups by what their mixers need
(runs whose mixers need the same heads, head size and window share a group and a
block table), names the per-request state tensors that mixers declare, and runs
    embedding -> runs in order -> final norm at the wanted rows -> head.
"""
from __future__ import annotations

import torch

from ..cache import CacheGroupSpec, StateSpec
from ..parts import BLOCKS, EMBEDDINGS, HEADS, NORMS, CacheRef, KVNeed, ModelPlan, Residual, StateNeed


class ComposedModel:
    def __init__(self, plan: ModelPlan, dtype: torch.dtype):
        self.plan, self.dtype = plan, dtype
        kw = dict(hidden_size=plan.hidden_size, model_dtype=dtype)
        self.embedding = EMBEDDINGS.build(plan.embedding, **kw)
        self.blocks = [BLOCKS.build(b, **kw) for b in plan.blocks]
        self.final_norm = NORMS.build(plan.final_norm, **kw)
        self.head = HEADS.build(plan.head, embedding=self.embedding, **kw)
        self.group_specs, self.state_specs, self.cache_refs = self._assign_caches()
        # captured decode steps replay launches and run a step twice when they are captured (see parts/base.py)
        self.graph_safe = not self.state_specs and all(getattr(p, "graph_safe", False) for p in self.parts() + self.blocks)
        self.loaded = False

    def _assign_caches(self):
        keys, layers, states, refs = [], [], [], []
        for i, run in enumerate(self.plan.runs):
            if run.cache_from is not None:
                src = refs[run.cache_from]
                refs.append(CacheRef(src.group, src.layer, False, src.state_names))
                continue
            need = self.blocks[run.block].cache_need()
            if isinstance(need, KVNeed):
                key = (need.kv_heads, need.head_dim, need.window)
                if key not in keys:
                    keys.append(key)
                    layers.append(0)
                g = keys.index(key)
                refs.append(CacheRef(group=g, layer=layers[g]))
                layers[g] += 1
            elif isinstance(need, StateNeed):
                names = {}
                for name, shape, dt in need.tensors:
                    names[name] = f"run{i}.{name}"
                    states.append(StateSpec(names[name], tuple(shape), dt))
                refs.append(CacheRef(state_names=names))
            elif need is None:
                refs.append(CacheRef())
            else:
                raise TypeError(f"run {i}: cache_need() returned {need!r}; expected KVNeed, StateNeed or None")
        groups = []
        for (kvh, hd, window), n in zip(keys, layers):
            name = ("all" if window is None else f"window{window}") + f"-{kvh}x{hd}"
            groups.append(CacheGroupSpec(name, n, kvh, hd, window))
        return groups, states, refs

    # -- weights -------------------------------------------------------------------
    def parts(self):
        out = [self.embedding]
        for b in self.blocks:
            out.extend(b.parts())
        out.extend([self.final_norm, self.head])
        return out

    def param_specs(self) -> list:
        seen, out = set(), []
        for part in self.parts():
            for ps in part.param_specs():
                if ps.name in seen:
                    continue
                seen.add(ps.name)
                out.append(ps)
        return out

    def load(self, fetch) -> None:
        for part in self.parts():
            part.load(fetch)
        self.loaded = True

    def weight_bytes(self) -> int:
        """Bytes of every weight a step reads once (the tied table counts once)."""
        seen, total = set(), 0
        for part in self.parts():
            for t in vars(part).values():
                if isinstance(t, torch.Tensor) and t.data_ptr() not in seen and t.dim() >= 1 and t.numel() > 1:
                    seen.add(t.data_ptr())
                    total += t.numel() * t.element_size()
        return total

    # -- one step ------------------------------------------------------------------
    def forward(self, ctx) -> torch.Tensor:
        residual = Residual(self.embedding(ctx.token_ids, ctx))
        for run, ref in zip(self.plan.runs, self.cache_refs):
            self.blocks[run.block](residual, ctx, ref)
        if ctx.want_rows.shape[0] == 0:
            return torch.empty((0, self.plan.vocab_size), dtype=torch.float32, device=ctx.token_ids.device)
        hidden = self.final_norm.rows(residual, ctx.want_rows, ctx)
        return self.head(hidden, ctx)
