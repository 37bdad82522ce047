"""A model put together from parts according to a :class:`ModelSpec`.

The reference wires one fixed module tree (engine/model/llama.py:22-68).  Here the tree is
data: parts are built by kind, the run order is a list, and cache needs are collected from
the mixers and sorted into cache groups.
"""

from __future__ import annotations

import math
from typing import Any

from ..cache.manager import PagedGroupSpec, StateGroupSpec
from ..config.spec import ModelSpec
from ..parts.base import BuildEnv, CacheBinding, PagedKVRequest, Part, StateRequest, WeightDecl
from ..parts.registry import build_part


def _walk(part: Part):
    yield part
    for child in part.parts():
        yield from _walk(child)


class Model:
    def __init__(self, spec: ModelSpec, dtype: str, max_positions: int, device=None) -> None:
        spec.validate()
        self.spec = spec
        self.env = BuildEnv(spec.hidden_size, dtype, max_positions, {}, device)
        self.positions = {n: build_part("position", p, self.env) for n, p in spec.positions.items()}
        self.env.positions = self.positions
        self.embedding = build_part("embedding", spec.embedding, self.env)
        self.blocks = [build_part("block", layer.block, self.env, layer=layer) for layer in spec.layers]
        self.final_norm = build_part("norm", spec.final_norm, self.env)
        self.head = build_part("head", spec.head, self.env)
        self.stream_parts = {n: build_part("stream", p, self.env) for n, p in spec.stream_parts.items()}
        # the embedding's output is kept for the step when a stream part reads it again later
        self.keeps_embedding = any(getattr(p, "needs_embedding", False) for p in self.stream_parts.values())
        self._plan_cache()

    # --- parts and weights ------------------------------------------------------------------

    def all_parts(self):
        for p in self.positions.values():
            yield from _walk(p)
        yield from _walk(self.embedding)
        for b in self.blocks:
            yield from _walk(b)
        yield from _walk(self.final_norm)
        yield from _walk(self.head)
        for p in self.stream_parts.values():
            yield from _walk(p)

    @property
    def captures(self) -> bool:
        """Whether every part's step can be captured as a launch sequence."""
        return all(getattr(part, "captures", True) for part in self.all_parts())

    def declared_weights(self) -> dict[str, WeightDecl]:
        out: dict[str, WeightDecl] = {}
        for part in self.all_parts():
            for name, decl in part.weights().items():
                if name in out and out[name] != decl:
                    raise ValueError(f"tensor {name!r} is declared twice with different shapes")
                out[name] = decl
        return out

    def load(self, tensors: dict[str, Any]) -> None:
        """Hand every part its tensors (already on the device)."""
        for part in self.all_parts():
            part.bind({n: tensors[n] for n in part.weights()}, self.env)
        if hasattr(self.head, "tie") and not self.head.weights():
            self.head.tie(self.embedding.table)

    # --- cache ------------------------------------------------------------------------------

    def _plan_cache(self) -> None:
        """Sort the run order's cache needs into groups of equal requests.  A mixer may ask for
        several caches (a tuple of requests: two mixers side by side, a mixer wrapped in another);
        its binding is then a tuple in the same order.  The embedding may ask for a state too."""
        paged: list[tuple[PagedKVRequest, int]] = []  # request, layers so far
        state: list[tuple[StateRequest, int]] = []
        self.bindings: list = []
        requests: list = []

        def assign(req):
            if req is None:
                return None
            if isinstance(req, tuple):
                return tuple(assign(r) for r in req)
            table = paged if isinstance(req, PagedKVRequest) else state
            for gi, (known, count) in enumerate(table):
                if known == req:
                    table[gi] = (known, count + 1)
                    return CacheBinding(gi if table is paged else -1 - gi, count)
            table.append((req, 1))
            gi = len(table) - 1
            return CacheBinding(gi if table is paged else -1 - gi, 0)

        def borrowed(binding):
            if binding is None:
                return None
            if isinstance(binding, tuple):
                return tuple(borrowed(b) for b in binding)
            return CacheBinding(binding.group, binding.slot, writes=False)

        for entry in self.spec.schedule:
            req = self.blocks[entry.layer].mixer.cache_request()
            requests.append(req)
            if entry.cache_from is not None:
                donor = self.bindings[entry.cache_from]
                if donor is None or requests[entry.cache_from] != req:
                    raise ValueError(
                        f"layer {entry.layer} cannot borrow the cache of run-order entry "
                        f"{entry.cache_from}: their cache needs differ")
                self.bindings.append(borrowed(donor))
                continue
            self.bindings.append(assign(req))
        ask = getattr(self.embedding, "cache_request", None)
        self.embedding_binding = assign(ask()) if ask is not None else None
        self.paged_groups = [PagedGroupSpec(n, r.num_kv_heads, r.head_dim, r.window, r.value_dim, r.chunk,
                                            r.keep_first)
                             for r, n in paged]
        self.state_groups = [StateGroupSpec(n, tuple(r.shape)) for r, n in state]
        # Context groups are listed paged first, then state: remap the negative indices.
        n_paged = len(self.paged_groups)

        def remap(b):
            if b is None:
                return None
            if isinstance(b, tuple):
                return tuple(remap(x) for x in b)
            return b if b.group >= 0 else CacheBinding(n_paged + (-1 - b.group), b.slot, b.writes)

        self.bindings = [remap(b) for b in self.bindings]
        self.embedding_binding = remap(self.embedding_binding)

    def footprint(self):
        """Parameters (every declared tensor once) and cache per token and per request, counted
        from the parts themselves: what an architecture's own ``footprint`` callable would say."""
        from ..config.model_config import Footprint

        parameters = sum(math.prod(d.shape) for d in self.declared_weights().values())
        per_token = sum(g.num_layers * g.values_per_token for g in self.paged_groups)
        per_request = sum(g.num_layers * math.prod(g.shape) for g in self.state_groups)
        return Footprint(parameters, per_token, per_request)

    # --- forward ----------------------------------------------------------------------------

    def forward(self, ctx, logit_rows):
        """Run the step's tokens through the run order; return 32-bit logits at
        ``logit_rows`` (indices into the step's flat tokens), or None if there are none."""
        if self.embedding_binding is not None:
            h = self.embedding.forward(ctx.token_ids, ctx, self.embedding_binding)
        else:
            h = self.embedding.forward(ctx.token_ids, ctx)
        for pos in self.positions.values():
            pos.apply_to_embedding(h, ctx)
        x0 = None
        if self.keeps_embedding:
            import torch

            x0 = ctx.ws.buffer("embedding.out", h.shape[0], h.shape[1], torch.float32)
            x0.copy_(h)
        delta, scale = None, 1.0  # the pending delta and the factor it is to be added with
        post = None  # what the block that left the pending delta wants done to it before it is added
        for entry, binding in zip(self.spec.schedule, self.bindings):
            block = self.blocks[entry.layer]
            if entry.before is not None:
                part = self.stream_parts[entry.before]
                # a stream part that only adds something to the stream joins the pending add (and the
                # next norm's kernel) where it can
                folded = None
                if delta is not None and scale == 1.0 and hasattr(part, "fold"):
                    folded = part.fold(post, x0)
                if folded is not None:
                    post = folded
                else:
                    # the stream part sees the whole stream: what is pending is added first
                    if delta is not None:
                        self._settle(h, delta, scale, post, ctx)
                        delta, scale, post = None, 1.0, None
                    part.forward(h, x0, ctx)
            if post is None:
                delta = block.forward(h, delta, ctx, binding, delta_scale=scale)
            else:
                delta = block.forward(h, delta, ctx, binding, delta_scale=scale, delta_post=post)
            scale = block.residual_mult
            post = getattr(block, "output_post", None)
        if logit_rows is None or logit_rows.shape[0] == 0:
            # Nothing is read back, but the last add still belongs to the step.
            return None
        if post is None:
            x = self.final_norm.add_norm(h, delta, ctx, rows=logit_rows, tag="norm.final", delta_scale=scale)
        else:
            x = self.final_norm.add_norm(h, delta, ctx, rows=logit_rows, tag="norm.final", delta_scale=scale,
                                         delta_post=post)
        return self.head.forward(x, ctx)

    def _settle(self, h, delta, scale, post, ctx) -> None:
        """Add what is pending to the residual stream (no normalised output is wanted)."""
        if post is not None:
            post.settle(h, delta, ctx)
        elif scale == 1.0:
            ctx.ops.sandwich_norm(h, delta, None, None, 0.0, None, 0.0, None)
        else:
            h.add_((delta if delta.dim() == 2 else delta.sum(0)) * scale)


def declared_weights(spec: ModelSpec) -> dict[str, WeightDecl]:
    """Names and shapes of every tensor a model of this description reads."""
    return Model(spec, "bfloat16", max_positions=1).declared_weights()
