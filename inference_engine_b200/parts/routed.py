"""A feed-forward made of many small gated experts, of which every token uses a few.

Routing: scores are the softmax over all experts of ``router(x)`` (plus a bias per expert, if the
router has one: ``router_bias``), in 32-bit.  The experts form
``groups`` equal groups of neighbours; a group's score is its best expert's; only experts of the
``keep_groups`` best groups can be chosen (``groups = keep_groups = 1``: no such limit).  The
``top`` allowed experts with the largest scores are taken, and their scores, divided by their sum
(+ 1e-20), weigh the experts' outputs (without groups this is the softmax over the chosen logits).
``scoring="sigmoid"``: a score is the sigmoid of the expert's logit; a ``correction`` per expert (a
tensor, if named) is added to the scores for the choice of groups and experts alone, a group is ranked
by its best ``group_top`` corrected scores added up, and the weights are the chosen experts' plain
scores over their sum.  ``weight_scale`` multiplies the weights.

An expert: ``g = min(gate(x), limit)``, ``u = clamp(up(x), -limit, limit)``,
``y = g * sigmoid(alpha * g) * (u + up_offset)``, output ``down(y)``; no biases.  ``limit``,
``alpha`` and ``up_offset`` are parameters (``limit=None``: nothing is clamped).

The experts' matrices are stacked (``[experts, 2, ff, hidden]`` gates then ups, and
``[experts, hidden, ff]``), a step's (token, expert) pairs are sorted by expert on the device, and
two grouped products run over the sorted list; nothing about the routing is read by the host.  The
result is ``[top, N, hidden]``: slice ``j`` holds the weighted output of every token's ``j``-th
choice, and the next norm adds the slices in order, like the parts of a split matrix product.
"""

from __future__ import annotations

from .base import BuildEnv, FeedForward, WeightDecl
from .registry import register_part


@register_part("feed_forward", "routed_experts")
class RoutedExperts(FeedForward):
    def __init__(self, *, router: str, expert_prefix: str, experts: int, top: int, groups: int,
                 keep_groups: int, hidden_size: int, intermediate_size: int, limit: float | None,
                 alpha: float, up_offset: float, dtype, router_bias: str | None = None, scoring: str = "softmax",
                 correction: str | None = None, group_top: int = 1, weight_scale: float = 1.0) -> None:
        if not 1 <= top <= experts:
            raise ValueError(f"top ({top}) must be between 1 and the number of experts ({experts})")
        if groups < 1 or experts % groups or not 1 <= keep_groups <= groups:
            raise ValueError(f"{experts} experts cannot form {groups} equal groups of which {keep_groups} are kept")
        if top > keep_groups * (experts // groups):
            raise ValueError(f"top ({top}) exceeds the experts of the {keep_groups} kept groups")
        if scoring not in ("softmax", "sigmoid"):
            raise ValueError(f"scores are a 'softmax' or 'sigmoid' of the router's logits, not {scoring!r}")
        if scoring == "softmax" and (correction is not None or group_top != 1):
            raise ValueError("a correction of the choice and groups scored by several experts go with sigmoid scores")
        if group_top not in (1, 2):
            raise ValueError("a group is scored by its best expert or by its best two")
        self.router_name, self.expert_prefix, self.router_bias_name = router, expert_prefix, router_bias
        self.router_bias = None
        self.scoring, self.correction_name, self.correction = scoring, correction, None
        self.group_top, self.weight_scale = int(group_top), float(weight_scale)
        self.experts, self.top, self.groups, self.keep_groups = experts, top, groups, keep_groups
        self.hidden_size, self.intermediate_size = hidden_size, intermediate_size
        self.limit = None if limit is None else float(limit)
        self.alpha, self.up_offset, self.dtype = float(alpha), float(up_offset), dtype
        self.w_router = self.w_gate_up = self.w_down = None

    @classmethod
    def from_spec(cls, params: dict, env: BuildEnv, **_):
        return cls(router=params["router"], expert_prefix=params["expert_prefix"],
                   experts=params["experts"], top=params["top"], groups=params.get("groups", 1),
                   keep_groups=params.get("keep_groups", 1),
                   hidden_size=params.get("hidden_size", env.hidden_size),
                   intermediate_size=params["intermediate_size"], limit=params.get("limit"),
                   alpha=params.get("alpha", 1.702), up_offset=params.get("up_offset", 1.0),
                   dtype=env.torch_dtype, router_bias=params.get("router_bias"),
                   scoring=params.get("scoring", "softmax"), correction=params.get("correction"),
                   group_top=params.get("group_top", 1), weight_scale=params.get("weight_scale", 1.0))

    def _name(self, e: int, which: str) -> str:
        return f"{self.expert_prefix}{e}.{which}"

    def weights(self) -> dict[str, WeightDecl]:
        h, i = self.hidden_size, self.intermediate_size
        out = {self.router_name: WeightDecl((self.experts, h), "vector")}
        if self.router_bias_name is not None:
            out[self.router_bias_name] = WeightDecl((self.experts,), "vector")
        if self.correction_name is not None:
            # (drawn as zeros in the random-weights mode: a random correction, the same for every token,
            # would send all tokens to the same few experts)
            out[self.correction_name] = WeightDecl((self.experts,), "vector", "zeros")
        for e in range(self.experts):
            out[self._name(e, "gate")] = WeightDecl((i, h))
            out[self._name(e, "up")] = WeightDecl((i, h))
            out[self._name(e, "down")] = WeightDecl((h, i))
        return out

    def bind(self, tensors, env: BuildEnv) -> None:
        import torch

        self.w_router = tensors[self.router_name].float().contiguous()  # routing is 32-bit
        if self.router_bias_name is not None:
            self.router_bias = tensors[self.router_bias_name].float().contiguous()
        if self.correction_name is not None:
            self.correction = tensors[self.correction_name].float().contiguous()
        self.w_gate_up = torch.stack([
            torch.stack([tensors[self._name(e, "gate")].to(self.dtype), tensors[self._name(e, "up")].to(self.dtype)])
            for e in range(self.experts)]).contiguous()
        self.w_down = torch.stack([tensors[self._name(e, "down")].to(self.dtype)
                                   for e in range(self.experts)]).contiguous()

    def forward(self, x, ctx):
        import torch

        n = x.shape[0]
        ids = ctx.ws.buffer("moe.ids", n, self.top, torch.int32)
        weights = ctx.ws.buffer("moe.weights", n, self.top, torch.float32)
        if self.scoring != "softmax" or self.weight_scale != 1.0:
            ctx.ops.route_topk(x, self.w_router, self.groups, self.keep_groups, ids, weights, bias=self.router_bias,
                               scoring=self.scoring, correction=self.correction, group_top=self.group_top,
                               weight_scale=self.weight_scale)
        elif self.router_bias is None:
            ctx.ops.route_topk(x, self.w_router, self.groups, self.keep_groups, ids, weights)
        else:
            ctx.ops.route_topk(x, self.w_router, self.groups, self.keep_groups, ids, weights, bias=self.router_bias)
        return ctx.ops.routed_experts(x, ids, weights, self.w_gate_up, self.w_down,
                                      limit=self.limit, alpha=self.alpha, up_offset=self.up_offset,
                                      ws=ctx.ws, tag="moe")
