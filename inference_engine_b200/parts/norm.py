"""Root-mean-square norm over the last dimension, with the residual add fused in.

Formula (engine/model/layers.py:41-43): ``normed = x * rsqrt(mean(x^2) + eps)`` in 32-bit,
then ``weight * normed``.  The residual stream is kept in 32-bit here, so square, mean,
rsqrt and both products are 32-bit and the result is rounded once to the compute dtype.
"""

from __future__ import annotations

from .base import BuildEnv, Norm, WeightDecl
from .registry import register_part


@register_part("norm", "rms")
class RMSNorm(Norm):
    """``offset``: what is added to the stored weight (1 for weights stored around zero, so that the
    factor is ``1 + w``; 0 for weights stored around one)."""

    def __init__(self, weight: str, size: int, eps: float, dtype, offset: float = 0.0) -> None:
        self.weight_name, self.size, self.eps, self.dtype = weight, int(size), float(eps), dtype
        self.offset = float(offset)
        self.weight = None

    @classmethod
    def from_spec(cls, params: dict, env: BuildEnv, **_):
        return cls(params["weight"], params.get("size", env.hidden_size), params["eps"],
                   env.torch_dtype, params.get("offset", 0.0))

    def weights(self) -> dict[str, WeightDecl]:
        init = "normal" if self.offset else "ones_plus_normal"
        return {self.weight_name: WeightDecl((self.size,), "vector", init)}

    def bind(self, tensors, env: BuildEnv) -> None:
        self.weight = (tensors[self.weight_name].float() + self.offset).contiguous()

    def add_norm(self, h, delta, ctx, rows=None, tag: str = "norm", delta_scale: float = 1.0,
                 delta_post: "PostNorm | None" = None):
        n = h.shape[0] if rows is None else rows.shape[0]
        out = ctx.ws.buffer(tag, n, self.size, self.dtype)
        if delta_post is not None:
            # something is done to the delta before it is added (it is normalised and takes its bias,
            # or passes a learned gate): one kernel for that, the add and this norm
            if delta_scale != 1.0:
                raise ValueError("a delta that is treated before the add has no residual multiplier")
            delta_post.add_norm(h, delta, ctx, self.weight, self.eps, out, rows)
        elif delta_scale == 1.0:
            ctx.ops.rmsnorm(h, delta, self.weight, self.eps, out, rows)
        else:
            ctx.ops.rmsnorm(h, delta, self.weight, self.eps, out, rows, delta_scale=float(delta_scale))
        return out


class PostNorm:
    """What a block wants done to a sublayer's output before it enters the residual stream: a bias
    (or None), then an RMS norm.  Carried beside the pending delta to whoever adds it."""

    def __init__(self, norm: RMSNorm, bias=None) -> None:
        self.norm, self.bias = norm, bias

    def add_norm(self, h, delta, ctx, weight, eps, out, rows) -> None:
        """``h += norm(delta + bias)`` (not with ``rows``); ``out = rms(h) * weight``."""
        ctx.ops.sandwich_norm(h, delta, self.bias, self.norm.weight, self.norm.eps, weight, eps, out, rows)

    def settle(self, h, delta, ctx) -> None:
        """``h += norm(delta + bias)`` with no normalised output."""
        ctx.ops.sandwich_norm(h, delta, self.bias, self.norm.weight, self.norm.eps, None, 0.0, None)


class AddedTerms:
    """What enters the residual stream together with a pending delta, in the same add: the output of
    a second sublayer that read the same input (``second``: whole, or in parts like a delta), a bias
    row of the sublayer that left the delta (``bias``), and a second stream of the rows' shape
    (``rows_like_stream``: the embedding's output that a looped model adds again before a pass).
    ``h += delta + second + bias + rows_like_stream`` and the next norm are one kernel."""

    def __init__(self, bias=None, second=None, rows_like_stream=None) -> None:
        self.bias, self.second, self.rows_like_stream = bias, second, rows_like_stream

    def with_stream_rows(self, x0) -> "AddedTerms":
        if self.rows_like_stream is not None:
            raise ValueError("one second stream per add")
        return AddedTerms(self.bias, self.second, x0)

    def add_norm(self, h, delta, ctx, weight, eps, out, rows) -> None:
        ctx.ops.sandwich_norm(h, delta, self.bias, None, 0.0, weight, eps, out, rows, second=self.second,
                              extra=self.rows_like_stream)

    def settle(self, h, delta, ctx) -> None:
        ctx.ops.sandwich_norm(h, delta, self.bias, None, 0.0, None, 0.0, None, second=self.second,
                              extra=self.rows_like_stream)


class ResidualGate:
    """A sublayer's output enters the residual stream through a gate: ``h += sigmoid(gate_pre + bias) *
    delta`` element by element.  ``gate_pre`` is the 32-bit pre-activation ``[N, hidden]`` of this
    step; carried beside the pending delta to whoever adds it, like :class:`PostNorm`."""

    def __init__(self, gate_pre, bias=None) -> None:
        self.gate_pre, self.bias = gate_pre, bias

    def add_norm(self, h, delta, ctx, weight, eps, out, rows) -> None:
        ctx.ops.gated_add_norm(h, delta, self.gate_pre, self.bias, weight, eps, out, rows)

    def settle(self, h, delta, ctx) -> None:
        ctx.ops.gated_add_norm(h, delta, self.gate_pre, self.bias, None, 0.0, None)


@register_part("norm", "layer")
class LayerNorm(Norm):
    """Layer norm over the last dimension with a weight and no bias, the residual add fused in:
    ``(x - mean(x)) / sqrt(mean((x - mean(x))^2) + eps) * weight``, all in 32-bit on the 32-bit
    residual stream; the result is rounded once to the compute dtype."""

    def __init__(self, weight: str, size: int, eps: float, dtype) -> None:
        self.weight_name, self.size, self.eps, self.dtype = weight, int(size), float(eps), dtype
        self.weight = None

    @classmethod
    def from_spec(cls, params: dict, env: BuildEnv, **_):
        return cls(params["weight"], params.get("size", env.hidden_size), params["eps"],
                   env.torch_dtype)

    def weights(self) -> dict[str, WeightDecl]:
        return {self.weight_name: WeightDecl((self.size,), "vector", "ones_plus_normal")}

    def bind(self, tensors, env: BuildEnv) -> None:
        self.weight = tensors[self.weight_name].float().contiguous()

    def add_norm(self, h, delta, ctx, rows=None, tag: str = "norm", delta_scale: float = 1.0):
        n = h.shape[0] if rows is None else rows.shape[0]
        out = ctx.ws.buffer(tag, n, self.size, self.dtype)
        ctx.ops.layernorm(h, delta, self.weight, self.eps, out, rows, delta_scale=float(delta_scale))
        return out
