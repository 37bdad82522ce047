"""Dense gated feed-forward: ``down(silu(gate(x)) * up(x))`` (engine/model/layers.py:277-281),
``silu(g) = g / (1 + exp(-g))`` evaluated in 32-bit.  Gate and up run as one matrix product
over the stacked weights.  Their rows alternate in blocks of 16 (16 gate rows, the 16 up rows
with the same indices, the next 16 gate rows, ...) when the width allows: every dot product is
unchanged, and a kernel that owns a tile of rows then holds each gate beside its up and can
apply the activation itself (``ops.gated_linear``).

With biases (``gate_bias``, ``up_bias``, ``down_bias``: tensor names) gate and up are stacked in
halves, their product comes back in the compute dtype and biases (added in 32-bit) and activation are one kernel; the down
projection's bias is not added here: the block's norm after the feed-forward takes it
(``output_bias``), so only a block with such a norm can hold a feed-forward with a down bias."""

from __future__ import annotations

from .base import BuildEnv, FeedForward, WeightDecl
from .registry import register_part


@register_part("feed_forward", "swiglu")
class SwiGLU(FeedForward):
    def __init__(self, *, gate_proj: str, up_proj: str, down_proj: str, hidden_size: int,
                 intermediate_size: int, dtype, gate_bias: str | None = None, up_bias: str | None = None,
                 down_bias: str | None = None) -> None:
        self.names = {"gate": gate_proj, "up": up_proj, "down": down_proj}
        self.bias_names = {"gate": gate_bias, "up": up_bias, "down": down_bias}
        if (gate_bias is None) != (up_bias is None):
            raise ValueError("gate and up have biases together or not at all")
        self.hidden_size, self.intermediate_size, self.dtype = hidden_size, intermediate_size, dtype
        self.w_gate_up = self.w_down = None
        self.bias_gate_up = self.output_bias = None
        self.interleave = 0

    ROW_BLOCK = 16  # gate and up rows alternate in blocks of this many

    @classmethod
    def from_spec(cls, params: dict, env: BuildEnv, **_):
        return cls(gate_proj=params["gate_proj"], up_proj=params["up_proj"],
                   down_proj=params["down_proj"],
                   hidden_size=params.get("hidden_size", env.hidden_size),
                   intermediate_size=params["intermediate_size"], dtype=env.torch_dtype,
                   gate_bias=params.get("gate_bias"), up_bias=params.get("up_bias"),
                   down_bias=params.get("down_bias"))

    def weights(self) -> dict[str, WeightDecl]:
        h, i = self.hidden_size, self.intermediate_size
        out = {
            self.names["gate"]: WeightDecl((i, h)),
            self.names["up"]: WeightDecl((i, h)),
            self.names["down"]: WeightDecl((h, i)),
        }
        for key, size in (("gate", i), ("up", i), ("down", h)):
            if self.bias_names[key] is not None:
                out[self.bias_names[key]] = WeightDecl((size,), "vector")
        return out

    def bind(self, tensors, env: BuildEnv) -> None:
        import torch

        gate, up = tensors[self.names["gate"]].to(self.dtype), tensors[self.names["up"]].to(self.dtype)
        i, h, b = self.intermediate_size, self.hidden_size, self.ROW_BLOCK
        if self.bias_names["down"] is not None:
            self.output_bias = tensors[self.bias_names["down"]].float().contiguous()
        if self.bias_names["gate"] is not None:
            self.bias_gate_up = torch.cat([tensors[self.bias_names["gate"]].float(),
                                           tensors[self.bias_names["up"]].float()]).contiguous()
        if self.bias_gate_up is not None:
            self.interleave = 0
            self.w_gate_up = torch.cat([gate, up]).contiguous()
        elif i % b == 0:
            self.interleave = b
            self.w_gate_up = torch.stack([gate.view(i // b, b, h), up.view(i // b, b, h)], dim=1).reshape(2 * i, h).contiguous()
        else:
            self.interleave = 0
            self.w_gate_up = torch.cat([gate, up]).contiguous()
        self.w_down = tensors[self.names["down"]].to(self.dtype).contiguous()

    def forward(self, x, ctx):
        import torch

        if self.bias_gate_up is not None:
            gate_up = ctx.ops.linear(x, self.w_gate_up, ws=ctx.ws, tag="ffn.gate_up", out_dtype=self.dtype)
            act = ctx.ws.buffer("ffn.act", x.shape[0], self.intermediate_size, self.dtype)
            ctx.ops.silu_mul_bias(gate_up, self.bias_gate_up, act)
        else:
            act = ctx.ops.gated_linear(x, self.w_gate_up, self.interleave, ws=ctx.ws, tag="ffn", out_dtype=self.dtype)
        return ctx.ops.linear(act, self.w_down, ws=ctx.ws, tag="ffn.delta", out_dtype=torch.float32,
                              allow_split=True)


@register_part("feed_forward", "relu2")
class SquaredReluFF(FeedForward):
    """Dense feed-forward without a gate: ``down(relu(up(x))^2)``.  The activation is evaluated in
    32-bit on the product's output and rounded once to the compute dtype."""

    def __init__(self, *, up_proj: str, down_proj: str, hidden_size: int, intermediate_size: int, dtype) -> None:
        self.names = {"up": up_proj, "down": down_proj}
        self.hidden_size, self.intermediate_size, self.dtype = hidden_size, intermediate_size, dtype
        self.w_up = self.w_down = None

    @classmethod
    def from_spec(cls, params: dict, env: BuildEnv, **_):
        return cls(up_proj=params["up_proj"], down_proj=params["down_proj"],
                   hidden_size=params.get("hidden_size", env.hidden_size),
                   intermediate_size=params["intermediate_size"], dtype=env.torch_dtype)

    def weights(self) -> dict[str, WeightDecl]:
        h, i = self.hidden_size, self.intermediate_size
        return {self.names["up"]: WeightDecl((i, h)), self.names["down"]: WeightDecl((h, i))}

    def bind(self, tensors, env: BuildEnv) -> None:
        self.w_up = tensors[self.names["up"]].to(self.dtype).contiguous()
        self.w_down = tensors[self.names["down"]].to(self.dtype).contiguous()

    def forward(self, x, ctx):
        import torch

        up = ctx.ops.linear(x, self.w_up, ws=ctx.ws, tag="ffn.up", out_dtype=self.dtype)
        act = ctx.ws.buffer("ffn.act", x.shape[0], self.intermediate_size, self.dtype)
        ctx.ops.relu_squared(up, act)
        return ctx.ops.linear(act, self.w_down, ws=ctx.ws, tag="ffn.delta", out_dtype=torch.float32,
                              allow_split=True)


@register_part("feed_forward", "polynorm")
class PolyNormFF(FeedForward):
    """Dense feed-forward without a gate: ``down(act(up(x)))`` with ``act(z) = a N(z) + b N(z^2) +
    c N(z^3) + e``: powers element by element, ``N`` divides a token's vector by its root mean square
    (eps inside the root), and ``(a, b, c, e)`` is a tensor of four numbers.  The first product's
    sums stay 32-bit for the activation, which rounds once to the compute dtype.  The first product
    can carry more rows (``accepts_input_rows``)."""

    accepts_input_rows = True

    def __init__(self, *, up_proj: str, down_proj: str, coeff: str, hidden_size: int, intermediate_size: int,
                 eps: float, dtype) -> None:
        self.names = {"up": up_proj, "down": down_proj, "coeff": coeff}
        self.hidden_size, self.intermediate_size, self.eps, self.dtype = hidden_size, intermediate_size, float(eps), dtype
        self.w_up = self.w_down = self.coeff = None

    @classmethod
    def from_spec(cls, params: dict, env: BuildEnv, **_):
        return cls(up_proj=params["up_proj"], down_proj=params["down_proj"], coeff=params["coeff"],
                   hidden_size=params.get("hidden_size", env.hidden_size),
                   intermediate_size=params["intermediate_size"], eps=params["eps"], dtype=env.torch_dtype)

    def weights(self) -> dict[str, WeightDecl]:
        h, i = self.hidden_size, self.intermediate_size
        return {self.names["up"]: WeightDecl((i, h)), self.names["down"]: WeightDecl((h, i)),
                self.names["coeff"]: WeightDecl((4,), "vector", "ones_plus_normal")}

    def bind(self, tensors, env: BuildEnv) -> None:
        self.w_up, self.extra_at = self._with_extra_rows([tensors[self.names["up"]].to(self.dtype)])
        self.w_down = tensors[self.names["down"]].to(self.dtype).contiguous()
        self.coeff = tensors[self.names["coeff"]].float().contiguous()

    def forward(self, x, ctx):
        import torch

        up = ctx.ops.linear(x, self.w_up, ws=ctx.ws, tag="ffn.up32", out_dtype=torch.float32)
        self.extra_out = self._extra_columns(up, self.extra_at)
        act = ctx.ws.buffer("ffn.act", x.shape[0], self.intermediate_size, self.dtype)
        ctx.ops.polynorm(up[:, : self.intermediate_size], self.coeff, self.eps, act)
        return ctx.ops.linear(act, self.w_down, ws=ctx.ws, tag="ffn.delta", out_dtype=torch.float32,
                              allow_split=True)
