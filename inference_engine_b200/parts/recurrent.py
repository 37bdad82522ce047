"""Recurrent mixers whose state is a matrix per head that decays and takes an outer product per
token, and a wrapper that passes a mixer's input through a short convolution first.

``conv_input``: the wrapped mixer reads ``h + conv(h)`` instead of ``h``, ``conv`` a causal
convolution over time on each channel (``taps`` taps, the last one weighs the token itself, zeros
before the request's start).  The last ``taps - 1`` inputs are kept per request in a state slot.

``hgrn2``: linear attention whose forget gate also decides what is written.  ``q = silu(W_q h)``,
``v = W_v h``, ``f = lower + (1 - lower) * sigmoid(W_f h + b_f)`` per head and channel;
``S <- diag(f) S + (1 - f) v^T``, ``o = S^T q``; each head's ``o`` is divided by its root mean
square over ``vdim`` and multiplied by a weight of size ``vdim`` that the heads share; ``W_o``.

``mlstm``: a matrix memory with exponential gates.  ``q = W_q h * dim^-1/2``, ``k = W_k h``,
``v = W_v h``; per head ``logi = cap * tanh((W_i h + b_i) / cap)`` and ``logf = logsigmoid(cap *
tanh((W_f h + b_f) / cap))``; with a running maximum ``m`` that starts at 0: ``m' = max(logf + m,
logi)``, ``S <- exp(logf + m - m') S + exp(logi - m') k v^T``, the normaliser ``n`` likewise with
``k`` alone, ``o = S^T q / (max(|n . q|, exp(-m')) + 1e-6)``; each head's ``o`` is divided by its root
mean square, the heads together are multiplied by a weight and by ``sigmoid(W_g h)``; ``W_o``.

``gla``: gated linear attention with a decay per key channel.  ``q = W_q h * dim^-1/2``, ``k = W_k h``,
``v = W_v h``; ``a = sigmoid(W_a2 (W_a1 h) + b)^(1 / tau)`` per head and channel, from a low-rank map of
the input; ``S <- diag(a) S + k v^T``, ``o = S^T q``; each head's ``o`` is divided by its root mean
square over ``vdim`` and multiplied by a weight of size ``vdim`` that the heads share; the heads
together are multiplied by ``silu(W_g h)``; ``W_o``.  Its input product can carry more rows of another
map of the same input (``accepts_input_rows``).

Gates, decays, the state and the read-out are 32-bit in every precision; the projections run in
the compute dtype with 32-bit sums.  The state lives in the request's state slot: ``S`` column by
column (``[heads, columns, dim]``; the normaliser is one more column), then the maxima.
"""

from __future__ import annotations

from ..config.spec import PartSpec
from .base import BuildEnv, Mixer, StateRequest, WeightDecl
from .registry import build_part, register_part


def _part_spec(raw) -> PartSpec:
    return raw if isinstance(raw, PartSpec) else PartSpec(raw["kind"], dict(raw.get("params", {})))


@register_part("mixer", "conv_input")
class ConvInput(Mixer):
    def __init__(self, weight: str, channels: int, taps: int, inner: Mixer, dtype) -> None:
        if taps < 1:
            raise ValueError("the convolution needs at least one tap")
        self.weight_name, self.channels, self.taps, self.inner, self.dtype = weight, channels, taps, inner, dtype
        self.weight = None

    @classmethod
    def from_spec(cls, params: dict, env: BuildEnv, **_):
        return cls(params["weight"], params.get("channels", env.hidden_size), int(params["taps"]),
                   build_part("mixer", _part_spec(params["inner"]), env), env.torch_dtype)

    @property
    def captures(self) -> bool:
        return getattr(self.inner, "captures", True)

    def parts(self):
        return [self.inner]

    def weights(self) -> dict[str, WeightDecl]:
        return {self.weight_name: WeightDecl((self.channels, self.taps), "vector")}

    def bind(self, tensors, env: BuildEnv) -> None:
        self.weight = tensors[self.weight_name].float().contiguous()

    def cache_request(self):
        return (StateRequest((max((self.taps - 1) * self.channels, 1),)), self.inner.cache_request())

    def forward(self, x, ctx, binding):
        own, inner = binding
        group = ctx.groups[own.group]
        y = ctx.ws.buffer("conv_input.out", x.shape[0], self.channels, self.dtype)
        ctx.ops.short_conv_residual(x, self.weight, group.state[own.slot], group.slots, ctx, y)
        return self.inner.forward(y, ctx, inner)


@register_part("mixer", "hgrn2")
class HGRN2(Mixer):
    allow_split = True  # whether the output projection may come back as partial sums

    def __init__(self, *, names: dict, hidden_size: int, heads: int, dim: int, vdim: int, eps: float, dtype) -> None:
        self.names, self.hidden_size = dict(names), hidden_size
        self.heads, self.dim, self.vdim, self.eps, self.dtype = heads, dim, vdim, float(eps), dtype
        self.qk_size, self.v_size = heads * dim, heads * vdim
        self.w_in = None

    @classmethod
    def from_spec(cls, params: dict, env: BuildEnv, **_):
        return cls(names=params["names"], hidden_size=params.get("hidden_size", env.hidden_size),
                   heads=params["heads"], dim=params["dim"], vdim=params["vdim"], eps=params["eps"],
                   dtype=env.torch_dtype)

    def weights(self) -> dict[str, WeightDecl]:
        n, h = self.names, self.hidden_size
        return {
            n["q"]: WeightDecl((self.qk_size, h)), n["f"]: WeightDecl((self.qk_size, h)),
            n["f_bias"]: WeightDecl((self.qk_size,), "vector"),
            n["lower"]: WeightDecl((self.qk_size,), "vector", "zeros"),
            n["v"]: WeightDecl((self.v_size, h)),
            n["out_norm"]: WeightDecl((self.vdim,), "vector", "ones_plus_normal"),
            n["o"]: WeightDecl((h, self.v_size)),
        }

    def bind(self, tensors, env: BuildEnv) -> None:
        import torch

        n = self.names
        self.w_in = torch.cat([tensors[n[k]].to(self.dtype) for k in ("q", "f", "v")]).contiguous()
        self.w_o = tensors[n["o"]].to(self.dtype).contiguous()
        self.f_bias = tensors[n["f_bias"]].float().contiguous()
        self.lower = tensors[n["lower"]].float().contiguous()
        self.out_norm = tensors[n["out_norm"]].float().contiguous()

    def cache_request(self) -> StateRequest:
        return StateRequest((self.heads * self.vdim * self.dim,))

    def forward(self, x, ctx, binding):
        import torch

        f32, n, qk = torch.float32, x.shape[0], self.qk_size
        group = ctx.groups[binding.group]
        ops, ws = ctx.ops, ctx.ws
        proj = ops.linear(x, self.w_in, ws=ws, tag="hgrn2.in", out_dtype=f32)
        write = ws.buffer("hgrn2.write", n, qk, f32)
        ops.hgrn2_gates(proj, self.f_bias, self.lower, write, qk)
        o = ws.buffer("hgrn2.o", n, self.v_size, f32)
        ops.gated_recurrence(proj[:, :qk], proj[:, qk: 2 * qk], write, None, proj[:, 2 * qk:],
                             group.state[binding.slot], group.slots, ctx, o, self.heads, self.dim, self.vdim,
                             self.vdim, 1.0)
        out = ws.buffer("hgrn2.out", n, self.v_size, self.dtype)
        ops.recurrence_readout(o, None, self.out_norm, self.eps, None, out, self.heads, self.vdim, self.vdim)
        return ops.linear(out, self.w_o, ws=ws, tag="hgrn2.delta", out_dtype=f32, allow_split=self.allow_split)


@register_part("mixer", "mlstm")
class MLSTM(Mixer):
    allow_split = True

    def __init__(self, *, names: dict, hidden_size: int, heads: int, dim: int, vdim: int, gate_cap: float,
                 eps: float, dtype) -> None:
        self.names, self.hidden_size = dict(names), hidden_size
        self.heads, self.dim, self.vdim, self.dtype = heads, dim, vdim, dtype
        self.gate_cap, self.eps = float(gate_cap), float(eps)
        self.qk_size, self.v_size = heads * dim, heads * vdim
        self.matrix_floats = heads * (vdim + 1) * dim  # S and, as one more column, the normaliser
        self.w_in = None

    @classmethod
    def from_spec(cls, params: dict, env: BuildEnv, **_):
        return cls(names=params["names"], hidden_size=params.get("hidden_size", env.hidden_size),
                   heads=params["heads"], dim=params["dim"], vdim=params["vdim"], gate_cap=params["gate_cap"],
                   eps=params["eps"], dtype=env.torch_dtype)

    def weights(self) -> dict[str, WeightDecl]:
        n, h = self.names, self.hidden_size
        return {
            n["q"]: WeightDecl((self.qk_size, h)), n["k"]: WeightDecl((self.qk_size, h)),
            n["v"]: WeightDecl((self.v_size, h)), n["g"]: WeightDecl((self.v_size, h)),
            n["i"]: WeightDecl((self.heads, h)), n["i_bias"]: WeightDecl((self.heads,), "vector"),
            n["f"]: WeightDecl((self.heads, h)), n["f_bias"]: WeightDecl((self.heads,), "vector"),
            n["out_norm"]: WeightDecl((self.v_size,), "vector", "ones_plus_normal"),
            n["o"]: WeightDecl((h, self.v_size)),
        }

    def bind(self, tensors, env: BuildEnv) -> None:
        import torch

        n = self.names
        self.w_in = torch.cat([tensors[n[k]].to(self.dtype) for k in ("q", "k", "v", "g", "i", "f")]).contiguous()
        self.w_o = tensors[n["o"]].to(self.dtype).contiguous()
        self.i_bias = tensors[n["i_bias"]].float().contiguous()
        self.f_bias = tensors[n["f_bias"]].float().contiguous()
        self.out_norm = tensors[n["out_norm"]].float().contiguous()

    def cache_request(self) -> StateRequest:
        return StateRequest((self.matrix_floats + self.heads,))

    def forward(self, x, ctx, binding):
        import torch

        f32, n, qk, vs, H = torch.float32, x.shape[0], self.qk_size, self.v_size, self.heads
        group = ctx.groups[binding.group]
        state = group.state[binding.slot]
        ops, ws = ctx.ops, ctx.ws
        proj = ops.linear(x, self.w_in, ws=ws, tag="mlstm.in", out_dtype=f32)
        at_g, at_i = 2 * qk + vs, 2 * qk + 2 * vs
        gates = ws.buffer("mlstm.gates", n, 3 * H, f32)
        ops.mlstm_gates(proj[:, at_i: at_i + H], proj[:, at_i + H: at_i + 2 * H], self.i_bias, self.f_bias,
                        self.gate_cap, state, self.matrix_floats, group.slots, ctx, gates, H)
        cols = self.vdim + 1
        o = ws.buffer("mlstm.o", n, H * cols, f32)
        ops.gated_recurrence(proj[:, :qk], None, proj[:, qk: 2 * qk], gates, proj[:, 2 * qk: at_g], state,
                             group.slots, ctx, o, H, self.dim, self.vdim, cols, self.dim ** -0.5)
        out = ws.buffer("mlstm.out", n, vs, self.dtype)
        ops.recurrence_readout(o, gates, self.out_norm, self.eps, proj[:, at_g: at_i], out, H, self.vdim, cols)
        return ops.linear(out, self.w_o, ws=ws, tag="mlstm.delta", out_dtype=f32, allow_split=self.allow_split)


@register_part("mixer", "gla")
class GatedLinearAttention(Mixer):
    allow_split = True
    accepts_input_rows = True

    def __init__(self, *, names: dict, hidden_size: int, heads: int, dim: int, vdim: int, rank: int, tau: float,
                 eps: float, dtype) -> None:
        if rank < 1 or not tau > 0:
            raise ValueError("the decay's low-rank map needs a rank of at least 1 and a positive tau")
        self.names, self.hidden_size = dict(names), hidden_size
        self.heads, self.dim, self.vdim, self.rank = heads, dim, vdim, int(rank)
        self.tau, self.eps, self.dtype = float(tau), float(eps), dtype
        self.qk_size, self.v_size = heads * dim, heads * vdim
        self.w_in = None

    @classmethod
    def from_spec(cls, params: dict, env: BuildEnv, **_):
        return cls(names=params["names"], hidden_size=params.get("hidden_size", env.hidden_size),
                   heads=params["heads"], dim=params["dim"], vdim=params["vdim"], rank=params["rank"],
                   tau=params["tau"], eps=params["eps"], dtype=env.torch_dtype)

    def weights(self) -> dict[str, WeightDecl]:
        n, h = self.names, self.hidden_size
        return {
            n["q"]: WeightDecl((self.qk_size, h)), n["k"]: WeightDecl((self.qk_size, h)),
            n["v"]: WeightDecl((self.v_size, h)), n["g"]: WeightDecl((self.v_size, h)),
            n["a1"]: WeightDecl((self.rank, h)), n["a2"]: WeightDecl((self.qk_size, self.rank)),
            n["a2_bias"]: WeightDecl((self.qk_size,), "vector"),
            n["out_norm"]: WeightDecl((self.vdim,), "vector", "ones_plus_normal"),
            n["o"]: WeightDecl((h, self.v_size)),
        }

    def bind(self, tensors, env: BuildEnv) -> None:
        import torch

        n = self.names
        self.w_in, self.extra_at = self._with_extra_rows(
            [tensors[n[k]].to(self.dtype) for k in ("q", "k", "v", "g", "a1")])
        self.w_o = tensors[n["o"]].to(self.dtype).contiguous()
        self.w_a2 = tensors[n["a2"]].float().contiguous()  # the decay's second map stays 32-bit
        self.a2_bias = tensors[n["a2_bias"]].float().contiguous()
        self.out_norm = tensors[n["out_norm"]].float().contiguous()

    def cache_request(self) -> StateRequest:
        return StateRequest((self.heads * self.vdim * self.dim,))

    def forward(self, x, ctx, binding):
        import torch

        f32, n, qk, vs = torch.float32, x.shape[0], self.qk_size, self.v_size
        group = ctx.groups[binding.group]
        ops, ws = ctx.ops, ctx.ws
        proj = ops.linear(x, self.w_in, ws=ws, tag="gla.in", out_dtype=f32)
        self.extra_out = self._extra_columns(proj, self.extra_at)
        at_g, at_a = 2 * qk + vs, 2 * qk + 2 * vs
        decay = ws.buffer("gla.decay", n, qk, f32)
        ops.lowrank_decay(proj[:, at_a: at_a + self.rank], self.w_a2, self.a2_bias, self.tau, decay)
        o = ws.buffer("gla.o", n, vs, f32)
        ops.gated_recurrence(proj[:, :qk], decay, proj[:, qk: 2 * qk], None, proj[:, 2 * qk: at_g],
                             group.state[binding.slot], group.slots, ctx, o, self.heads, self.dim, self.vdim,
                             self.vdim, self.dim ** -0.5)
        out = ws.buffer("gla.out", n, vs, self.dtype)
        ops.recurrence_readout(o, None, self.out_norm, self.eps, proj[:, at_g: at_a], out, self.heads, self.vdim,
                               self.vdim, gate_act="silu")
        return ops.linear(out, self.w_o, ws=ws, tag="gla.delta", out_dtype=f32, allow_split=self.allow_split)
