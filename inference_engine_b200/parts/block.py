"""Arrangements of a layer's parts.

``prenorm_residual`` (engine/model/layers.py:301-303): ``h = x + m * mixer(norm(x))``, then
``out = h + m * feed_forward(norm(h))``; ``m`` is the parameter ``residual_mult`` (1 unless the
model description says otherwise), and a layer without a feed-forward stops after its mixer.  The residual stream ``h`` is 32-bit and is updated in
place; each add is fused into the norm that follows it, so a block returns its
feed-forward's output as a pending ``delta`` for the next norm to add.

``sandwich_residual``: a norm before and after each sublayer, ``x <- x + post(mixer(pre(x)))`` and
``x <- x + post'(feed_forward(pre'(x)))``.  The norm after a sublayer, the add and the norm before the
next sublayer are one kernel: the block hands its last sublayer's raw output on as the pending delta
together with what is to be done to it before the add (``output_post``: an output bias, if the
sublayer has one, and the norm).

``gated_prenorm_residual``: the pre-norm arrangement with a learned gate on each sublayer's way into
the stream: ``x <- x + sigmoid(W1 h + b1) * mixer(h)`` with ``h = norm(x)``, then the same with
``W2``, ``b2`` and the feed-forward.  The gate reads what the sublayer reads.  Its product runs in
the compute dtype with 32-bit sums; sigmoid, multiplication and add are 32-bit and sit in the
kernel of the next norm (the pending delta travels with its gate: ``output_post``).  A mixer or
feed-forward that starts with one product over its input carries its gate's rows in that product.

``parallel_residual``: one norm, and both sublayers read its output: ``x <- x + mixer(h) +
feed_forward(h)`` with ``h = norm(x)``.  The two outputs stay apart (each whole or in the parts of a
split product) and are added, with the mixer's output bias if it has one, in the kernel of the
next norm: the mixer's output is the pending delta, the rest travels beside it (``output_post``).
"""

from __future__ import annotations

import os

from .base import Block, BuildEnv, CacheBinding, WeightDecl
from .norm import AddedTerms, PostNorm, ResidualGate
from .registry import build_part, register_part


def _adds_no_output_bias(mixer) -> None:
    """An arrangement that adds the mixer's output as it is cannot take a mixer that leaves its
    output bias to the add."""
    if getattr(mixer, "names", None) and mixer.names.get("o_bias"):
        raise ValueError("this arrangement of a layer does not add a mixer's output bias")


@register_part("block", "prenorm_residual")
class PreNormResidualBlock(Block):
    def __init__(self, mixer, feed_forward, pre_mixer, pre_feed_forward, residual_mult: float = 1.0) -> None:
        _adds_no_output_bias(mixer)
        self.mixer, self.feed_forward = mixer, feed_forward
        self.pre_mixer, self.pre_feed_forward = pre_mixer, pre_feed_forward
        self.residual_mult = float(residual_mult)

    @classmethod
    def from_spec(cls, params: dict, env: BuildEnv, *, layer, **_):
        has_ff = layer.feed_forward is not None
        return cls(
            build_part("mixer", layer.mixer, env),
            build_part("feed_forward", layer.feed_forward, env) if has_ff else None,
            build_part("norm", layer.norms["pre_mixer"], env),
            build_part("norm", layer.norms["pre_feed_forward"], env) if has_ff else None,
            params.get("residual_mult", 1.0),
        )

    def parts(self):
        both = [self.pre_mixer, self.mixer, self.pre_feed_forward, self.feed_forward]
        return [p for p in both if p is not None]

    def forward(self, h, delta, ctx, binding: CacheBinding | None, delta_scale: float = 1.0):
        x = self.pre_mixer.add_norm(h, delta, ctx, tag="norm.mixer", delta_scale=delta_scale)
        mixed = self.mixer.forward(x, ctx, binding)
        if self.feed_forward is None:
            return mixed
        x = self.pre_feed_forward.add_norm(h, mixed, ctx, tag="norm.ffn", delta_scale=self.residual_mult)
        return self.feed_forward.forward(x, ctx)


@register_part("block", "parallel_residual")
class ParallelResidualBlock(Block):
    """The norm ``pre_mixer`` feeds the mixer and the feed-forward alike.  A mixer with an output
    bias leaves it to the add (``output_bias``)."""

    def __init__(self, mixer, feed_forward, pre_mixer) -> None:
        self.mixer, self.feed_forward, self.pre_mixer = mixer, feed_forward, pre_mixer
        self.residual_mult = 1.0
        self._pending: AddedTerms | None = None

    @classmethod
    def from_spec(cls, params: dict, env: BuildEnv, *, layer, **_):
        return cls(build_part("mixer", layer.mixer, env),
                   build_part("feed_forward", layer.feed_forward, env) if layer.feed_forward is not None else None,
                   build_part("norm", layer.norms["pre_mixer"], env))

    def parts(self):
        return [p for p in (self.pre_mixer, self.mixer, self.feed_forward) if p is not None]

    @property
    def output_post(self) -> AddedTerms | None:
        """What is added together with the delta this block's last forward left pending."""
        return self._pending

    def forward(self, h, delta, ctx, binding: CacheBinding | None, delta_scale: float = 1.0, delta_post=None):
        if delta_post is None:
            x = self.pre_mixer.add_norm(h, delta, ctx, tag="norm.mixer", delta_scale=delta_scale)
        else:
            x = self.pre_mixer.add_norm(h, delta, ctx, tag="norm.mixer", delta_scale=delta_scale,
                                        delta_post=delta_post)
        mixed = self.mixer.forward(x, ctx, binding)
        fed = self.feed_forward.forward(x, ctx) if self.feed_forward is not None else None
        bias = getattr(self.mixer, "output_bias", None)
        self._pending = AddedTerms(bias, fed) if (bias is not None or fed is not None) else None
        return mixed


@register_part("block", "sandwich_residual")
class SandwichResidualBlock(Block):
    """Norms ``pre_mixer``, ``post_mixer`` and, with a feed-forward, ``pre_feed_forward`` and
    ``post_feed_forward``.  A feed-forward with an output bias leaves it to the post norm's kernel
    (``output_bias``)."""

    def __init__(self, mixer, feed_forward, norms: dict) -> None:
        _adds_no_output_bias(mixer)
        self.mixer, self.feed_forward, self.norms = mixer, feed_forward, norms
        self.residual_mult = 1.0

    @classmethod
    def from_spec(cls, params: dict, env: BuildEnv, *, layer, **_):
        has_ff = layer.feed_forward is not None
        names = ["pre_mixer", "post_mixer"] + (["pre_feed_forward", "post_feed_forward"] if has_ff else [])
        return cls(build_part("mixer", layer.mixer, env),
                   build_part("feed_forward", layer.feed_forward, env) if has_ff else None,
                   {n: build_part("norm", layer.norms[n], env) for n in names})

    def parts(self):
        return [*self.norms.values(), self.mixer] + ([self.feed_forward] if self.feed_forward is not None else [])

    @property
    def output_post(self) -> PostNorm:
        if self.feed_forward is None:
            return PostNorm(self.norms["post_mixer"])
        return PostNorm(self.norms["post_feed_forward"], getattr(self.feed_forward, "output_bias", None))

    def forward(self, h, delta, ctx, binding, delta_scale: float = 1.0, delta_post: PostNorm | None = None):
        x = self.norms["pre_mixer"].add_norm(h, delta, ctx, tag="norm.mixer", delta_scale=delta_scale,
                                             delta_post=delta_post)
        mixed = self.mixer.forward(x, ctx, binding)
        if self.feed_forward is None:
            return mixed
        x = self.norms["pre_feed_forward"].add_norm(h, mixed, ctx, tag="norm.ffn",
                                                    delta_post=PostNorm(self.norms["post_mixer"]))
        return self.feed_forward.forward(x, ctx)


@register_part("block", "gated_prenorm_residual")
class GatedPreNormResidualBlock(Block):
    """Norms ``pre_mixer`` and, with a feed-forward, ``pre_feed_forward``.  Parameters: the tensor
    names ``mixer_gate``, ``mixer_gate_bias``, ``feed_forward_gate``, ``feed_forward_gate_bias`` (a
    bias name may be absent)."""

    def __init__(self, mixer, feed_forward, pre_mixer, pre_feed_forward, names: dict, hidden_size: int, dtype) -> None:
        _adds_no_output_bias(mixer)
        self.mixer, self.feed_forward = mixer, feed_forward
        self.pre_mixer, self.pre_feed_forward = pre_mixer, pre_feed_forward
        self.names, self.hidden_size, self.dtype = dict(names), int(hidden_size), dtype
        self.residual_mult = 1.0
        self.w_gate: dict = {}
        self.gate_bias: dict = {}
        self._pending: ResidualGate | None = None

    @classmethod
    def from_spec(cls, params: dict, env: BuildEnv, *, layer, **_):
        has_ff = layer.feed_forward is not None
        names = {k: params[k] for k in ("mixer_gate", "mixer_gate_bias") if params.get(k)}
        if has_ff:
            names.update({k: params[k] for k in ("feed_forward_gate", "feed_forward_gate_bias") if params.get(k)})
        for needed in ["mixer_gate"] + (["feed_forward_gate"] if has_ff else []):
            if needed not in names:
                raise ValueError(f"the gated block needs the tensor name {needed!r}")
        return cls(
            build_part("mixer", layer.mixer, env),
            build_part("feed_forward", layer.feed_forward, env) if has_ff else None,
            build_part("norm", layer.norms["pre_mixer"], env),
            build_part("norm", layer.norms["pre_feed_forward"], env) if has_ff else None,
            names, params.get("hidden_size", env.hidden_size), env.torch_dtype,
        )

    def parts(self):
        both = [self.pre_mixer, self.mixer, self.pre_feed_forward, self.feed_forward]
        return [p for p in both if p is not None]

    def weights(self) -> dict[str, WeightDecl]:
        h = self.hidden_size
        out = {}
        for which in ("mixer_gate", "feed_forward_gate"):
            if which in self.names:
                out[self.names[which]] = WeightDecl((h, h))
            if which + "_bias" in self.names:
                out[self.names[which + "_bias"]] = WeightDecl((h,), "vector")
        return out

    def bind(self, tensors, env: BuildEnv) -> None:
        for which in ("mixer_gate", "feed_forward_gate"):
            if which in self.names:
                self.w_gate[which] = tensors[self.names[which]].to(self.dtype).contiguous()
                bias = self.names.get(which + "_bias")
                self.gate_bias[which] = tensors[bias].float().contiguous() if bias else None
        # The mixer's gate reads what the mixer reads: a mixer that starts with one product over its
        # input takes the gate's rows into that product (this runs before the mixer's own bind).
        # The same for a feed-forward and its gate.
        if os.environ.get("IE_B200_GATE_IN_MIXER", "1") != "0":
            for which, part in (("mixer_gate", self.mixer), ("feed_forward_gate", self.feed_forward)):
                if part is not None and part.accepts_input_rows:
                    part.take_input_rows(self.w_gate[which])
                    self.w_gate[which] = None

    def _gate(self, which: str, x, ctx) -> ResidualGate:
        import torch

        # (the product may come back as partial sums if the kernel set says so: the kernel that applies
        # the gate adds them)
        pre = ctx.ops.linear(x, self.w_gate[which], ws=ctx.ws, tag="resgate." + which, out_dtype=torch.float32,
                             allow_split=getattr(ctx.ops, "gate_split", False))
        return ResidualGate(pre, self.gate_bias[which])

    @property
    def output_post(self) -> ResidualGate:
        """The gate of the delta this block's last forward left pending."""
        return self._pending

    def forward(self, h, delta, ctx, binding: CacheBinding | None, delta_scale: float = 1.0, delta_post=None):
        if delta_post is None:
            x = self.pre_mixer.add_norm(h, delta, ctx, tag="norm.mixer", delta_scale=delta_scale)
        else:
            x = self.pre_mixer.add_norm(h, delta, ctx, tag="norm.mixer", delta_scale=delta_scale,
                                        delta_post=delta_post)
        in_mixer = self.w_gate["mixer_gate"] is None
        gate = None if in_mixer else self._gate("mixer_gate", x, ctx)
        mixed = self.mixer.forward(x, ctx, binding)
        if in_mixer:
            gate = ResidualGate(self.mixer.extra_out, self.gate_bias["mixer_gate"])
        if self.feed_forward is None:
            self._pending = gate
            return mixed
        x = self.pre_feed_forward.add_norm(h, mixed, ctx, tag="norm.ffn", delta_post=gate)
        if self.w_gate["feed_forward_gate"] is not None:
            self._pending = self._gate("feed_forward_gate", x, ctx)
            return self.feed_forward.forward(x, ctx)
        out = self.feed_forward.forward(x, ctx)
        self._pending = ResidualGate(self.feed_forward.extra_out, self.gate_bias["feed_forward_gate"])
        return out
