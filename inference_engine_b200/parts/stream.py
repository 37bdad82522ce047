"""Operations on the whole residual stream between layers (category ``stream``).

``reinject``: ``x <- W [x; x0]`` with ``x0`` the embedding's output of the same token and ``W`` of
shape ``[width, 2 width]`` (the stream's part first).  A model whose layers run several times in a
row with the same weights applies it before each pass.  The product runs in the compute dtype with
32-bit sums; its result is the new 32-bit stream.

``add_embedding``: ``x <- x + x0``, the embedding's output added again (a looped model before every
pass but the first).  Where the stream still waits for a pending delta, the add joins that delta's
add in the kernel of the next norm (``fold``); by itself it is one 32-bit add.
"""

from __future__ import annotations

from .base import BuildEnv, Part, WeightDecl
from .registry import register_part


@register_part("stream", "reinject")
class Reinject(Part):
    category = "stream"
    needs_embedding = True  # the model keeps the embedding's output of the step for this part

    def __init__(self, weight: str, hidden_size: int, dtype) -> None:
        self.weight_name, self.hidden_size, self.dtype = weight, int(hidden_size), dtype
        self.weight = None

    @classmethod
    def from_spec(cls, params: dict, env: BuildEnv, **_):
        return cls(params["weight"], params.get("hidden_size", env.hidden_size), env.torch_dtype)

    def weights(self) -> dict[str, WeightDecl]:
        return {self.weight_name: WeightDecl((self.hidden_size, 2 * self.hidden_size))}

    def bind(self, tensors, env: BuildEnv) -> None:
        self.weight = tensors[self.weight_name].to(self.dtype).contiguous()

    def forward(self, h, x0, ctx) -> None:
        both = ctx.ws.buffer("stream.both", h.shape[0], 2 * self.hidden_size, self.dtype)
        ctx.ops.concat_cast(h, x0, both)
        ctx.ops.linear(both, self.weight, out=h, tag="stream.reinject")


@register_part("stream", "add_embedding")
class AddEmbedding(Part):
    category = "stream"
    needs_embedding = True

    @classmethod
    def from_spec(cls, params: dict, env: BuildEnv, **_):
        return cls()

    def fold(self, post, x0):
        """The pending delta's companion with ``x0`` taken in, or None if this add cannot join it (the
        delta is treated before it is added: normalised, or gated)."""
        from .norm import AddedTerms

        if post is None:
            return AddedTerms(rows_like_stream=x0)
        if isinstance(post, AddedTerms) and post.rows_like_stream is None:
            return post.with_stream_rows(x0)
        return None

    def forward(self, h, x0, ctx) -> None:
        ctx.ops.weighted_sum(h, 1.0, x0, 1.0, h)
