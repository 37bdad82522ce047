"""Token embedding and the output head.

Embedding: ``x = table[token_ids]`` with no scaling (engine/model/llama.py:25,61), or times the
constant ``scale`` of a model that has one; the rows are widened to the 32-bit residual stream.  Head: ``logits = x @ W^T`` in 32-bit out, no
bias (engine/model/llama.py:36,68), times ``logit_scale`` where a model has one; with tied embeddings ``W`` is the embedding table
itself (engine/model/loader.py:91-92), one buffer.
"""

from __future__ import annotations

from .base import BuildEnv, CacheBinding, Part, StateRequest, WeightDecl
from .registry import register_part


@register_part("embedding", "token")
class TokenEmbedding(Part):
    category = "embedding"

    def __init__(self, weight: str, vocab_size: int, hidden_size: int, dtype, scale: float = 1.0) -> None:
        self.weight_name, self.vocab_size, self.hidden_size = weight, vocab_size, hidden_size
        self.dtype, self.table, self.scale = dtype, None, float(scale)

    @classmethod
    def from_spec(cls, params: dict, env: BuildEnv, **_):
        return cls(params["weight"], params["vocab_size"], env.hidden_size, env.torch_dtype,
                   params.get("scale", 1.0))

    def weights(self) -> dict[str, WeightDecl]:
        return {self.weight_name: WeightDecl((self.vocab_size, self.hidden_size), "table")}

    def bind(self, tensors, env: BuildEnv) -> None:
        self.table = tensors[self.weight_name].to(self.dtype).contiguous()

    def forward(self, token_ids, ctx):
        import torch

        h = ctx.ws.buffer("residual", token_ids.shape[0], self.hidden_size, torch.float32)
        if self.scale == 1.0:
            ctx.ops.embedding(self.table, token_ids, h)
        else:
            ctx.ops.embedding(self.table, token_ids, h, self.scale)
        return h


@register_part("embedding", "token_bigram")
class TokenBigramEmbedding(TokenEmbedding):
    """Token embedding plus a hashed bigram embedding: row ``(previous * mul_prev + token * mul_cur)
    mod buckets`` of a second table, whose last row (number ``buckets``) serves a request's first
    token.  The token before a step's first one is part of the request's state: it lives in a
    state slot on the device (the integer's bits in a 32-bit word), so a step launched on tokens
    the device is still sampling finds it too."""

    def __init__(self, weight: str, bigram: str, vocab_size: int, hidden_size: int, dtype, buckets: int,
                 mul_prev: int, mul_cur: int) -> None:
        super().__init__(weight, vocab_size, hidden_size, dtype)
        if buckets < 1:
            raise ValueError("the bigram table needs at least one bucket")
        self.bigram_name, self.buckets = bigram, int(buckets)
        self.mul_prev, self.mul_cur = int(mul_prev), int(mul_cur)
        self.bigram = None

    @classmethod
    def from_spec(cls, params: dict, env: BuildEnv, **_):
        return cls(params["weight"], params["bigram"], params["vocab_size"], env.hidden_size, env.torch_dtype,
                   params["buckets"], params["mul_prev"], params["mul_cur"])

    def weights(self) -> dict[str, WeightDecl]:
        return {**super().weights(),
                self.bigram_name: WeightDecl((self.buckets + 1, self.hidden_size), "table")}

    def bind(self, tensors, env: BuildEnv) -> None:
        super().bind(tensors, env)
        self.bigram = tensors[self.bigram_name].to(self.dtype).contiguous()

    def cache_request(self) -> StateRequest:
        return StateRequest((1,))

    def forward(self, token_ids, ctx, binding: CacheBinding):
        import torch

        group = ctx.groups[binding.group]
        h = ctx.ws.buffer("residual", token_ids.shape[0], self.hidden_size, torch.float32)
        ctx.ops.bigram_embedding(self.table, self.bigram, token_ids, ctx, group.state[binding.slot], group.slots,
                                 h, self.buckets, self.mul_prev, self.mul_cur)
        return h


@register_part("head", "linear")
class LinearHead(Part):
    category = "head"

    def __init__(self, weight: str | None, vocab_size: int, hidden_size: int, dtype,
                 logit_scale: float = 1.0, softcap: float | None = None) -> None:
        self.weight_name, self.vocab_size, self.hidden_size = weight, vocab_size, hidden_size
        self.dtype, self.weight = dtype, None
        self.logit_scale = float(logit_scale)  # the 32-bit logits are multiplied by it
        # ... and then squashed into (-softcap, softcap): c * tanh(logits / c), if the model caps them
        self.softcap = None if not softcap else float(softcap)
        if self.softcap is not None and not self.softcap > 0:
            raise ValueError("the cap of the logits must be positive")

    @classmethod
    def from_spec(cls, params: dict, env: BuildEnv, **_):
        # weight=None means tied: the model hands over the embedding table at bind time.
        return cls(params.get("weight"), params["vocab_size"], env.hidden_size, env.torch_dtype,
                   params.get("logit_scale", 1.0), params.get("softcap"))

    def weights(self) -> dict[str, WeightDecl]:
        if self.weight_name is None:
            return {}
        return {self.weight_name: WeightDecl((self.vocab_size, self.hidden_size))}

    def bind(self, tensors, env: BuildEnv) -> None:
        if self.weight_name is not None:
            self.weight = tensors[self.weight_name].to(self.dtype).contiguous()

    def tie(self, table) -> None:
        self.weight = table

    def forward(self, x, ctx):
        import torch

        logits = ctx.ws.buffer("logits", x.shape[0], self.vocab_size, torch.float32, rows_cap=None)
        ctx.ops.linear(x, self.weight, logits, tag="head")
        if self.softcap is not None:
            ctx.ops.scale_softcap_(logits, self.logit_scale, self.softcap)
        elif self.logit_scale != 1.0:
            ctx.ops.scale_(logits, self.logit_scale)
        return logits
