"""Grouped-query softmax attention over the paged cache with a sink, a window and a gate per head.

``q = W_q h (+ b_q)``, ``k = W_k h (+ b_k)``, ``v = W_v h (+ b_v)``; value rows may have another size
than key rows.  With ``value_norm`` each value head is divided by its root mean square over
``vdim`` (eps inside the root, no weight) before it is cached.  Queries and keys are rotated by
their position only if a position encoding is named; without one positions do not enter the scores.
``score = q . k * scale``; a query sees itself and the ``window - 1`` positions before it (no
window: everything before it); pages behind the window are given back.  With a sink the softmax's
denominator holds one more term ``exp(sink[head])`` that has no key and no value.  With a head gate
the head's result is multiplied by ``sigmoid(W_g h)[head]`` (one number per head, from the mixer's
input) before the output projection.  Query head ``h`` uses key/value head ``h // (heads /
kv_heads)``.  Scores, weights, the value norm and the gate are 32-bit.

Queries, keys, values and the head gates come from one matrix product over the row-concatenated
weights, which can carry more rows of another map of the same input (``accepts_input_rows``);
biases, value norm and the cache write are one kernel; the gate is applied where the attention
kernel writes its result.
"""

from __future__ import annotations

from .base import BuildEnv, CacheBinding, Mixer, PagedKVRequest, WeightDecl
from .registry import register_part


@register_part("mixer", "sink_attention")
class SinkAttention(Mixer):
    allow_split = True
    accepts_input_rows = True

    def __init__(self, *, names: dict, hidden_size: int, heads: int, kv_heads: int, dim: int, vdim: int,
                 scale: float, window: int | None, value_norm: bool, eps: float, position, dtype) -> None:
        if heads % kv_heads:
            raise ValueError(f"heads ({heads}) not divisible by kv_heads ({kv_heads})")
        if window is not None and window < 1:
            raise ValueError("a window holds at least the query's own position")
        for needed in ("q", "k", "v", "o"):
            if not names.get(needed):
                raise ValueError(f"the attention needs the tensor name {needed!r}")
        biases = [bool(names.get(b)) for b in ("q_bias", "k_bias", "v_bias")]
        if any(biases) and not all(biases):
            raise ValueError("queries, keys and values have biases together or not at all")
        self.names = {k: v for k, v in names.items() if v}
        self.hidden_size, self.heads, self.kv_heads, self.dim, self.vdim = hidden_size, heads, kv_heads, dim, vdim
        self.scale, self.window, self.value_norm, self.eps = float(scale), window, bool(value_norm), float(eps)
        self.position, self.dtype = position, dtype
        self.qkv_size = (heads + kv_heads) * dim + kv_heads * vdim
        self.w_in = self.w_o = self.bias = self.sinks = None

    @classmethod
    def from_spec(cls, params: dict, env: BuildEnv, **_):
        position = env.positions[params["position"]] if params.get("position") else None
        return cls(names=params["names"], hidden_size=params.get("hidden_size", env.hidden_size),
                   heads=params["heads"], kv_heads=params["kv_heads"], dim=params["dim"], vdim=params["vdim"],
                   scale=params["scale"], window=params.get("window"), value_norm=params.get("value_norm", False),
                   eps=params.get("eps", 1e-6), position=position, dtype=env.torch_dtype)

    def weights(self) -> dict[str, WeightDecl]:
        n, h = self.names, self.hidden_size
        out = {
            n["q"]: WeightDecl((self.heads * self.dim, h)), n["k"]: WeightDecl((self.kv_heads * self.dim, h)),
            n["v"]: WeightDecl((self.kv_heads * self.vdim, h)), n["o"]: WeightDecl((h, self.heads * self.vdim)),
        }
        if "q_bias" in n:
            out[n["q_bias"]] = WeightDecl((self.heads * self.dim,), "vector")
            out[n["k_bias"]] = WeightDecl((self.kv_heads * self.dim,), "vector")
            out[n["v_bias"]] = WeightDecl((self.kv_heads * self.vdim,), "vector")
        if "sink" in n:
            out[n["sink"]] = WeightDecl((self.heads,), "vector")
        if "head_gate" in n:
            out[n["head_gate"]] = WeightDecl((self.heads, h))
        return out

    def bind(self, tensors, env: BuildEnv) -> None:
        import torch

        n = self.names
        rows = [tensors[n[k]].to(self.dtype) for k in "qkv"]
        if "head_gate" in n:
            rows.append(tensors[n["head_gate"]].to(self.dtype))
        self.w_in, self.extra_at = self._with_extra_rows(rows)
        self.w_o = tensors[n["o"]].to(self.dtype).contiguous()
        if "q_bias" in n:
            self.bias = torch.cat([tensors[n[k]].float() for k in ("q_bias", "k_bias", "v_bias")]).contiguous()
        if "sink" in n:
            self.sinks = tensors[n["sink"]].float().contiguous()

    def cache_request(self) -> PagedKVRequest:
        return PagedKVRequest(self.kv_heads, self.dim, self.window, value_dim=self.vdim)

    def forward(self, x, ctx, binding: CacheBinding):
        import torch

        n = x.shape[0]
        group = ctx.groups[binding.group]
        k_cache, v_cache = group.k[binding.slot], group.v[binding.slot]
        ops, ws = ctx.ops, ctx.ws
        proj = ops.linear(x, self.w_in, ws=ws, tag="sinkattn.in", out_dtype=torch.float32)
        self.extra_out = self._extra_columns(proj, self.extra_at)
        q = ws.buffer("sinkattn.q", n, self.heads * self.dim, self.dtype)
        table = self.position.rotary_table() if self.position is not None else None
        rot_dims = self.position.rotary_dim if self.position is not None else 0
        ops.qk_norm_rope_write(proj, ctx.positions, table, rot_dims, None, None, self.eps, q, k_cache, v_cache,
                               group.slot_mapping if binding.writes else None, self.heads, self.kv_heads,
                               self.dim, self.vdim, group.page_size, bias=self.bias, value_norm=self.value_norm)
        gate = proj[:, self.qkv_size: self.qkv_size + self.heads] if "head_gate" in self.names else None
        out = ws.buffer("sinkattn.out", n, self.heads * self.vdim, self.dtype)
        ops.sink_attention(q, k_cache, v_cache, group.block_tables, ctx, self.heads, self.kv_heads, self.dim,
                           self.vdim, group.page_size, self.scale, self.window, self.sinks, gate, out)
        return ops.linear(out, self.w_o, ws=ws, tag="sinkattn.delta", out_dtype=torch.float32,
                          allow_split=self.allow_split)
