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

Variants by parameters.  ``values="keys"``: there is no value projection; the values are the keys as
projected (with their bias), before the rotation, so the cache holds a rotated and a plain copy of
each key row, and only queries and keys may have biases.  ``softcap``: a score ``s`` becomes
``softcap * tanh(s / softcap)`` before the softmax.  ``sink_value``: the sink is this constant for
every head instead of a learned tensor (0: the denominator's extra term is ``exp(0)``).
``keep_first`` (with a window): the first positions of a request stay visible to all its later
queries, at their own positions, and their pages are kept.  A rotary encoding of either layout
(halves or interleaved pairs) on the first ``rotary_dim`` entries of each head.  ``o_bias`` among
the names: a bias of the output projection, which the part leaves to whoever adds its output to the
residual stream (``output_bias``).

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
                 scale: float, window: int | None, value_norm: bool, eps: float, position, dtype,
                 values: str = "projected", softcap: float | None = None, sink_value: float | None = None,
                 keep_first: int = 0) -> None:
        if heads % kv_heads:
            raise ValueError(f"heads ({heads}) not divisible by kv_heads ({kv_heads})")
        if window is not None and window < 1:
            raise ValueError("a window holds at least the query's own position")
        if values not in ("projected", "keys"):
            raise ValueError(f"values are 'projected' or 'keys', not {values!r}")
        self.values_from_keys = values == "keys"
        if self.values_from_keys and (vdim != dim or value_norm or names.get("v") or names.get("v_bias")):
            raise ValueError("values that are the keys have the keys' size, no projection, no bias and no norm")
        self.projected = ("q", "k") if self.values_from_keys else ("q", "k", "v")
        for needed in (*self.projected, "o"):
            if not names.get(needed):
                raise ValueError(f"the attention needs the tensor name {needed!r}")
        self.bias_names = tuple(p + "_bias" for p in self.projected)
        biases = [bool(names.get(b)) for b in self.bias_names]
        if any(biases) and not all(biases):
            raise ValueError("queries, keys and values have biases together or not at all")
        if softcap is not None and not softcap > 0:
            raise ValueError("the cap of the scores must be positive")
        if sink_value is not None and names.get("sink"):
            raise ValueError("the sink is a learned tensor or a constant, not both")
        if keep_first < 0 or (keep_first and window is None):
            raise ValueError("first positions are kept beside a window, and there cannot be fewer than none")
        self.names = {k: v for k, v in names.items() if v}
        self.hidden_size, self.heads, self.kv_heads, self.dim, self.vdim = hidden_size, heads, kv_heads, dim, vdim
        self.scale, self.window, self.value_norm, self.eps = float(scale), window, bool(value_norm), float(eps)
        self.position, self.dtype = position, dtype
        self.softcap = None if softcap is None else float(softcap)
        self.sink_value = None if sink_value is None else float(sink_value)
        self.keep_first = int(keep_first)
        self.qkv_size = (heads + kv_heads) * dim + (0 if self.values_from_keys else kv_heads * vdim)
        self.w_in = self.w_o = self.bias = self.sinks = self.output_bias = None

    @classmethod
    def from_spec(cls, params: dict, env: BuildEnv, **_):
        position = env.positions[params["position"]] if params.get("position") else None
        return cls(names=params["names"], hidden_size=params.get("hidden_size", env.hidden_size),
                   heads=params["heads"], kv_heads=params["kv_heads"], dim=params["dim"], vdim=params["vdim"],
                   scale=params["scale"], window=params.get("window"), value_norm=params.get("value_norm", False),
                   eps=params.get("eps", 1e-6), position=position, dtype=env.torch_dtype,
                   values=params.get("values", "projected"), softcap=params.get("softcap"),
                   sink_value=params.get("sink_value"), keep_first=params.get("keep_first") or 0)

    def weights(self) -> dict[str, WeightDecl]:
        n, h = self.names, self.hidden_size
        out = {
            n["q"]: WeightDecl((self.heads * self.dim, h)), n["k"]: WeightDecl((self.kv_heads * self.dim, h)),
            n["o"]: WeightDecl((h, self.heads * self.vdim)),
        }
        if not self.values_from_keys:
            out[n["v"]] = WeightDecl((self.kv_heads * self.vdim, h))
        if "q_bias" in n:
            out[n["q_bias"]] = WeightDecl((self.heads * self.dim,), "vector")
            out[n["k_bias"]] = WeightDecl((self.kv_heads * self.dim,), "vector")
            if not self.values_from_keys:
                out[n["v_bias"]] = WeightDecl((self.kv_heads * self.vdim,), "vector")
        if "o_bias" in n:
            out[n["o_bias"]] = WeightDecl((h,), "vector")
        if "sink" in n:
            out[n["sink"]] = WeightDecl((self.heads,), "vector")
        if "head_gate" in n:
            out[n["head_gate"]] = WeightDecl((self.heads, h))
        return out

    def bind(self, tensors, env: BuildEnv) -> None:
        import torch

        n = self.names
        rows = [tensors[n[k]].to(self.dtype) for k in self.projected]
        if "head_gate" in n:
            rows.append(tensors[n["head_gate"]].to(self.dtype))
        self.w_in, self.extra_at = self._with_extra_rows(rows)
        self.w_o = tensors[n["o"]].to(self.dtype).contiguous()
        if "q_bias" in n:
            self.bias = torch.cat([tensors[n[k]].float() for k in self.bias_names]).contiguous()
        if "o_bias" in n:
            self.output_bias = tensors[n["o_bias"]].float().contiguous()
        if "sink" in n:
            self.sinks = tensors[n["sink"]].float().contiguous()
        elif self.sink_value is not None:
            self.sinks = torch.full((self.heads,), self.sink_value, dtype=torch.float32, device=self.w_o.device)

    def cache_request(self) -> PagedKVRequest:
        return PagedKVRequest(self.kv_heads, self.dim, self.window, value_dim=self.vdim, keep_first=self.keep_first)

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
                               self.dim, self.vdim, group.page_size, bias=self.bias, value_norm=self.value_norm,
                               values_from_keys=self.values_from_keys,
                               interleaved=getattr(self.position, "layout", "halves") == "interleaved")
        gate = proj[:, self.qkv_size: self.qkv_size + self.heads] if "head_gate" in self.names else None
        out = ws.buffer("sinkattn.out", n, self.heads * self.vdim, self.dtype)
        ops.sink_attention(q, k_cache, v_cache, group.block_tables, ctx, self.heads, self.kv_heads, self.dim,
                           self.vdim, group.page_size, self.scale, self.window, self.sinks, gate, out,
                           softcap=self.softcap, keep_first=self.keep_first)
        return ops.linear(out, self.w_o, ws=ws, tag="sinkattn.delta", out_dtype=torch.float32,
                          allow_split=self.allow_split)
