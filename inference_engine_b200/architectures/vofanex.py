"""Vofanex: a decoder-only model of gated-linear-attention layers and windowed attention layers,
whose sublayers enter the residual stream through learned gates.

Configuration keys: ``vocab``, ``width``, ``norm.eps``, ``embedding.scale`` and ``layers``; each
layer gives its ``type`` (``gla`` or ``attention``), the mixer's sizes and constants under ``mixer``
and its feed-forward under ``mlp`` (``null``: none; ``kind`` ``dense``: an ungated feed-forward with
the PolyNorm activation; ``kind`` ``moe``: ``router.experts`` small gated experts of ``expert.ff``
units, of which a token uses ``router.top``).  ``max_positions`` is optional: nothing in the model
depends on a position's number.  Tensors: ``embed``, ``l<i>.norm1`` / ``norm2``, ``l<i>.rg1`` /
``rg1.b`` / ``rg2`` / ``rg2.b`` (the residual gates), ``l<i>.mix.*``, ``l<i>.mlp.*``, ``final.norm``,
``head``.

The model: token embedding times a constant.  A layer is pre-norm (RMS norm with a weight); what a
sublayer returns is multiplied, element by element, by the sigmoid of a linear map of the sublayer's
own input before it is added.  ``gla`` mixers keep a matrix state per head that decays per key
channel (``tau`` sharpens the decay; the rank of the decay's low-rank map is the shape of
``mix.a1``, or the optional key ``decay_rank``).  ``attention`` mixers are grouped-query softmax
attention without any rotation, with biases on queries, keys and values, value heads of unit root
mean square, a sliding window (``mask.size``; absent: none), a learned sink per head in the
softmax's denominator and a sigmoid gate per head.  No torch import here.
"""

from __future__ import annotations

import math
from dataclasses import dataclass
from typing import Any

from ..config.model_config import ConfigError, Footprint, id_tuple
from ..config.registry import register_architecture
from ..config.spec import LayerSpec, ModelSpec, PartSpec, ScheduleEntry
from .rugedra import read_tensor_shapes

NAME = "Vofanex"
LAYER_TYPES = ("gla", "attention")
NO_POSITION_LIMIT = 1 << 30  # the model has no position table: its length is the cache's business


def _need(raw, key: str, kind, where: str):
    if not isinstance(raw, dict) or key not in raw or raw[key] is None:
        raise ConfigError(f"config.json: {where} is missing the key {key!r}")
    try:
        return kind(raw[key])
    except (TypeError, ValueError) as exc:
        raise ConfigError(f"config.json: {where}.{key} = {raw[key]!r} is not a {kind.__name__}") from exc


def _parse_mixer(kind: str, raw: dict, where: str) -> dict:
    if kind == "gla":
        out = {k: _need(raw, k, int, where) for k in ("heads", "dim", "vdim")}
        out["tau"] = _need(raw, "tau", float, where)
        if not out["tau"] > 0 or not math.isfinite(out["tau"]):
            raise ConfigError(f"config.json: {where}.tau must be a positive number")
        out["decay_rank"] = int(raw["decay_rank"]) if raw.get("decay_rank") is not None else None
    else:
        out = {k: _need(raw, k, int, where) for k in ("heads", "dim", "vdim")}
        # (a mixer that does not share keys and values among heads need not say so)
        out["kv_heads"] = _need(raw, "kv_heads", int, where) if raw.get("kv_heads") is not None else out["heads"]
        out["scale"] = _need(raw, "scale", float, where)
        if out["kv_heads"] < 1 or out["heads"] % out["kv_heads"]:
            raise ConfigError(f"config.json: {where}.heads is not a multiple of kv_heads")
        mask = raw.get("mask") or {}
        out["window"] = int(mask["size"]) if mask.get("size") is not None else None
        if out["window"] is not None and out["window"] < 1:
            raise ConfigError(f"config.json: {where}.mask.size must be at least 1")
    for k in ("heads", "dim", "vdim"):
        if out[k] < 1:
            raise ConfigError(f"config.json: {where}.{k} must be at least 1")
    return out


def _parse_mlp(raw, where: str):
    if raw is None:
        return None
    kind = _need(raw, "kind", str, where)
    if kind == "dense":
        return {"kind": "dense", "ff": _need(raw, "ff", int, where)}
    if kind != "moe":
        raise ConfigError(f"config.json: {where}.kind = {kind!r} is neither 'dense' nor 'moe'")
    expert, router = raw.get("expert") or {}, raw.get("router") or {}
    out = {"kind": "moe", "ff": _need(expert, "ff", int, where + ".expert"),
           "experts": _need(router, "experts", int, where + ".router"),
           "top": _need(router, "top", int, where + ".router")}
    if not 1 <= out["top"] <= out["experts"]:
        raise ConfigError(f"config.json: {where}.router.top must be between 1 and the number of experts")
    return out


@dataclass(frozen=True)
class VofanexLayer:
    type: str
    mixer: dict
    mlp: dict | None


@dataclass(frozen=True)
class VofanexConfig:
    architecture: str
    vocab_size: int
    hidden_size: int
    max_position_embeddings: int
    norm_eps: float
    embedding_scale: float
    layers: tuple[VofanexLayer, ...]
    eos_token_ids: tuple[int, ...] = ()
    torch_dtype: str = "bfloat16"

    @classmethod
    def from_dict(cls, raw: dict[str, Any]) -> "VofanexConfig":
        listed = raw.get("layers")
        if not isinstance(listed, list) or not listed:
            raise ConfigError("config.json: 'layers' must list at least one layer")
        layers = []
        for i, entry in enumerate(listed):
            where = f"layers[{i}]"
            kind = _need(entry, "type", str, where)
            if kind not in LAYER_TYPES:
                raise ConfigError(f"config.json: {where}.type = {kind!r} is not one of {LAYER_TYPES}")
            layers.append(VofanexLayer(kind, _parse_mixer(kind, entry.get("mixer") or {}, where + ".mixer"),
                                       _parse_mlp(entry.get("mlp"), where + ".mlp")))
        cfg = cls(
            architecture=str(raw.get("architecture", NAME)),
            vocab_size=_need(raw, "vocab", int, "the model"),
            hidden_size=_need(raw, "width", int, "the model"),
            max_position_embeddings=int(raw.get("max_positions") or NO_POSITION_LIMIT),
            norm_eps=_need(raw.get("norm") or {}, "eps", float, "norm"),
            embedding_scale=float((raw.get("embedding") or {}).get("scale", 1.0)),
            layers=tuple(layers),
            eos_token_ids=id_tuple(raw.get("eos_token_id")),
            torch_dtype=str(raw.get("torch_dtype", "bfloat16")),
        )
        for key in ("vocab_size", "hidden_size", "max_position_embeddings"):
            if getattr(cfg, key) < 1:
                raise ConfigError(f"config.json: {key} must be >= 1")
        if not cfg.norm_eps > 0 or not math.isfinite(cfg.norm_eps):
            raise ConfigError("config.json: norm.eps must be a positive number")
        if not math.isfinite(cfg.embedding_scale):
            raise ConfigError("config.json: embedding.scale must be a number")
        return cfg

    def complete_from_folder(self, model_dir) -> "VofanexConfig":
        return self.with_tensor_shapes(read_tensor_shapes(model_dir))

    def with_tensor_shapes(self, shapes: dict[str, tuple[int, ...]]) -> "VofanexConfig":
        """Fill in the size only a tensor's shape gives: the rank of a ``gla`` mixer's decay map."""
        layers = []
        for i, layer in enumerate(self.layers):
            mixer = dict(layer.mixer)
            name = f"l{i}.mix.a1"
            if layer.type == "gla" and mixer.get("decay_rank") is None and name in shapes:
                mixer["decay_rank"] = int(shapes[name][0])
            layers.append(VofanexLayer(layer.type, mixer, layer.mlp))
        return VofanexConfig(**{**self.__dict__, "layers": tuple(layers)})


def _mixer_spec(cfg: VofanexConfig, i: int, layer: VofanexLayer) -> PartSpec:
    p, m = f"l{i}.mix", layer.mixer
    if layer.type == "gla":
        if m.get("decay_rank") is None:
            raise ConfigError(f"layers[{i}].mixer: the rank of a1 is known neither from the tensor's shape nor "
                              "from 'decay_rank'")
        return PartSpec("gla", {
            "names": {"q": f"{p}.q", "k": f"{p}.k", "v": f"{p}.v", "g": f"{p}.g", "a1": f"{p}.a1", "a2": f"{p}.a2",
                      "a2_bias": f"{p}.a2.b", "out_norm": f"{p}.norm", "o": f"{p}.o"},
            "heads": m["heads"], "dim": m["dim"], "vdim": m["vdim"], "rank": m["decay_rank"], "tau": m["tau"],
            "eps": cfg.norm_eps})
    return PartSpec("sink_attention", {
        "names": {"q": f"{p}.q", "k": f"{p}.k", "v": f"{p}.v", "q_bias": f"{p}.q.b", "k_bias": f"{p}.k.b",
                  "v_bias": f"{p}.v.b", "sink": f"{p}.sink", "head_gate": f"{p}.g", "o": f"{p}.o"},
        "heads": m["heads"], "kv_heads": m["kv_heads"], "dim": m["dim"], "vdim": m["vdim"], "scale": m["scale"],
        "window": m["window"], "value_norm": True, "eps": cfg.norm_eps, "position": None})


def _mlp_spec(cfg: VofanexConfig, i: int, mlp: dict | None) -> PartSpec | None:
    if mlp is None:
        return None
    p = f"l{i}.mlp"
    if mlp["kind"] == "dense":
        return PartSpec("polynorm", {"up_proj": f"{p}.up", "down_proj": f"{p}.down", "coeff": f"{p}.act",
                                     "intermediate_size": mlp["ff"], "eps": cfg.norm_eps})
    # experts: down(silu(gate(x)) * up(x)); nothing is clamped, the router has a bias
    return PartSpec("routed_experts", {
        "router": f"{p}.router", "router_bias": f"{p}.router.b", "expert_prefix": f"{p}.e",
        "experts": mlp["experts"], "top": mlp["top"], "groups": 1, "keep_groups": 1,
        "intermediate_size": mlp["ff"], "limit": None, "alpha": 1.0, "up_offset": 0.0})


def vofanex_spec(cfg: VofanexConfig) -> ModelSpec:
    layers = []
    for i, layer in enumerate(cfg.layers):
        norms = {"pre_mixer": PartSpec("rms", {"weight": f"l{i}.norm1", "eps": cfg.norm_eps})}
        gates = {"mixer_gate": f"l{i}.rg1", "mixer_gate_bias": f"l{i}.rg1.b"}
        if layer.mlp is not None:
            norms["pre_feed_forward"] = PartSpec("rms", {"weight": f"l{i}.norm2", "eps": cfg.norm_eps})
            gates.update(feed_forward_gate=f"l{i}.rg2", feed_forward_gate_bias=f"l{i}.rg2.b")
        layers.append(LayerSpec(prefix=f"l{i}", block=PartSpec("gated_prenorm_residual", gates),
                                mixer=_mixer_spec(cfg, i, layer), feed_forward=_mlp_spec(cfg, i, layer.mlp),
                                norms=norms))
    return ModelSpec(
        architecture=cfg.architecture, vocab_size=cfg.vocab_size, hidden_size=cfg.hidden_size,
        max_position_embeddings=cfg.max_position_embeddings,
        embedding=PartSpec("token", {"weight": "embed", "vocab_size": cfg.vocab_size, "scale": cfg.embedding_scale}),
        positions={}, layers=tuple(layers), schedule=tuple(ScheduleEntry(i) for i in range(len(layers))),
        final_norm=PartSpec("rms", {"weight": "final.norm", "eps": cfg.norm_eps}),
        head=PartSpec("linear", {"weight": "head", "vocab_size": cfg.vocab_size}),
        eos_token_ids=cfg.eos_token_ids)


def vofanex_footprint(cfg: VofanexConfig) -> Footprint:
    h = cfg.hidden_size
    params = cfg.vocab_size * h * 2 + h
    per_token = per_request = 0
    for layer in cfg.layers:
        m = layer.mixer
        params += h + h * h + h  # the norm and the mixer's residual gate
        if layer.type == "gla":
            qk, v, r = m["heads"] * m["dim"], m["heads"] * m["vdim"], m.get("decay_rank") or 0
            params += 2 * qk * h + 2 * v * h + r * h + qk * r + qk + m["vdim"] + h * v
            per_request += qk * m["vdim"]
        else:
            q, k, v = m["heads"] * m["dim"], m["kv_heads"] * m["dim"], m["kv_heads"] * m["vdim"]
            params += (q + k + v) * (h + 1) + m["heads"] * (h + 1) + h * m["heads"] * m["vdim"]
            per_token += k + v
        if layer.mlp is not None:
            params += h + h * h + h
            if layer.mlp["kind"] == "dense":
                params += 2 * layer.mlp["ff"] * h + 4
            else:
                params += layer.mlp["experts"] * (3 * layer.mlp["ff"] * h + h + 1)
    return Footprint(params, per_token, per_request)


def describe_vofanex(cfg: VofanexConfig) -> list[str]:
    kinds = [layer.type + ("" if layer.mlp is None else "+" + layer.mlp["kind"]) for layer in cfg.layers]
    fp = vofanex_footprint(cfg)
    windows = sorted({layer.mixer["window"] for layer in cfg.layers
                      if layer.type == "attention" and layer.mixer["window"] is not None})
    return [
        f"architecture        {cfg.architecture}",
        f"layers / width      {len(cfg.layers)} / {cfg.hidden_size}",
        f"layer kinds         {', '.join(kinds)}",
        f"attention windows   {', '.join(map(str, windows)) if windows else 'none'}",
        f"parameters          {fp.parameters / 1e9:.3f} B",
        f"cache per token     {fp.cache_bytes_per_token(2)} B (bf16), state per request {fp.state_values_per_request * 4} B",
    ]


register_architecture(NAME, VofanexConfig, vofanex_spec, describe_vofanex, vofanex_footprint)
