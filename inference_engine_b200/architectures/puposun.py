"""Puposun: a decoder-only model of parallel layers (one norm feeds the mixer and the feed-forward,
both outputs are added to the stream at once), two kinds of attention whose values are their
unrotated keys, mixtures of experts routed by sigmoid scores, and a run of layers that is looped.

Configuration keys: ``vocab``, ``width``, ``norm.eps``, ``embedding.scale``, ``logit_softcap``
(absent: the logits are not capped), ``loop`` (``start``, ``stop``, ``times``; absent: every layer
once) and ``layers``; each layer gives its ``type`` (``attention`` or ``attention_2``), the mixer's
sizes and constants under ``mixer`` (``heads``, ``kv_heads``, ``dim``, ``vdim``, ``scale``,
``rot.dims`` / ``rot.base``, ``softcap``, ``mask.size`` / ``mask.keep_first``; what is absent does not
exist) and its feed-forward under ``mlp`` (``null``: none; ``kind`` ``moe``: ``router.experts`` gated
experts of ``expert.ff`` units, ``router.top`` per token, ``router.groups.count`` / ``keep``,
``router.scale``).  ``max_positions`` is optional.  Tensors: ``embed``, ``l<i>.norm1``,
``l<i>.mix.q`` / ``k`` / ``o`` (``attention``: with ``.b`` biases; ``attention_2``: with the head gates
``g``), ``l<i>.mlp.router`` / ``correction`` / ``e<j>.gate`` / ``up`` / ``down``, ``final.norm``, ``head``.

The model: token embedding times a constant.  A layer: ``x <- x + mixer(h) + feed_forward(h)`` with
``h = rms(x) * norm1``.  Both mixers are grouped-query softmax attention with ``v = k`` as projected,
before the rotation.  ``attention``: rotation of pairs ``(i, i + dims / 2)``, biases on queries, keys
and the output, scores capped by ``softcap * tanh(s / softcap)``, every earlier position visible, and a
term ``exp(0)`` in the softmax's denominator that has neither key nor value (a sink).  ``attention_2``: rotation of pairs
``(2i, 2i + 1)``, no biases, a sliding window that also keeps the first ``keep_first`` positions
visible, a sigmoid gate per head.  The router scores experts by the sigmoid of its logits, chooses
by score plus a stored correction, within the groups whose two best such values add up highest, and
weighs the chosen by their plain scores over their sum, times a constant.  Layers ``loop.start ..
loop.stop - 1`` run ``loop.times`` times in a row with the same weights and a cache of their own per
pass; before each pass but the first the embedding's output is added to the stream.  The logits are
capped like the scores.  No torch import here.
"""

from __future__ import annotations

import math
from dataclasses import dataclass
from typing import Any

from ..config.model_config import ConfigError, Footprint, id_tuple
from ..config.registry import register_architecture
from ..config.spec import LayerSpec, ModelSpec, PartSpec, ScheduleEntry

NAME = "Puposun"
LAYER_TYPES = ("attention", "attention_2")
ROTARY_LAYOUT = {"attention": "halves", "attention_2": "interleaved"}
NO_POSITION_LIMIT = 1 << 30  # rotary tables are as long as the engine's longest request


def _need(raw, key: str, kind, where: str):
    if not isinstance(raw, dict) or key not in raw or raw[key] is None:
        raise ConfigError(f"config.json: {where} is missing the key {key!r}")
    try:
        return kind(raw[key])
    except (TypeError, ValueError) as exc:
        raise ConfigError(f"config.json: {where}.{key} = {raw[key]!r} is not a {kind.__name__}") from exc


def _positive(value: float, what: str) -> float:
    if not value > 0 or not math.isfinite(value):
        raise ConfigError(f"config.json: {what} must be a positive number")
    return value


def _parse_mixer(raw: dict, where: str) -> dict:
    out = {k: _need(raw, k, int, where) for k in ("heads", "dim", "vdim")}
    out["kv_heads"] = _need(raw, "kv_heads", int, where) if raw.get("kv_heads") is not None else out["heads"]
    for k in ("heads", "kv_heads", "dim", "vdim"):
        if out[k] < 1:
            raise ConfigError(f"config.json: {where}.{k} must be at least 1")
    if out["heads"] % out["kv_heads"]:
        raise ConfigError(f"config.json: {where}.heads is not a multiple of kv_heads")
    if out["vdim"] != out["dim"]:
        raise ConfigError(f"config.json: {where}.vdim must equal dim (the values are the keys)")
    out["scale"] = _need(raw, "scale", float, where)
    rot = raw.get("rot") or {}
    out["rot_dims"] = int(rot.get("dims") or 0)
    out["rot_base"] = _positive(_need(rot, "base", float, where + ".rot"), where + ".rot.base") if out["rot_dims"] else 1.0
    if out["rot_dims"] < 0 or out["rot_dims"] % 2 or out["rot_dims"] > out["dim"]:
        raise ConfigError(f"config.json: {where}.rot.dims must be even and at most dim")
    out["softcap"] = _positive(float(raw["softcap"]), where + ".softcap") if raw.get("softcap") is not None else None
    mask = raw.get("mask") or {}
    out["window"] = int(mask["size"]) if mask.get("size") is not None else None
    out["keep_first"] = int(mask.get("keep_first") or 0) if out["window"] is not None else 0
    if out["window"] is not None and out["window"] < 1:
        raise ConfigError(f"config.json: {where}.mask.size must be at least 1")
    if out["keep_first"] < 0:
        raise ConfigError(f"config.json: {where}.mask.keep_first cannot be negative")
    return out


def _parse_mlp(raw, where: str):
    if raw is None:
        return None
    kind = _need(raw, "kind", str, where)
    if kind != "moe":
        raise ConfigError(f"config.json: {where}.kind = {kind!r} is not 'moe'")
    expert, router = raw.get("expert") or {}, raw.get("router") or {}
    groups = router.get("groups") or {}
    out = {"kind": "moe", "ff": _need(expert, "ff", int, where + ".expert"),
           "experts": _need(router, "experts", int, where + ".router"),
           "top": _need(router, "top", int, where + ".router"),
           "scale": float(router["scale"]) if router.get("scale") is not None else 1.0,
           "groups": int(groups.get("count") or 1), "keep": int(groups.get("keep") or groups.get("count") or 1)}
    if out["ff"] < 1 or out["experts"] < 1:
        raise ConfigError(f"config.json: {where} needs at least one expert of at least one unit")
    if out["groups"] < 1 or out["experts"] % out["groups"] or not 1 <= out["keep"] <= out["groups"]:
        raise ConfigError(f"config.json: {where}.router.groups: {out['experts']} experts cannot form "
                          f"{out['groups']} equal groups of which {out['keep']} are kept")
    if not 1 <= out["top"] <= out["keep"] * (out["experts"] // out["groups"]):
        raise ConfigError(f"config.json: {where}.router.top must be between 1 and the experts of the kept groups")
    return out


@dataclass(frozen=True)
class PuposunLayer:
    type: str
    mixer: dict
    mlp: dict | None


@dataclass(frozen=True)
class PuposunConfig:
    architecture: str
    vocab_size: int
    hidden_size: int
    max_position_embeddings: int
    norm_eps: float
    embedding_scale: float
    logit_softcap: float | None
    loop: tuple[int, int, int] | None  # (start, stop, times)
    layers: tuple[PuposunLayer, ...]
    eos_token_ids: tuple[int, ...] = ()
    torch_dtype: str = "bfloat16"

    @classmethod
    def from_dict(cls, raw: dict[str, Any]) -> "PuposunConfig":
        listed = raw.get("layers")
        if not isinstance(listed, list) or not listed:
            raise ConfigError("config.json: 'layers' must list at least one layer")
        layers = []
        for i, entry in enumerate(listed):
            where = f"layers[{i}]"
            kind = _need(entry, "type", str, where)
            if kind not in LAYER_TYPES:
                raise ConfigError(f"config.json: {where}.type = {kind!r} is not one of {LAYER_TYPES}")
            layers.append(PuposunLayer(kind, _parse_mixer(entry.get("mixer") or {}, where + ".mixer"),
                                       _parse_mlp(entry.get("mlp"), where + ".mlp")))
        loop = raw.get("loop")
        cap = raw.get("logit_softcap")
        cfg = cls(
            architecture=str(raw.get("architecture", NAME)),
            vocab_size=_need(raw, "vocab", int, "the model"),
            hidden_size=_need(raw, "width", int, "the model"),
            max_position_embeddings=int(raw.get("max_positions") or NO_POSITION_LIMIT),
            norm_eps=_need(raw.get("norm") or {}, "eps", float, "norm"),
            embedding_scale=float((raw.get("embedding") or {}).get("scale", 1.0)),
            logit_softcap=_positive(float(cap), "logit_softcap") if cap is not None else None,
            loop=(_need(loop, "start", int, "loop"), _need(loop, "stop", int, "loop"),
                  _need(loop, "times", int, "loop")) if loop else None,
            layers=tuple(layers),
            eos_token_ids=id_tuple(raw.get("eos_token_id")),
            torch_dtype=str(raw.get("torch_dtype", "bfloat16")),
        )
        for key in ("vocab_size", "hidden_size", "max_position_embeddings"):
            if getattr(cfg, key) < 1:
                raise ConfigError(f"config.json: {key} must be >= 1")
        _positive(cfg.norm_eps, "norm.eps")
        if not math.isfinite(cfg.embedding_scale):
            raise ConfigError("config.json: embedding.scale must be a number")
        if cfg.loop is not None:
            start, stop, times = cfg.loop
            if not 0 <= start <= stop <= len(layers) or times < 0:
                raise ConfigError("config.json: loop needs 0 <= start <= stop <= number of layers and times >= 0")
        return cfg

    def run_order(self) -> list[tuple[int, bool]]:
        """(layer, whether a pass of the loop after the first starts with it), in the order the layers run."""
        n = len(self.layers)
        if self.loop is None:
            return [(i, False) for i in range(n)]
        start, stop, times = self.loop
        order = [(i, False) for i in range(start)]
        for t in range(times):
            order += [(i, t > 0 and i == start) for i in range(start, stop)]
        return order + [(i, False) for i in range(stop, n)]


def _rotary_name(layer: PuposunLayer) -> str | None:
    m = layer.mixer
    if not m["rot_dims"]:
        return None
    return f"rot_{ROTARY_LAYOUT[layer.type]}_{m['rot_dims']}_{m['rot_base']!r}"


def _mixer_spec(cfg: PuposunConfig, i: int, layer: PuposunLayer) -> PartSpec:
    p, m = f"l{i}.mix", layer.mixer
    names = {"q": f"{p}.q", "k": f"{p}.k", "o": f"{p}.o"}
    params = {"heads": m["heads"], "kv_heads": m["kv_heads"], "dim": m["dim"], "vdim": m["vdim"],
              "scale": m["scale"], "values": "keys", "softcap": m["softcap"], "window": m["window"],
              "keep_first": m["keep_first"], "value_norm": False, "eps": cfg.norm_eps,
              "position": _rotary_name(layer)}
    if layer.type == "attention":
        names.update(q_bias=f"{p}.q.b", k_bias=f"{p}.k.b", o_bias=f"{p}.o.b")
        params["sink_value"] = 0.0  # one more term exp(0) in the softmax's denominator
    else:
        names["head_gate"] = f"{p}.g"
    return PartSpec("sink_attention", {"names": names, **params})


def _mlp_spec(i: int, mlp: dict | None) -> PartSpec | None:
    if mlp is None:
        return None
    p = f"l{i}.mlp"
    # experts: down(silu(gate(x)) * up(x)); nothing is clamped
    return PartSpec("routed_experts", {
        "router": f"{p}.router", "correction": f"{p}.correction", "expert_prefix": f"{p}.e",
        "experts": mlp["experts"], "top": mlp["top"], "groups": mlp["groups"], "keep_groups": mlp["keep"],
        "scoring": "sigmoid", "group_top": 2, "weight_scale": mlp["scale"],
        "intermediate_size": mlp["ff"], "limit": None, "alpha": 1.0, "up_offset": 0.0})


def puposun_spec(cfg: PuposunConfig) -> ModelSpec:
    layers, positions = [], {}
    for i, layer in enumerate(cfg.layers):
        name = _rotary_name(layer)
        if name is not None:
            positions.setdefault(name, PartSpec("rotary", {
                "rotary_dim": layer.mixer["rot_dims"], "theta": layer.mixer["rot_base"],
                "layout": ROTARY_LAYOUT[layer.type]}))
        layers.append(LayerSpec(prefix=f"l{i}", block=PartSpec("parallel_residual", {}),
                                mixer=_mixer_spec(cfg, i, layer), feed_forward=_mlp_spec(i, layer.mlp),
                                norms={"pre_mixer": PartSpec("rms", {"weight": f"l{i}.norm1", "eps": cfg.norm_eps})}))
    order = cfg.run_order()
    looped = any(again for _, again in order)
    head = {"weight": "head", "vocab_size": cfg.vocab_size}
    if cfg.logit_softcap is not None:
        head["softcap"] = cfg.logit_softcap
    return ModelSpec(
        architecture=cfg.architecture, vocab_size=cfg.vocab_size, hidden_size=cfg.hidden_size,
        max_position_embeddings=cfg.max_position_embeddings,
        embedding=PartSpec("token", {"weight": "embed", "vocab_size": cfg.vocab_size, "scale": cfg.embedding_scale}),
        positions=positions, layers=tuple(layers),
        schedule=tuple(ScheduleEntry(i, before="loop_in" if again else None) for i, again in order),
        final_norm=PartSpec("rms", {"weight": "final.norm", "eps": cfg.norm_eps}),
        head=PartSpec("linear", head), eos_token_ids=cfg.eos_token_ids,
        stream_parts={"loop_in": PartSpec("add_embedding", {})} if looped else {})


def puposun_footprint(cfg: PuposunConfig) -> Footprint:
    h = cfg.hidden_size
    params = cfg.vocab_size * h * 2 + h
    runs: dict[int, int] = {}
    for i, _ in cfg.run_order():
        runs[i] = runs.get(i, 0) + 1
    per_token = 0
    for i, layer in enumerate(cfg.layers):
        m = layer.mixer
        q, k = m["heads"] * m["dim"], m["kv_heads"] * m["dim"]
        params += h + (q + k) * h + h * m["heads"] * m["vdim"]
        params += (q + k + h) if layer.type == "attention" else m["heads"] * h
        per_token += runs.get(i, 0) * (k + m["kv_heads"] * m["vdim"])  # a rotated and a plain copy of the keys
        if layer.mlp is not None:
            params += layer.mlp["experts"] * (3 * layer.mlp["ff"] * h + h + 1)
    return Footprint(params, per_token, 0)


def describe_puposun(cfg: PuposunConfig) -> list[str]:
    kinds = [layer.type + ("" if layer.mlp is None else "+moe") for layer in cfg.layers]
    fp = puposun_footprint(cfg)
    windows = sorted({(layer.mixer["window"], layer.mixer["keep_first"]) for layer in cfg.layers
                      if layer.mixer["window"] is not None})
    loop = "none" if cfg.loop is None else f"layers {cfg.loop[0]}..{cfg.loop[1] - 1} x {cfg.loop[2]}"
    return [
        f"architecture        {cfg.architecture}",
        f"layers / width      {len(cfg.layers)} / {cfg.hidden_size}",
        f"layer kinds         {', '.join(kinds)}",
        f"loop                {loop}",
        f"attention windows   {', '.join(f'{w} (+ first {k})' for w, k in windows) if windows else 'none'}",
        f"parameters          {fp.parameters / 1e9:.3f} B",
        f"cache per token     {fp.cache_bytes_per_token(2)} B (bf16)",
    ]


register_architecture(NAME, PuposunConfig, puposun_spec, describe_puposun, puposun_footprint)
