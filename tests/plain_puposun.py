"""A plain, slow Puposun in PyTorch (64-bit unless asked otherwise): whole sequences, no cache, one
function per mechanism.

The oracle of the Puposun tests.  It shares no code with the engine: it takes the configuration as
the dictionary ``config.json`` holds and the tensors by their stored names.

The model: ``x = embed[token] * embedding.scale``.  Layers ``loop.start .. loop.stop - 1`` run
``loop.times`` times in a row with the same weights; before every pass but the first the embedding's
output is added to ``x``.  A layer is parallel: with ``h = rms(x) * norm1``,
``x <- x + mixer(h) + feed_forward(h)``.  Mixers: ``attention`` (values are the unrotated keys,
rotate-half rotation, capped scores, a zero sink in the softmax, biases) and ``attention_2`` (values
are the unrotated keys, interleaved rotation, a sliding window that also keeps the first tokens, a
sigmoid gate per head).  The feed-forward is a mixture of gated experts with sigmoid scores, a
correction that only steers the choice, and groups scored by their two best experts.  The logits
are capped by ``c * tanh(logits / c)``.
"""

from __future__ import annotations

import torch


def rms_norm(x, weight, eps):
    y = x / torch.sqrt(x.pow(2).mean(-1, keepdim=True) + eps)
    return y if weight is None else y * weight


def rotate(x, positions, dims, base, layout):
    """x: [T, heads, dim]; the first ``dims`` entries of every head are rotated by the position."""
    if not dims:
        return x
    half = dims // 2
    i = torch.arange(half, dtype=x.dtype)
    freq = torch.pow(torch.tensor(float(base), dtype=x.dtype), -2.0 * i / dims)
    ang = positions.to(x.dtype)[:, None] * freq[None, :]
    cos, sin = ang.cos()[:, None, :], ang.sin()[:, None, :]
    out = x.clone()
    if layout == "halves":
        u, v = x[..., :half], x[..., half:dims]
        out[..., :half] = u * cos - v * sin
        out[..., half:dims] = v * cos + u * sin
    else:
        u, v = x[..., 0:dims:2], x[..., 1:dims:2]
        out[..., 0:dims:2] = u * cos - v * sin
        out[..., 1:dims:2] = v * cos + u * sin
    return out


def visible(T, window=None, keep_first=0):
    """[T, T] mask: query i sees key j <= i if i - j < window or j < keep_first."""
    i = torch.arange(T)[:, None]
    j = torch.arange(T)[None, :]
    ok = j <= i
    if window is not None:
        ok = ok & ((i - j < window) | (j < keep_first))
    return ok


def attention_core(q, k, v, scale, mask, softcap=None, sink=False):
    """q: [T, H, d], k: [T, G, d], v: [T, G, dv] -> [T, H, dv]."""
    T, H, _ = q.shape
    G = k.shape[1]
    rep = H // G
    out = torch.zeros(T, H, v.shape[-1], dtype=q.dtype)
    for h in range(H):
        g = h // rep
        s = (q[:, h] @ k[:, g].T) * scale
        if softcap is not None:
            s = softcap * torch.tanh(s / softcap)
        s = s.masked_fill(~mask, float("-inf"))
        if sink:
            m = torch.clamp(s.max(-1, keepdim=True).values, min=0.0)
            e = torch.exp(s - m)
            p = e / (torch.exp(-m) + e.sum(-1, keepdim=True))
        else:
            p = torch.softmax(s, dim=-1)
        out[:, h] = p @ v[:, g]
    return out


def mixer_attention(w, p, h, m):
    """Rotate-half rotation, capped scores, zero sink, biases; the values are the unrotated keys."""
    T = h.shape[0]
    H, G, d = m["heads"], m["kv_heads"], m["dim"]
    q = (h @ w[p + ".q"].T + w[p + ".q.b"]).view(T, H, d)
    k = (h @ w[p + ".k"].T + w[p + ".k.b"]).view(T, G, d)
    v = k
    pos = torch.arange(T)
    rot = m.get("rot") or {}
    q = rotate(q, pos, rot.get("dims", 0), rot.get("base", 1.0), "halves")
    kr = rotate(k, pos, rot.get("dims", 0), rot.get("base", 1.0), "halves")
    o = attention_core(q, kr, v, m["scale"], visible(T), m.get("softcap"), sink=True)
    return o.reshape(T, -1) @ w[p + ".o"].T + w[p + ".o.b"]


def mixer_attention_2(w, p, h, m):
    """Interleaved rotation, window with kept first tokens, a gate per head; values are the unrotated keys."""
    T = h.shape[0]
    H, G, d = m["heads"], m["kv_heads"], m["dim"]
    q = (h @ w[p + ".q"].T).view(T, H, d)
    k = (h @ w[p + ".k"].T).view(T, G, d)
    v = k
    pos = torch.arange(T)
    rot = m.get("rot") or {}
    q = rotate(q, pos, rot.get("dims", 0), rot.get("base", 1.0), "interleaved")
    kr = rotate(k, pos, rot.get("dims", 0), rot.get("base", 1.0), "interleaved")
    mask_cfg = m.get("mask") or {}
    mask = visible(T, mask_cfg.get("size"), mask_cfg.get("keep_first", 0))
    o = attention_core(q, kr, v, m["scale"], mask)
    gate = torch.sigmoid(h @ w[p + ".g"].T)  # [T, H]
    o = o * gate[:, :, None]
    return o.reshape(T, -1) @ w[p + ".o"].T


def route(w, p, h, mlp, margins=None):
    """(ids [T, top], weights [T, top]) of the mixture's router.  ``margins``: a list that receives, per
    token, how far the last chosen expert's corrected score is above the best one that was not chosen,
    and how far the last kept group's score is above the best one that was dropped."""
    r = mlp["router"]
    E, top = r["experts"], r["top"]
    groups = r.get("groups") or {"count": 1, "keep": 1}
    s = torch.sigmoid(h @ w[p + ".router"].T)
    choice = s + w[p + ".correction"]
    per = E // groups["count"]
    if groups["keep"] < groups["count"]:
        by_group = choice.view(-1, groups["count"], per)
        gscore = by_group.topk(min(2, per), dim=-1).values.sum(-1)
        kept = gscore.topk(groups["keep"], dim=-1).indices
        if margins is not None:
            ranked = gscore.sort(-1, descending=True).values
            margins.extend((ranked[:, groups["keep"] - 1] - ranked[:, groups["keep"]]).tolist())
        allowed = torch.zeros_like(gscore, dtype=torch.bool).scatter_(1, kept, True)
        choice = choice.masked_fill(~allowed[:, :, None].expand(-1, -1, per).reshape(-1, E), float("-inf"))
    ids = choice.topk(top, dim=-1).indices
    if margins is not None and top < (choice > float("-inf")).sum(-1).min():
        ranked = choice.sort(-1, descending=True).values
        margins.extend((ranked[:, top - 1] - ranked[:, top]).tolist())
    picked = s.gather(1, ids)
    weights = picked / (picked.sum(-1, keepdim=True) + 1e-20) * r["scale"]
    return ids, weights


def feed_forward_moe(w, p, h, mlp, margins=None):
    ids, weights = route(w, p, h, mlp, margins)
    out = torch.zeros(h.shape[0], w[p + ".e0.down"].shape[0], dtype=h.dtype)
    for t in range(h.shape[0]):
        for j in range(ids.shape[1]):
            e = int(ids[t, j])
            g = h[t] @ w[f"{p}.e{e}.gate"].T
            u = h[t] @ w[f"{p}.e{e}.up"].T
            out[t] += weights[t, j] * ((torch.nn.functional.silu(g) * u) @ w[f"{p}.e{e}.down"].T)
    return out


def run_order(cfg):
    """(layer, whether a later pass of the loop starts with it) in the order the layers run."""
    n = len(cfg["layers"])
    loop = cfg.get("loop")
    if not loop:
        return [(i, False) for i in range(n)]
    start, stop, times = loop["start"], loop["stop"], loop["times"]
    order = [(i, False) for i in range(start)]
    for t in range(times):
        order += [(i, t > 0 and i == start) for i in range(start, stop)]
    return order + [(i, False) for i in range(stop, n)]


def forward(cfg, w, tokens, dtype=torch.float64, return_layers=False, margins=None):
    """Logits [T, vocab] of a whole sequence (and the stream after every layer run)."""
    tokens = torch.as_tensor(tokens, dtype=torch.long)
    w = {k: v.to(dtype) for k, v in w.items()}
    x0 = w["embed"][tokens] * float((cfg.get("embedding") or {}).get("scale", 1.0))
    x = x0.clone()
    eps = cfg["norm"]["eps"]
    seen = []
    for i, again in run_order(cfg):
        layer = cfg["layers"][i]
        if again:
            x = x + x0
        h = rms_norm(x, w[f"l{i}.norm1"], eps)
        mix = (mixer_attention if layer["type"] == "attention" else mixer_attention_2)(w, f"l{i}.mix", h, layer["mixer"])
        if layer.get("mlp") is not None:
            mix = mix + feed_forward_moe(w, f"l{i}.mlp", h, layer["mlp"], margins)
        x = x + mix
        seen.append(x.clone())
    logits = rms_norm(x, w["final.norm"], eps) @ w["head"].T
    cap = cfg.get("logit_softcap")
    if cap:
        logits = cap * torch.tanh(logits / cap)
    return (logits, torch.stack(seen)) if return_layers else logits
