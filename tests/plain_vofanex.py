"""A plain, slow, whole-sequence implementation of the Vofanex design, one function per mechanism.

Written from the design's equations only; it shares no code with the package.  Everything runs
in the dtype of the weights it is given (the tests pass 64-bit copies).  ``forward`` returns the
logits of every position of one sequence.
"""

from __future__ import annotations

import torch


def rms(x, eps):
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def embed(tokens, W, cfg):
    return W["embed"][torch.tensor(tokens)] * cfg["embedding"]["scale"]


def sink_window_softmax(scores, sink, window):
    """scores: [H, T, T] (query, key).  Position i sees j with 0 <= i - j < window; the denominator
    holds one more term exp(sink[h]) that has no value."""
    H, T, _ = scores.shape
    i = torch.arange(T)[:, None]
    j = torch.arange(T)[None, :]
    seen = (i - j >= 0) & (i - j < window)
    masked = scores.masked_fill(~seen, float("-inf"))
    top = torch.maximum(masked.max(-1).values, sink[:, None])  # [H, T]
    e = torch.exp(masked - top[..., None])
    return e / (e.sum(-1) + torch.exp(sink[:, None] - top))[..., None]


def attention(h, W, p, m, eps):
    """Grouped-query attention without rotation: biased projections, unit-RMS values, a window, a
    sink in the softmax and a gate per head."""
    T = h.shape[0]
    H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = (h @ W[p + ".q"].T + W[p + ".q.b"]).view(T, H, d)
    k = (h @ W[p + ".k"].T + W[p + ".k.b"]).view(T, G, d)
    v = rms((h @ W[p + ".v"].T + W[p + ".v.b"]).view(T, G, dv), eps)
    group = torch.arange(H) // (H // G)
    scores = torch.einsum("thd,shd->hts", q, k[:, group]) * m["scale"]
    window = (m.get("mask") or {}).get("size") or T  # (no mask: every earlier position is seen)
    weights = sink_window_softmax(scores, W[p + ".sink"], window)
    o = torch.einsum("hts,shv->thv", weights, v[:, group])
    gate = torch.sigmoid(h @ W[p + ".g"].T)  # [T, H]
    return (o * gate[..., None]).reshape(T, H * dv) @ W[p + ".o"].T


def gla_recurrence(q, k, v, alpha):
    """q, k, alpha: [T, H, d]; v: [T, H, dv].  S_t = diag(alpha_t) S_(t-1) + k_t v_t^T; o_t = S_t^T q_t."""
    T, H, d = q.shape
    S = q.new_zeros(H, d, v.shape[-1])
    out = []
    for t in range(T):
        S = alpha[t][:, :, None] * S + k[t][:, :, None] * v[t][:, None, :]
        out.append(torch.einsum("hdv,hd->hv", S, q[t]))
    return torch.stack(out)


def gla(h, W, p, m, eps):
    T = h.shape[0]
    H, d, dv = m["heads"], m["dim"], m["vdim"]
    q = (h @ W[p + ".q"].T).view(T, H, d) * d ** -0.5
    k = (h @ W[p + ".k"].T).view(T, H, d)
    v = (h @ W[p + ".v"].T).view(T, H, dv)
    z = (h @ W[p + ".a1"].T) @ W[p + ".a2"].T + W[p + ".a2.b"]
    alpha = torch.sigmoid(z).pow(1.0 / m["tau"]).view(T, H, d)
    o = rms(gla_recurrence(q, k, v, alpha), eps) * W[p + ".norm"]
    g = h @ W[p + ".g"].T
    return (o.reshape(T, H * dv) * (g * torch.sigmoid(g))) @ W[p + ".o"].T


def polynorm(z, coeff, eps):
    a, b, c, e = coeff
    return a * rms(z, eps) + b * rms(z ** 2, eps) + c * rms(z ** 3, eps) + e


def dense_ff(h, W, p, eps):
    return polynorm(h @ W[p + ".up"].T, W[p + ".act"], eps) @ W[p + ".down"].T


def route(h, W, p, top):
    """Chosen experts [T, top] and their weights: softmax over the chosen logits only."""
    z = h @ W[p + ".router"].T + W[p + ".router.b"]
    best = torch.topk(z, top, dim=-1)
    return best.indices, torch.softmax(best.values, dim=-1)


def expert(h, W, p):
    g = h @ W[p + ".gate"].T
    return ((g * torch.sigmoid(g)) * (h @ W[p + ".up"].T)) @ W[p + ".down"].T


def router_margin(h, W, p, top):
    """The smallest gap, over the tokens, between the last chosen logit and the best one not chosen
    (infinite when every expert is chosen): how far the choice is from a close call."""
    z = h @ W[p + ".router"].T + W[p + ".router.b"]
    if top >= z.shape[-1]:
        return float("inf")
    best = torch.topk(z, top + 1, dim=-1).values
    return float((best[:, top - 1] - best[:, top]).min())


def moe_ff(h, W, p, mlp, margins=None):
    if margins is not None:
        margins.append(router_margin(h, W, p, mlp["router"]["top"]))
    ids, weights = route(h, W, p, mlp["router"]["top"])
    out = torch.zeros_like(h)
    for t in range(h.shape[0]):
        for e, w in zip(ids[t].tolist(), weights[t]):
            out[t] += w * expert(h[t: t + 1], W, f"{p}.e{e}")[0]
    return out


def residual_gate(h, W, name):
    return torch.sigmoid(h @ W[name].T + W[name + ".b"])


def layer(x, W, i, entry, eps, margins=None):
    p = f"l{i}"
    h = rms(x, eps) * W[p + ".norm1"]
    mix = attention if entry["type"] == "attention" else gla
    x = x + residual_gate(h, W, p + ".rg1") * mix(h, W, p + ".mix", entry["mixer"], eps)
    mlp = entry.get("mlp")
    if mlp is None:
        return x
    h = rms(x, eps) * W[p + ".norm2"]
    y = dense_ff(h, W, p + ".mlp", eps) if mlp["kind"] == "dense" else moe_ff(h, W, p + ".mlp", mlp, margins)
    return x + residual_gate(h, W, p + ".rg2") * y


def forward(cfg, weights, tokens, dtype=torch.float64, layers_out=None, margins=None):
    W = {n: (t.to(dtype) if t.is_floating_point() else t) for n, t in weights.items()}
    eps = cfg["norm"]["eps"]
    x = embed(tokens, W, cfg)
    for i, entry in enumerate(cfg["layers"]):
        x = layer(x, W, i, entry, eps, margins)
        if layers_out is not None:
            layers_out.append(x.clone())
    return (rms(x, eps) * W["final.norm"]) @ W["head"].T
