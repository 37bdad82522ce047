"""Small Vofanex configurations and random weights for the tests.  Sizes are odd on purpose: head
counts that are not powers of two, several key/value heads, key and value sizes that differ,
windows of one position, of a few and wider than any prompt, an attention layer that comes first,
a layer without a feed-forward, experts of which one or all are used, ranks and taus that differ
from layer to layer, an embedding scale of one and of something else, nothing a multiple of four
where it need not be."""

from __future__ import annotations

import torch


def gla(heads, dim, vdim, tau=4.0):
    return "gla", {"heads": heads, "dim": dim, "vdim": vdim, "tau": tau}


def attention(heads, kv_heads, dim, vdim, window=None, scale=None):
    out = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim,
           "scale": dim ** -0.5 if scale is None else scale}
    if window:
        out["mask"] = {"size": window}
    return "attention", out


def dense(ff):
    return {"kind": "dense", "ff": ff}


def moe(experts, top, ff):
    return {"kind": "moe", "expert": {"ff": ff}, "router": {"experts": experts, "top": top}}


def config(width, vocab, layers, *, scale=1.7, eps=1e-5):
    return {"architecture": "Vofanex", "vocab": vocab, "width": width, "norm": {"eps": eps},
            "embedding": {"scale": scale},
            "layers": [{"type": t, "mixer": m, "mlp": f} for (t, m), f in layers]}


# the rank of each gla layer's decay map (the shape of its a1), by layer index
RANKS = {"mixed": {0: 5, 2: 3, 4: 9}, "attention_first": {1: 2, 3: 7}, "odd": {0: 1, 1: 4}, "wide": {0: 16, 2: 24}}

# recurrent and windowed layers in turn; grouped and ungrouped key/value heads; windows of 10 and 7
MIXED = config(72, 131, [
    (gla(3, 12, 20, tau=8.0), dense(40)),
    (attention(6, 2, 16, 24, window=10), moe(5, 2, 24)),
    (gla(2, 20, 8, tau=3.5), None),
    (attention(3, 3, 8, 12, window=7, scale=0.4), dense(56)),
    (gla(6, 4, 12, tau=1.0), moe(4, 1, 16)),
])
# attention first; a window wider than any prompt and one of a single position; every expert used
ATTENTION_FIRST = config(64, 97, [
    (attention(4, 2, 16, 8, window=500), dense(96)),
    (gla(2, 16, 16, tau=12.0), moe(3, 3, 20)),
    (attention(2, 1, 24, 40, window=1), None),
    (gla(4, 8, 8, tau=2.0), dense(32)),
], scale=1.0)
# nothing a multiple of four: sizes the kernels' 16-byte paths do not take
ODD = config(50, 61, [
    (gla(1, 5, 3, tau=5.0), moe(7, 3, 9)),
    (gla(5, 6, 10, tau=2.5), dense(30)),
    (attention(5, 5, 6, 10, window=13), dense(22)),
    (attention(3, 1, 10, 6), moe(2, 1, 14)),  # no window: every earlier position is seen
], scale=0.5)
# sizes the bfloat16 tensor-core kernels take, windows that span several tiles and pages of 16
WIDE = config(128, 211, [
    (gla(4, 32, 64, tau=20.0), dense(192)),
    (attention(8, 2, 64, 32, window=100), moe(8, 2, 64)),
    (gla(2, 64, 32, tau=6.0), dense(160)),
    (attention(4, 4, 32, 64, window=40), dense(128)),
    (attention(6, 3, 128, 128, window=257), None),
], scale=2.0)

CONFIGS = {"mixed": MIXED, "attention_first": ATTENTION_FIRST, "odd": ODD}
ALL_CONFIGS = dict(CONFIGS, wide=WIDE)


def name_of(cfg: dict) -> str:
    return next(n for n, c in ALL_CONFIGS.items() if c is cfg)


def tensor_shapes(cfg: dict, ranks: dict[int, int]) -> dict[str, tuple[int, ...]]:
    h = cfg["width"]
    shapes = {"embed": (cfg["vocab"], h), "final.norm": (h,), "head": (cfg["vocab"], h)}
    for i, layer in enumerate(cfg["layers"]):
        p, m = f"l{i}", layer["mixer"]
        shapes[f"{p}.norm1"] = (h,)
        shapes[f"{p}.rg1"], shapes[f"{p}.rg1.b"] = (h, h), (h,)
        if layer["type"] == "gla":
            qk, v, r = m["heads"] * m["dim"], m["heads"] * m["vdim"], ranks[i]
            shapes.update({f"{p}.mix.q": (qk, h), f"{p}.mix.k": (qk, h), f"{p}.mix.v": (v, h), f"{p}.mix.g": (v, h),
                           f"{p}.mix.o": (h, v), f"{p}.mix.norm": (m["vdim"],), f"{p}.mix.a1": (r, h),
                           f"{p}.mix.a2": (qk, r), f"{p}.mix.a2.b": (qk,)})
        else:
            q, k, v = m["heads"] * m["dim"], m["kv_heads"] * m["dim"], m["kv_heads"] * m["vdim"]
            shapes.update({f"{p}.mix.q": (q, h), f"{p}.mix.q.b": (q,), f"{p}.mix.k": (k, h), f"{p}.mix.k.b": (k,),
                           f"{p}.mix.v": (v, h), f"{p}.mix.v.b": (v,), f"{p}.mix.sink": (m["heads"],),
                           f"{p}.mix.g": (m["heads"], h), f"{p}.mix.o": (h, m["heads"] * m["vdim"])})
        mlp = layer["mlp"]
        if mlp is None:
            continue
        shapes[f"{p}.norm2"] = (h,)
        shapes[f"{p}.rg2"], shapes[f"{p}.rg2.b"] = (h, h), (h,)
        if mlp["kind"] == "dense":
            shapes.update({f"{p}.mlp.up": (mlp["ff"], h), f"{p}.mlp.down": (h, mlp["ff"]), f"{p}.mlp.act": (4,)})
        else:
            ff, n = mlp["expert"]["ff"], mlp["router"]["experts"]
            shapes[f"{p}.mlp.router"], shapes[f"{p}.mlp.router.b"] = (n, h), (n,)
            for e in range(n):
                shapes.update({f"{p}.mlp.e{e}.gate": (ff, h), f"{p}.mlp.e{e}.up": (ff, h),
                               f"{p}.mlp.e{e}.down": (h, ff)})
    return shapes


def make_weights(cfg: dict, seed: int = 0, ranks: dict[int, int] | None = None) -> dict:
    """Random weights, stored as bfloat16 values.  Matrices are N(0, 1/sqrt(fan-in)); norm weights
    around one.  Query and key projections are scaled up so that attention is peaked (with flat
    attention a lost key moves the output by one part in dozens and hides in the tolerance); sinks
    are of the scores' size, so that leaving one out moves the weights; the decays' biases are
    positive and their maps small, so that the states forget slowly and early tokens matter; router
    biases and logits are spread so that the chosen experts are not a close call."""
    ranks = RANKS[name_of(cfg)] if ranks is None else ranks
    g = torch.Generator().manual_seed(seed)
    out = {}
    for name, shape in tensor_shapes(cfg, ranks).items():
        last = name.rsplit(".", 1)[-1]
        if name.endswith(("norm1", "norm2", "final.norm", "mix.norm")):
            t = 1.0 + 0.1 * torch.randn(shape, generator=g)
        elif name.endswith("mlp.act"):
            t = torch.tensor([0.9, 0.4, -0.3, 0.1]) + 0.1 * torch.randn(shape, generator=g)
        elif name.endswith("mix.sink"):
            t = 1.0 + torch.randn(shape, generator=g)
        elif name.endswith("a2.b"):
            t = 2.5 + torch.randn(shape, generator=g)
        elif name.endswith("router.b"):
            t = torch.randn(shape, generator=g)
        elif last == "b":
            t = 0.3 * torch.randn(shape, generator=g)
        elif name in ("embed",):
            t = torch.randn(shape, generator=g)
        else:
            t = torch.randn(shape, generator=g) / shape[-1] ** 0.5
            if name.endswith(("mix.q", "mix.k")):
                t = t * 2.5
            if name.endswith("mlp.router"):
                t = t * 3.0
        out[name] = t.to(torch.bfloat16)
    return out
