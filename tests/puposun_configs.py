"""Small Puposun configurations and random weights for the tests.  Sizes are odd on purpose: head
counts that are not powers of two, one, several and as many key/value heads as query heads, rotations
of a part of a head, of all of it and none, windows of one position, of a few and wider than any
prompt, more kept first positions than the window holds and none, a layer without a feed-forward,
routers without groups, with all groups kept and with some, one expert per token and all of them,
loops that start at the first layer, end at the last, run once, or are absent, capped and uncapped
scores and logits, nothing a multiple of four where it need not be."""

from __future__ import annotations

import torch


def attention(heads, kv_heads, dim, rot=None, base=10000.0, softcap=None, scale=None):
    out = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": dim,
           "scale": dim ** -0.5 if scale is None else scale}
    if rot:
        out["rot"] = {"dims": rot, "base": base}
    if softcap:
        out["softcap"] = softcap
    return "attention", out


def attention_2(heads, kv_heads, dim, rot=None, base=10000.0, window=None, keep_first=0, scale=None):
    out = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": dim,
           "scale": dim ** -0.5 if scale is None else scale}
    if rot:
        out["rot"] = {"dims": rot, "base": base}
    if window:
        out["mask"] = {"size": window, "keep_first": keep_first}
    return "attention_2", out


def moe(experts, top, ff, groups=1, keep=1, scale=1.0):
    router = {"experts": experts, "top": top, "scale": scale}
    if groups > 1:
        router["groups"] = {"count": groups, "keep": keep}
    return {"kind": "moe", "expert": {"ff": ff}, "router": router}


def config(width, vocab, layers, *, scale=1.7, eps=1e-5, loop=None, logit_softcap=None):
    out = {"architecture": "Puposun", "vocab": vocab, "width": width, "norm": {"eps": eps},
           "embedding": {"scale": scale},
           "layers": [{"type": t, "mixer": m, "mlp": f} for (t, m), f in layers]}
    if loop:
        out["loop"] = dict(zip(("start", "stop", "times"), loop))
    if logit_softcap:
        out["logit_softcap"] = logit_softcap
    return out


# both kinds of attention in turn, the middle two layers looped twice; grouped, ungrouped and single
# key/value heads; a rotation of half a head, of a whole one, of a third and none
MIXED = config(72, 131, [
    (attention(6, 2, 16, rot=8, softcap=5.0), moe(8, 2, 24, groups=4, keep=2, scale=1.5)),
    (attention_2(3, 3, 8, rot=8, window=10, keep_first=3), moe(5, 1, 16)),
    (attention_2(4, 1, 12, rot=4, base=500.0, window=7), None),
    (attention(2, 2, 20, scale=0.3), moe(6, 3, 20, groups=2, keep=1)),
], loop=(1, 3, 2), logit_softcap=12.0)
# nothing a multiple of four; more kept positions than the window holds; every expert used; an
# attention_2 layer without a window (every earlier position is seen); no loop, logits not capped
ODD = config(50, 61, [
    (attention_2(5, 5, 6, rot=6, window=13, keep_first=17), moe(7, 7, 9)),
    (attention(3, 1, 10, rot=10, softcap=50.0), None),
    (attention_2(2, 1, 14), moe(4, 2, 14, groups=2, keep=2, scale=0.5)),
], scale=0.5)
# the loop starts at the first layer and runs three times; a window of one position beside two kept
# ones; a window wider than any prompt; an embedding scale of one
LOOP_FIRST = config(64, 97, [
    (attention(4, 2, 16, rot=16, softcap=8.0), moe(4, 2, 20, groups=2, keep=1, scale=2.2)),
    (attention_2(4, 4, 16, rot=2, window=1, keep_first=2), moe(3, 1, 12)),
    (attention_2(2, 2, 8, rot=8, window=500, keep_first=4), None),
], scale=1.0, loop=(0, 2, 3), logit_softcap=25.0)
# the loop ends with the last layer and runs once (nothing is added again)
LOOP_LAST = config(48, 83, [
    (attention_2(2, 1, 24, rot=12, window=9, keep_first=1), moe(6, 2, 10, groups=3, keep=2)),
    (attention(3, 3, 16, rot=4, base=77.0), moe(2, 1, 18)),
], loop=(1, 2, 1), logit_softcap=6.0)
# sizes the bfloat16 tensor-core kernels take, windows that span several tiles and pages of 16, kept
# positions that fill more than a tile of 64 keys
WIDE = config(128, 211, [
    (attention(8, 2, 64, rot=32, softcap=15.0), moe(8, 2, 64, groups=4, keep=2, scale=2.0)),
    (attention_2(4, 4, 32, rot=32, window=100, keep_first=5), moe(8, 3, 32, groups=2, keep=1)),
    (attention_2(6, 3, 128, rot=64, base=2e5, window=257, keep_first=70), None),
    (attention(4, 1, 48, rot=48, base=3e4, softcap=30.0), moe(4, 1, 48)),
], scale=2.0, loop=(1, 3, 2), logit_softcap=20.0)

CONFIGS = {"mixed": MIXED, "odd": ODD, "loop_first": LOOP_FIRST, "loop_last": LOOP_LAST}
ALL_CONFIGS = dict(CONFIGS, wide=WIDE)


def tensor_shapes(cfg: dict) -> dict[str, tuple[int, ...]]:
    h = cfg["width"]
    shapes = {"embed": (cfg["vocab"], h), "final.norm": (h,), "head": (cfg["vocab"], h)}
    for i, layer in enumerate(cfg["layers"]):
        p, m = f"l{i}", layer["mixer"]
        q, k = m["heads"] * m["dim"], m["kv_heads"] * m["dim"]
        shapes[f"{p}.norm1"] = (h,)
        shapes.update({f"{p}.mix.q": (q, h), f"{p}.mix.k": (k, h), f"{p}.mix.o": (h, m["heads"] * m["vdim"])})
        if layer["type"] == "attention":
            shapes.update({f"{p}.mix.q.b": (q,), f"{p}.mix.k.b": (k,), f"{p}.mix.o.b": (h,)})
        else:
            shapes[f"{p}.mix.g"] = (m["heads"], h)
        mlp = layer["mlp"]
        if mlp is None:
            continue
        ff, n = mlp["expert"]["ff"], mlp["router"]["experts"]
        shapes[f"{p}.mlp.router"], shapes[f"{p}.mlp.correction"] = (n, h), (n,)
        for e in range(n):
            shapes.update({f"{p}.mlp.e{e}.gate": (ff, h), f"{p}.mlp.e{e}.up": (ff, h), f"{p}.mlp.e{e}.down": (h, ff)})
    return shapes


def make_weights(cfg: dict, seed: int = 0) -> dict:
    """Random weights, stored as bfloat16 values.  Matrices are N(0, 1/sqrt(fan-in)); norm weights
    around one.  Query and key projections are scaled up so that attention is peaked (with flat
    attention a lost key moves the output by one part in dozens and hides in the tolerance) and the
    capped scores do reach the cap's bend; the routers' logits are spread and their corrections are
    as large as the differences between scores, so that the correction decides who is chosen and the
    choice is not a close call; the biases are of the projections' size."""
    g = torch.Generator().manual_seed(seed)
    out = {}
    for name, shape in tensor_shapes(cfg).items():
        last = name.rsplit(".", 1)[-1]
        if last in ("norm1", "norm"):
            t = 1.0 + 0.1 * torch.randn(shape, generator=g)
        elif last == "correction":
            t = 0.4 * torch.randn(shape, generator=g)
        elif last == "b":
            t = 0.3 * torch.randn(shape, generator=g)
        elif name == "embed":
            t = torch.randn(shape, generator=g)
        else:
            t = torch.randn(shape, generator=g) / shape[-1] ** 0.5
            if name.endswith(("mix.q", "mix.k")):
                t = t * 2.5
            if name.endswith(("mlp.router", "mix.g")):
                t = t * 3.0
        out[name] = t.to(torch.bfloat16)
    return out
