"""The Puposun design in the engine against the plain whole-sequence implementation
(`tests/plain_puposun.py`): whole prompts, token-by-token decoding, portions down to two tokens,
mixed batches with pages and slots used again, configurations of odd sizes; every mechanism alone
against its plain function, with inputs made so that a key just inside or just outside a window, a
kept first key, a sink that is left out, a cap that is not applied or a wrong expert shows; on the
CPU through the plain stand-ins of the kernels, on the GPU through the kernels in both precisions;
long decoding; greedy generation through the engine's own entry point and scheduler."""

from __future__ import annotations

from types import SimpleNamespace

import pytest
import torch

from tests import helpers as H
from tests import plain_puposun as P
from tests import puposun_configs as V

LENGTHS = [50, 21, 37, 64, 9, 1]
BF16_TOL = dict(atol=0.35, rtol=0.0, pos_rel_rms=0.08, rel_rms=0.04)
# (under these names the run's summary lists this file's comparisons: their bounds are measured)
LABEL = {"float32": "float32, Puposun", "bfloat16": "bfloat16, Puposun"}
DEVICES = ["cpu", pytest.param("cuda", marks=pytest.mark.gpu)]
D = torch.float64


def _requests(cfg, lengths=LENGTHS, seed=700):
    return {f"r{i}": torch.randint(0, cfg["vocab"], (n,), generator=torch.Generator().manual_seed(seed + i)).tolist()
            for i, n in enumerate(lengths)}


def _want(cfg, weights, requests):
    return {rid: P.forward(cfg, weights, toks, D).float() for rid, toks in requests.items()}


def _float32_bound(cfg, weights, requests, want) -> dict:
    """Three times what rounding alone does to the plain implementation when it runs in 32-bit
    instead of 64-bit, and never below the engine's fixed bound for tiny models.  A lost key, a
    window that is one off or a sink left out moves logits by 1e-2 and more."""
    worst = max(float((P.forward(cfg, weights, toks, torch.float32) - want[rid]).abs().max())
                for rid, toks in requests.items())
    return dict(atol=max(3 * worst, H.TOL["float32"]["atol"]), rtol=H.TOL["float32"]["rtol"])


def _bfloat16_bound(tmp_path, cfg, weights, requests, want) -> dict:
    """Three times what rounding does to the same requests on the plain stand-ins of the kernels run
    in bfloat16 (activations rounded between the parts, as the kernels round them), and never below
    the fixed bounds."""
    from tests.ref_ops import RefOps

    room = sum(H.round64(len(t)) for t in requests.values())
    got = H.collect(_session(tmp_path / "bound", cfg, weights, "bfloat16", "cpu", RefOps(), room, 16),
                    H.trace_whole(requests))
    tol = dict(BF16_TOL)
    for rid in requests:
        diff = (got[rid].double() - want[rid].double()).abs()
        pos_rel = diff.pow(2).mean(-1).sqrt() / want[rid].double().pow(2).mean(-1).sqrt().clamp_min(1e-12)
        rel = float(diff.pow(2).mean().sqrt() / want[rid].double().pow(2).mean().sqrt())
        tol["atol"] = max(tol["atol"], 3 * float(diff.max()))
        tol["pos_rel_rms"] = max(tol["pos_rel_rms"], 3 * float(pos_rel.max()))
        tol["rel_rms"] = max(tol["rel_rms"], 3 * rel)
    return tol


def _bound(tmp_path, dtype, cfg, weights, requests, want):
    return (_float32_bound(cfg, weights, requests, want) if dtype == "float32"
            else _bfloat16_bound(tmp_path, cfg, weights, requests, want))


def _session(tmp_path, cfg, weights, dtype, device, ops, max_tokens, page_size):
    from inference_engine_b200.engine.replay import ReplaySession

    folder = H.write_model_dir(tmp_path / f"m{abs(hash(str(cfg))) % 10**8}", cfg, weights)
    return ReplaySession(folder, dtype, max_tokens, device=device, ops=ops, page_size=page_size)


def _run_all_modes(tmp_path, name, dtype, device, ops, page_size=4, lengths=LENGTHS):
    cfg = V.ALL_CONFIGS[name]
    weights = V.make_weights(cfg, seed=11)
    requests = _requests(cfg, lengths)
    want = _want(cfg, weights, requests)
    tol = _bound(tmp_path, dtype, cfg, weights, requests, want)
    mixed, peak = H.trace_mixed(requests, seed=5, tail=7, max_portion=15)
    whole_room = sum(H.round64(len(t)) for t in requests.values())
    results = {}
    for mode, (trace, room) in {"whole": (H.trace_whole(requests), whole_room),
                                "tail": (H.trace_decode_tail(requests, 14), whole_room),
                                "portions": (H.trace_portions(requests, (5, 2, 13, 3, 2, 8)), whole_room),
                                "mixed": (mixed, peak)}.items():
        session = _session(tmp_path, cfg, weights, dtype, device, ops, room, page_size)
        got = H.collect(session, trace)
        for rid in requests:
            H.assert_close(got[rid], want[rid], LABEL[dtype], f"puposun {name} {mode} {rid}", tol)
        # everything went back to the pools
        assert session.cache.num_free_pages == [p.num_pages for p in session.cache.pools]
        assert session.cache.slots.num_free == session.cache.slots.num_slots
        results[mode] = got
    return results


def test_the_test_weights_make_no_close_call_in_the_routers():
    """The groups and experts the plain implementation chooses are chosen by a margin that rounding
    does not reach, so a difference in the logits is a fault and not another expert."""
    for name, cfg in V.CONFIGS.items():
        weights = V.make_weights(cfg, seed=11)
        margins = []
        for toks in _requests(cfg, [30, 13, 21, 9, 1]).values():
            P.forward(cfg, weights, toks, D, margins=margins)
        assert margins and min(margins) > 1e-4, name


@pytest.mark.parametrize("name", list(V.CONFIGS))
def test_every_way_of_cutting_on_the_plain_kernels(tmp_path, name):
    from tests.ref_ops import RefOps

    _run_all_modes(tmp_path, name, "float32", "cpu", RefOps(), lengths=[30, 13, 21, 9, 1])


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", list(V.CONFIGS))
def test_every_way_of_cutting_on_the_gpu(tmp_path, name, dtype):
    from inference_engine_b200.kernels import get_ops

    results = _run_all_modes(tmp_path, name, dtype, "cuda", get_ops("cuda"), lengths=[150, 21, 67, 64, 9, 1, 33])
    if dtype == "float32":  # a row's arithmetic does not depend on the cutting or the batch at all
        for mode in ("tail", "portions", "mixed"):
            for rid, rows in results["whole"].items():
                assert torch.equal(rows, results[mode][rid]), f"{name} {mode} {rid}: 32-bit logits differ by cutting"
    get_ops("cuda").check_errors()


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_a_wider_model_with_long_prompts(tmp_path, dtype):
    """Prompts of hundreds of tokens over several windows and many pages of 16, sizes that reach the
    tensor-core attention in bfloat16, kept first positions that fill more than a tile of keys."""
    from inference_engine_b200.kernels import get_ops

    cfg = V.WIDE
    weights = V.make_weights(cfg, seed=21)
    requests = _requests(cfg, [420, 130, 257, 64], seed=900)
    want = _want(cfg, weights, requests)
    tol = _bound(tmp_path, dtype, cfg, weights, requests, want)
    mixed, peak = H.trace_mixed(requests, seed=8, tail=20, max_portion=90)
    room = sum(H.round64(len(t)) for t in requests.values())
    before = dict(get_ops("cuda").launch_counts)
    results = {}
    for mode, (trace, space) in {"whole": (H.trace_whole(requests), room),
                                 "tail": (H.trace_decode_tail(requests, 40), room),
                                 "portions": (H.trace_portions(requests, (70, 2, 129, 3, 64, 33)), room),
                                 "mixed": (mixed, peak)}.items():
        session = _session(tmp_path / mode, cfg, weights, dtype, "cuda", get_ops("cuda"), space, 16)
        results[mode] = H.collect(session, trace)
        for rid in requests:
            H.assert_close(results[mode][rid], want[rid], LABEL[dtype], f"wide {mode} {rid}", tol)
        assert session.cache.num_free_pages == [p.num_pages for p in session.cache.pools]
    ran = get_ops("cuda").launch_counts.get("sink_attention_mma", 0) - before.get("sink_attention_mma", 0)
    if dtype == "float32":
        assert ran == 0
        for mode in ("tail", "portions", "mixed"):
            for rid in requests:
                assert torch.equal(results["whole"][rid], results[mode][rid]), (mode, rid)
    else:
        assert ran > 0  # (the tensor-core kernel did serve these sizes)
    get_ops("cuda").check_errors()


# --- what the model is made of ---------------------------------------------------------------------


def test_layout_of_the_model_and_its_caches():
    from inference_engine_b200.config import build_model_spec, config_from_dict
    from inference_engine_b200.engine.model import Model

    spec = build_model_spec(config_from_dict(V.MIXED))
    model = Model(spec, "float32", 64)
    assert [type(b).__name__ for b in model.blocks] == ["ParallelResidualBlock"] * 4
    assert [type(b.mixer).__name__ for b in model.blocks] == ["SinkAttention"] * 4
    assert [type(b.feed_forward).__name__ for b in model.blocks] == [
        "RoutedExperts", "RoutedExperts", "NoneType", "RoutedExperts"]
    # layers 1 and 2 run twice; the second pass starts by adding the embedding's output again
    assert [(e.layer, e.before) for e in spec.schedule] == [
        (0, None), (1, None), (2, None), (1, "loop_in"), (2, None), (3, None)]
    assert model.keeps_embedding
    # every run of a layer has a cache slot of its own in its group
    assert len({(b.group, b.slot) for b in model.bindings}) == 6
    groups = sorted((g.num_kv_heads, g.head_dim, g.value_dim, g.window, g.keep_first, g.num_layers)
                    for g in model.paged_groups)
    assert groups == [(1, 12, 12, 7, 0, 2), (2, 16, 16, None, 0, 1), (2, 20, 20, None, 0, 1), (3, 8, 8, 10, 3, 2)]
    assert not model.state_groups
    first, second = model.blocks[0].mixer, model.blocks[1].mixer
    assert first.values_from_keys and first.softcap == 5.0 and first.sink_value == 0.0 and first.position.layout == "halves"
    assert second.softcap is None and second.sink_value is None and second.position.layout == "interleaved"
    assert (second.window, second.keep_first) == (10, 3) and second.position.rotary_dim == 8
    assert model.blocks[3].mixer.position is None  # (a layer whose configuration names no rotation)
    router = model.blocks[0].feed_forward
    assert (router.scoring, router.group_top, router.groups, router.keep_groups, router.weight_scale) == ("sigmoid", 2, 4, 2, 1.5)
    assert model.head.softcap == 12.0 and model.embedding.scale == 1.7
    assert set(model.declared_weights()) == set(V.tensor_shapes(V.MIXED))
    # no loop, or one that runs once: nothing is added again, and the embedding's output is not kept
    for raw in (V.ODD, V.LOOP_LAST):
        plain = Model(build_model_spec(config_from_dict(raw)), "float32", 64)
        assert not plain.keeps_embedding and not plain.stream_parts
    assert Model(build_model_spec(config_from_dict(V.ODD)), "float32", 64).head.softcap is None


@pytest.mark.parametrize("name", list(V.ALL_CONFIGS))
def test_footprint_formula_counts_what_the_model_declares(name):
    from inference_engine_b200.architectures.puposun import puposun_footprint
    from inference_engine_b200.config import build_model_spec, config_from_dict
    from inference_engine_b200.engine.model import Model

    cfg = config_from_dict(V.ALL_CONFIGS[name])
    assert puposun_footprint(cfg) == Model(build_model_spec(cfg), "float32", 64).footprint()


def test_configuration_errors():
    from inference_engine_b200.config import ConfigError, config_from_dict

    layer = V.MIXED["layers"]
    with pytest.raises(ConfigError, match="type"):
        config_from_dict(dict(V.MIXED, layers=[dict(layer[0], type="other")]))
    with pytest.raises(ConfigError, match="kv_heads"):
        config_from_dict(dict(V.MIXED, layers=[dict(layer[0], mixer=dict(layer[0]["mixer"], kv_heads=4))]))
    with pytest.raises(ConfigError, match="vdim"):
        config_from_dict(dict(V.MIXED, layers=[dict(layer[0], mixer=dict(layer[0]["mixer"], vdim=8))]))
    with pytest.raises(ConfigError, match="rot"):
        config_from_dict(dict(V.MIXED, layers=[dict(layer[0], mixer=dict(layer[0]["mixer"], rot={"dims": 7, "base": 10.0}))]))
    with pytest.raises(ConfigError, match="softcap"):
        config_from_dict(dict(V.MIXED, layers=[dict(layer[0], mixer=dict(layer[0]["mixer"], softcap=0.0))]))
    with pytest.raises(ConfigError, match="top"):
        config_from_dict(dict(V.MIXED, layers=[dict(layer[0], mlp=V.moe(8, 5, 8, groups=4, keep=2))]))
    with pytest.raises(ConfigError, match="groups"):
        config_from_dict(dict(V.MIXED, layers=[dict(layer[0], mlp=V.moe(8, 2, 8, groups=3, keep=2))]))
    with pytest.raises(ConfigError, match="kind"):
        config_from_dict(dict(V.MIXED, layers=[dict(layer[0], mlp={"kind": "dense", "ff": 8})]))
    with pytest.raises(ConfigError, match="loop"):
        config_from_dict(dict(V.MIXED, loop={"start": 2, "stop": 5, "times": 2}))
    with pytest.raises(ConfigError, match="eps"):
        config_from_dict({k: v for k, v in V.MIXED.items() if k != "norm"})


def test_an_output_bias_needs_an_arrangement_that_adds_it():
    from inference_engine_b200.config.spec import LayerSpec, PartSpec
    from inference_engine_b200.parts.base import BuildEnv
    from inference_engine_b200.parts.registry import build_part

    mixer = PartSpec("sink_attention", {"names": {"q": "q", "k": "k", "o": "o", "o_bias": "ob"}, "heads": 2, "kv_heads": 1,
                                        "dim": 4, "vdim": 4, "scale": 0.5, "values": "keys", "window": None})
    norm = PartSpec("rms", {"weight": "n", "eps": 1e-5})
    layer = LayerSpec("l", PartSpec("prenorm_residual"), mixer, None, {"pre_mixer": norm})
    env = BuildEnv(8, "float32", 16, {})
    with pytest.raises(ValueError, match="output bias"):
        build_part("block", layer.block, env, layer=layer)
    parallel = build_part("block", PartSpec("parallel_residual"), env, layer=layer)
    assert parallel.feed_forward is None and "ob" in parallel.mixer.weights()


def test_kept_first_pages_stay_and_pages_behind_the_window_go_back():
    from inference_engine_b200.cache.manager import CacheManager, PagedGroupSpec

    groups = [PagedGroupSpec(1, 1, 8, window=10, value_dim=8, keep_first=6), PagedGroupSpec(1, 1, 8, window=10, value_dim=8),
              PagedGroupSpec(1, 1, 8)]
    cache = CacheManager(groups, [], 16, 4, 2)
    cache.add_request("a")
    cache.grow("a", 0, 23)
    assert cache.pages_held("a") == [6, 6, 6]
    cache.release_behind_window("a", 23)  # the next query, at 23, sees 14..23 (and 0..5): pages before 12 go
    assert cache.table(0, "a")[:4] == [cache.table(0, "a")[0], cache.table(0, "a")[1], -1, cache.table(0, "a")[3]]
    assert min(cache.table(0, "a")[:2]) >= 0 and cache.table(1, "a")[:3] == [-1] * 3
    assert cache.pages_held("a") == [5, 3, 6]
    cache.check_invariants()
    # growing on needs pages for the new positions only: the kept ones are still held
    assert cache.pages_needed("a", 23, 41) == [5, 5, 5]
    cache.grow("a", 23, 41)
    cache.release_behind_window("a", 41)
    assert [p >= 0 for p in cache.table(0, "a")] == [True, True] + [False] * 6 + [True] * 3
    cache.check_invariants()
    # after its pages were taken away (a preempted request) the kept pages are asked for again
    cache.release_pages("a")
    assert cache.pages_needed("a", 0, 8) == [2, 2, 2]
    cache.free("a")
    assert cache.num_free_pages == [16, 16, 16]


# --- every mechanism alone, against its plain function -------------------------------------------


def _ops(device):
    if device == "cpu":
        from tests.ref_ops import RefOps

        return RefOps()
    from inference_engine_b200.kernels import get_ops

    return get_ops("cuda")


def _ctx(lens, starts, device, slots=None):
    """The parts of a step's context the kernels read, for requests with `lens` new tokens that
    start at positions `starts`."""
    b = len(lens)
    cu = [0]
    for n in lens:
        cu.append(cu[-1] + n)
    seq = [i for i, n in enumerate(lens) for _ in range(n)]
    pos = [s + t for s, n in zip(starts, lens) for t in range(n)]
    i32 = lambda x: torch.tensor(x, dtype=torch.int32, device=device)  # noqa: E731
    return SimpleNamespace(num_tokens=cu[-1], num_seqs=b, seq_of_token=i32(seq), positions=i32(pos), cu_q=i32(cu),
                           q_starts=cu[:-1], q_lens=list(lens), start_positions=list(starts), max_q_len=max(lens),
                           ctx_lens=i32([s + n for s, n in zip(starts, lens)]), bounds=None, padded=False,
                           slots=i32(slots if slots is not None else list(range(b))), ws=None)


def _paged(x, page_size, pages_total, order, device):
    """Rows [T, G, d] into a cache [pages, G, page_size, d] at the pages `order` names."""
    T, G, d = x.shape
    cache = torch.full((pages_total + 1, G, page_size, d), 9.0, device=device)  # (unused rows hold nonsense)
    for t in range(T):
        cache[order[t // page_size], :, t % page_size] = x[t].to(device)
    return cache


def _plain_attention(q, k, v, scale, window, keep_first, softcap, sink, gate):
    """q [T, H, d], k [T, G, d], v [T, G, d], gate [T, H] (before the sigmoid) -> [T, H, d]."""
    o = P.attention_core(q, k, v, scale, P.visible(q.shape[0], window, keep_first), softcap, sink)
    return o if gate is None else o * torch.sigmoid(gate)[..., None]


def _standout_inputs(T, H, G, d, window, keep_first, g, boost_q=25.0):
    """Queries and keys in which one key per query stands out (its score far above the others'): by
    turns the oldest key the window still holds, the one before it (which must not be seen unless
    it is kept), the last kept key and the first one that is not kept."""
    k = torch.randn(T, G, d, generator=g) * 0.01
    q = torch.randn(T, H, d, generator=g) * 0.01
    for t in range(T):
        oldest = max(t - window + 1, 0) if window else 0
        # (without a window: a key far back for every other query; the rest have flat scores, where a
        # sink's share of the weights is largest)
        target = [oldest, oldest - 1, keep_first - 1, keep_first][t % 4] if window else (t // 4 if t % 2 else -1)
        if 0 <= target <= t:
            k[target, :, t % d] += 1.0
            q[t, :, t % d] += boost_q
    return q, k


@pytest.mark.parametrize("device", DEVICES)
@pytest.mark.parametrize("window,keep_first", [(None, 0), (1, 0), (1, 2), (5, 3), (12, 6), (7, 17), (150, 4)])
@pytest.mark.parametrize("softcap,sink", [(None, False), (6.0, True)])
def test_attention_sees_its_window_and_the_kept_first_keys(device, window, keep_first, softcap, sink):
    """One key per query stands out: just inside or just outside the window, or at the edge of the
    kept first positions.  Prompt portions and single tokens, scattered pages of 4 whose borders the
    kept positions and the window cross, grouped heads, gates per head; with capped scores (the key
    that stands out reaches far into the cap's bend) and a zero sink, and without either."""
    ops = _ops(device)
    g = torch.Generator().manual_seed(3)
    T, H, G, d, ps = 45, 4, 2, 48, 4
    q, k = _standout_inputs(T, H, G, d, window, keep_first, g)
    v = torch.randn(T, G, d, generator=g)
    gate = torch.randn(T, H, generator=g) * 2
    scale = 0.6
    want = _plain_attention(q.to(D), k.to(D), v.to(D), scale, window, keep_first, softcap, sink, gate.to(D)).float()
    if window and keep_first and window + keep_first < T:
        # the made-up inputs do tell a kept key from one that is not, and the window's edge
        other = _plain_attention(q.to(D), k.to(D), v.to(D), scale, window, keep_first - 1, softcap, sink, gate.to(D)).float()
        assert (want - other).abs().max() > 0.05
        other = _plain_attention(q.to(D), k.to(D), v.to(D), scale, window + 1, keep_first, softcap, sink, gate.to(D)).float()
        assert (want - other).abs().max() > 0.05
    if softcap:
        # (a query that sees one key alone gives it all the weight the sink leaves, capped or not)
        for changed in ((None, sink), (softcap, False)) if window != 1 else ((softcap, False),):
            other = _plain_attention(q.to(D), k.to(D), v.to(D), scale, window, keep_first, *changed, gate.to(D)).float()
            assert (want - other).abs().max() > 0.05  # (a cap or a sink that is left out shows)
    order = [7, 2, 11, 0, 5, 9, 3, 10, 1, 8, 6, 4]
    kc, vc = _paged(k, ps, 12, order, device), _paged(v, ps, 12, order, device)
    tables = torch.tensor([order], dtype=torch.int32, device=device)
    sinks = torch.zeros(H, device=device) if sink else None
    got, at = [], 0
    for n in [13, 1, 1, 2, 20, 1, 7]:
        ctx = _ctx([n], [at], device)
        out = torch.zeros(n, H * d, device=device)
        wide = torch.cat([torch.zeros(n, 3), gate[at: at + n]], dim=1).to(device)  # (gates beside other columns)
        ops.sink_attention(q[at: at + n].reshape(n, -1).to(device).contiguous(), kc, vc, tables, ctx, H, G, d, d, ps,
                           scale, window, sinks, wide[:, 3:], out, softcap=softcap, keep_first=keep_first)
        got.append(out.cpu().view(n, H, d))
        at += n
    torch.testing.assert_close(torch.cat(got), want, atol=1e-4, rtol=1e-4)


@pytest.mark.gpu
@pytest.mark.parametrize("d,window,keep_first,softcap", [
    (16, 50, 3, None), (64, None, 0, 10.0), (128, 160, 70, None), (48, 64, 64, 4.0), (128, 1, 5, None),
    (80, 65, 130, 25.0), (256, 200, 1, None), (96, None, 0, 12.0), (64, 90, 7, None)])
def test_attention_on_the_tensor_cores(d, window, keep_first, softcap):
    """The bfloat16 kernel against the plain function: portions that start and end inside windows,
    kept positions and tiles of 64, two requests of unequal length in one step (one of them a single
    token), scattered pages, a key per query that stands out at an edge, a zero sink where the
    scores are capped, gates; steps of few tokens cut the keys among blocks (also without a window)."""
    from inference_engine_b200.kernels import get_ops

    ops, g = get_ops("cuda"), torch.Generator().manual_seed(d + (window or 0))
    T, H, G, ps = 333, 6, 2, 16
    bf = lambda x: x.to(torch.bfloat16).float()  # noqa: E731
    k = torch.randn(T, G, d, generator=g) * 0.3
    q = torch.randn(T, H, d, generator=g) * 0.3
    v = bf(torch.randn(T, G, d, generator=g))
    for t in range(0, T, 3):
        oldest = max(t - window + 1, 0) if window else 0
        target = [oldest, oldest - 1, keep_first - 1, keep_first][(t // 3) % 4] if window else t // 2
        if 0 <= target <= t:
            k[target, :, t % d] += 2.0
            q[t, :, t % d] += 8.0
    q, k = bf(q), bf(k)
    sink = softcap is not None
    gate = torch.randn(T, H, generator=g) * 2
    scale = 0.7
    want = _plain_attention(q.to(D), k.to(D), v.to(D), scale, window, keep_first, softcap, sink, gate.to(D)).float()
    pages = -(-T // ps)
    order = torch.randperm(pages + 3, generator=g).tolist()[:pages]
    kc = _paged(k, ps, pages + 3, order, "cuda").to(torch.bfloat16)
    vc = _paged(v, ps, pages + 3, order, "cuda").to(torch.bfloat16)
    other = [pages + 3] * pages  # the second request: one token on the scratch page
    tables = torch.tensor([order, other], dtype=torch.int32, device="cuda")
    kc[pages + 3], vc[pages + 3] = 0.5, 0.25
    sinks = torch.zeros(H, device="cuda") if sink else None
    before = ops.launch_counts.get("sink_attention_mma", 0), ops.launch_counts.get("sink_attention_merge", 0)
    got, at = [], 0
    portions = [70, 33, 1, 2, 5, 130, 1, 8, 83]  # (few tokens: the key tiles are cut among blocks)
    for n in portions:
        ctx = _ctx([n, 1], [at, 0], "cuda")
        qq = torch.cat([q[at: at + n].reshape(n, -1), torch.ones(1, H * d)]).to("cuda", torch.bfloat16)
        gg = torch.cat([gate[at: at + n], torch.zeros(1, H)]).cuda()
        out = torch.zeros(n + 1, H * d, device="cuda", dtype=torch.bfloat16)
        ops.sink_attention(qq, kc, vc, tables, ctx, H, G, d, d, ps, scale, window, sinks, gg, out, softcap=softcap,
                           keep_first=keep_first)
        got.append(out[:n].float().cpu().view(n, H, d))
        # the stranger's one key: its weight against the sink's (if any), its gate one half
        s = torch.tensor(d * 0.5 * scale, dtype=D)
        s = softcap * torch.tanh(s / softcap) if softcap else s
        lone = 0.5 * 0.25 * (torch.exp(s) / (torch.exp(s) + 1.0) if sink else torch.tensor(1.0, dtype=D))
        torch.testing.assert_close(out[n].float().cpu(), torch.full((H * d,), float(lone)), atol=2e-3, rtol=2e-2)
        at += n
    ops.check_errors()
    assert at == T and ops.launch_counts.get("sink_attention_mma", 0) == before[0] + len(portions)
    assert ops.launch_counts.get("sink_attention_merge", 0) > before[1]  # (the steps of few tokens were cut)
    # (weights keep 16 bits of mantissa in the second product; outputs are rounded to bfloat16)
    torch.testing.assert_close(torch.cat(got), want, atol=0.015, rtol=0.01)


@pytest.mark.gpu
def test_far_keys_in_long_decoding_without_a_window():
    """Single tokens at contexts of thousands of positions, where the keys are cut among many blocks:
    each query's key that stands out lies far back (among the first positions, or thousands before
    it), in both precisions' kernels."""
    from inference_engine_b200.kernels import get_ops

    ops, g = get_ops("cuda"), torch.Generator().manual_seed(9)
    T, H, G, d, ps = 4500, 4, 1, 64, 16
    bf = lambda x: x.to(torch.bfloat16).float()  # noqa: E731
    k, v = bf(torch.randn(T, G, d, generator=g) * 0.3), bf(torch.randn(T, G, d, generator=g))
    probes = [T - 1, T - 2, 4099, 4031, 2500, 70]
    far = {T - 1: 3, T - 2: 1100, 4099: 4035, 4031: 64, 2500: 0, 70: 63}
    q = torch.randn(T, H, d, generator=g) * 0.3
    for i, (t, target) in enumerate(far.items()):  # (a dimension of its own for every probe)
        q[:, :, 5 + i], k[:, :, 5 + i] = 0.0, 0.0
        k[target, :, 5 + i] = 3.0
        q[t, :, 5 + i] = 12.0
    q, k = bf(q), bf(k)
    scale, softcap = 0.5, 30.0
    pages = -(-T // ps)
    order = torch.randperm(pages, generator=g).tolist()
    tables = torch.tensor([order], dtype=torch.int32, device="cuda")
    for dtype, tol in ((torch.bfloat16, 0.02), (torch.float32, 2e-4)):
        kc, vc = _paged(k, ps, pages, order, "cuda").to(dtype), _paged(v, ps, pages, order, "cuda").to(dtype)
        for t in probes:
            s = torch.einsum("hd,kgd->hk", q[t].to(D), k[: t + 1].to(D)) * scale
            s = softcap * torch.tanh(s / softcap)
            p = torch.exp(s) / (1.0 + torch.exp(s).sum(-1, keepdim=True))
            want = (p @ v[: t + 1, 0].to(D)).float()
            assert p[:, far[t]].min() > 0.5  # (the far key carries the result)
            out = torch.zeros(1, H * d, device="cuda", dtype=dtype)
            ops.sink_attention(q[t].reshape(1, -1).to("cuda", dtype), kc, vc, tables, _ctx([1], [t], "cuda"), H, G, d, d,
                               ps, scale, None, torch.zeros(H, device="cuda"), None, out, softcap=softcap)
            torch.testing.assert_close(out.float().cpu().view(H, d), want, atol=tol, rtol=tol)
    ops.check_errors()


@pytest.mark.parametrize("device", DEVICES)
@pytest.mark.parametrize("interleaved,rot", [(False, 0), (False, 6), (False, 10), (True, 4), (True, 10)])
def test_rotated_keys_plain_values_and_cache_rows(device, interleaved, rot):
    """Queries and keys take their biases and are rotated on their first `rot` entries, by pairs of
    either layout; the cached values are the keys with their bias, before the rotation; rows land
    where the slot mapping says; the columns behind the keys (head gates) are left alone."""
    ops, g = _ops(device), torch.Generator().manual_seed(8)
    n, H, G, d, ps = 9, 3, 2, 10, 4
    size = (H + G) * d
    proj = torch.randn(n, size + H, generator=g)
    bias = torch.randn(size, generator=g)
    pos = torch.tensor([0, 1, 2, 3, 17, 18, 19, 5, 6])
    base = 50.0
    full = proj[:, :size].to(D) + bias.to(D)
    layout = "interleaved" if interleaved else "halves"
    q = P.rotate(full[:, : H * d].view(n, H, d), pos, rot, base, layout)
    k_plain = full[:, H * d:].view(n, G, d)
    k = P.rotate(k_plain, pos, rot, base, layout)
    table = None
    if rot:
        freq = base ** (-torch.arange(0, rot, 2, dtype=D) / rot)
        ang = torch.arange(20, dtype=D)[:, None] * freq[None, :]
        table = torch.stack((ang.cos(), ang.sin()), dim=1).float().to(device)
    q_out = torch.zeros(n, H * d, device=device)
    kc, vc = torch.zeros(9, G, ps, d, device=device), torch.zeros(9, G, ps, d, device=device)
    slots = torch.tensor([p + 8 for p in pos.tolist()], dtype=torch.int32, device=device)  # pages 2..6
    ops.qk_norm_rope_write(proj.to(device), pos.to(torch.int32).to(device), table, rot, None, None, 1e-5, q_out, kc, vc,
                           slots, H, G, d, d, ps, bias=bias.to(device), values_from_keys=True, interleaved=interleaved)
    torch.testing.assert_close(q_out.cpu(), q.reshape(n, -1).float(), atol=1e-5, rtol=1e-5)
    for i, s in enumerate(slots.tolist()):
        torch.testing.assert_close(kc[s // ps, :, s % ps].cpu(), k[i].float(), atol=1e-5, rtol=1e-5)
        torch.testing.assert_close(vc[s // ps, :, s % ps].cpu(), k_plain[i].float(), atol=1e-6, rtol=1e-6)
    if rot:  # (the rotation does move the keys, so values taken after it would show)
        assert (k - k_plain)[4:].abs().max() > 0.1


@pytest.mark.parametrize("device", DEVICES)
@pytest.mark.parametrize("experts,top,groups,keep", [(9, 3, 1, 1), (8, 2, 4, 2), (18, 3, 3, 1), (6, 6, 3, 3), (12, 1, 6, 1),
                                                     (4, 2, 4, 3), (64, 8, 8, 4), (2, 1, 1, 1)])
def test_router_with_sigmoid_scores_and_a_correction(device, experts, top, groups, keep):
    """The correction decides which groups and experts are chosen (it is as large as the scores, and
    pushes many corrected scores below zero, so that a dropped group's experts must rank below every
    one of them and not at zero); a group is ranked by its two best corrected scores; the weights are the
    chosen experts' plain scores over their sum, times the scale."""
    ops, g = _ops(device), torch.Generator().manual_seed(experts + top)
    n, hidden = 33, 40
    x = torch.randn(n, hidden, generator=g)
    W = {"r.router": torch.randn(experts, hidden, generator=g) / hidden ** 0.5 * 2,
         "r.correction": torch.randn(experts, generator=g) - 0.9}
    mlp = {"router": {"experts": experts, "top": top, "scale": 2.5, "groups": {"count": groups, "keep": keep}}}
    W64 = {k: t.to(D) for k, t in W.items()}
    ids_want, w_want = P.route(W64, "r", x.to(D), mlp)
    plain = dict(W64, **{"r.correction": torch.zeros(experts, dtype=D)})
    if top < experts:  # (without the correction others would be chosen)
        assert not torch.equal(ids_want.sort(-1).values, P.route(plain, "r", x.to(D), mlp)[0].sort(-1).values)
    ids = torch.zeros(n, top, dtype=torch.int32, device=device)
    weights = torch.zeros(n, top, device=device)
    ops.route_topk(x.to(device), W["r.router"].to(device), groups, keep, ids, weights, scoring="sigmoid",
                   correction=W["r.correction"].to(device), group_top=2, weight_scale=2.5)
    got = torch.zeros(n, experts).scatter_(1, ids.long().cpu(), weights.cpu())
    want = torch.zeros(n, experts, dtype=D).scatter_(1, ids_want, w_want).float()
    torch.testing.assert_close(got, want, atol=1e-5, rtol=1e-5)
    torch.testing.assert_close(weights.sum(-1).cpu(), torch.full((n,), 2.5), atol=1e-5, rtol=1e-5)
    if 1 < keep < groups and experts // groups > 1:
        # ranking the groups by their best expert alone would keep other groups for some token
        best = (torch.sigmoid(x.to(D) @ W64["r.router"].T) + W64["r.correction"]).view(n, groups, -1)
        by_one = best.max(-1).values.topk(keep, dim=-1).indices.sort(-1).values
        by_two = best.topk(2, dim=-1).values.sum(-1).topk(keep, dim=-1).indices.sort(-1).values
        assert not torch.equal(by_one, by_two)


@pytest.mark.parametrize("device", DEVICES)
@pytest.mark.parametrize("hidden", [50, 72, 1100])
def test_two_sublayers_a_bias_and_a_second_stream_in_one_add(device, hidden):
    """h += mixer + feed-forward + bias + the embedding's output, and the next norm of h: the outputs
    whole or in parts, any of the terms absent, for all rows or chosen ones (then h stays as it is),
    and without a following norm."""
    ops, g = _ops(device), torch.Generator().manual_seed(hidden)
    n, eps = 7, 1e-5
    h, first = torch.randn(n, hidden, generator=g), torch.randn(2, n, hidden, generator=g) * 3
    second, x0 = torch.randn(3, n, hidden, generator=g) * 2, torch.randn(n, hidden, generator=g) * 4
    bias, w = torch.randn(hidden, generator=g), torch.randn(hidden, generator=g)
    dev = lambda t: None if t is None else t.to(device)  # noqa: E731
    for a in (first, first[0]):
        for b in (second, second[1], None):
            for bb in (bias, None):
                for extra in (x0, None):
                    total = (a.to(D).sum(0) if a.dim() == 3 else a.to(D))
                    if b is not None:
                        total = total + (b.to(D).sum(0) if b.dim() == 3 else b.to(D))
                    total = total + (0 if bb is None else bb.to(D)) + (0 if extra is None else extra.to(D))
                    h_want = h.to(D) + total
                    out_want = P.rms_norm(h_want, w.to(D), eps)
                    hd, out = h.clone().to(device), torch.zeros(n, hidden, device=device)
                    ops.sandwich_norm(hd, dev(a), dev(bb), None, 0.0, dev(w), eps, out, second=dev(b), extra=dev(extra))
                    torch.testing.assert_close(hd.cpu(), h_want.float(), atol=1e-5, rtol=1e-5)
                    torch.testing.assert_close(out.cpu(), out_want.float(), atol=1e-5, rtol=1e-5)
                    rows = torch.tensor([5, 0], dtype=torch.int32, device=device)
                    hd2, out2 = h.clone().to(device), torch.zeros(2, hidden, device=device, dtype=torch.bfloat16)
                    ops.sandwich_norm(hd2, dev(a), dev(bb), None, 0.0, dev(w), eps, out2, rows, second=dev(b), extra=dev(extra))
                    torch.testing.assert_close(out2.float().cpu(), out_want.float()[[5, 0]], atol=3e-2, rtol=2e-2)
                    assert torch.equal(hd2.cpu(), h)
                    hd3 = h.clone().to(device)
                    ops.sandwich_norm(hd3, dev(a), dev(bb), None, 0.0, None, 0.0, None, second=dev(b), extra=dev(extra))
                    torch.testing.assert_close(hd3.cpu(), h_want.float(), atol=1e-5, rtol=1e-5)


@pytest.mark.parametrize("device", DEVICES)
def test_capped_logits(device):
    ops = _ops(device)
    logits = torch.linspace(-90.0, 90.0, 1001).view(7, 143).contiguous()
    for factor, cap in ((1.0, 30.0), (0.5, 4.0)):
        t = logits.clone().to(device)
        ops.scale_softcap_(t, factor, cap)
        want = cap * torch.tanh(logits.to(D) * factor / cap)
        torch.testing.assert_close(t.cpu(), want.float(), atol=2e-6 * cap, rtol=1e-6)
        assert float(t.abs().max()) <= cap


def test_a_stream_add_joins_the_pending_add():
    """Before a later pass of the loop the embedding's output rides along with the pending outputs of
    the layer before (one add, in the next norm's kernel); where the pending output is treated before
    it is added, the stream is brought up to date first."""
    from inference_engine_b200.parts.norm import AddedTerms, PostNorm
    from inference_engine_b200.parts.stream import AddEmbedding

    part, x0 = AddEmbedding(), torch.ones(2, 4)
    alone = part.fold(None, x0)
    assert isinstance(alone, AddedTerms) and alone.rows_like_stream is x0 and alone.second is None
    second, bias = torch.zeros(3, 2, 4), torch.zeros(4)
    joined = part.fold(AddedTerms(bias, second), x0)
    assert joined.rows_like_stream is x0 and joined.second is second and joined.bias is bias
    assert part.fold(joined, x0) is None and part.fold(PostNorm(None), x0) is None


# --- long decoding and generation through the engine ------------------------------------------------


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_long_decoding_through_windows_and_pages(tmp_path, dtype):
    """400 tokens decoded one by one after a short prompt, across many windows and pages: the kept
    first positions stay while pages behind the windows go back (the pool is smaller than the
    sequence would need in the windowed layers alone; the layers that see everything hold it all)."""
    from inference_engine_b200.kernels import get_ops

    cfg = V.MIXED
    weights = V.make_weights(cfg, seed=3)
    toks = _requests(cfg, [410], seed=5)["r0"]
    want = P.forward(cfg, weights, toks, D).float()
    session = _session(tmp_path, cfg, weights, dtype, "cuda", get_ops("cuda"), 448, 16)
    got = H.collect(session, H.trace_decode_tail({"a": toks}, 400))["a"]
    H.assert_close(got, want, LABEL[dtype], "long decoding", _bound(tmp_path, dtype, cfg, weights, {"a": toks}, {"a": want}))


def test_pages_behind_the_windows_go_back_while_decoding(tmp_path):
    """On the plain kernels: after 70 positions the windowed groups hold their windows' pages and the
    kept first ones, the groups that see everything hold every page."""
    from tests.ref_ops import RefOps

    cfg = V.MIXED
    weights = V.make_weights(cfg, seed=3)
    toks = _requests(cfg, [70], seed=5)["r0"]
    session = _session(tmp_path, cfg, weights, "float32", "cpu", RefOps(), 128, 4)
    steps = H.trace_decode_tail({"a": toks}, 60)
    steps[-1]["end"] = []
    got = H.collect(session, steps)["a"]
    want = P.forward(cfg, weights, toks, D).float()
    H.assert_close(got, want, LABEL["float32"], "decoding on the plain kernels",
                   _float32_bound(cfg, weights, {"a": toks}, {"a": want}))
    held = {(g.window, g.keep_first): n for g, n in zip(session.cache.paged_groups, session.cache.pages_held("a"))}
    # the next query, at 70: window 10 sees 61.. (pages 15..17) and keeps page 0; window 7 sees 64.. (pages 16, 17)
    assert held == {(None, 0): 18, (10, 3): 4, (7, 0): 2}


def _greedy_plain(cfg, weights, prompt, count):
    ids = list(prompt)
    for _ in range(count):
        ids.append(int(P.forward(cfg, weights, ids, D)[-1].argmax()))
    return ids[len(prompt):]


def _generate(cfg, weights, device, **kw):
    from inference_engine_b200 import SamplingParams
    from inference_engine_b200.engine.llm_engine import LLMEngine
    from inference_engine_b200.engine.loading import model_from_tensors

    model, _ = model_from_tensors(cfg, weights, "float32", device, 128)
    engine = LLMEngine(model, None, (), num_blocks=48, block_size=8, max_num_seqs=3,
                       max_num_batched_tokens=16, debug_checks=True, **kw)
    prompts = {f"p{i}": _requests(cfg, [n], seed=90 + i)["r0"] for i, n in enumerate([5, 40, 23, 1, 31])}
    for rid, prompt in prompts.items():
        engine.add_request(rid, prompt, SamplingParams(max_tokens=10, temperature=0.0))
    got: dict[str, list[int]] = {rid: [] for rid in prompts}
    while engine.has_unfinished():
        for out in engine.step():
            got[out.request_id].append(out.token_id)
    engine.cache.check_invariants()
    assert engine.cache.slots.num_free == engine.cache.slots.num_slots
    return engine, prompts, got


def test_greedy_generation_on_the_plain_kernels():
    """The engine's own entry point and scheduler on the CPU stand-ins of the kernels."""
    from tests.ref_ops import RefOps

    cfg = V.LOOP_FIRST
    weights = V.make_weights(cfg, seed=4)
    _, prompts, got = _generate(cfg, weights, "cpu", ops=RefOps())
    for rid, prompt in prompts.items():
        assert got[rid] == _greedy_plain(cfg, weights, prompt, 10), rid


@pytest.mark.gpu
@pytest.mark.parametrize("name", ["mixed", "odd"])
def test_greedy_generation_through_the_engine(name):
    """`LLMEngine` with the scheduler cutting prompts into portions and batching requests (three at
    a time, so slots and pages serve one request after another), decode steps captured and launched
    ahead: the tokens are the plain implementation's greedy choices."""
    cfg = V.CONFIGS[name]
    weights = V.make_weights(cfg, seed=4)
    engine, prompts, got = _generate(cfg, weights, "cuda")
    assert engine.graphs is not None  # decode steps are captured
    for rid, prompt in prompts.items():
        assert got[rid] == _greedy_plain(cfg, weights, prompt, 10), rid


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_captured_short_steps_with_portions(tmp_path, dtype):
    """Portions and mixed batches replayed through captured launch sequences (launched for bounds,
    padded with tokens that belong to no request): key sizes the tensor-core attention takes, so in
    bfloat16 that kernel runs sized by the token bound.  Against the plain implementation; in 32-bit
    equal bit for bit to the eagerly launched steps."""
    from inference_engine_b200.engine.graphs import DecodeGraphs, MixedGraphs
    from inference_engine_b200.kernels import get_ops

    cfg = V.config(64, 89, [
        (V.attention(4, 2, 16, rot=8, softcap=7.0), V.moe(4, 2, 24, groups=2, keep=1, scale=1.5)),
        (V.attention_2(4, 2, 32, rot=32, window=24, keep_first=5), V.moe(6, 2, 16)),
        (V.attention_2(2, 1, 16, rot=6, window=9, keep_first=20), None),
    ], loop=(1, 3, 2), logit_softcap=15.0)
    weights = V.make_weights(cfg, seed=6)
    requests = _requests(cfg, [70, 45, 33, 90, 20, 60], seed=300)
    want = _want(cfg, weights, requests)
    tol = _bound(tmp_path, dtype, cfg, weights, requests, want)
    mixed, peak = H.trace_mixed(requests, seed=2, tail=6, max_portion=20)
    results = {}
    for captured in (True, False):
        for mode, (trace, room) in {"portions": (H.trace_portions(requests), 128), "mixed": (mixed, peak)}.items():
            session = _session(tmp_path / f"{mode}{captured}", cfg, weights, dtype, "cuda", get_ops("cuda"), room, 8)
            if captured:
                graphs = MixedGraphs(DecodeGraphs(session.runner, 256, max(64, -(-room // 8))))
                eager = session.runner.step
                session.runner.step = lambda entries, g=graphs, e=eager: g.run(entries) if g.can_run(entries) else e(entries)
            got = H.collect(session, trace)
            for rid in requests:
                H.assert_close(got[rid], want[rid], LABEL[dtype], f"captured={captured} {mode} {rid}", tol)
            if captured:
                assert graphs.replays > len(requests)
            results[(captured, mode)] = got
    if dtype == "float32":
        for mode in ("portions", "mixed"):
            for rid in requests:
                assert torch.equal(results[(True, mode)][rid], results[(False, mode)][rid]), (mode, rid)
    get_ops("cuda").check_errors()
