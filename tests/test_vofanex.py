"""The Vofanex design in the engine against the plain whole-sequence implementation
(`tests/plain_vofanex.py`): whole prompts, token-by-token decoding, portions down to two tokens,
mixed batches with pages and state slots used again, configurations of odd sizes; every mechanism
alone against its plain function, with inputs made so that a key just inside or just outside a
window, a sink that is left out, a lost state or a wrong expert shows; on the CPU through the plain
stand-ins of the kernels, on the GPU through the kernels in both precisions; long decoding; greedy
generation through the engine's own entry point and scheduler."""

from __future__ import annotations

from types import SimpleNamespace

import pytest
import torch

from tests import helpers as H
from tests import plain_vofanex as P
from tests import vofanex_configs as V

LENGTHS = [50, 21, 37, 64, 9, 1]
BF16_TOL = dict(atol=0.35, rtol=0.0, pos_rel_rms=0.08, rel_rms=0.04)
# (under these names the run's summary lists this file's comparisons: their bounds are measured)
LABEL = {"float32": "float32, Vofanex", "bfloat16": "bfloat16, Vofanex"}
DEVICES = ["cpu", pytest.param("cuda", marks=pytest.mark.gpu)]


def _requests(cfg, lengths=LENGTHS, seed=700):
    return {f"r{i}": torch.randint(0, cfg["vocab"], (n,), generator=torch.Generator().manual_seed(seed + i)).tolist()
            for i, n in enumerate(lengths)}


def _want(cfg, weights, requests):
    return {rid: P.forward(cfg, weights, toks, torch.float64).float() for rid, toks in requests.items()}


def _float32_bound(cfg, weights, requests, want) -> dict:
    """Three times what rounding alone does to the plain implementation when it runs in 32-bit
    instead of 64-bit, and never below the engine's fixed bound for tiny models.  A lost state, a
    wrong key or a sink left out moves logits by 1e-2 and more."""
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
            H.assert_close(got[rid], want[rid], LABEL[dtype], f"vofanex {name} {mode} {rid}", tol)
        # everything went back to the pools
        assert session.cache.num_free_pages == [p.num_pages for p in session.cache.pools]
        assert session.cache.slots.num_free == session.cache.slots.num_slots
        results[mode] = got
    return results


def test_the_test_weights_make_no_close_call_in_the_routers():
    """The experts the plain implementation chooses are chosen by a margin that rounding does not
    reach, so a difference in the logits is a fault and not another expert."""
    for name, cfg in V.CONFIGS.items():
        weights = V.make_weights(cfg, seed=11)
        margins = []
        for toks in _requests(cfg, [30, 13, 21, 9, 1]).values():
            P.forward(cfg, weights, toks, torch.float64, margins=margins)
        assert min(margins) > 1e-4, name


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
    tensor-core attention in bfloat16 and the wider instances of the recurrence."""
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

    cfg = config_from_dict(V.MIXED).with_tensor_shapes(V.tensor_shapes(V.MIXED, V.RANKS["mixed"]))
    model = Model(build_model_spec(cfg), "float32", 64)
    assert [type(b).__name__ for b in model.blocks] == ["GatedPreNormResidualBlock"] * 5
    assert [type(b.mixer).__name__ for b in model.blocks] == [
        "GatedLinearAttention", "SinkAttention", "GatedLinearAttention", "SinkAttention", "GatedLinearAttention"]
    assert [type(b.feed_forward).__name__ for b in model.blocks] == [
        "PolyNormFF", "RoutedExperts", "NoneType", "PolyNormFF", "RoutedExperts"]
    assert [b.mixer.rank for b in model.blocks if hasattr(b.mixer, "rank")] == [5, 3, 9]  # (from a1's shape)
    # a cache group per attention layer's sizes, with its window; a state per recurrent layer
    assert sorted((g.num_kv_heads, g.head_dim, g.value_dim, g.window) for g in model.paged_groups) == [
        (2, 16, 24, 10), (3, 8, 12, 7)]
    shapes = {g.shape: g.num_layers for g in model.state_groups}
    assert shapes == {(3 * 12 * 20,): 1, (2 * 20 * 8,): 1, (6 * 4 * 12,): 1}
    assert model.embedding.scale == 1.7
    no_window = Model(build_model_spec(config_from_dict(V.ODD).with_tensor_shapes(
        V.tensor_shapes(V.ODD, V.RANKS["odd"]))), "float32", 64)
    assert sorted((g.window is None) for g in no_window.paged_groups) == [False, True]


@pytest.mark.parametrize("name", list(V.ALL_CONFIGS))
def test_footprint_formula_counts_what_the_model_declares(name):
    from inference_engine_b200.architectures.vofanex import vofanex_footprint
    from inference_engine_b200.config import build_model_spec, config_from_dict
    from inference_engine_b200.engine.model import Model

    raw = V.ALL_CONFIGS[name]
    cfg = config_from_dict(raw).with_tensor_shapes(V.tensor_shapes(raw, V.RANKS[name]))
    assert vofanex_footprint(cfg) == Model(build_model_spec(cfg), "float32", 64).footprint()


def test_configuration_errors():
    from inference_engine_b200.config import ConfigError, build_model_spec, config_from_dict

    layer = V.MIXED["layers"]
    with pytest.raises(ConfigError, match="type"):
        config_from_dict(dict(V.MIXED, layers=[dict(layer[0], type="other")]))
    with pytest.raises(ConfigError, match="kv_heads"):
        config_from_dict(dict(V.MIXED, layers=[dict(layer[1], mixer=dict(layer[1]["mixer"], kv_heads=4))]))
    with pytest.raises(ConfigError, match="tau"):
        config_from_dict(dict(V.MIXED, layers=[dict(layer[0], mixer=dict(layer[0]["mixer"], tau=0.0))]))
    with pytest.raises(ConfigError, match="top"):
        config_from_dict(dict(V.MIXED, layers=[dict(layer[1], mlp=V.moe(3, 4, 8))]))
    with pytest.raises(ConfigError, match="kind"):
        config_from_dict(dict(V.MIXED, layers=[dict(layer[0], mlp={"kind": "other"})]))
    with pytest.raises(ConfigError, match="eps"):
        config_from_dict({k: v for k, v in V.MIXED.items() if k != "norm"})
    with pytest.raises(ConfigError, match="rank"):  # neither a tensor's shape nor a key gives the rank
        build_model_spec(config_from_dict(V.MIXED))
    with_key = dict(V.MIXED, layers=[dict(layer[0], mixer=dict(layer[0]["mixer"], decay_rank=6))])
    assert build_model_spec(config_from_dict(with_key)).layers[0].mixer.params["rank"] == 6


def test_pages_behind_the_window_go_back():
    from inference_engine_b200.cache.manager import CacheManager, PagedGroupSpec

    cache = CacheManager([PagedGroupSpec(1, 1, 8, window=10, value_dim=12), PagedGroupSpec(1, 1, 8)], [], 16, 4, 2)
    cache.add_request("a")
    cache.grow("a", 0, 23)
    assert cache.pages_held("a") == [6, 6]
    cache.release_behind_window("a", 23)  # the next query, at 23, sees 14..23: pages before 12 go
    assert cache.table(0, "a")[:3] == [-1] * 3 and cache.table(0, "a")[3] >= 0
    assert cache.pages_held("a") == [3, 6]
    cache.check_invariants()
    cache.free("a")
    assert cache.num_free_pages == [16, 16]


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
                           slots=i32(slots if slots is not None else list(range(b))))


def _paged(x, page_size, pages_total, order, device):
    """Rows [T, G, d] into a cache [pages, G, page_size, d] at the pages `order` names."""
    T, G, d = x.shape
    cache = torch.full((pages_total + 1, G, page_size, d), 9.0, device=device)  # (unused rows hold nonsense)
    for t in range(T):
        cache[order[t // page_size], :, t % page_size] = x[t].to(device)
    return cache


def _plain_sink_attention(q, k, v, scale, sink, window, gate):
    """q [T, H, d], k [T, G, d], v [T, G, dv], gate [T, H] (before the sigmoid) -> [T, H, dv]."""
    H, G = q.shape[1], k.shape[1]
    group = torch.arange(H) // (H // G)
    scores = torch.einsum("thd,shd->hts", q, k[:, group]) * scale
    if sink is None:
        sink = torch.full((H,), float("-inf"), dtype=q.dtype)  # (a term of size zero)
    weights = P.sink_window_softmax(scores, sink, window or q.shape[0])
    o = torch.einsum("hts,shv->thv", weights, v[:, group])
    return o if gate is None else o * torch.sigmoid(gate)[..., None]


@pytest.mark.parametrize("device", DEVICES)
@pytest.mark.parametrize("window", [None, 1, 2, 5, 12, 150])
def test_sink_attention_sees_exactly_its_window(device, window):
    """One key per query stands out (its score 25 above the others'): the oldest key the window still
    holds, or the one before it, which must not be seen; the sink takes a known share of what is
    left.  Prompt portions and single tokens, scattered pages, grouped heads, value rows of another
    size than key rows, gates per head."""
    ops = _ops(device)
    g = torch.Generator().manual_seed(3)
    T, H, G, d, dv, ps = 45, 4, 2, 48, 6, 4  # (a dimension of its own for every query)
    k = torch.randn(T, G, d, generator=g) * 0.01
    v = torch.randn(T, G, dv, generator=g)
    q = torch.randn(T, H, d, generator=g) * 0.01
    for t in range(T):
        oldest = max(t - window + 1, 0) if window else 0
        target = oldest if t % 2 == 0 else oldest - 1  # just inside / just outside (or before the start)
        if 0 <= target < T:
            k[target, :, t] += 1.0
            q[t, :, t] += 25.0
    sink = torch.tensor([2.0, -1.0, 0.5, 24.0])  # (the last one as large as the key that stands out)
    gate = torch.randn(T, H, generator=g) * 2
    D = torch.float64
    want = _plain_sink_attention(q.to(D), k.to(D), v.to(D), 1.0, sink.to(D), window, gate.to(D)).float()
    without = _plain_sink_attention(q.to(D), k.to(D), v.to(D), 1.0, None, window, gate.to(D)).float()
    assert (want - without).abs().max() > 0.05  # (the inputs do show a sink that is left out)
    order = [7, 2, 11, 0, 5, 9, 3, 10, 1, 8, 6, 4]
    kc, vc = _paged(k, ps, 12, order, device), _paged(v, ps, 12, order, device)
    tables = torch.tensor([order], dtype=torch.int32, device=device)
    for sinks, expect in ((sink, want), (None, without)):
        got, at = [], 0
        for n in [13, 1, 1, 2, 20, 1, 7]:
            ctx = _ctx([n], [at], device)
            out = torch.zeros(n, H * dv, device=device)
            # the gates sit beside other columns of a wider 32-bit buffer, as in the mixer
            wide = torch.cat([torch.zeros(n, 3), gate[at: at + n]], dim=1).to(device)
            ops.sink_attention(q[at: at + n].reshape(n, -1).to(device).contiguous(), kc, vc, tables, ctx, H, G, d,
                               dv, ps, 1.0, window, None if sinks is None else sinks.to(device), wide[:, 3:], out)
            got.append(out.cpu().view(n, H, dv))
            at += n
        torch.testing.assert_close(torch.cat(got), expect, atol=1e-4, rtol=1e-4)
    if window and window > 1 and 2 * window + 1 < T:  # the made-up inputs do tell inside from outside
        seen = without.abs().amax(2)[:, 0] / torch.sigmoid(gate[:, 0])
        t = 2 * window  # an even position looks just inside, the next one just outside
        far_in = v[t - window + 1, 0].abs().max()
        assert abs(seen[t] - far_in) < 1e-3 * far_in + 1e-4 and not torch.allclose(want[t], want[t + 1])


@pytest.mark.gpu
@pytest.mark.parametrize("d,dv,window", [(16, 32, 50), (64, 64, None), (128, 128, 160), (48, 16, 64), (128, 64, 1),
                                         (80, 112, 65), (256, 256, 200)])
def test_sink_attention_on_the_tensor_cores(d, dv, window):
    """The bfloat16 kernel against the plain function: portions that start and end inside windows
    and tiles of 64, two requests of unequal length in one step (one of them a single token), scattered
    pages, a key per query that stands out just inside or just outside the window, sinks, gates."""
    from inference_engine_b200.kernels import get_ops

    ops, g = get_ops("cuda"), torch.Generator().manual_seed(d + dv)
    T, H, G, ps = 333, 6, 2, 16
    bf = lambda x: x.to(torch.bfloat16).float()  # noqa: E731
    k = bf(torch.randn(T, G, d, generator=g) * 0.3)
    v = bf(torch.randn(T, G, dv, generator=g))
    q = bf(torch.randn(T, H, d, generator=g) * 0.3)
    for t in range(0, T, 3):
        oldest = max(t - window + 1, 0) if window else 0
        target = oldest if t % 2 == 0 else oldest - 1
        if 0 <= target < T:
            k[target, :, t % d] += 2.0
            q[t, :, t % d] += 8.0
    q, k = bf(q), bf(k)
    sink = torch.linspace(-2.0, 6.0, H)
    gate = torch.randn(T, H, generator=g) * 2
    scale = 0.7
    D = torch.float64
    want = _plain_sink_attention(q.to(D), k.to(D), v.to(D), scale, sink.to(D), window, gate.to(D)).float()
    pages = -(-T // ps)
    order = torch.randperm(pages + 3, generator=g).tolist()[:pages]
    kc = _paged(k, ps, pages + 3, order, "cuda").to(torch.bfloat16)
    vc = _paged(v, ps, pages + 3, order, "cuda").to(torch.bfloat16)
    other = [pages + 3] * pages  # the second request: one token on the scratch page
    tables = torch.tensor([order, other], dtype=torch.int32, device="cuda")
    kc[pages + 3], vc[pages + 3] = 0.5, 0.25
    before = ops.launch_counts.get("sink_attention_mma", 0)
    got, at = [], 0
    portions = [70, 33, 1, 2, 5, 130, 1, 8, 83]  # (few tokens: the window's key tiles are cut among blocks)
    for n in portions:
        ctx = _ctx([n, 1], [at, 0], "cuda")
        qq = torch.cat([q[at: at + n].reshape(n, -1), torch.ones(1, H * d)]).to("cuda", torch.bfloat16)
        gg = torch.cat([gate[at: at + n], torch.zeros(1, H)]).cuda()
        out = torch.zeros(n + 1, H * dv, device="cuda", dtype=torch.bfloat16)
        ops.sink_attention(qq, kc, vc, tables, ctx, H, G, d, dv, ps, scale, window, sink.cuda(), gg, out)
        got.append(out[:n].float().cpu().view(n, H, dv))
        # the stranger's one key: its weight against the sink's, its gate one half
        s = torch.tensor(d * 0.5 * scale, dtype=D)
        lone = (0.5 * 0.25 * torch.exp(s) / (torch.exp(s) + torch.exp(sink.to(D)))).float()[:, None]
        torch.testing.assert_close(out[n].float().cpu().view(H, dv), lone.expand(H, dv), atol=2e-3, rtol=2e-2)
        at += n
    ops.check_errors()
    assert at == T and ops.launch_counts.get("sink_attention_mma", 0) == before + len(portions)  # (the kernel under test did run)
    # (weights keep 16 bits of mantissa in the second product; outputs are rounded to bfloat16)
    torch.testing.assert_close(torch.cat(got), want, atol=0.015, rtol=0.01)


@pytest.mark.parametrize("device", DEVICES)
@pytest.mark.parametrize("heads,dim,vdim,rank,tau", [(3, 12, 20, 5, 8.0), (1, 5, 3, 1, 1.0), (2, 48, 16, 16, 32.0),
                                                     (2, 100, 40, 7, 2.5), (1, 130, 8, 300, 4.0), (1, 260, 33, 3, 64.0)])
def test_gated_linear_attention_in_pieces(device, heads, dim, vdim, rank, tau):
    """The decay from its low-rank map and the recurrence over 61 tokens cut into pieces of 1 to 17
    tokens, from and to a state slot, against the whole-sequence functions; the first token leaves
    a mark that slow decays keep, so a state that is lost or starts anywhere but at zero shows; a
    second request beside it must not disturb it."""
    ops, g = _ops(device), torch.Generator().manual_seed(dim)
    T, D = 61, torch.float64
    q = torch.randn(T, heads, dim, generator=g)
    k = torch.randn(T, heads, dim, generator=g)
    v = torch.randn(T, heads, vdim, generator=g)
    k[0], v[0] = 3.0, 5.0  # (the first token's mark)
    y = torch.randn(T, rank, generator=g)
    w2 = torch.randn(heads * dim, rank, generator=g) / rank ** 0.5
    bias = torch.randn(heads * dim, generator=g) + 3.0
    alpha = torch.sigmoid(y.to(D) @ w2.to(D).T + bias.to(D)).pow(1.0 / tau).view(T, heads, dim)
    want = P.gla_recurrence(q.to(D) * dim ** -0.5, k.to(D), v.to(D), alpha).float()
    forgot = P.gla_recurrence(q[1:].to(D) * dim ** -0.5, k[1:].to(D), v[1:].to(D), alpha[1:]).float()
    assert (want[-1] - forgot[-1]).abs().max() > 1e-2  # (the last token still feels the first)
    state = torch.zeros(3, heads * vdim * dim, device=device)
    state[1] = 7.0  # another request's slot: left alone
    got, decays, at = [], [], 0
    for n in [1, 17, 2, 8, 1, 1, 16, 9, 6]:
        # the request (slot 2) beside a stranger (slot 0) that brings 3 tokens of noise
        ctx = _ctx([3, n], [0, at], device, slots=[0, 2])
        rows = lambda x, w: torch.cat([torch.randn(3, w, generator=g), x[at: at + n].reshape(n, -1)]).to(device)  # noqa: E731
        # the low-rank input sits in the last columns of a wider buffer, as in the mixer
        wide = torch.cat([torch.zeros(3 + n, 2, device=device), rows(y, rank)], dim=1)
        decay = torch.zeros(3 + n, heads * dim, device=device)
        ops.lowrank_decay(wide[:, 2:], w2.to(device), bias.to(device), tau, decay)
        out = torch.zeros(3 + n, heads * vdim, device=device)
        ops.gated_recurrence(rows(q, heads * dim), decay, rows(k, heads * dim), None, rows(v, heads * vdim), state,
                             ctx.slots, ctx, out, heads, dim, vdim, vdim, dim ** -0.5)
        got.append(out[3:].cpu().view(n, heads, vdim))
        decays.append(decay[3:].cpu().view(n, heads, dim))
        at += n
    torch.testing.assert_close(torch.cat(decays), alpha.float(), atol=2e-6, rtol=2e-6)
    torch.testing.assert_close(torch.cat(got), want, atol=3e-4, rtol=3e-4)
    assert torch.all(state[1] == 7.0)


@pytest.mark.parametrize("device", DEVICES)
@pytest.mark.parametrize("heads,vdim", [(3, 20), (1, 3), (5, 64), (2, 200)])
def test_read_out_norm_with_a_silu_gate(device, heads, vdim):
    ops, g = _ops(device), torch.Generator().manual_seed(vdim)
    n, eps, D = 9, 1e-5, torch.float64
    o = torch.randn(n, heads, vdim, generator=g) * 4
    w = torch.randn(vdim, generator=g) + 1  # one weight for every head
    pre = torch.randn(n, heads * vdim, generator=g) * 2
    want = (P.rms(o.to(D), eps) * w.to(D)).reshape(n, -1) * (pre.to(D) * torch.sigmoid(pre.to(D)))
    for dtype, tol in ((torch.float32, 1e-5), (torch.bfloat16, 2e-2)):
        out = torch.zeros(n, heads * vdim, device=device, dtype=dtype)
        wide = torch.cat([torch.zeros(n, 5), pre], dim=1).to(device)  # (the gate is a view of a wider buffer)
        ops.recurrence_readout(o.reshape(n, -1).to(device), None, w.to(device), eps, wide[:, 5:], out, heads, vdim,
                               vdim, gate_act="silu")
        torch.testing.assert_close(out.float().cpu(), want.float(), atol=tol, rtol=tol)


@pytest.mark.parametrize("device", DEVICES)
@pytest.mark.parametrize("inter", [1, 24, 30, 1096, 5000])
def test_polynorm_activation(device, inter):
    """a N(z) + b N(z^2) + c N(z^3) + e with each power divided by its own root mean square; rows of
    very different sizes, so that a norm shared between the powers or taken over the batch shows."""
    ops, g = _ops(device), torch.Generator().manual_seed(inter)
    n, eps, D = 6, 1e-5, torch.float64
    z = torch.randn(n, inter, generator=g) * torch.tensor([0.01, 0.3, 1.0, 3.0, 10.0, 1e-4])[:, None]
    coeff = torch.tensor([0.8, -0.6, 0.45, 0.1])
    want = P.polynorm(z.to(D), coeff.to(D), eps).float()
    out = torch.zeros(n, inter, device=device)
    ops.polynorm(z.to(device), coeff.to(device), eps, out)
    torch.testing.assert_close(out.cpu(), want, atol=2e-5, rtol=2e-5)
    out16 = torch.zeros(n, inter, device=device, dtype=torch.bfloat16)
    ops.polynorm(z.to(device), coeff.to(device), eps, out16)
    torch.testing.assert_close(out16.float().cpu(), want, atol=2e-2, rtol=2e-2)
    # the rows may be the first columns of a wider product
    wide = torch.cat([z, torch.full((n, 7), 50.0)], dim=1).to(device)
    out_w = torch.zeros(n, inter, device=device)
    ops.polynorm(wide[:, :inter], coeff.to(device), eps, out_w)
    torch.testing.assert_close(out_w.cpu(), want, atol=2e-5, rtol=2e-5)


@pytest.mark.parametrize("device", DEVICES)
@pytest.mark.parametrize("hidden", [50, 72, 1100])
def test_gated_add_and_norm_in_one_kernel(device, hidden):
    """h += sigmoid(W h' + b) * delta and the next norm of h, with the delta whole or in two partial
    sums, with and without a bias, for all rows or for chosen ones (then h stays as it is), and
    without a following norm."""
    ops, g = _ops(device), torch.Generator().manual_seed(hidden)
    n, eps, D = 7, 1e-5, torch.float64
    h, delta = torch.randn(n, hidden, generator=g), torch.randn(2, n, hidden, generator=g) * 3
    pre, bias, w = torch.randn(n, hidden, generator=g) * 2, torch.randn(hidden, generator=g), torch.randn(hidden, generator=g)
    for b in (bias, None):
        gate = torch.sigmoid(pre.to(D) + (0 if b is None else b.to(D)))
        dev_b = None if b is None else b.to(device)
        for parts in (delta, delta[0]):
            whole = parts.to(D).sum(0) if parts.dim() == 3 else parts.to(D)
            h_want = h.to(D) + gate * whole
            out_want = P.rms(h_want, eps) * w.to(D)
            hd, out = h.clone().to(device), torch.zeros(n, hidden, device=device)
            ops.gated_add_norm(hd, parts.to(device), pre.to(device), dev_b, w.to(device), eps, out)
            torch.testing.assert_close(hd.cpu(), h_want.float(), atol=1e-5, rtol=1e-5)
            torch.testing.assert_close(out.cpu(), out_want.float(), atol=1e-5, rtol=1e-5)
            rows = torch.tensor([5, 0], dtype=torch.int32, device=device)
            hd2, out2 = h.clone().to(device), torch.zeros(2, hidden, device=device)
            ops.gated_add_norm(hd2, parts.to(device), pre.to(device), dev_b, w.to(device), eps, out2, rows)
            torch.testing.assert_close(out2.cpu(), out_want.float()[[5, 0]], atol=1e-5, rtol=1e-5)
            assert torch.equal(hd2.cpu(), h)
            hd3 = h.clone().to(device)
            ops.gated_add_norm(hd3, parts.to(device), pre.to(device), dev_b, None, 0.0, None)
            torch.testing.assert_close(hd3.cpu(), h_want.float(), atol=1e-5, rtol=1e-5)
            # the gate may be some columns of a wider product (on a 16-byte boundary or not)
            for lead in (4, 3):
                wide = torch.cat([torch.full((n, lead), 9.0), pre, torch.full((n, 2), 9.0)], dim=1).to(device)
                hd5, out5 = h.clone().to(device), torch.zeros(n, hidden, device=device)
                ops.gated_add_norm(hd5, parts.to(device), wide[:, lead: lead + hidden], dev_b, w.to(device), eps, out5)
                torch.testing.assert_close(hd5.cpu(), h_want.float(), atol=1e-5, rtol=1e-5)
                torch.testing.assert_close(out5.cpu(), out_want.float(), atol=1e-5, rtol=1e-5)
            # the gate's product may arrive in parts too
            halves = torch.stack([pre * 0.25, pre * 0.75]).to(device)
            hd4, out4 = h.clone().to(device), torch.zeros(n, hidden, device=device)
            ops.gated_add_norm(hd4, parts.to(device), halves, dev_b, w.to(device), eps, out4)
            torch.testing.assert_close(hd4.cpu(), h_want.float(), atol=1e-5, rtol=1e-5)
            torch.testing.assert_close(out4.cpu(), out_want.float(), atol=1e-5, rtol=1e-5)


@pytest.mark.parametrize("device", DEVICES)
@pytest.mark.parametrize("experts,top", [(9, 3), (5, 1), (3, 3), (2, 1), (7, 6), (64, 8)])
def test_router_with_a_bias_weighs_only_the_chosen(device, experts, top):
    """The bias decides who is chosen (it is as large as the logits), and the weights are the
    softmax over the chosen logits alone."""
    ops, g = _ops(device), torch.Generator().manual_seed(experts)
    n, hidden, D = 33, 40, torch.float64
    x = torch.randn(n, hidden, generator=g)
    W = {"r.router": torch.randn(experts, hidden, generator=g) / hidden ** 0.5 * 2,
         "r.router.b": torch.randn(experts, generator=g) * 2}
    ids_want, w_want = P.route(x.to(D), {k: t.to(D) for k, t in W.items()}, "r", top)
    no_bias = P.route(x.to(D), {"r.router": W["r.router"].to(D), "r.router.b": torch.zeros(experts, dtype=D)}, "r", top)[0]
    if top < experts:
        assert not torch.equal(ids_want.sort(-1).values, no_bias.sort(-1).values)
    ids = torch.zeros(n, top, dtype=torch.int32, device=device)
    weights = torch.zeros(n, top, device=device)
    ops.route_topk(x.to(device), W["r.router"].to(device), 1, 1, ids, weights, bias=W["r.router.b"].to(device))
    got = torch.zeros(n, experts).scatter_(1, ids.long().cpu(), weights.cpu())
    want = torch.zeros(n, experts, dtype=D).scatter_(1, ids_want, w_want).float()
    torch.testing.assert_close(got, want, atol=1e-5, rtol=1e-5)
    torch.testing.assert_close(weights.sum(-1).cpu(), torch.ones(n), atol=1e-5, rtol=1e-5)


@pytest.mark.parametrize("device", DEVICES)
def test_biases_unit_values_and_cache_rows(device):
    """Queries, keys and values take their biases; each value head is divided by its root mean square
    before it is cached; nothing is rotated; rows land where the slot mapping says."""
    ops, g = _ops(device), torch.Generator().manual_seed(8)
    n, H, G, d, dv, ps, eps, D = 9, 3, 2, 10, 14, 4, 1e-5, torch.float64
    size = (H + G) * d + G * dv
    proj = torch.randn(n, size + H, generator=g)  # (the head gates' columns follow and are left alone)
    bias = torch.randn(size, generator=g)
    pos = torch.tensor([0, 1, 2, 3, 17, 18, 19, 5, 6])
    full = proj[:, :size].to(D) + bias.to(D)
    q = full[:, : H * d]
    k = full[:, H * d: (H + G) * d].view(n, G, d)
    v = P.rms(full[:, (H + G) * d:].view(n, G, dv), eps)
    q_out = torch.zeros(n, H * d, device=device)
    kc, vc = torch.zeros(9, G, ps, d, device=device), torch.zeros(9, G, ps, dv, device=device)
    slots = torch.tensor([p + 8 for p in pos.tolist()], dtype=torch.int32, device=device)  # pages 2..6
    ops.qk_norm_rope_write(proj.to(device), pos.to(torch.int32).to(device), None, 0, None, None, eps, q_out, kc, vc,
                           slots, H, G, d, dv, ps, bias=bias.to(device), value_norm=True)
    torch.testing.assert_close(q_out.cpu(), q.float(), atol=1e-6, rtol=1e-6)
    for i, s in enumerate(slots.tolist()):
        torch.testing.assert_close(kc[s // ps, :, s % ps].cpu(), k[i].float(), atol=1e-6, rtol=1e-6)
        torch.testing.assert_close(vc[s // ps, :, s % ps].cpu(), v[i].float(), atol=1e-5, rtol=1e-5)
        torch.testing.assert_close(vc[s // ps, :, s % ps].cpu().pow(2).mean(-1), torch.ones(G), atol=1e-3, rtol=1e-3)


@pytest.mark.parametrize("device", DEVICES)
def test_embedding_rows_times_the_scale(device):
    ops, g = _ops(device), torch.Generator().manual_seed(2)
    table = torch.randn(23, 50, generator=g)
    ids = torch.tensor([0, 22, 7, 7, 13], dtype=torch.int32)
    for dtype in (torch.float32, torch.bfloat16):
        t = table.to(dtype)
        out = torch.zeros(5, 50, device=device)
        ops.embedding(t.to(device), ids.to(device), out, 1.7)
        want = P.embed(ids.tolist(), {"embed": t.double()}, {"embedding": {"scale": 1.7}}).float()
        torch.testing.assert_close(out.cpu(), want, atol=1e-6, rtol=1e-6)


# --- long decoding and generation through the engine ------------------------------------------------


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_long_decoding_through_state_and_pages(tmp_path, dtype):
    """400 tokens decoded one by one after a short prompt, across many windows and pages: the
    recurrent states and the cached rows carry what they must, and pages behind the windows go back
    (the pool is smaller than the sequence)."""
    from inference_engine_b200.kernels import get_ops

    cfg = V.MIXED
    weights = V.make_weights(cfg, seed=3)
    toks = _requests(cfg, [410], seed=5)["r0"]
    want = P.forward(cfg, weights, toks, torch.float64).float()
    session = _session(tmp_path, cfg, weights, dtype, "cuda", get_ops("cuda"), 448, 16)
    got = H.collect(session, H.trace_decode_tail({"a": toks}, 400))["a"]
    H.assert_close(got, want, LABEL[dtype], "long decoding", _bound(tmp_path, dtype, cfg, weights, {"a": toks}, {"a": want}))


def _greedy_plain(cfg, weights, prompt, count):
    ids = list(prompt)
    for _ in range(count):
        ids.append(int(P.forward(cfg, weights, ids, torch.float64)[-1].argmax()))
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

    cfg = V.ATTENTION_FIRST
    weights = V.make_weights(cfg, seed=4)
    _, prompts, got = _generate(cfg, weights, "cpu", ops=RefOps())
    for rid, prompt in prompts.items():
        assert got[rid] == _greedy_plain(cfg, weights, prompt, 10), rid


@pytest.mark.gpu
@pytest.mark.parametrize("name", ["mixed", "odd"])
def test_greedy_generation_through_the_engine(name):
    """`LLMEngine` with the scheduler cutting prompts into portions and batching requests (three at
    a time, so state slots and pages serve one request after another), decode steps captured and
    launched ahead: the tokens are the plain implementation's greedy choices."""
    cfg = V.CONFIGS[name]
    weights = V.make_weights(cfg, seed=4)
    engine, prompts, got = _generate(cfg, weights, "cuda")
    assert engine.graphs is not None  # decode steps are captured, with per-request state too
    for rid, prompt in prompts.items():
        assert got[rid] == _greedy_plain(cfg, weights, prompt, 10), rid


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_captured_short_steps_with_portions(tmp_path, dtype):
    """Portions and mixed batches replayed through captured launch sequences (launched for bounds,
    padded with tokens that belong to no request): key and value sizes the tensor-core attention
    takes, so in bfloat16 that kernel runs sized by the token bound.  Against the plain
    implementation; in 32-bit equal bit for bit to the eagerly launched steps."""
    from inference_engine_b200.engine.graphs import DecodeGraphs, MixedGraphs
    from inference_engine_b200.kernels import get_ops

    cfg = V.config(64, 89, [
        (V.gla(2, 16, 24, tau=6.0), V.dense(48)),
        (V.attention(4, 2, 16, 32, window=24), V.moe(4, 2, 24)),
        (V.attention(2, 1, 32, 16, window=9), None),
        (V.gla(3, 8, 8, tau=2.0), V.dense(40)),
    ])
    weights = V.make_weights(cfg, seed=6, ranks={0: 4, 3: 6})
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
