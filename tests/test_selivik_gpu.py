"""The Selivik design on the GPU against the plain implementation
(tests/plain_selivik.py): every mechanism alone, then whole models through the
engine's step function, cut and batched in every way, then greedy generation
through the scheduler.

float32 must match every row closely; bfloat16 is held to the rounding of
bfloat16 operands in front of the products (a few 1e-2 of a row's length), and
where experts are routed to most rows (a choice at a near tie may flip under
that rounding).  Where random inputs would hide a fault (one far key, a
window's edge, the kept first positions, a sink), inputs are made so that it
shows, and the test checks on the plain side that they do.
"""
from __future__ import annotations

import numpy as np
import pytest
import torch

import plain_selivik as plain
from helpers import run_trace_on_engine, trace_mixed, trace_portions, trace_tail_decoded, trace_whole
from potivik_helpers import PartHarness, ids_for, make_part, rel_rows
from selivik_helpers import (CFG_A, CFG_B, CFG_C, CFG_D, CONFIGS, att, build, dense, lat, make_weights, moe, one_layer,
                             part_spec, random_config)

pytestmark = pytest.mark.gpu

DTYPES = {"float32": torch.float32, "bfloat16": torch.bfloat16}
TOL = {"float32": 2e-4, "bfloat16": 4e-2}
DEV = "cuda:0"
F64 = torch.float64


def gen(seed):
    return torch.Generator().manual_seed(seed)


def bf(t):
    return t.to(torch.bfloat16).to(torch.float32)


def dbl(W):
    return {k: v.double() for k, v in W.items()}


def check_rows(got, want, dtype: str, what: str = "", tol=None, most: bool = False):
    e = rel_rows(got, want)
    if dtype == "bfloat16":
        # a row that is short because its terms cancel (a head of one value, say) carries the rounding of terms
        # as long as other rows': it is measured against a typical row's length
        want64 = np.asarray(want, np.float64)
        lengths = np.linalg.norm(want64, axis=-1)
        e = np.linalg.norm(np.asarray(got, np.float64) - want64, axis=-1) / np.maximum(lengths, 0.3 * np.median(lengths) + 1e-30)
    tol = TOL[dtype] if tol is None else tol
    if most and dtype == "bfloat16":
        assert np.median(e) <= tol and (e <= tol).mean() >= 0.9 and e.max() <= 1.0, \
            f"{what}: median {np.median(e):.3g}, {(e > tol).sum()} of {e.size} rows beyond {tol}"
        return
    assert e.max() <= tol, f"{what}: row {int(e.argmax())} differs by {e.max():.3g} (tolerance {tol})"


def local(W, names: dict):
    """{local name: tensor} for a part whose plan binds local names to checkpoint names."""
    return {k: W[v] for k, v in names.items()}


def plain_mixer(cfg, i, W, h):
    lay = cfg["layers"][i]
    return plain.MIXERS[lay["type"]](h.double(), dbl(W), f"l{i}.mix.", lay["mixer"], float(cfg["norm"]["eps"]))


def part_of(cfg, i, W, dtype, role="mixer"):
    category, kind, params, names = part_spec(cfg, i, role)
    return make_part(category, kind, params, local(W, names), DTYPES[dtype])


def layers_of(kind):
    return [(cfg, i) for cfg in (CFG_A, CFG_B, CFG_C, CFG_D) for i, lay in enumerate(cfg["layers"]) if kind(lay)]


# ---------------------------------------------------------------------------
# mechanisms alone
# ---------------------------------------------------------------------------

@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("d", [44, 64, 336, 2100])
def test_norm_whose_weight_is_stored_around_zero(d, dtype):
    g = gen(1)
    w = bf(torch.randn(d, generator=g) * 0.2)
    x = torch.randn(9, d, generator=g) * 3.0
    part = make_part("norm", "rmsnorm_rows", {"dim": d, "eps": 1e-5, "gain_offset": 1.0}, {"weight": w}, DTYPES[dtype])
    got = part.forward(x.to(DEV)).float().cpu()
    want = plain.norm_around_zero(x.double(), w.double(), 1e-5)
    check_rows(got, want, dtype, tol=1e-6 if dtype == "float32" else 6e-3)
    # a weight of zero is a gain of one, not of zero
    assert rel_rows(want, plain.rms(x.double(), 1e-5) * w.double()).min() > 0.5


class Rows:
    """What a runner needs of a step when an operation only walks over rows."""
    def __init__(self, n):
        z = torch.zeros(1, dtype=torch.int32, device=DEV)
        self.n_tokens, self.n_requests, self.n_want, self.max_ctx_len = n, 1, 0, 1
        self.token_ids = self.tok_req = self.tok_pos = self.q_start = self.q_len = self.start_pos = self.want_rows = z


@pytest.mark.parametrize("d", [44, 46, 336, 1536, 5000])
@pytest.mark.parametrize("branches", [("mixer",), ("mixer", "ffn")])
def test_scaled_sum_of_branches_and_the_norm_behind_it(d, branches):
    from gibbs_b200.parts.base import Runtime
    from gibbs_b200.parts.runner import Eager
    g = gen(2)
    n, mult = (7 if d == 1536 else 70), 0.37               # (64 rows and more of up to 1,024 entries: a warp a row)
    scales = {b: bf(1.0 + 0.4 * torch.randn(d, generator=g)) for b in branches}
    x, ys = torch.randn(n, d, generator=g), [torch.randn(n, d, generator=g) for _ in branches]
    part = make_part("branch_sum", "scaled_sum", {"dim": d, "mult": mult, "branches": branches}, scales)
    norm = make_part("norm", "rmsnorm_rows", {"dim": d, "eps": 1e-5, "gain_offset": 1.0},
                     {"weight": bf(torch.randn(d, generator=g) * 0.2)})
    want = x.double() + mult * sum(scales[b].double() * y.double() for b, y in zip(branches, ys))
    for then in (None, norm):
        xs = x.to(DEV).clone()
        h = part.add(Eager(Runtime(torch.float32, torch.device(DEV)), Rows(n)), xs, [y.to(DEV) for y in ys], then=then)
        assert rel_rows(xs.cpu(), want).max() < 1e-6
        if then is not None:
            assert rel_rows(h.cpu(), plain.rms(want, 1e-5) * (1.0 + norm.gain.cpu().double() - 1.0)).max() < 1e-5


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("cfg,layer", layers_of(lambda lay: True))
def test_mixer_alone_whole_cut_and_decoded(cfg, layer, dtype):
    """One mixer with a cache of its own: the whole input at once, in portions down to two tokens and one, and
    with its last 45 tokens one by one; twelve pages, so pages come back and go out again."""
    d = cfg["width"]
    W = make_weights(cfg, 5)
    part = part_of(cfg, layer, W, dtype)
    T = 150
    h = bf(torch.randn(T, d, generator=gen(6)))
    want = plain_mixer(cfg, layer, W, h)
    hz = PartHarness(part, n_pages=12, page_size=16, n_slots=2)
    for rid, cuts in (("whole", [T]), ("cut", [2, 3, 17, 2, 31, 16, 1, 5, 64, 7]), ("decoded", [T - 45, 1])):
        got = hz.run_cut(rid, h, cuts)
        check_rows(got, want, dtype, what=f"{cfg['layers'][layer]['type']}, {rid}")
        hz.close(rid)


def _matters(fn, h, hot, query):
    """How much the plain output at ``query`` moves when the input at ``hot`` is replaced."""
    h2 = h.clone()
    h2[hot] = bf(torch.randn(h.shape[1], generator=gen(99)))
    a, b = fn(h)[query], fn(h2)[query]
    return float((a - b).norm() / a.norm())


def _pointed_attention(window, keep_first, T, hot, query, vdim=8, seed=7):
    """An attention whose query at ``query`` points at the key of ``hot``: that score stands far above all others.
    Keys read the input's first 32 entries, queries the next 32, so the query token's own key is an ordinary one."""
    d, H, G, dim = 128, 2, 1, 32
    m = att(H, G, dim, vdim, 1.0, window=window, keep_first=keep_first, softcap=50.0, rot=(10000.0, 8), factor=2.0)
    g = gen(seed)
    W = {"q": torch.zeros(H * dim, d), "k": torch.zeros(G * dim, d), "v": bf(torch.randn(G * vdim, d, generator=g) / 8),
         "q.b": torch.zeros(H * dim), "k.b": torch.zeros(G * dim), "v.b": torch.zeros(G * vdim),
         "sink": torch.tensor([1.0, -2.0]), "o": bf(torch.randn(d, H * vdim, generator=g) / 4)}
    for i in range(dim):
        W["k"][i, i] = 1.0
        for hh in range(H):
            W["q"][hh * dim + i, 32 + i] = 1.0
    h = bf(torch.randn(T, d, generator=g))
    h[query, 32:32 + dim] = h[hot, :dim]
    # (the first 8 entries turn with the position: the rest, 24 of 32 entries, carries the score)
    h[query, 32:40] = 0.0
    return m, W, h


POINTED = [
    # window, kept first, tokens, hot key, query
    (44, 5, 120, 56, 99),         # the last position inside the window
    (44, 5, 120, 55, 99),         # the first one outside
    (44, 5, 120, 4, 99),          # the last kept first position
    (44, 5, 120, 5, 99),          # the first one that is not kept
    (44, 5, 120, 0, 99),          # the first token of the sequence
    (44, 0, 120, 0, 99),          # ... which a window without kept positions does not see
    (44, 5, 120, 0, 30),          # a query whose window still reaches the start
    (16, 17, 120, 16, 95),        # kept positions beyond a page: the first row of the second page
    (16, 17, 120, 17, 95),
    (16, 16, 120, 80, 95),        # a window of one page
    (16, 16, 120, 79, 95),
    (64, 32, 200, 128, 191),      # a window of one key tile of the tensor-core kernel, kept: one tile of the generic
    (64, 32, 200, 127, 191),
    (64, 32, 200, 31, 191),
    (64, 32, 200, 32, 191),
    (100, 70, 300, 69, 299),      # more kept positions than a key tile
    (100, 70, 300, 70, 299),
    (100, 70, 300, 200, 299),
    (100, 70, 300, 199, 299),
    (7, 30, 120, 29, 60),         # more kept positions than the window is long
    (7, 30, 120, 30, 60),
    (1, 1, 50, 0, 40),            # a window of the position itself
    (1, 1, 50, 39, 40),
    (None, None, 400, 3, 399),    # no window: a key hundreds of positions back
    (None, None, 400, 16, 399),   # ... at a page's first row
    (None, None, 400, 63, 399),   # ... at a key tile's last row
]


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("decoded", [False, True])
@pytest.mark.parametrize("vdim", [8, 32])                     # 32: in bfloat16 the tensor-core kernel runs
@pytest.mark.parametrize("window,keep_first,T,hot,query", POINTED)
def test_attention_finds_the_one_key_that_matters(window, keep_first, T, hot, query, vdim, decoded, dtype):
    m, W, h = _pointed_attention(window, keep_first, T, hot, query, vdim)
    cfg = one_layer("attention", m, h.shape[1])
    fn = lambda x: plain.attention(x.double(), dbl(W), "", m, 1e-5)
    want = fn(h)
    visible = window is None or query - hot < window or hot < (keep_first or 0)
    moved = _matters(fn, h, hot, query)
    assert (moved > 0.3) == visible, f"the inputs do not show it: visible={visible}, moved {moved:.3g}"
    category, kind, params, _ = part_spec(cfg, 0, "mixer")
    part = make_part(category, kind, params, W, DTYPES[dtype])
    hz = PartHarness(part, n_pages=32, page_size=16)
    got = hz.run_cut("r", h, [query - 10, 1] if decoded else [T])
    e = rel_rows(got, want)
    loose = TOL[dtype] if dtype == "float32" else 0.1
    assert e[query] <= (TOL[dtype] if visible else loose), f"query row differs by {e[query]:.3g}"
    assert e.max() <= loose


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_the_sink_the_cap_and_the_norm_behind_the_rotation_show(dtype):
    """The first rows see few keys, so the sink weighs most there; scores far beyond the cap; heads of unequal
    length, which a norm per head makes equal: each changes the plain output, and the engine follows."""
    m = att(4, 2, 16, 12, 2.0, window=30, keep_first=2, softcap=4.0, rot=(100.0, 16), factor=1.0)
    cfg = one_layer("attention", m, 64)
    W = make_weights(cfg, 3)
    Wm = {k[len("l0.mix."):]: v for k, v in W.items() if k.startswith("l0.mix.")}
    h = bf(torch.randn(80, 64, generator=gen(4)) * 2.0)
    want = plain.attention(h.double(), dbl(Wm), "", m, 1e-5)
    no_sink = dict(dbl(Wm), sink=torch.full((4,), -1e9, dtype=F64))
    assert rel_rows(plain.attention(h.double(), no_sink, "", m, 1e-5)[:3], want[:3]).max() > 0.05
    assert rel_rows(plain.attention(h.double(), dbl(Wm), "", dict(m, softcap=None), 1e-5), want).max() > 0.05
    # (the sink is not capped: a sink beyond the cap still differs from one at the cap)
    big = dict(dbl(Wm), sink=torch.full((4,), 9.0, dtype=F64))
    at_cap = dict(dbl(Wm), sink=torch.full((4,), 4.0, dtype=F64))
    assert rel_rows(plain.attention(h.double(), big, "", m, 1e-5), plain.attention(h.double(), at_cap, "", m, 1e-5)).max() > 0.05
    for sink in (Wm["sink"], torch.full((4,), 9.0)):
        Ws = dict(Wm, sink=sink)
        category, kind, params, _ = part_spec(cfg, 0, "mixer")
        part = make_part(category, kind, params, Ws, DTYPES[dtype])
        hz = PartHarness(part, n_pages=16, page_size=16)
        for rid, cuts in (("whole", [80]), ("decoded", [1])):
            check_rows(hz.run_cut(rid, h, cuts), plain.attention(h.double(), dbl(Ws), "", m, 1e-5), dtype, what=rid)
            hz.close(rid)


def _pointed_latent(T, hot, query, seed=11):
    """A latent attention whose query at ``query`` is the latent of ``hot``: that score stands far above the rest.
    The queries' latent passes the input's entries 64.. through; the gate reads entries 96.. ."""
    d, H, dim, dr, vdim, r, rq = 128, 2, 32, 4, 8, 32, 32
    m = lat(H, dim, dr, vdim, r, rq, 1.0)
    g = gen(seed)
    W = {"dq": torch.zeros(rq, d), "dq.norm": torch.ones(rq), "uq": torch.zeros(H * (dim + dr), rq),
         "dkv": torch.zeros(r + dr, d), "dkv.norm": torch.ones(r), "uk": torch.zeros(H * dim, r),
         "uv": bf(torch.randn(H * vdim, r, generator=g) / 4), "g": bf(torch.randn(H * vdim, d, generator=g) / 6),
         "o": bf(torch.randn(d, H * vdim, generator=g) / 4)}
    W["g"][:, :96] = 0.0
    for i in range(r):
        W["dkv"][i, i] = 1.0
        W["dq"][i, 64 + i] = 1.0
        for hh in range(H):
            W["uk"][hh * dim + i, i] = 1.0
            W["uq"][hh * (dim + dr) + i, i] = 1.0
    for j in range(dr):                                     # a small rotated part on both sides
        W["dkv"][r + j] = bf(torch.randn(d, generator=g) / 40)
        for hh in range(H):
            W["uq"][hh * (dim + dr) + dim + j] = bf(torch.randn(rq, generator=g) / 20)
    h = bf(torch.randn(T, d, generator=g))
    h[query, 64:64 + r] = h[hot, :r]                        # normed, query and latent agree: score 32 against about +-6
    return m, W, h


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("decoded", [False, True])
@pytest.mark.parametrize("T,hot,query", [(400, 0, 399), (400, 3, 399), (400, 16, 399), (400, 31, 399), (400, 32, 399),
                                         (120, 47, 48), (700, 1, 650)])
def test_latent_attention_finds_a_far_key_and_its_gate_shows(T, hot, query, decoded, dtype):
    m, W, h = _pointed_latent(T, hot, query)
    fn = lambda x: plain.latent_attention(x.double(), dbl(W), "", m, 1e-5)
    want = fn(h)
    assert _matters(fn, h, hot, query) > 0.3
    # a gate per output element is not a gate per head: the mean gate of a head gives another output
    gl = h.double() @ W["g"].double().T
    per_head = torch.sigmoid(gl).reshape(T, 2, 8).mean(-1, keepdim=True).expand(T, 2, 8).reshape(T, 16)
    ungated = plain.latent_attention(h.double(), dict(dbl(W), g=torch.zeros_like(W["g"], dtype=F64)), "", m, 1e-5) * 2.0
    assert rel_rows(want, ungated).max() > 0.05 and float((torch.sigmoid(gl) - per_head).abs().max()) > 0.1
    category, kind, params, _ = part_spec(one_layer("latent_attention", m, h.shape[1]), 0, "mixer")
    part = make_part(category, kind, params, W, DTYPES[dtype])
    hz = PartHarness(part, n_pages=48, page_size=16)
    got = hz.run_cut("r", h, [query - 10, 1] if decoded else [T])
    e = rel_rows(got, want)
    assert e[query] <= TOL[dtype], f"query row differs by {e[query]:.3g}"
    assert e.max() <= (TOL[dtype] if dtype == "float32" else 0.1)


def test_router_picks_by_logits_with_their_bias_and_weighs_by_the_chosen_ones_alone():
    """Inputs for which every clause decides: the bias changes who wins; the weights sum to one over the chosen
    and are not the softmax over all; choosing every expert gives the softmax over all."""
    d, E = 32, 6
    g = gen(5)
    for top in (1, 2, 6):
        f = moe(E, top, 16)
        cfg = one_layer("attention", att(1, 1, 8, 8, 0.3), d, mlp=f)
        W = make_weights(cfg, 6)
        W["l0.mlp.router.b"] = torch.tensor([0.0, 3.0, -3.0, 0.5, 0.0, -0.5])
        h = bf(torch.randn(50, d, generator=g))
        p = "l0.mlp."
        idx, wts = plain.route(h.double(), dbl(W), p, top)
        free_idx, _ = plain.route(h.double(), dict(dbl(W), **{p + "router.b": torch.zeros(E, dtype=F64)}), p, top)
        z = h.double() @ W[p + "router"].double().T + W[p + "router.b"].double()
        assert torch.allclose(wts.sum(-1), torch.ones(50, dtype=F64))
        if top < E:
            assert not torch.equal(idx.sort(-1).values, free_idx.sort(-1).values)
            assert (torch.softmax(z, -1).gather(1, idx) - wts).abs().max() > 0.05
        category, kind, params, names = part_spec(cfg, 0, "ffn")
        part = make_part(category, kind, params, local(W, names), torch.float32)
        got = PartHarness(part).feed("r", h)
        want = plain.experts(h.double(), dbl(W), p, f)
        check_rows(got, want, "float32", what=f"top {top}")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("cfg,layer", layers_of(lambda lay: lay["mlp"] is not None))
def test_feed_forward_alone_and_one_token_against_the_batch(cfg, layer, dtype):
    W = make_weights(cfg, 8)
    f = cfg["layers"][layer]["mlp"]
    part = part_of(cfg, layer, W, dtype, role="ffn")
    h = bf(torch.randn(70, cfg["width"], generator=gen(9)))
    p = f"l{layer}.mlp."
    want = plain.dense_unit(h.double(), dbl(W), p) if f["kind"] == "dense" else plain.experts(h.double(), dbl(W), p, f)
    hz = PartHarness(part)
    got = hz.feed("all", h)
    check_rows(got, want, dtype, most=f["kind"] == "moe")
    one = torch.cat([hz.feed(f"one{t}", h[t:t + 1]) for t in (0, 33, 69)], 0)
    check_rows(one, got[[0, 33, 69]], dtype, tol=1e-5 if dtype == "float32" else 2e-2, most=f["kind"] == "moe")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_batches_of_unequal_requests_through_one_mixer(dtype):
    """Three requests through each mixer in the same steps, portions beside single tokens, against each alone."""
    for cfg in (CFG_A, CFG_D):
        W = make_weights(cfg, 5)
        for layer in range(4):
            part = part_of(cfg, layer, W, dtype)
            hs = {rid: bf(torch.randn(n, cfg["width"], generator=gen(20 + n))) for rid, n in (("a", 70), ("b", 5), ("c", 33))}
            want = {rid: plain_mixer(cfg, layer, W, h) for rid, h in hs.items()}
            hz = PartHarness(part, n_pages=16, page_size=16, n_slots=3)
            at = {rid: 0 for rid in hs}
            got = {rid: [] for rid in hs}
            for st in ({"a": 40, "b": 1, "c": 2}, {"a": 1, "b": 1}, {"a": 1, "c": 30, "b": 2}, {"a": 28, "c": 1, "b": 1}):
                res = hz.feed_many({rid: hs[rid][at[rid]:at[rid] + n] for rid, n in st.items()})
                for rid, n in st.items():
                    got[rid].append(res[rid])
                    at[rid] += n
            for rid in hs:
                assert at[rid] == hs[rid].shape[0]
                check_rows(torch.cat(got[rid], 0), want[rid], dtype, what=f"layer {layer}, {rid}")


# (three query heads a kv head, keys of 32 and values of 96 entries, a window and kept positions that are no multiples
# of a page or a key tile)
CFG_TC = one_layer("attention", att(6, 2, 32, 96, 0.2, window=50, keep_first=13, softcap=10.0, rot=(1000.0, 16), factor=4.0), 96)


@pytest.mark.parametrize("cfg,layer", [(CFG_D, 0), (CFG_D, 2), (CFG_D, 4), (CFG_TC, 0)])
def test_tensor_core_attention_against_the_generic_kernel(cfg, layer, monkeypatch):
    """bfloat16: the two kernels read the same pages; the tensor-core one reads the queries in bfloat16 too.
    Whole, cut at odd places (tiles that straddle the window's and the kept positions' edges) and decoded."""
    from gibbs_b200.parts import gated_attention
    W = make_weights(cfg, 5)
    T = 300
    h = bf(torch.randn(T, cfg["width"], generator=gen(6)))
    want = plain_mixer(cfg, layer, W, h)
    outs = {}
    for tc in (True, False):
        monkeypatch.setattr(gated_attention, "USE_TENSOR_CORES", tc)
        part = part_of(cfg, layer, W, "bfloat16")
        hz = PartHarness(part, n_pages=24, page_size=16)
        for rid, cuts in (("whole", [T]), ("cut", [37, 2, 90, 1, 1, 64, 5]), ("decoded", [T - 40, 1])):
            outs[(tc, rid)] = hz.run_cut(rid, h, cuts)
            check_rows(outs[(tc, rid)], want, "bfloat16", what=f"tensor cores {tc}, {rid}")
            hz.close(rid)
    for rid in ("whole", "cut", "decoded"):
        assert not torch.equal(outs[(True, rid)], outs[(False, rid)])          # (two kernels did run)
        assert rel_rows(outs[(True, rid)], outs[(False, rid)]).max() < 2e-2


# ---------------------------------------------------------------------------
# whole models through the engine
# ---------------------------------------------------------------------------

_CACHE: dict = {}


def model_and_truth(name: str, dtype: str, lengths=(1, 2, 23, 61, 130)):
    """A model, some requests, and the plain implementation's logits for them."""
    key = (name, dtype)
    if key not in _CACHE:
        cfg, seed = CONFIGS[name]
        W, model = build(cfg, seed, dtype)
        reqs = {f"r{n}": ids_for(cfg, 100 + n, n) for n in lengths}
        tkey = ("truth", name)
        if tkey not in _CACHE:
            _CACHE[tkey] = {rid: plain.forward(cfg, W, ids).numpy() for rid, ids in reqs.items()}
        _CACHE[key] = (cfg, model, reqs, _CACHE[tkey])
    return _CACHE[key]


def engine_for(model, n_pages=64, page_size=16, max_requests=4, cap=512, **kw):
    from gibbs_b200 import Engine
    return Engine(model, n_pages=n_pages, page_size=page_size, max_requests=max_requests, max_step_tokens=cap,
                  max_context=cap, guard_cache=True, **kw)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B", "C", "D"])
def test_whole_decoded_and_cut_prompts_match_the_plain_implementation(name, dtype):
    cfg, model, reqs, truth = model_and_truth(name, dtype)
    eng = engine_for(model)
    assert eng.plan is not None, eng.plan_refusal
    for what, steps in (("whole", trace_whole(reqs)), ("decoded", trace_tail_decoded(reqs, tail=40)),
                        ("cut", trace_portions(reqs)), ("cut in twos", trace_portions(reqs, sizes=(2,)))):
        got = run_trace_on_engine(eng, steps)
        for rid in reqs:
            check_rows(got[rid], truth[rid], dtype, what=f"{name} {what} {rid}", most=True)


@pytest.mark.parametrize("name", ["A", "B", "C", "D"])
def test_layer_by_layer_in_float32(name):
    """The residual stream after every layer, through the parts' forward methods."""
    cfg, model, reqs, _ = model_and_truth(name, "float32")
    W = make_weights(cfg, CONFIGS[name][1])
    ids = reqs["r61"]
    _, layers = plain.forward(cfg, W, ids, streams=True)
    eng = engine_for(model, use_plan=False, use_graphs=False)
    seen = []
    originals = [b.forward for b in model.blocks]
    try:
        for b, orig in zip(model.blocks, originals):
            def fw(x, step, caches, orig=orig):
                orig(x, step, caches)
                seen.append(x.tensor().clone())
            b.forward = fw
        from gibbs_b200 import StepEntry
        eng.open("x")
        eng.step([StepEntry("x", ids, [len(ids) - 1])])
        eng.close("x")
    finally:
        for b in model.blocks:
            del b.forward
    assert len(seen) == len(cfg["layers"])
    for i, x in enumerate(seen):
        assert rel_rows(x.cpu(), layers[i]).max() <= 1e-4, f"layer {i}"


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B", "D"])
def test_plan_and_forward_methods_give_the_same_bits(name, dtype):
    cfg, model, reqs, _ = model_and_truth(name, dtype)
    steps = trace_mixed(reqs, capacity_tokens=320, seed=3)
    a = run_trace_on_engine(engine_for(model, n_pages=20), steps)
    b = run_trace_on_engine(engine_for(model, n_pages=20, use_plan=False, use_graphs=False), steps)
    for rid in reqs:
        assert np.array_equal(a[rid], b[rid]), rid


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B", "C", "D"])
def test_mixed_batches_with_pages_used_again(name, dtype):
    """Up to three live requests in a pool that holds little more than the live ones, portions beside single
    tokens: against the plain implementation, and against each request run alone."""
    cfg, model, reqs, truth = model_and_truth(name, dtype)
    more = dict(reqs)
    for k in range(4):                                        # more requests than the engine runs at a time
        more[f"again{k}"] = ids_for(cfg, 500 + k, 40 + 17 * k)
    for seed in (0, 1):
        eng = engine_for(model, n_pages=20, max_requests=3)   # 320 tokens of pages
        got = run_trace_on_engine(eng, trace_mixed(more, capacity_tokens=320, max_live=3, seed=seed))
        assert eng.cache.free_pages() == [20] * len(eng.cache.groups)
        for rid in reqs:
            check_rows(got[rid], truth[rid], dtype, what=f"{name} mixed {rid}", most=True)
        alone = run_trace_on_engine(engine_for(model), trace_whole(more))
        for rid in more:
            check_rows(got[rid], alone[rid], dtype, what=f"{rid}: batch against alone",
                       tol=1e-4 if dtype == "float32" else TOL[dtype], most=True)


@pytest.mark.parametrize("seed", [2, 5, 8, 13, 21, 34, 55, 89])
def test_random_configurations_in_float32(seed):
    """Sizes, options and the order of layers drawn at random, whole, cut, decoded and in mixed batches, against
    the plain implementation in float64."""
    from gibbs_b200.config import parse_config
    from gibbs_b200.parts.model import build_model
    from gibbs_b200.weights import TensorDict
    cfg = random_config(seed)
    W = make_weights(cfg, seed)
    model = build_model(parse_config(cfg).plan(), TensorDict({k: v.to(torch.bfloat16) for k, v in W.items()}),
                        torch.float32, DEV)
    reqs = {f"r{n}": ids_for(cfg, seed * 7 + n, n) for n in (1, 2, 37, 90)}
    truth = {rid: plain.forward(cfg, W, ids).numpy() for rid, ids in reqs.items()}
    for what, steps in (("whole", trace_whole(reqs)), ("cut", trace_portions(reqs)),
                        ("decoded", trace_tail_decoded(reqs, tail=30)),
                        ("mixed", trace_mixed(reqs, capacity_tokens=256, max_live=3, seed=seed))):
        eng = engine_for(model, n_pages=16, max_requests=3, cap=256)
        got = run_trace_on_engine(eng, steps)
        for rid in reqs:
            check_rows(got[rid], truth[rid], "float32", what=f"{what} {rid}", tol=3e-4)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_long_decoding_past_windows_and_pages(dtype):
    """260 tokens decoded one by one after a two-token prompt: every window edge, the end of the kept positions
    and every page edge is passed by single tokens (inside CUDA graphs), and pages a window has passed come back."""
    cfg, model, _, _ = model_and_truth("D", dtype)
    W = make_weights(cfg, CONFIGS["D"][1])
    ids = ids_for(cfg, 77, 262)
    truth = plain.forward(cfg, W, ids).numpy()
    eng = engine_for(model, n_pages=20)
    got = run_trace_on_engine(eng, trace_tail_decoded({"long": ids}, tail=260))
    e = rel_rows(got["long"], truth)
    if dtype == "float32":
        assert e.max() <= TOL[dtype], f"first wrong position {int(np.nonzero(e > TOL[dtype])[0][0])}"
    else:
        check_rows(got["long"], truth, dtype, most=True)
    assert min(eng.cache.free_pages()) == 20


def test_pages_behind_a_window_go_back_but_those_of_kept_positions_stay():
    """A request of 200 tokens in an engine whose windowed groups have far fewer pages than the request: the window's
    pages plus the kept first positions' plus a step's."""
    cfg, model, _, _ = model_and_truth("D", "float32")
    from gibbs_b200 import Engine
    probe = Engine(model, n_pages=4, max_requests=1, max_step_tokens=64, max_context=256)
    rules = sorted(str(g.window) + "/" + str(g.keep_first) for g in probe.cache.groups)
    assert rules == ["100/20", "48/4", "None/0"], rules
    # window 100 + 20 kept + a step of 30: 2 + 8 + 2 pages; window 48 + 4 kept: 1 + 4 + 3
    pools = {("window", 100, 20): 12, ("window", 48, 4): 8, None: 16}
    eng = Engine(model, n_pages=pools, page_size=16, max_requests=1, max_step_tokens=64, max_context=256, guard_cache=True)
    W = make_weights(cfg, CONFIGS["D"][1])
    ids = ids_for(cfg, 78, 200)
    truth = plain.forward(cfg, W, ids).numpy()
    got = run_trace_on_engine(eng, trace_portions({"r": ids}, sizes=(16, 1, 1, 30, 2)))
    check_rows(got["r"], truth, "float32", what="pages behind windows")


def test_greedy_generation_through_the_scheduler():
    """Generator -> Scheduler -> Engine.step -> sampler: the tokens are those the plain implementation
    picks, fed back one by one; several prompts of unequal length at once."""
    from gibbs_b200 import Generator, SamplingParams
    cfg, model, _, _ = model_and_truth("B", "float32")
    W = make_weights(cfg, CONFIGS["B"][1])
    gen_ = Generator(model, ctx=256, page_size=16, n_pages=40, max_running=4, max_batch_tokens=48)
    prompts = [ids_for(cfg, 900 + k, n) for k, n in enumerate((3, 50, 19))]
    outs = gen_.generate(prompts, SamplingParams(max_new_tokens=12, temperature=0.0), stop_at_eos=False)
    for p, out in zip(prompts, outs):
        seq = list(p)
        for tok in out:
            logits = plain.forward(cfg, W, seq)[-1]
            top2 = torch.topk(logits, 2).values
            if float(top2[0] - top2[1]) > 1e-3:               # (no verdict on a tie)
                assert int(logits.argmax()) == tok, f"after {len(seq)} tokens"
            seq.append(tok)
        assert len(out) == 12


def test_command_line_from_a_configuration_to_tokens(tmp_path, capsys):
    """config.json -> random weights on disk -> --arch-dump, --probe-top5 and a greedy continuation, all
    through the command line's own entry point."""
    import json
    from gibbs_b200.engine.cli import main
    cfg_path = tmp_path / "cfg.json"
    cfg_path.write_text(json.dumps(CFG_A))
    folder = tmp_path / "model"
    assert main(["--random", str(cfg_path), "--save", str(folder), "--seed", "3", "--dtype", "float32"]) == 0
    capsys.readouterr()
    assert main(["-m", str(folder), "--arch-dump"]) == 0
    dump = json.loads(capsys.readouterr().out)
    assert dump["architecture"] == "Selivik"
    prompt = ids_for(CFG_A, 5, 9)
    ids = ",".join(map(str, prompt))
    assert main(["-m", str(folder), "--dtype", "float32", "--probe-top5", ids, "--ctx", "128"]) == 0
    top = json.loads(capsys.readouterr().out)
    from gibbs_b200.weights import Checkpoint
    ck = Checkpoint(folder)
    W = {n: ck.tensor(n) for n in ck.names()}
    cfg = json.loads((folder / "config.json").read_text())
    logits = plain.forward(cfg, W, prompt)[-1]
    assert top["ids"][0] == int(logits.argmax())
    assert abs(top["logits"][0] - float(logits.max())) < 1e-3
    assert main(["-m", str(folder), "--dtype", "float32", "--prompt-ids", ids, "--max-tokens", "5", "--temperature", "0",
                 "--ctx", "128"]) == 0
    out = capsys.readouterr().out
    generated = [int(t) for t in out.split("Output:\n")[1].splitlines()[0].split(",")]
    assert len(generated) == 5 and generated[0] == top["ids"][0]


@pytest.mark.parametrize("heads,dim,rot_dim,vdim,kv_rank,q_rank", [(4, 16, 8, 16, 64, 24), (3, 8, 16, 20, 24, 8), (5, 24, 8, 8, 136, 40),
                                                                 (16, 32, 32, 32, 256, 96), (8, 32, 64, 16, 512, 64),
                                                                 (64, 8, 8, 8, 40, 16), (1, 16, 24, 16, 8, 16)])
def test_tensor_core_latent_attention_with_a_rotated_part_against_the_generic_kernel(heads, dim, rot_dim, vdim, kv_rank, q_rank,
                                                                                    monkeypatch):
    """bfloat16: the kernel that takes steps with portions of prompts, with cache rows of a latent and a rotated part
    (together 32 to 576 entries, also no multiples of 16), against the plain implementation and the generic kernel:
    whole, cut so that tiles end inside key tiles and pages, decoded, and a portion beside single tokens."""
    from gibbs_b200.parts import latent_attention
    cfg = one_layer("latent_attention", lat(heads, dim, rot_dim, vdim, kv_rank, q_rank, 0.3), 64)
    W = make_weights(cfg, 15)
    T = 330
    h = bf(torch.randn(T, 64, generator=gen(16)))
    want = plain_mixer(cfg, 0, W, h)
    outs = {}
    for tc in (True, False):
        monkeypatch.setattr(latent_attention, "USE_TENSOR_CORES", tc)
        part = part_of(cfg, 0, W, "bfloat16")
        hz = PartHarness(part, n_pages=64, page_size=16)
        for rid, cuts in (("whole", [T]), ("cut", [70, 9, 130, 1, 65, 55]), ("decoded", [T - 30, 1])):
            outs[(tc, rid)] = hz.run_cut(rid, h, cuts)
            # (the tensor-core kernel reads the absorbed queries in bfloat16 too: a little more where the latent is short)
            check_rows(outs[(tc, rid)], want, "bfloat16", what=f"tensor cores {tc}, {rid}", tol=5e-2)
            hz.close(rid)
        first = hz.feed_many({"a": h[:200], "b": h[:100]})
        second = hz.feed_many({"a": h[200:201], "b": h[100:T]})
        third = hz.feed_many({"a": h[201:T]})
        outs[(tc, "mixed a")] = torch.cat([first["a"], second["a"], third["a"]], 0)
        outs[(tc, "mixed b")] = torch.cat([first["b"], second["b"]], 0)
        check_rows(outs[(tc, "mixed a")], want, "bfloat16", what=f"tensor cores {tc}, mixed a", tol=5e-2)
        check_rows(outs[(tc, "mixed b")], want, "bfloat16", what=f"tensor cores {tc}, mixed b", tol=5e-2)
    assert not torch.equal(outs[(True, "whole")], outs[(False, "whole")])       # (two kernels did run)
    for rid in ("whole", "cut", "mixed a", "mixed b"):
        assert rel_rows(outs[(True, rid)], outs[(False, rid)]).max() < 5e-2


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_the_norm_taken_by_the_sum_in_front_of_it_changes_nothing(dtype, monkeypatch):
    """A layer's norm runs inside the kernel that completes the layer in front of it; built without that, the model
    gives the same logits up to the order in which a row's squares are added."""
    from gibbs_b200.parts import block
    cfg, seed = CONFIGS["D"]
    reqs = {f"r{n}": ids_for(cfg, 300 + n, n) for n in (1, 37, 90)}
    steps = trace_mixed(reqs, capacity_tokens=256, max_live=3, seed=2)
    outs = []
    for fuse in (True, False):
        monkeypatch.setattr(block, "FUSE_NEXT_NORM", fuse)
        _, model = build(cfg, seed, dtype)
        assert (model.blocks[0]._next is not None) == fuse
        eng = engine_for(model, n_pages=16, max_requests=3, cap=256)
        assert eng.plan is not None
        outs.append(run_trace_on_engine(eng, steps))
    for rid in reqs:
        check_rows(outs[0][rid], outs[1][rid], dtype, what=rid, tol=2e-5 if dtype == "float32" else TOL[dtype], most=True)


@pytest.mark.parametrize("act", ["gelu_tanh", "silu"])
@pytest.mark.parametrize("d,ff,rows", [(128, 256, 70), (96, 128, 5), (336, 64, 300), (64, 1024, 33)])
def test_gated_unit_in_the_epilogue_of_its_product_against_the_kernel_of_its_own(d, ff, rows, act, monkeypatch):
    """bfloat16, widths that are multiples of 64: gate and up are one tensor-core product whose epilogue applies
    act(g) * u in the form g * sigmoid(alpha * (g + cubic * g^3)); against the 32-bit product followed by the
    activation kernel (the named function itself), and against float64."""
    from gibbs_b200.parts import mlp
    g = gen(31)
    W = {"gate": bf(torch.randn(ff, d, generator=g) * (2.0 / d ** 0.5)), "up": bf(torch.randn(ff, d, generator=g) / d ** 0.5),
         "down": bf(torch.randn(d, ff, generator=g) / ff ** 0.5)}
    h = bf(torch.randn(rows, d, generator=g) * 1.5)
    z = h.double() @ W["gate"].double().T
    a = plain.gelu_tanh(z) if act == "gelu_tanh" else z * torch.sigmoid(z)
    want = (a * (h.double() @ W["up"].double().T)) @ W["down"].double().T
    outs = {}
    for fuse in (True, False):
        monkeypatch.setattr(mlp, "FUSE_GATED_UNIT", fuse)
        part = make_part("feed_forward", "gated_mlp", {"hidden": d, "inner": ff, "act": act}, W, torch.bfloat16)
        assert part.fused == fuse
        outs[fuse] = PartHarness(part).feed("r", h)
        check_rows(outs[fuse], want, "bfloat16", what=f"fused {fuse}", tol=1.5e-2)
    assert rel_rows(outs[True], outs[False]).max() < 1e-2


@pytest.mark.parametrize("heads,dim,rot_dim,vdim,kv_rank,q_rank", [(4, 16, 8, 16, 64, 24), (16, 8, 16, 8, 40, 16), (2, 16, 8, 16, 264, 16),
                                                                 (8, 16, 32, 16, 288, 32)])
def test_a_long_prompt_whose_key_tiles_two_blocks_share(heads, dim, rot_dim, vdim, kv_rank, q_rank):
    """bfloat16: a step of one long portion has few tiles of rows, so every tile's key tiles are cut in two halves
    whose partial results a second kernel merges; a row may see nothing of the second half.  Whole (700 tokens) and
    as a portion of 600 behind 100 tokens, against the plain implementation."""
    cfg = one_layer("latent_attention", lat(heads, dim, rot_dim, vdim, kv_rank, q_rank, 0.3), 64)
    W = make_weights(cfg, 17)
    T = 700
    h = bf(torch.randn(T, 64, generator=gen(18)))
    want = plain_mixer(cfg, 0, W, h)
    part = part_of(cfg, 0, W, "bfloat16")
    hz = PartHarness(part, n_pages=96, page_size=16)
    for rid, cuts in (("whole", [T]), ("behind", [100, 600])):
        check_rows(hz.run_cut(rid, h, cuts), want, "bfloat16", what=rid, tol=5e-2)
        hz.close(rid)
