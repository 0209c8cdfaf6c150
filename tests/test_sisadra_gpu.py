"""The Sisadra design on the GPU against the plain implementation
(tests/plain_sisadra.py): every mechanism alone, then whole models through the
engine's step function, cut and batched in every way, then greedy generation
through the scheduler.

float32 must match every row closely; bfloat16 is held to the rounding of
bfloat16 operands in front of the products (a few 1e-2 of a row's length).
Where random inputs would hide a fault (one far key, a block's edge, a sink,
the first tokens), inputs are made so that it shows, and the test checks on
the plain side that they do.
"""
from __future__ import annotations

import math

import numpy as np
import pytest
import torch

import plain_sisadra as plain
from helpers import run_trace_on_engine, trace_mixed, trace_portions, trace_tail_decoded, trace_whole
from potivik_helpers import PartHarness, ids_for, make_part, rel_rows
from sisadra_helpers import (CFG_A, CFG_B, CFG_C, CFG_D, CONFIGS, att, build, delta, lat, make_weights, mixer_part, one_layer,
                             random_config)

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


def check_rows(got, want, dtype: str, what: str = "", tol=None):
    e = rel_rows(got, want)
    tol = TOL[dtype] if tol is None else tol
    assert e.max() <= tol, f"{what}: row {int(e.argmax())} differs by {e.max():.3g} (tolerance {tol})"


def plain_mixer(cfg, i, W, h):
    layer = cfg["layers"][i]
    return plain.MIXERS[layer["type"]](h.double(), dbl(plain.sub(W, f"l{i}.mix.")), layer["mixer"], float(cfg["norm"]["eps"]))


def part_of(cfg, i, W, dtype):
    kind, params = mixer_part(cfg, i)
    return make_part("mixer", kind, params, plain.sub(W, f"l{i}.mix."), DTYPES[dtype])


# ---------------------------------------------------------------------------
# mechanisms alone
# ---------------------------------------------------------------------------

class EmbeddingHarness:
    """The pair embedding alone, with a cache manager and step builder of its own (the id before a
    portion is state in the request's slot)."""

    def __init__(self, part, n_slots=2):
        from gibbs_b200.cache import CacheManager
        from gibbs_b200.engine.step import StepBuilder
        self.part = part
        self.cache = CacheManager([(part.cache_needs(), None)], 4, 16, n_slots, part.rt.dtype, part.rt.device, 512, guard=True)
        self.builder = StepBuilder(self.cache, part.rt.device, n_slots, 512)

    def feed_many(self, portions: dict) -> dict:
        from gibbs_b200.engine.step import StepEntry
        rcs, entries = [], []
        for rid, ids in portions.items():
            if rid not in self.cache.live:
                self.cache.open(rid)
            rcs.append(self.cache.live[rid])
            entries.append(StepEntry(rid, list(ids), []))
        self.cache.reserve_all([(rc, rc.length + len(e.tokens)) for rc, e in zip(rcs, entries)])
        step, caches = self.builder.build(entries, rcs)
        out = self.part.forward(step.token_ids, step, caches[0])
        torch.cuda.synchronize()
        for rc, e in zip(rcs, entries):
            self.cache.advance(rc, rc.length + len(e.tokens))
        self.cache.check()
        res, at = {}, 0
        for rid, ids in portions.items():
            res[rid] = out[at:at + len(ids)].cpu()
            at += len(ids)
        return res


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("buckets,mul_prev,mul_cur", [(53, 7, 11), (1, 3, 5), (4093, 2000000011, 1999999973)])
def test_pair_embedding_carries_the_token_before_across_portions_and_slots(dtype, buckets, mul_prev, mul_cur):
    g = gen(1)
    V, d, scale = 77, 52, 3.0
    table, pairs = bf(torch.randn(V, d, generator=g)), bf(torch.randn(buckets + 1, d, generator=g))
    part = make_part("embedding", "pair_embedding", {"vocab": V, "dim": d, "scale": scale, "buckets": buckets,
                                                     "mul_prev": mul_prev, "mul_cur": mul_cur},
                     {"weight": table, "pairs": pairs}, DTYPES[dtype])
    seqs = {rid: torch.randint(0, V, (n,), generator=g).tolist() for rid, n in (("a", 40), ("b", 9), ("c", 23), ("d", 2))}
    want = {rid: plain.embed(ids, table.double(), scale, pairs.double(), buckets, mul_prev, mul_cur) for rid, ids in seqs.items()}
    # the first token's row is not the row the hash of (anything, token) gives
    hz = EmbeddingHarness(part, n_slots=2)
    got = {rid: [] for rid in seqs}
    # a and b side by side in unequal portions (b decodes); then c and d in the slots a and b leave
    plan = [{"a": 3, "b": 2}, {"a": 1, "b": 1}, {"b": 1}, {"a": 30, "b": 1}, {"a": 6, "b": 4}]
    plan2 = [{"c": 1, "d": 1}, {"c": 20, "d": 1}, {"c": 2}]
    at = {rid: 0 for rid in seqs}
    for group, steps in ((("a", "b"), plan), (("c", "d"), plan2)):
        for st in steps:
            res = hz.feed_many({rid: seqs[rid][at[rid]:at[rid] + n] for rid, n in st.items()})
            for rid, n in st.items():
                got[rid].append(res[rid])
                at[rid] += n
        for rid in group:
            assert at[rid] == len(seqs[rid])
            hz.cache.close(rid)
    for rid in seqs:
        out = torch.cat(got[rid], 0)
        assert out.dtype == torch.float32
        assert rel_rows(out, want[rid]).max() < 1e-6, rid
    first = plain.embed(seqs["c"][:1], table.double(), scale, pairs.double(), buckets, mul_prev, mul_cur)
    assert torch.allclose(first[0], table[seqs["c"][0]].double() * scale + pairs[buckets].double())


MIXER_CASES = [(CFG_A, 0), (CFG_A, 1), (CFG_A, 2), (CFG_A, 3), (CFG_B, 0), (CFG_B, 1), (CFG_B, 2), (CFG_B, 3), (CFG_B, 4),
               (CFG_C, 0), (CFG_C, 1), (CFG_C, 2), (CFG_C, 3), (CFG_D, 0), (CFG_D, 1), (CFG_D, 2), (CFG_D, 3), (CFG_D, 4)]


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("cfg,layer", MIXER_CASES)
def test_mixer_alone_whole_cut_and_decoded(cfg, layer, dtype):
    """One mixer with a cache of its own: the whole input at once, in portions down to two tokens and one, and
    with its last 45 tokens one by one; twelve pages and three slots, so pages and slots come back and go out again."""
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


# -- one key that matters ------------------------------------------------------------------

def _pointed_differential(block, T, hot, query, vdim=8, seed=7):
    """A differential attention whose first map, at the query position, scores ``hot`` far above all other
    keys, and whose second map is flat (its queries are zero).  Keys read the input's first 64 entries,
    queries its last 64, so the query token's own key is an ordinary one."""
    d, H, G, dim = 128, 2, 1, 32
    m = att(H, G, dim, vdim, 1.0, 0.3, block=block)
    g = gen(seed)
    W = {"q": torch.zeros(H * 2 * dim, d), "k": torch.zeros(G * 2 * dim, d), "v": bf(torch.randn(G * vdim, d, generator=g) / 8),
         "q.b": torch.zeros(H * 2 * dim), "k.b": torch.zeros(G * 2 * dim), "v.b": torch.zeros(G * vdim),
         "q.norm": torch.full((dim,), 1.5), "k.norm": torch.full((dim,), 1.5), "o": bf(torch.randn(d, H * vdim, generator=g) / 4),
         "o.b": torch.zeros(d)}
    for n in ("lq1", "lk1", "lq2", "lk2"):
        W[n] = bf(torch.randn(dim, generator=g) * 0.1)
    for i in range(dim):
        W["k"][i, i] = 1.0                     # map 1 of the keys; map 2 reads the next entries
        W["k"][dim + i, dim + i] = 1.0
        for hh in range(H):
            W["q"][hh * 2 * dim + i, 64 + i] = 1.0          # map 1 of every head; map 2 stays zero
    h = bf(torch.randn(T, d, generator=g))
    h[query, 64:64 + dim] = h[hot, :dim]       # normed, the query's first map is the hot key: score 72 against about +-13
    return m, W, h


POINTED = [
    (40, 120, 80, 99),        # the first position of the query's block
    (40, 120, 79, 99),        # the last one of the block before
    (40, 120, 0, 39),         # the first token of the sequence, in the same block
    (40, 120, 0, 40),         # ... and from the next block's first position
    (16, 120, 80, 95),        # blocks of one page
    (16, 120, 79, 95),
    (32, 120, 64, 95),        # blocks of one key tile
    (32, 120, 63, 95),
    (64, 200, 128, 191),
    (64, 200, 127, 191),
    (19, 120, 95, 113),       # blocks that are no multiple of a page: 95 = 5 * 19
    (19, 120, 94, 113),
    (None, 400, 3, 399),      # no mask: a key hundreds of positions back
    (None, 400, 16, 399),     # ... at a page's first row
    (None, 400, 31, 399),     # ... at a key tile's last row
    (300, 400, 300, 399),     # long blocks: far but inside
    (300, 400, 299, 399),     # ... and outside
]


def _matters(fn, h, hot, query):
    """How much the plain output at ``query`` moves when the input at ``hot`` is replaced."""
    h2 = h.clone()
    h2[hot] = bf(torch.randn(h.shape[1], generator=gen(99)))
    a, b = fn(h)[query], fn(h2)[query]
    return float((a - b).norm() / a.norm())


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("decoded", [False, True])
@pytest.mark.parametrize("vdim", [8, 32])                     # 32: in bfloat16 the tensor-core kernel runs
@pytest.mark.parametrize("block,T,hot,query", POINTED)
def test_differential_attention_finds_the_one_key_that_matters(block, T, hot, query, vdim, decoded, dtype):
    m, W, h = _pointed_differential(block, T, hot, query, vdim)
    cfg = one_layer("attention", m, h.shape[1])
    fn = lambda x: plain.differential_attention(x.double(), dbl(W), m, 1e-5)
    want = fn(h)
    visible = block is None or query // block == hot // block
    moved = _matters(fn, h, hot, query)
    assert (moved > 0.3) == visible, f"the inputs do not show it: visible={visible}, moved {moved:.3g}"
    kind, params = mixer_part(cfg, 0)
    part = make_part("mixer", kind, params, W, DTYPES[dtype])
    hz = PartHarness(part, n_pages=32, page_size=16)
    got = hz.run_cut("r", h, [query - 10, 1] if decoded else [T])
    e = rel_rows(got, want)
    # (scores eight times as wide as a model's: where no key stands out, the rounding of keys and queries to
    # bfloat16 shows in the sharp softmax)
    loose = TOL[dtype] if dtype == "float32" else 0.1
    assert e[query] <= (TOL[dtype] if visible else loose), f"query row differs by {e[query]:.3g}"
    assert e.max() <= loose


def _pointed_latent(T, hot, query, seed=11):
    """A latent attention whose query at ``query`` is the latent of ``hot``: that score stands far above the rest."""
    d, H, dim, vdim, r = 128, 2, 32, 8, 32
    m = lat(H, dim, vdim, r, 1.0)
    g = gen(seed)
    W = {"q": torch.zeros(H * dim, d), "dkv": torch.zeros(r, d), "dkv.norm": torch.ones(r), "uk": torch.zeros(H * dim, r),
         "uv": bf(torch.randn(H * vdim, r, generator=g) / 4), "sink": torch.tensor([2.0, -1.0]),
         "o": bf(torch.randn(d, H * vdim, generator=g) / 4)}
    for i in range(r):
        W["dkv"][i, i] = 1.0
        for hh in range(H):
            W["uk"][hh * dim + i, i] = 1.0
            W["q"][hh * dim + i, 64 + i] = 1.0
    h = bf(torch.randn(T, d, generator=g))
    c = h[hot, :r].double()
    h[query, 64:64 + r] = bf((c / c.pow(2).mean().sqrt()).float())      # score 32 against about +-6
    return m, W, h


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("decoded", [False, True])
@pytest.mark.parametrize("T,hot,query", [(400, 0, 399), (400, 3, 399), (400, 16, 399), (400, 31, 399), (400, 32, 399),
                                         (120, 47, 48), (700, 1, 650)])
def test_latent_attention_finds_a_far_key_and_its_sink_shows(T, hot, query, decoded, dtype):
    m, W, h = _pointed_latent(T, hot, query)
    fn = lambda x: plain.latent_attention(x.double(), dbl(W), m, 1e-5)
    want = fn(h)
    assert _matters(fn, h, hot, query) > 0.3
    # the sink shows: without it (a sink of -1e9 adds nothing) the first rows, which see few keys, differ
    no_sink = dict(dbl(W), sink=torch.full((2,), -1e9, dtype=F64))
    assert rel_rows(plain.latent_attention(h.double(), no_sink, m, 1e-5)[:3], want[:3]).max() > 0.05
    kind, params = mixer_part(one_layer("latent_attention", m, h.shape[1]), 0)
    part = make_part("mixer", kind, params, W, DTYPES[dtype])
    hz = PartHarness(part, n_pages=48, page_size=16)
    got = hz.run_cut("r", h, [query - 10, 1] if decoded else [T])
    e = rel_rows(got, want)
    assert e[query] <= TOL[dtype], f"query row differs by {e[query]:.3g}"
    assert e.max() <= (TOL[dtype] if dtype == "float32" else 0.1)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_delta_rule_remembers_the_first_token_over_hundreds_of_steps(dtype):
    """Decays close to one: what the first token wrote is still read 300 tokens later, whole and decoded; with
    strong decays it is not (both on the plain side, so that the comparison means something)."""
    d = 64
    m = delta(2, 1, 64, 8, 3, 4, 4)             # (keys of 64 entries: 300 later writes do not wipe the first one out)
    cfg = one_layer("channel_delta", m, d)
    W = plain.sub(make_weights(cfg, 3), "l0.mix.")
    W["A_log"] = torch.tensor([-9.0, -8.0])
    T = 300
    h = bf(torch.randn(T, d, generator=gen(4)))
    fn = lambda x: plain.channel_delta(x.double(), dbl(W), m, 1e-5)
    assert _matters(fn, h, 0, T - 1) > 0.02
    Wf = dict(W, A_log=torch.tensor([1.0, 1.5]))
    assert _matters(lambda x: plain.channel_delta(x.double(), dbl(Wf), m, 1e-5), h, 0, T - 1) < 1e-6
    want = fn(h)
    kind, params = mixer_part(cfg, 0)
    part = make_part("mixer", kind, params, W, DTYPES[dtype])
    hz = PartHarness(part, n_slots=2)
    for rid, cuts in (("whole", [T]), ("decoded", [2, 1]), ("cut", [7, 2, 50, 3])):
        check_rows(hz.run_cut(rid, h, cuts), want, dtype, what=f"delta rule, {rid}")
        hz.close(rid)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_batches_of_unequal_requests_through_one_mixer(dtype):
    """Three requests through each kind of mixer in the same steps, portions beside single tokens, against
    each request alone."""
    cfg = CFG_A
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


# (three query heads a kv head, keys of 32 and values of 96 entries, blocks of 50: no multiple of a page or key tile)
CFG_TC = one_layer("attention", att(6, 2, 32, 96, 0.2, 0.4, block=50, rot=(1000.0, 16), scaling=(4.0, 1.0, 4.0, 64)), 96)


@pytest.mark.parametrize("cfg,layer", [(CFG_D, 0), (CFG_D, 4), (CFG_TC, 0)])
def test_tensor_core_attention_against_the_generic_kernel(cfg, layer, monkeypatch):
    """bfloat16: the two kernels read the same pages; the tensor-core one reads the queries in bfloat16 too.
    Whole, cut at odd places (tiles that straddle blocks) and decoded."""
    from gibbs_b200.parts import diff_attention
    W = make_weights(cfg, 5)
    T = 300
    h = bf(torch.randn(T, cfg["width"], generator=gen(6)))
    want = plain_mixer(cfg, layer, W, h)
    outs = {}
    for tc in (True, False):
        monkeypatch.setattr(diff_attention, "USE_TENSOR_CORES", tc)
        part = part_of(cfg, layer, W, "bfloat16")
        hz = PartHarness(part, n_pages=24, page_size=16)
        for rid, cuts in (("whole", [T]), ("cut", [37, 2, 90, 1, 1, 64, 5]), ("decoded", [T - 40, 1])):
            outs[(tc, rid)] = hz.run_cut(rid, h, cuts)
            check_rows(outs[(tc, rid)], want, "bfloat16", what=f"tensor cores {tc}, {rid}")
            hz.close(rid)
    for rid in ("whole", "cut", "decoded"):
        assert not torch.equal(outs[(True, rid)], outs[(False, rid)])          # (two kernels did run)
        assert rel_rows(outs[(True, rid)], outs[(False, rid)]).max() < 2e-2


@pytest.mark.parametrize("heads,dim,vdim,kv_rank", [(4, 16, 16, 64), (3, 8, 20, 24), (5, 24, 8, 136), (16, 32, 32, 256),
                                                    (6, 16, 24, 320), (8, 32, 16, 512), (64, 8, 8, 40), (1, 16, 16, 8)])
def test_tensor_core_latent_attention_against_the_generic_kernel(heads, dim, vdim, kv_rank, monkeypatch):
    """bfloat16: every width class of the kernel that takes steps with portions of prompts (latents of 8 to 512
    entries, also no multiples of 64; 1 to 64 heads, also counts that do not divide a tile's 64 rows), against the
    plain implementation and the generic kernel: whole, cut so that tiles end inside key tiles and pages, decoded
    (which the generic kernel does either way), and a portion beside single tokens of another request."""
    from gibbs_b200.parts import latent_attention
    cfg = one_layer("latent_attention", lat(heads, dim, vdim, kv_rank, 0.3), 64)
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
            check_rows(outs[(tc, rid)], want, "bfloat16", what=f"tensor cores {tc}, {rid}")
            hz.close(rid)
        # a portion of one request beside single tokens of another, in one step
        first = hz.feed_many({"a": h[:200], "b": h[:100]})
        second = hz.feed_many({"a": h[200:201], "b": h[100:T]})
        third = hz.feed_many({"a": h[201:T]})
        outs[(tc, "mixed a")] = torch.cat([first["a"], second["a"], third["a"]], 0)
        outs[(tc, "mixed b")] = torch.cat([first["b"], second["b"]], 0)
        check_rows(outs[(tc, "mixed a")], want, "bfloat16", what=f"tensor cores {tc}, mixed a")
        check_rows(outs[(tc, "mixed b")], want, "bfloat16", what=f"tensor cores {tc}, mixed b")
    assert not torch.equal(outs[(True, "whole")], outs[(False, "whole")])       # (two kernels did run)
    # (the tensor-core path also rounds the inputs of the two per-head products to bfloat16, as products do)
    for rid in ("whole", "cut", "mixed a", "mixed b"):
        assert rel_rows(outs[(True, rid)], outs[(False, rid)]).max() < 4e-2


@pytest.mark.parametrize("heads,kv_heads,dim,vdim", [(2, 1, 4, 4), (3, 3, 12, 20), (2, 2, 20, 72), (4, 2, 32, 8), (2, 1, 48, 36),
                                                     (4, 1, 64, 64), (1, 1, 100, 12), (2, 1, 128, 40), (1, 1, 160, 16),
                                                     (2, 2, 256, 24)])
def test_delta_rule_with_split_columns_against_one_thread_a_column(heads, kv_heads, dim, vdim, monkeypatch):
    """32-bit: every size class of the kernel that spreads a column of the state over several lanes, against the
    plain recurrence and against the kernel with one thread a column.  Whole, cut and decoded, two slots."""
    from gibbs_b200.parts import delta_rule
    cfg = one_layer("channel_delta", delta(heads, kv_heads, dim, vdim, 3, 4, 4), 48)
    W = make_weights(cfg, 9)
    T = 90
    h = bf(torch.randn(T, 48, generator=gen(10)))
    want = plain_mixer(cfg, 0, W, h)
    outs = {}
    for split in (True, False):
        monkeypatch.setattr(delta_rule, "SPLIT_COLUMNS", split)
        part = part_of(cfg, 0, W, "float32")
        hz = PartHarness(part, n_slots=2)
        for rid, cuts in (("whole", [T]), ("cut", [2, 15, 1, 16, 17, 2, 33, 4]), ("decoded", [T - 40, 1])):
            outs[(split, rid)] = hz.run_cut(rid, h, cuts)
            check_rows(outs[(split, rid)], want, "float32", what=f"split {split}, {rid}")
            hz.close(rid)
    for rid in ("whole", "cut", "decoded"):
        assert rel_rows(outs[(True, rid)], outs[(False, rid)]).max() < 1e-5


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
            check_rows(got[rid], truth[rid], dtype, what=f"{name} {what} {rid}")


@pytest.mark.parametrize("name", ["A", "B", "C", "D"])
def test_layer_by_layer_in_float32(name):
    """The residual stream after every layer, through the parts' forward methods."""
    cfg, model, reqs, _ = model_and_truth(name, "float32")
    W = make_weights(cfg, CONFIGS[name][1])
    ids = reqs["r61"]
    layers = []
    plain.forward(cfg, W, ids, layers_out=layers)
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
def test_mixed_batches_with_pages_and_slots_used_again(name, dtype):
    """Up to three live requests in a pool that holds little more than the live ones and has three slots,
    portions beside single tokens: against the plain implementation, and against each request run alone."""
    cfg, model, reqs, truth = model_and_truth(name, dtype)
    more = dict(reqs)
    for k in range(4):                                        # more requests than slots: slots and pages go round
        more[f"again{k}"] = ids_for(cfg, 500 + k, 40 + 17 * k)
    for seed in (0, 1):
        eng = engine_for(model, n_pages=20, max_requests=3)   # 320 tokens of pages
        got = run_trace_on_engine(eng, trace_mixed(more, capacity_tokens=320, max_live=3, seed=seed))
        assert eng.cache.free_pages() == [20] * len(eng.cache.groups)
        for rid in reqs:
            check_rows(got[rid], truth[rid], dtype, what=f"{name} mixed {rid}")
        alone = run_trace_on_engine(engine_for(model), trace_whole(more))
        for rid in more:
            check_rows(got[rid], alone[rid], dtype, what=f"{rid}: batch against alone",
                       tol=1e-4 if dtype == "float32" else TOL[dtype])


@pytest.mark.parametrize("seed", [2, 5, 8, 13, 21, 34, 55, 89])
def test_random_configurations_in_float32(seed):
    """Sizes, options and the order of layers drawn at random (one to six layers of the three kinds; blocks of
    one position and none; with and without rotation, stretching, pair table and cap; convolutions of one
    tap), whole, cut, decoded and in mixed batches, against the plain implementation in float64."""
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


def test_long_decoding_past_blocks_and_pages():
    """260 tokens decoded one by one after a two-token prompt: every block edge and page edge is passed
    by single tokens, and pages of blocks left behind come back."""
    cfg, model, _, _ = model_and_truth("A", "float32")
    W = make_weights(cfg, CONFIGS["A"][1])
    ids = ids_for(cfg, 77, 262)
    truth = plain.forward(cfg, W, ids).numpy()
    eng = engine_for(model, n_pages=20)
    got = run_trace_on_engine(eng, trace_tail_decoded({"long": ids}, tail=260))
    e = rel_rows(got["long"], truth)
    assert e.max() <= TOL["float32"], f"first wrong position {int(np.nonzero(e > TOL['float32'])[0][0])}"
    assert min(eng.cache.free_pages()) == 20


def test_pages_of_blocks_left_behind_go_back_to_the_pool():
    """A request of 200 tokens in an engine whose groups for blocks of 19 and of 48 positions have four and six
    pages of 16: enough for a block and a step of 30 tokens, far less than the request."""
    cfg, model, _, _ = model_and_truth("A", "float32")
    from gibbs_b200 import Engine
    probe = Engine(model, n_pages=4, max_requests=1, max_step_tokens=64, max_context=256)
    assert sorted((g.block or 0) for g in probe.cache.groups) == [0, 19, 48]
    pools = {("block", 19): 4, ("block", 48): 6, None: 16}
    eng = Engine(model, n_pages=pools, page_size=16, max_requests=1, max_step_tokens=64, max_context=256, guard_cache=True)
    W = make_weights(cfg, CONFIGS["A"][1])
    ids = ids_for(cfg, 78, 200)
    truth = plain.forward(cfg, W, ids).numpy()
    got = run_trace_on_engine(eng, trace_portions({"r": ids}, sizes=(16, 1, 1, 30, 2)))
    check_rows(got["r"], truth, "float32", what="pages of blocks")


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
    assert dump["architecture"] == "Sisadra"
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
