"""Sisadra without a GPU: configuration, refusals, plan, tensor names, ranks read from a checkpoint's shapes,
cache bookkeeping of pages kept by blocks, and the plain implementation's own properties."""
from __future__ import annotations

import copy

import numpy as np
import pytest
import torch

import plain_sisadra as plain
from sisadra_helpers import CFG_A, CFG_B, CFG_C, CFG_D, make_weights, random_config


def test_detected_by_its_name_and_laid_out_as_a_plan():
    from gibbs_b200.config import SisadraConfig, parse_config
    conf = parse_config(CFG_A)
    assert isinstance(conf, SisadraConfig)
    plan = conf.plan()
    assert plan.architecture == "Sisadra" and len(plan.layers) == 4
    assert [l.mixer.kind for l in plan.layers] == ["gated_delta_rule", "differential_attention", "latent_attention",
                                                   "differential_attention"]
    assert plan.embedding.kind == "pair_embedding" and plan.embedding.params["scale"] == 3.0
    assert (plan.embedding.params["buckets"], plan.embedding.params["mul_prev"], plan.embedding.params["mul_cur"]) == (53, 7, 11)
    assert plan.head.params["softcap"] == 8.0 and plan.final_norm.kind == "layernorm"
    m0, m1, m2, m3 = (layer.mixer.params for layer in plan.layers)
    assert (m0["decay_rank"], m0["gate_rank"], m0["conv"], m0["unit_eps"], m0["q_scale"]) == (5, 9, 3, 1e-6, 8 ** -0.5)
    assert m1["mask"] == ("blocks", 19) and m1["rot_dims"] == 8 and m1["rot_scaling"]["factor"] == 4.0 and m1["diff"] == 0.25
    assert m2["sink"] and not m2["gate"] and m2["rot_dim"] == 0 and m2["window"] is None
    assert m3["mask"] == ("blocks", 48) and m3["rot_scaling"] is None
    assert [r for r, _, _ in plan.layers[1].parts] == ["mixer_norm", "mixer"]          # no feed-forward
    assert plan.layers[0].ffn.kind == "dense_mlp" and plan.layers[0].ffn.params["act"] == "gelu"
    assert "l1.norm2" in plan.ignorable
    # no pair table, no cap, no mask, no rotation
    pb = parse_config(CFG_B).plan()
    assert pb.embedding.kind == "token_embedding" and pb.head.params["softcap"] == 0.0
    assert pb.layers[0].mixer.params["mask"] is None and pb.layers[3].mixer.params["rot_dims"] == 0


@pytest.mark.parametrize("cfg", [CFG_A, CFG_B, CFG_C, CFG_D, random_config(4), random_config(9), random_config(17)])
def test_tensor_names_and_shapes(cfg):
    from gibbs_b200.config import parse_config
    from gibbs_b200.weights.loader import expected_tensors
    want = {k: tuple(v.shape) for k, v in make_weights(cfg, 1).items()}
    got = {k: d.shapes[0] for k, d in expected_tensors(parse_config(cfg).plan()).items()}
    assert got == want


def test_ranks_come_from_the_checkpoints_shapes_when_it_is_there():
    from gibbs_b200.config import ConfigError, parse_config
    cfg = copy.deepcopy(CFG_A)
    m = cfg["layers"][0]["mixer"]
    del m["decay_rank"], m["gate_rank"]
    with pytest.raises(ConfigError, match="rank"):
        parse_config(cfg)
    with pytest.raises(ConfigError, match="rank"):
        parse_config(cfg, ["l0.mix.a1", "l0.mix.g1"])            # names alone say nothing
    conf = parse_config(cfg, {"l0.mix.a1": (3, 64), "l0.mix.g1": (11, 64)})
    assert conf.ranks[0] == (3, 11) and conf.ranks[1] is None
    p = conf.plan().layers[0].mixer.params
    assert (p["decay_rank"], p["gate_rank"]) == (3, 11)
    # written out again, the configuration carries them: random weights of the same sizes can be made from it
    again = parse_config(conf.to_dict())
    assert again.ranks == conf.ranks
    # a checkpoint's shapes win over keys
    assert parse_config(CFG_A, {"l0.mix.a1": (2, 64), "l0.mix.g1": (9, 64)}).ranks[0] == (2, 9)


def _broken(path, value):
    cfg = copy.deepcopy(CFG_A)
    d = cfg
    for k in path[:-1]:
        d = d[k]
    if value is KeyError:
        del d[path[-1]]
    else:
        d[path[-1]] = value
    return cfg


@pytest.mark.parametrize("path,value", [
    (("width",), KeyError), (("norm",), KeyError), (("layers",), []), (("vocab",), KeyError),
    (("layers", 0, "type"), "conv"), (("layers", 0, "mixer", "dim"), KeyError), (("layers", 0, "mixer", "conv"), 0),
    (("layers", 1, "mixer", "kv_heads"), 4),                       # 6 heads over 4
    (("layers", 1, "mixer", "rot", "dims"), 7), (("layers", 1, "mixer", "rot", "dims"), 18),
    (("layers", 1, "mixer", "rot", "scaling", "low"), KeyError), (("layers", 1, "mixer", "diff"), KeyError),
    (("layers", 1, "mixer", "mask", "size"), 0), (("layers", 2, "mixer", "kv_rank"), KeyError),
    (("layers", 2, "mixer", "scale"), KeyError), (("layers", 0, "mlp", "kind"), "moe"), (("layers", 0, "mlp", "ff"), KeyError),
    (("embedding", "bigram", "buckets"), 0), (("embedding", "bigram", "mul_cur"), KeyError),
])
def test_refusals(path, value):
    from gibbs_b200.config import ConfigError, parse_config
    with pytest.raises(ConfigError):
        parse_config(_broken(path, value))


def test_stretched_frequencies_against_the_plain_rule():
    from gibbs_b200.parts.position import stretched_inv_freq
    cases = [(10000.0, 64, (8.0, 1.0, 4.0, 64)), (500000.0, 32, (8.0, 1.0, 4.0, 8192)), (100.0, 8, None),
             (1000.0, 8, (4.0, 1.0, 3.0, 40)), (30.0, 2, (2.0, 1.0, 2.0, 16)), (10.0, 6, (32.0, 1.0, 4.0, 1024))]
    branches = set()
    for base, dims, sc in cases:
        scaling = dict(zip(("factor", "low", "high", "original"), sc)) if sc else None
        want = plain.stretched_frequencies(base, dims, scaling)
        got = stretched_inv_freq(dims, base, scaling)
        assert got.dtype == np.float32 and np.allclose(got, want.numpy(), rtol=2e-7, atol=0)
        if sc:
            f = plain.stretched_frequencies(base, dims, None)
            for a, b in zip(want.tolist(), f.tolist()):
                branches.add("kept" if a == b else "slowed" if abs(a - b / sc[0]) <= 1e-15 * b else "blended")
    assert branches == {"kept", "slowed", "blended"}


def test_pages_kept_by_blocks_go_back_as_soon_as_a_request_has_left_them():
    from gibbs_b200.cache import CacheManager
    from gibbs_b200.parts.base import PagedKV, SlotState
    needs = [([PagedKV(1, 8, None, 4, block=10)], None), ([PagedKV(2, 4)], None), ([PagedKV(1, 8, None, 4, block=10)], None),
             ([SlotState((1,), torch.int32)], None)]
    m = CacheManager(needs, {("block", 10): 6, None: 16}, 4, 2, torch.float32, "cpu", 64)
    assert [(g.block, g.window) for g in m.groups] == [(10, None), (None, None)]
    assert m.groups[0].entries == [(0, 0), (2, 0)]
    with pytest.raises(ValueError, match="not both"):
        PagedKV(1, 8, window=5, block=10)
    rc = m.open("a")
    m.reserve(rc, 9); m.advance(rc, 9)                 # block 0: pages 0, 1, 2
    assert m.free_pages() == [3, 13]
    m.reserve(rc, 12); m.advance(rc, 12)               # 9 is still of block 0: nothing goes back before the step
    assert m.free_pages() == [3, 13]
    m.reserve(rc, 13); m.advance(rc, 13)               # a step that starts at 12 reads from 10 on: pages 0 and 1 are free
    assert m.free_pages() == [4, 12] and rc.block_tables[0][:2] == [-1, -1] and rc.block_tables[0][2] >= 0
    m.reserve(rc, 31); m.advance(rc, 31)               # a long step: pages 2 .. 7 held (the block of position 13 on)
    assert rc.block_tables[0][:2] == [-1, -1] and m.free_pages()[0] == 0
    m.reserve(rc, 32); m.advance(rc, 32)               # starts at 31, block 30: page 7 on
    assert rc.block_tables[0][:7] == [-1] * 7 and m.free_pages()[0] == 5
    m.check()
    m.close("a")
    assert m.free_pages() == [6, 16]


def test_the_plain_delta_rule_written_as_one_product_per_token():
    """S_t = diag(g_t) S_(t-1) (I - beta_t k_t k_t^T applied after the decay) + beta_t k_t v_t^T: the plain
    function against the closed form of one step, and a state that forgets under a decay of zero."""
    g = torch.Generator().manual_seed(0)
    T, dim, vdim = 7, 5, 3
    q, k, v = (torch.randn(T, n, generator=g, dtype=torch.float64) for n in (dim, dim, vdim))
    beta, decay = torch.rand(T, generator=g, dtype=torch.float64), torch.rand(T, dim, generator=g, dtype=torch.float64)
    out = plain.delta_rule(q, k, v, beta, decay)
    S = torch.zeros(dim, vdim, dtype=torch.float64)
    for t in range(T):
        D = torch.diag(decay[t]) @ S
        S = (torch.eye(dim, dtype=torch.float64) - beta[t] * torch.outer(k[t], k[t])) @ D + beta[t] * torch.outer(k[t], v[t])
        assert torch.allclose(out[t], S.T @ q[t], atol=1e-12)
    decay[3] = 0.0
    out2 = plain.delta_rule(q, k, v, beta, decay)
    fresh = plain.delta_rule(q[3:], k[3:], v[3:], beta[3:], decay[3:])
    assert torch.allclose(out2[3:], fresh, atol=1e-12)


def test_the_plain_model_is_causal_and_its_blocks_cut_what_a_position_sees():
    W = make_weights(CFG_A, 2)
    ids = [int(t) for t in torch.randint(0, CFG_A["vocab"], (60,), generator=torch.Generator().manual_seed(3))]
    a = plain.forward(CFG_A, W, ids)
    b = plain.forward(CFG_A, W, ids[:41])
    assert torch.allclose(a[:41], b, atol=1e-9)
    # attention alone: position 19 (first of its block of 19) sees only itself
    m = CFG_A["layers"][1]["mixer"]
    w = {k: v.double() for k, v in plain.sub(W, "l1.mix.").items()}
    h = torch.randn(40, CFG_A["width"], dtype=torch.float64, generator=torch.Generator().manual_seed(4))
    h2 = h.clone()
    h2[:19] = torch.randn(19, CFG_A["width"], dtype=torch.float64, generator=torch.Generator().manual_seed(5))
    x, y = plain.differential_attention(h, w, m, 1e-5), plain.differential_attention(h2, w, m, 1e-5)
    assert torch.allclose(x[19:38], y[19:38], atol=1e-12) and not torch.allclose(x[18], y[18], atol=1e-3)
