"""Selivik without a GPU: configuration, refusals, plan, tensor names, random weights, cache bookkeeping of
windows that keep a sequence's first positions, and the plain implementation's own properties."""
from __future__ import annotations

import copy
import math

import pytest
import torch

import plain_selivik as plain
from selivik_helpers import CFG_A, CFG_B, CFG_C, CFG_D, make_weights, random_config


def test_detected_by_its_name_and_laid_out_as_a_plan():
    from gibbs_b200.config import SelivikConfig, parse_config
    conf = parse_config(CFG_A)
    assert isinstance(conf, SelivikConfig)
    plan = conf.plan()
    assert plan.architecture == "Selivik" and len(plan.layers) == 4
    assert [l.block for l in plan.layers] == ["parallel_residual"] * 4
    assert [l.mixer.kind for l in plan.layers] == ["gated_attention", "latent_attention", "gated_attention", "latent_attention"]
    assert plan.embedding.kind == "token_embedding" and plan.embedding.params["scale"] == 3.0
    assert plan.final_norm.kind == "rmsnorm_rows" and plan.final_norm.params["gain_offset"] == 1.0
    m0, m1, m2, m3 = (layer.mixer.params for layer in plan.layers)
    assert (m0["window"], m0["keep_first"], m0["softcap"], m0["rot_dims"], m0["rot_factor"]) == (19, 3, 5.0, 8, 4.0)
    assert m0["rot_pairs"] == "halves" and m0["qk_norm"] == "head_after_rot" and m0["sink"] == "learned" and not m0["gate"]
    assert (m1["q_rank"], m1["kv_rank"], m1["rot_dim"], m1["rot_dims"], m1["gate"]) == (10, 24, 6, 4, "outputs")
    assert m2["window"] is None and m2["keep_first"] == 0 and m2["softcap"] == 0.0 and m2["rot_factor"] == 1.0
    assert [r for r, _, _ in plan.layers[2].parts] == ["norm", "mixer", "sum"]          # no feed-forward
    assert plan.layers[2].sum.params["branches"] == ("mixer",) and "l2.ls2" in plan.ignorable
    assert plan.layers[0].sum.params == {"dim": 64, "mult": 0.7, "branches": ("mixer", "ffn")}
    f0, f1 = plan.layers[0].ffn, plan.layers[1].ffn
    assert f0.kind == "routed_glu" and (f0.params["experts"], f0.params["top"], f0.params["expert_inner"]) == (5, 2, 24)
    assert (f0.params["scores"], f0.params["normalise"], f0.params["weight_on"], f0.params["router_bias"]) == \
        ("logits", "softmax", "output", True)
    assert f1.kind == "gated_mlp" and f1.params["act"] == "gelu_tanh" and f1.params["inner"] == 40
    assert parse_config(CFG_B).plan().layers[0].sum.params["mult"] == 1.0


@pytest.mark.parametrize("cfg", [CFG_A, CFG_B, CFG_C, CFG_D, random_config(4), random_config(9), random_config(17)])
def test_tensor_names_and_shapes(cfg):
    from gibbs_b200.config import parse_config
    from gibbs_b200.weights.loader import expected_tensors
    want = {k: tuple(v.shape) for k, v in make_weights(cfg, 1).items()}
    got = {k: d.shapes[0] for k, d in expected_tensors(parse_config(cfg).plan()).items()}
    assert got == want


def _broken(path, value=None, drop=False):
    cfg = copy.deepcopy(CFG_A)
    node = cfg
    for key in path[:-1]:
        node = node[key]
    if drop:
        del node[path[-1]]
    else:
        node[path[-1]] = value
    return cfg


@pytest.mark.parametrize("cfg,match", [
    (_broken(["vocab"], drop=True), "vocab"),
    (_broken(["norm"], drop=True), "norm"),
    (_broken(["layers"], []), "non-empty"),
    (_broken(["layers", 0, "type"], "convolution"), "unknown mixer type"),
    (_broken(["layers", 0, "mixer", "kv_heads"], 4), "multiple"),
    (_broken(["layers", 0, "mixer", "rot", "dims"], 7), "rotated dimensions"),
    (_broken(["layers", 0, "mixer", "rot", "dims"], 18), "rotated dimensions"),
    (_broken(["layers", 0, "mixer", "rot", "scaling", "factor"], 0.0), "stretched"),
    (_broken(["layers", 0, "mixer", "mask", "size"], 0), "window"),
    (_broken(["layers", 0, "mixer", "mask", "keep_first"], -1), "kept"),
    (_broken(["layers", 0, "mixer", "scale"], drop=True), "scale"),
    (_broken(["layers", 1, "mixer", "q_rank"], drop=True), "q_rank"),
    (_broken(["layers", 1, "mixer", "rot", "dims"], 8), "rot_dim"),
    (_broken(["layers", 0, "mlp", "kind"], "conv"), "unknown mlp kind"),
    (_broken(["layers", 0, "mlp", "router", "top"], 6), "top 6 of 5"),
    (_broken(["layers", 1, "mlp", "ff"], drop=True), "ff"),
])
def test_refusals_name_what_is_wrong(cfg, match):
    from gibbs_b200.config import ConfigError, parse_config
    with pytest.raises(ConfigError, match=match):
        parse_config(cfg)


def test_random_weights_keep_norm_weights_at_zero_and_scales_at_one(tmp_path):
    from gibbs_b200.config import parse_config
    from gibbs_b200.weights import random_tensors
    W = dict(random_tensors(parse_config(CFG_A).plan(), 3, torch.float32))
    assert set(W) == set(make_weights(CFG_A, 1))
    assert float(W["l0.norm1"].abs().max()) == 0.0 and float(W["final.norm"].abs().max()) == 0.0
    assert torch.equal(W["l1.ls1"], torch.ones(64)) and torch.equal(W["l1.ls2"], torch.ones(64))
    assert torch.equal(W["l1.mix.dkv.norm"], torch.ones(24)) and torch.equal(W["l1.mix.dq.norm"], torch.ones(10))
    assert 0.0 < float(W["l0.mix.sink"].abs().max()) < 0.2


def test_pages_behind_a_window_go_back_and_those_of_the_first_positions_stay():
    from gibbs_b200.cache import CacheManager
    from gibbs_b200.parts.base import PagedKV
    need = PagedKV(1, 8, window=40, v_head_dim=4, keep_first=20)
    assert need.retention == ("window", 40, 20)
    assert PagedKV(1, 8, window=40).retention == 40
    with pytest.raises(ValueError):
        PagedKV(1, 8, keep_first=3)
    cm = CacheManager([([need], None)], 9, 16, 2, torch.float32, "cpu", 1024)
    rc = cm.open("a")
    held = lambda: [i for i, p in enumerate(rc.block_tables[0]) if p >= 0]
    cm.reserve(rc, 60), cm.advance(rc, 60)
    assert held() == [0, 1, 2, 3]
    cm.reserve(rc, 100), cm.advance(rc, 100)          # a step from position 60 reads from 21: nothing has passed yet
    assert held() == [0, 1, 2, 3, 4, 5, 6]
    cm.reserve(rc, 130), cm.advance(rc, 130)          # from 100: reads from 61 = page 3; pages 0 and 1 hold the first 20
    assert held() == [0, 1, 3, 4, 5, 6, 7, 8]
    assert cm.free_pages() == [1]
    cm.reserve(rc, 160), cm.advance(rc, 160)          # from 130: reads from 91 = page 5
    assert held() == [0, 1, 5, 6, 7, 8, 9]
    view = cm.views([torch.zeros(1, 64, dtype=torch.int32)], torch.zeros(1, dtype=torch.int32), [0])[0][0]
    assert view.window == 40 and view.keep_first == 20
    cm.close("a")
    cm.check()
    assert cm.free_pages() == [9]


def test_the_plain_implementation_sees_what_the_design_says():
    seen = plain.window_with_first(12, 4, 2)
    assert [int(j) for j in torch.nonzero(seen[9]).flatten()] == [0, 1, 6, 7, 8, 9]
    assert [int(j) for j in torch.nonzero(seen[3]).flatten()] == [0, 1, 2, 3]
    assert [int(j) for j in torch.nonzero(plain.window_with_first(12, 1, 0)[5]).flatten()] == [5]
    # the sink only joins the denominator
    s = torch.tensor([[0.0, 1.0, 2.0]], dtype=torch.float64)
    w = plain.softmax_seen(s, torch.ones(1, 3, dtype=torch.bool), sink=1.0)
    e = [math.exp(v) for v in (0.0, 1.0, 2.0, 1.0)]
    assert abs(float(w.sum()) - (1.0 - e[3] / sum(e))) < 1e-12
    # turning does not change a pair's length, halves and neighbours pair differently
    x = torch.arange(8, dtype=torch.float64).reshape(1, 8) + 1.0
    f = plain.frequencies(100.0, 4, 2.0)
    assert torch.allclose(f, torch.tensor([0.5, 0.05], dtype=torch.float64))
    pos = torch.tensor([3])
    a, b = plain.rotate_halves(x, pos, f), plain.rotate_neighbours(x, pos, f)
    assert torch.allclose(a[0, 4:], x[0, 4:]) and torch.allclose(b[0, 4:], x[0, 4:])
    assert abs(float(a[0, 0] ** 2 + a[0, 2] ** 2) - (1.0 + 9.0)) < 1e-12
    assert abs(float(b[0, 0] ** 2 + b[0, 1] ** 2) - (1.0 + 4.0)) < 1e-12
    assert not torch.allclose(a, b)
