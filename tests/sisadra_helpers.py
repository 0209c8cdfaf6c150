"""Shared by the Sisadra tests: small configurations that differ in every size,
option and order of layers, weights with realistic scales (all values exactly
representable in bfloat16, so that both compute dtypes and the plain
implementation read the same numbers), and builders."""
from __future__ import annotations

import math
import random

import torch


def att(heads, kv_heads, dim, vdim, scale, diff, block=None, rot=None, scaling=None):
    m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale, "diff": diff}
    if block is not None:
        m["mask"] = {"size": block}
    if rot is not None:
        m["rot"] = {"base": rot[0], "dims": rot[1]}
        if scaling is not None:
            m["rot"]["scaling"] = dict(zip(("factor", "low", "high", "original"), scaling))
    return m


def lat(heads, dim, vdim, kv_rank, scale):
    return {"heads": heads, "dim": dim, "vdim": vdim, "kv_rank": kv_rank, "scale": scale}


def delta(heads, kv_heads, dim, vdim, conv, decay_rank, gate_rank):
    return {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "conv": conv, "decay_rank": decay_rank,
            "gate_rank": gate_rank}


def dense(ff):
    return {"kind": "dense", "ff": ff}


def layer(kind, mixer, mlp=None):
    return {"type": kind, "mixer": mixer, "mlp": mlp}


# A: three query heads a kv head, values narrower than a map's keys, blocks of 19 (no multiple of a page), partial
# rotation with stretched wavelengths on both sides of the blend, a delta rule with two heads a key head and ranks that
# differ, a latent wider than the heads' keys, layers without a feed-forward
CFG_A = {
    "architecture": "Sisadra", "vocab": 300, "width": 64, "norm": {"eps": 1e-5}, "logit_softcap": 8.0,
    "embedding": {"scale": 3.0, "bigram": {"buckets": 53, "mul_prev": 7, "mul_cur": 11}},
    "layers": [
        layer("channel_delta", delta(4, 2, 8, 12, 3, 5, 9), dense(96)),
        layer("attention", att(6, 2, 16, 12, 0.3, 0.25, block=19, rot=(1000.0, 8), scaling=(4.0, 1.0, 3.0, 40)), None),
        layer("latent_attention", lat(3, 8, 20, 24, 0.4), dense(40)),
        layer("attention", att(2, 2, 8, 8, 0.5, 0.6, block=48, rot=(100.0, 8)), dense(64)),
    ],
}
# B: ten query heads a kv head (twenty maps: more than a block's warps), values of 40 entries, no mask in one attention
# layer and no rotation in another, a convolution of one tap and one of five, one head, no pair table, no cap
CFG_B = {
    "architecture": "Sisadra", "vocab": 257, "width": 96, "norm": {"eps": 1e-6}, "embedding": {"scale": 0.5},
    "layers": [
        layer("attention", att(10, 1, 12, 40, 0.3, 0.1, rot=(50000.0, 4)), dense(128)),
        layer("channel_delta", delta(1, 1, 40, 33, 1, 4, 4), None),
        layer("latent_attention", lat(5, 24, 8, 16, 0.2), None),
        layer("attention", att(4, 2, 32, 72, 0.2, 0.5, block=64), dense(32)),
        layer("channel_delta", delta(6, 3, 16, 16, 5, 7, 2), dense(48)),
    ],
}
# C: sizes that are multiples of nothing, blocks of one position and of two, one bucket, a latent of 3 entries, heads of
# one value, a key of 70 entries in the delta rule (beyond 64), multipliers that overflow 32 bits
CFG_C = {
    "architecture": "Sisadra", "vocab": 97, "width": 44, "norm": {"eps": 1e-5}, "logit_softcap": 30.0,
    "embedding": {"scale": 1.0, "bigram": {"buckets": 1, "mul_prev": 3, "mul_cur": 5}},
    "layers": [
        layer("attention", att(1, 1, 10, 7, 0.4, 0.3, block=1, rot=(30.0, 2)), dense(9)),
        layer("latent_attention", lat(1, 6, 1, 3, 0.5), dense(20)),
        layer("channel_delta", delta(2, 1, 70, 3, 2, 1, 3), None),
        layer("attention", att(5, 5, 6, 3, 0.5, 0.8, block=2, rot=(10000.0, 6), scaling=(8.0, 1.0, 4.0, 16)), None),
    ],
}
# D: sizes of the kind real layers have (keys of 64 and 128, values of 64 and 128), a long block, every kind of mixer
CFG_D = {
    "architecture": "Sisadra", "vocab": 211, "width": 128, "norm": {"eps": 1e-5}, "logit_softcap": 20.0,
    "embedding": {"scale": 2.0, "bigram": {"buckets": 4093, "mul_prev": 1000003, "mul_cur": 999983}},
    "layers": [
        layer("attention", att(4, 2, 64, 64, 0.125, 0.3, block=100, rot=(10000.0, 64), scaling=(8.0, 1.0, 4.0, 64)), dense(256)),
        layer("channel_delta", delta(4, 2, 64, 64, 4, 16, 16), dense(128)),
        layer("latent_attention", lat(4, 64, 64, 128, 0.125), dense(128)),
        layer("channel_delta", delta(2, 2, 128, 128, 4, 8, 8), None),
        layer("attention", att(2, 1, 128, 128, 0.09, 0.5, rot=(500.0, 32)), None),
    ],
}
CONFIGS = {"A": (CFG_A, 31), "B": (CFG_B, 32), "C": (CFG_C, 33), "D": (CFG_D, 34)}


def random_config(seed: int) -> dict:
    """A configuration of the design with every size, option and the order of layers drawn at random."""
    rng = random.Random(seed)
    d = rng.choice([24, 32, 40, 64, 72, 128])
    layers = []
    for _ in range(rng.randint(1, 6)):
        kind = rng.choice(["attention", "latent_attention", "channel_delta"])
        if kind == "attention":
            G = rng.choice([1, 2, 3])
            dim = rng.choice([2, 4, 8, 16, 24, 32, 40])
            m = att(G * rng.choice([1, 2, 4]), G, dim, rng.choice([1, 3, 8, 16, 33, 64]), rng.choice([0.2, 0.35, 0.5]),
                    rng.choice([0.1, 0.3, 0.8]), block=rng.choice([None, 1, 2, 7, 16, 17, 40, 100]))
            if rng.random() < 0.8:
                m["rot"] = {"base": rng.choice([10.0, 1000.0, 500000.0]), "dims": rng.choice(range(2, dim + 1, 2))}
                if rng.random() < 0.6:
                    m["rot"]["scaling"] = {"factor": rng.choice([2.0, 8.0, 32.0]), "low": 1.0, "high": rng.choice([2.0, 4.0]),
                                           "original": rng.choice([16, 64, 1024])}
        elif kind == "latent_attention":
            m = lat(rng.choice([1, 2, 5, 8]), rng.choice([2, 8, 16, 24, 64]), rng.choice([1, 4, 16, 40]),
                    rng.choice([3, 8, 32, 48]), rng.choice([0.2, 0.35]))
        else:
            G = rng.choice([1, 2, 3])
            m = delta(G * rng.choice([1, 2, 3]), G, rng.choice([2, 8, 16, 32, 40]), rng.choice([1, 8, 16, 33, 64]),
                      rng.choice([1, 2, 4, 5]), rng.choice([1, 4, 16]), rng.choice([2, 8]))
        layers.append(layer(kind, m, None if rng.random() < 0.3 else dense(rng.choice([4, 9, 16, 64, 100]))))
    cfg = {"architecture": "Sisadra", "vocab": rng.choice([50, 97, 256]), "width": d, "norm": {"eps": rng.choice([1e-5, 1e-6])},
           "embedding": {"scale": rng.choice([1.0, 0.7, 6.0])}, "layers": layers}
    if rng.random() < 0.7:
        cfg["embedding"]["bigram"] = {"buckets": rng.choice([1, 13, 509]), "mul_prev": rng.choice([1, 31, 65537]),
                                      "mul_cur": rng.choice([1, 17, 99991])}
    if rng.random() < 0.7:
        cfg["logit_softcap"] = rng.choice([5.0, 15.0, 50.0])
    return cfg


def _bf16_exact(t: torch.Tensor) -> torch.Tensor:
    return t.to(torch.bfloat16).to(torch.float32)


def make_weights(cfg: dict, seed: int) -> dict:
    """name -> float32 tensor (bfloat16-exact values) for every tensor of the design."""
    g = torch.Generator().manual_seed(seed)
    d, V = cfg["width"], cfg["vocab"]
    W = {}

    def mat(name, out, inp, scale=1.0):
        W[name] = torch.randn(out, inp, generator=g) * (scale / math.sqrt(inp))

    def vec(name, n, scale=1.0, mean=0.0):
        W[name] = mean + scale * torch.randn(n, generator=g)

    W["embed"] = torch.randn(V, d, generator=g) / max(float(cfg["embedding"].get("scale", 1.0)), 1.0)
    big = cfg["embedding"].get("bigram")
    if big:
        W["bigram"] = torch.randn(big["buckets"] + 1, d, generator=g) * 0.7
    for i, layer in enumerate(cfg["layers"]):
        p, m, kind = f"l{i}.", layer["mixer"], layer["type"]
        H, dim, vdim = m["heads"], m["dim"], m["vdim"]
        vec(p + "norm1", d, 0.15, 1.0)
        if kind == "attention":
            G = m["kv_heads"]
            mat(p + "mix.q", H * 2 * dim, d, 1.5), mat(p + "mix.k", G * 2 * dim, d, 1.5), mat(p + "mix.v", G * vdim, d, 1.5)
            # (heads and maps of unequal size: a norm per head and map is then no norm over more)
            W[p + "mix.q"] *= (1.0 + torch.arange(H * 2 * dim) // dim % 3).unsqueeze(1).float()
            vec(p + "mix.q.b", H * 2 * dim, 0.3), vec(p + "mix.k.b", G * 2 * dim, 0.3), vec(p + "mix.v.b", G * vdim, 0.3)
            vec(p + "mix.q.norm", dim, 0.3, 1.6), vec(p + "mix.k.norm", dim, 0.3, 1.6)     # sharp maps: the two differ
            for n in ("lq1", "lk1", "lq2", "lk2"):
                vec(p + "mix." + n, dim, 0.9 / math.sqrt(dim))
            mat(p + "mix.o", d, H * vdim), vec(p + "mix.o.b", d, 0.2)
        elif kind == "latent_attention":
            r = m["kv_rank"]
            mat(p + "mix.q", H * dim, d, 2.0), mat(p + "mix.dkv", r, d), vec(p + "mix.dkv.norm", r, 0.2, 1.0)
            mat(p + "mix.uk", H * dim, r, 2.0), mat(p + "mix.uv", H * vdim, r, 1.5), vec(p + "mix.sink", H, 1.5, 0.5)
            mat(p + "mix.o", d, H * vdim)
        else:
            G, K, ra, rg = m["kv_heads"], m["conv"], m["decay_rank"], m["gate_rank"]
            mat(p + "mix.q", G * dim, d, 1.5), mat(p + "mix.k", G * dim, d, 1.5), mat(p + "mix.v", H * vdim, d, 1.5)
            for n, c in (("q", G * dim), ("k", G * dim), ("v", H * vdim)):
                W[p + f"mix.{n}.conv"] = torch.randn(c, K, generator=g) * (0.8 / math.sqrt(K)) + 0.3
            mat(p + "mix.b", H, d, 2.0)
            # decays from nearly one to strong forgetting, different for every head and channel
            W[p + "mix.A_log"] = torch.linspace(-2.5, 0.7, H) + 0.1 * torch.randn(H, generator=g)
            vec(p + "mix.dt_bias", H * dim, 1.0, -0.5)
            mat(p + "mix.a1", ra, d), mat(p + "mix.a2", H * dim, ra, 2.0)
            mat(p + "mix.g1", rg, d), mat(p + "mix.g2", H * vdim, rg, 2.0)
            vec(p + "mix.norm", vdim, 0.2, 1.0), mat(p + "mix.o", d, H * vdim)
        f = layer.get("mlp")
        if f is not None:
            vec(p + "norm2", d, 0.15, 1.0)
            mat(p + "mlp.up", f["ff"], d, 1.5), mat(p + "mlp.down", d, f["ff"])
    vec("final.norm", d, 0.15, 1.0)
    mat("head", V, d, 3.0)
    return {k: _bf16_exact(v) for k, v in W.items()}


def build(cfg: dict, seed: int, dtype: str, device="cuda:0"):
    """(weights, model on the device) of a configuration."""
    from gibbs_b200.config import parse_config
    from gibbs_b200.engine.loading import parse_dtype
    from gibbs_b200.parts.model import build_model
    from gibbs_b200.weights import TensorDict
    W = make_weights(cfg, seed)
    conf = parse_config(cfg)
    model = build_model(conf.plan(), TensorDict({k: v.to(torch.bfloat16) for k, v in W.items()}), parse_dtype(dtype), device)
    model.config = conf
    return W, model


def mixer_part(cfg: dict, i: int):
    """(registry kind, params) the design's plan hands the mixer of layer i."""
    from gibbs_b200.config import parse_config
    spec = parse_config(cfg).plan().layers[i].mixer
    return spec.kind, dict(spec.params)


def one_layer(kind: str, mixer: dict, d: int, eps: float = 1e-5) -> dict:
    """A configuration around one mixer, for tests of a mechanism alone."""
    return {"architecture": "Sisadra", "vocab": 32, "width": d, "norm": {"eps": eps}, "embedding": {"scale": 1.0},
            "layers": [layer(kind, mixer, None)]}
