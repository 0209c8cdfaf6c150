"""Shared by the Selivik tests: small configurations that differ in every size,
option and order of layers, weights with realistic scales (all values exactly
representable in bfloat16, so that both compute dtypes and the plain
implementation read the same numbers), and builders."""
from __future__ import annotations

import math
import random

import torch


def att(heads, kv_heads, dim, vdim, scale, window=None, keep_first=None, softcap=None, rot=None, factor=None):
    m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale}
    if window is not None:
        m["mask"] = {"size": window}
        if keep_first is not None:
            m["mask"]["keep_first"] = keep_first
    if softcap is not None:
        m["softcap"] = softcap
    m["rot"] = {"base": rot[0], "dims": rot[1]} if rot is not None else {"base": 10000.0, "dims": 0}
    if factor is not None:
        m["rot"]["scaling"] = {"factor": factor}
    return m


def lat(heads, dim, rot_dim, vdim, kv_rank, q_rank, scale, base=10000.0, dims=None):
    return {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "kv_rank": kv_rank, "q_rank": q_rank,
            "scale": scale, "rot": {"base": base, "dims": rot_dim if dims is None else dims}}


def dense(ff):
    return {"kind": "dense", "ff": ff}


def moe(experts, top, ff):
    return {"kind": "moe", "expert": {"ff": ff}, "router": {"experts": experts, "top": top}}


def layer(kind, mixer, mlp=None):
    return {"type": kind, "mixer": mixer, "mlp": mlp}


# A: three query heads a kv head, values narrower than keys, a window that is no multiple of a page with three kept
# first positions, partial rotation, a rotated part of which only four entries turn, a layer without a feed-forward,
# a layer without a window, one expert of several and two of five
CFG_A = {
    "architecture": "Selivik", "vocab": 300, "width": 64, "norm": {"eps": 1e-5}, "residual_mult": 0.7,
    "embedding": {"scale": 3.0},
    "layers": [
        layer("attention", att(6, 2, 16, 12, 0.3, window=19, keep_first=3, softcap=5.0, rot=(1000.0, 8), factor=4.0), moe(5, 2, 24)),
        layer("latent_attention", lat(3, 8, 6, 20, 24, 10, 0.4, base=100.0, dims=4), dense(40)),
        layer("attention", att(2, 2, 8, 8, 0.5, softcap=None, rot=(100.0, 8)), None),
        layer("latent_attention", lat(2, 12, 4, 8, 16, 24, 0.3), moe(3, 1, 16)),
    ],
}
# B: ten query heads a kv head (more than a block's warps), values of 40 entries, a window without kept positions, more
# kept positions than the window is long, every expert chosen, a multiplier of one, five heads of latent attention
CFG_B = {
    "architecture": "Selivik", "vocab": 257, "width": 96, "norm": {"eps": 1e-6}, "residual_mult": 1.0,
    "embedding": {"scale": 0.5},
    "layers": [
        layer("attention", att(10, 1, 12, 40, 0.3, window=40, softcap=12.0, rot=(50000.0, 4)), dense(128)),
        layer("latent_attention", lat(5, 24, 8, 8, 16, 40, 0.2), moe(4, 4, 32)),
        layer("attention", att(4, 2, 32, 72, 0.2, window=7, keep_first=30, softcap=30.0, rot=(10000.0, 32), factor=8.0), None),
        layer("latent_attention", lat(1, 16, 2, 16, 8, 8, 0.25), dense(32)),
        layer("attention", att(3, 3, 20, 20, 0.22, window=64, keep_first=16, rot=(500.0, 20), factor=2.0), moe(7, 3, 20)),
    ],
}
# C: sizes that are multiples of nothing, a window of one position with one kept, a latent of 3 entries, one expert,
# one head, values of one entry, a query latent of one entry
CFG_C = {
    "architecture": "Selivik", "vocab": 97, "width": 44, "norm": {"eps": 1e-5}, "residual_mult": 0.25,
    "embedding": {"scale": 1.0},
    "layers": [
        layer("attention", att(1, 1, 10, 7, 0.4, window=1, keep_first=1, softcap=3.0, rot=(30.0, 2)), dense(9)),
        layer("latent_attention", lat(1, 6, 2, 1, 3, 1, 0.5), moe(1, 1, 20)),
        layer("attention", att(5, 5, 6, 3, 0.5, window=2, keep_first=0, rot=(10000.0, 6), factor=8.0), moe(6, 5, 9)),
        layer("latent_attention", lat(7, 2, 2, 3, 5, 3, 0.7), None),
    ],
}
# D: sizes of the kind real layers have (keys and values of 64 and 128 entries: the tensor-core kernels run in
# bfloat16; experts whose width is a multiple of 64), a window longer than a key tile, kept positions beyond a page
CFG_D = {
    "architecture": "Selivik", "vocab": 211, "width": 128, "norm": {"eps": 1e-5}, "residual_mult": 0.5,
    "embedding": {"scale": 11.0},
    "layers": [
        layer("attention", att(8, 2, 64, 64, 0.11, window=100, keep_first=20, softcap=25.0, rot=(250000.0, 64), factor=4.0),
              moe(8, 2, 64)),
        layer("latent_attention", lat(4, 64, 32, 64, 128, 96, 0.1), dense(256)),
        layer("attention", att(2, 1, 128, 32, 0.09, window=48, keep_first=4, softcap=20.0, rot=(500.0, 32)), moe(4, 2, 128)),
        layer("latent_attention", lat(2, 32, 16, 32, 64, 64, 0.15), None),
        layer("attention", att(8, 2, 32, 96, 0.18, rot=(10000.0, 32)), dense(64)),
    ],
}
CONFIGS = {"A": (CFG_A, 41), "B": (CFG_B, 42), "C": (CFG_C, 43), "D": (CFG_D, 44)}


def random_config(seed: int) -> dict:
    """A configuration of the design with every size, option and the order of layers drawn at random."""
    rng = random.Random(seed)
    d = rng.choice([24, 32, 40, 64, 72, 128])
    layers = []
    for _ in range(rng.randint(1, 6)):
        kind = rng.choice(["attention", "latent_attention"])
        if kind == "attention":
            G = rng.choice([1, 2, 3])
            dim = rng.choice([2, 4, 8, 16, 24, 32, 40, 64])
            window = rng.choice([None, 1, 2, 7, 16, 17, 40, 100])
            m = att(G * rng.choice([1, 2, 4]), G, dim, rng.choice([1, 3, 8, 16, 33, 64]), rng.choice([0.2, 0.35, 0.5]),
                    window=window, keep_first=rng.choice([None, 0, 1, 5, 16, 33]) if window else None,
                    softcap=rng.choice([None, 4.0, 30.0]),
                    rot=(rng.choice([10.0, 1000.0, 500000.0]), rng.choice(range(0, dim + 1, 2))),
                    factor=rng.choice([None, 1.0, 8.0]))
        else:
            dr = rng.choice([2, 4, 8, 16])
            m = lat(rng.choice([1, 2, 5, 8]), rng.choice([2, 8, 16, 24, 64]), dr, rng.choice([1, 4, 16, 40]),
                    rng.choice([3, 8, 32, 48]), rng.choice([1, 6, 16, 40]), rng.choice([0.2, 0.35]),
                    base=rng.choice([10.0, 10000.0]), dims=rng.choice([dr, dr, dr - 2]))
        f = rng.random()
        if f < 0.25:
            mlp = None
        elif f < 0.55:
            mlp = dense(rng.choice([4, 9, 16, 64, 100]))
        else:
            E = rng.choice([1, 2, 5, 9])
            mlp = moe(E, rng.randint(1, E), rng.choice([3, 8, 20, 64]))
        layers.append(layer(kind, m, mlp))
    return {"architecture": "Selivik", "vocab": rng.choice([50, 97, 256]), "width": d,
            "norm": {"eps": rng.choice([1e-5, 1e-6])}, "residual_mult": rng.choice([1.0, 0.5, 0.3]),
            "embedding": {"scale": rng.choice([1.0, 0.7, 6.0])}, "layers": layers}


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
    for i, lay in enumerate(cfg["layers"]):
        p, m, kind = f"l{i}.", lay["mixer"], lay["type"]
        H, dim, vdim = m["heads"], m["dim"], m["vdim"]
        vec(p + "norm1", d, 0.15)                              # stored around zero
        vec(p + "ls1", d, 0.3, 1.0), vec(p + "ls2", d, 0.3, 0.8)
        if kind == "attention":
            G = m["kv_heads"]
            mat(p + "mix.q", H * dim, d, 1.5), mat(p + "mix.k", G * dim, d, 1.5), mat(p + "mix.v", G * vdim, d, 1.5)
            # (heads of unequal size: a norm per head is then no norm over more)
            W[p + "mix.q"] *= (1.0 + torch.arange(H * dim) // dim % 3).unsqueeze(1).float()
            vec(p + "mix.q.b", H * dim, 0.3), vec(p + "mix.k.b", G * dim, 0.3), vec(p + "mix.v.b", G * vdim, 0.3)
            vec(p + "mix.sink", H, 1.5, 0.5)
            mat(p + "mix.o", d, H * vdim)
        else:
            r, rq, dr = m["kv_rank"], m["q_rank"], m["rot_dim"]
            mat(p + "mix.dq", rq, d), vec(p + "mix.dq.norm", rq, 0.2, 1.0), mat(p + "mix.uq", H * (dim + dr), rq, 2.0)
            mat(p + "mix.dkv", r + dr, d, 1.5), vec(p + "mix.dkv.norm", r, 0.2, 1.0)
            mat(p + "mix.uk", H * dim, r, 2.0), mat(p + "mix.uv", H * vdim, r, 1.5)
            mat(p + "mix.g", H * vdim, d, 2.0), mat(p + "mix.o", d, H * vdim)
        f = lay.get("mlp")
        if f is None:
            del W[p + "ls2"]
        elif f["kind"] == "dense":
            mat(p + "mlp.gate", f["ff"], d, 1.5), mat(p + "mlp.up", f["ff"], d, 1.5), mat(p + "mlp.down", d, f["ff"])
        else:
            E, ff = f["router"]["experts"], f["expert"]["ff"]
            mat(p + "mlp.router", E, d, 2.0), vec(p + "mlp.router.b", E, 0.5)
            for e in range(E):
                mat(p + f"mlp.e{e}.gate", ff, d, 1.5), mat(p + f"mlp.e{e}.up", ff, d, 1.5), mat(p + f"mlp.e{e}.down", d, ff)
    vec("final.norm", d, 0.15)
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


def part_spec(cfg: dict, i: int, role: str):
    """(category, registry kind, params, {local name: checkpoint name}) of a part of layer i in the design's plan."""
    from gibbs_b200.config import parse_config
    for r, category, spec in parse_config(cfg).plan().layers[i].parts:
        if r == role:
            return category, spec.kind, dict(spec.params), dict(spec.tensors)
    raise KeyError(role)


def one_layer(kind: str, mixer: dict, d: int, mlp=None, eps: float = 1e-5) -> dict:
    """A configuration around one layer, for tests of a mechanism alone."""
    return {"architecture": "Selivik", "vocab": 32, "width": d, "norm": {"eps": eps}, "residual_mult": 1.0,
            "embedding": {"scale": 1.0}, "layers": [layer(kind, mixer, mlp)]}
