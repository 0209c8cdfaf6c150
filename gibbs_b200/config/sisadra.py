"""Configuration of the Sisadra design and its plan.

Sisadra is a decoder-only model whose config.json lists its layers one by one
(``layers``: ``type``, ``mixer``, ``mlp`` or null).  A layer is pre-norm with
layer norms (gain, no bias): x += mixer(ln(x)), then, unless its ``mlp`` is
null, x += ff(ln(x)).  The embedded tokens are multiplied by
``embedding.scale`` and a row of a pair table, chosen by a hash of (token
before, token), is added (``embedding.bigram``: ``buckets``, ``mul_prev``,
``mul_cur``).  The model ends with its norm, the head and a soft cap on the
logits (``logit_softcap``).

Mixers (``type``):

``attention``          differential attention: two softmax maps per head over the
                       same values, grouped keys and values, biases, RMS norm per
                       head and map, rotation in halves of the first ``rot.dims``
                       entries with stretched long wavelengths (``rot.scaling``),
                       positions seen in blocks of ``mask.size`` counted from 0.
``latent_attention``   keys and values of every head from one normed latent of
                       ``kv_rank`` entries per position, no positions, causal, a
                       learned sink per head in the softmax.
``channel_delta``      a gated delta rule with one decay per head and key
                       channel, short convolutions of ``conv`` taps on q, k and v,
                       low-rank decay and gate projections.

Feed-forward ``dense``: W_down gelu(W_up h) with the exact gelu.

Tensor names: ``embed``, ``bigram``, ``final.norm``, ``head``; layer i's start with
``l<i>.``: ``norm1``, ``norm2``, ``mix.*``, ``mlp.{up,down}``.

The ranks of the low-rank projections are no keys of config.json: they are read
from the shapes of ``mix.a1`` and ``mix.g1`` when a checkpoint is at hand, and
from the keys ``decay_rank`` / ``gate_rank`` of the mixer otherwise (random
weights).

Constants the design fixes: 1e-6 under the root of the delta rule's unit norms,
q times dim^-1/2 there, two maps per attention head, plain norm gains.
"""
from __future__ import annotations

import copy
from dataclasses import dataclass, field
from typing import Optional

from .lfm2 import ConfigError
from .plan import LayerSpec, ModelPlan, OrderEntry, PartSpec

DEFAULT_CONTEXT = 131072          # config.json names no longest context; pools are sized by the engine's caller

MIXERS = ("attention", "latent_attention", "channel_delta")


def _need(d, key: str, where: str):
    if not isinstance(d, dict) or d.get(key) is None:
        raise ConfigError(f"config.json: {where} has no '{key}'")
    return d[key]


@dataclass(frozen=True)
class SisadraConfig:
    raw: dict
    # per layer: (decay rank, gate rank) of a channel_delta mixer, else None
    ranks: tuple = field(default_factory=tuple)

    # -- what the rest of the framework asks a configuration -----------------------------
    @property
    def vocab_size(self) -> int:
        return int(self.raw["vocab"])

    @property
    def hidden_size(self) -> int:
        return int(self.raw["width"])

    @property
    def num_hidden_layers(self) -> int:
        return len(self.raw["layers"])

    @property
    def max_position_embeddings(self) -> int:
        return int(self.raw.get("max_context") or DEFAULT_CONTEXT)

    @property
    def eos_token_ids(self) -> tuple:
        eos = self.raw.get("eos_token_id")
        return () if eos is None else tuple(int(e) for e in (eos if isinstance(eos, (list, tuple)) else [eos]))

    @property
    def norm_eps(self) -> float:
        return float(self.raw["norm"]["eps"])

    @classmethod
    def from_dict(cls, cfg: dict, tensor_names=None) -> "SisadraConfig":
        """``tensor_names``: the checkpoint's tensor names; when it is a mapping from name to shape, the
        low-rank projections' ranks are read from it."""
        raw = copy.deepcopy(cfg)
        shapes = tensor_names if hasattr(tensor_names, "get") else {}
        ranks = []
        for i, layer in enumerate(raw.get("layers") or []):
            if not isinstance(layer, dict) or layer.get("type") != "channel_delta":
                ranks.append(None)
                continue
            m = layer.get("mixer") or {}
            pair = []
            for tensor, key in (("a1", "decay_rank"), ("g1", "gate_rank")):
                shape = shapes.get(f"l{i}.mix.{tensor}")
                if shape is not None:
                    pair.append(int(shape[0]))
                elif m.get(key) is not None:
                    pair.append(int(m[key]))
                else:
                    raise ConfigError(f"layers[{i}]: the rank of '{tensor}' comes from the checkpoint's tensor "
                                      f"l{i}.mix.{tensor} or from the mixer's '{key}'; neither is there")
            ranks.append(tuple(pair))
        out = cls(raw, tuple(ranks))
        out.check()
        return out

    def check(self) -> None:
        c = self.raw
        for key in ("vocab", "width", "layers"):
            _need(c, key, "the model")
        _need(_need(c, "norm", "the model"), "eps", "norm")
        if not isinstance(c["layers"], list) or not c["layers"]:
            raise ConfigError("config.json: 'layers' is a non-empty list")
        big = (c.get("embedding") or {}).get("bigram")
        if big is not None:
            for k in ("buckets", "mul_prev", "mul_cur"):
                _need(big, k, "embedding.bigram")
            if int(big["buckets"]) < 1:
                raise ConfigError(f"embedding.bigram: {big['buckets']} buckets")
        for i, layer in enumerate(c["layers"]):
            where = f"layers[{i}]"
            kind = _need(layer, "type", where)
            if kind not in MIXERS:
                raise ConfigError(f"{where}: unknown mixer type '{kind}'; Sisadra knows {list(MIXERS)}")
            m = _need(layer, "mixer", where)
            for k in ("heads", "dim", "vdim"):
                _need(m, k, where + ".mixer")
            if kind in ("attention", "channel_delta"):
                _need(m, "kv_heads", where + ".mixer")
                if int(m["kv_heads"]) < 1 or int(m["heads"]) % int(m["kv_heads"]):
                    raise ConfigError(f"{where}: {m['heads']} heads are not a multiple of {m['kv_heads']} kv heads")
            if kind == "attention":
                _need(m, "scale", where + ".mixer"), _need(m, "diff", where + ".mixer")
                rot = m.get("rot")
                if rot is not None:
                    _need(rot, "base", where + ".mixer.rot"), _need(rot, "dims", where + ".mixer.rot")
                    if int(rot["dims"]) % 2 or not 0 <= int(rot["dims"]) <= int(m["dim"]):
                        raise ConfigError(f"{where}: {rot['dims']} rotated dimensions must be even and at most dim "
                                          f"{m['dim']}")
                    sc = rot.get("scaling")
                    if sc is not None:
                        for k in ("factor", "low", "high", "original"):
                            _need(sc, k, where + ".mixer.rot.scaling")
                size = (m.get("mask") or {}).get("size")
                if size is not None and int(size) < 1:
                    raise ConfigError(f"{where}: blocks of {size} positions")
            elif kind == "latent_attention":
                _need(m, "scale", where + ".mixer"), _need(m, "kv_rank", where + ".mixer")
            else:
                if int(_need(m, "conv", where + ".mixer")) < 1:
                    raise ConfigError(f"{where}: a convolution of {m['conv']} taps")
            f = layer.get("mlp")
            if f is not None:
                fk = _need(f, "kind", where + ".mlp")
                if fk != "dense":
                    raise ConfigError(f"{where}: unknown mlp kind '{fk}'; Sisadra knows 'dense'")
                _need(f, "ff", where + ".mlp")

    def to_dict(self) -> dict:
        """config.json again; the ranks a checkpoint's shapes gave become keys of their mixers, so that
        random weights for the same sizes can be made from the result."""
        d = copy.deepcopy(self.raw)
        for layer, pair in zip(d["layers"], self.ranks):
            if pair is not None:
                layer["mixer"]["decay_rank"], layer["mixer"]["gate_rank"] = pair
        return d

    def dump(self) -> dict:
        return self.to_dict()

    # -- plan ------------------------------------------------------------------------------
    def plan(self) -> ModelPlan:
        c = self.raw
        d, vocab, eps = self.hidden_size, self.vocab_size, self.norm_eps

        def norm(tensor):
            return PartSpec("layernorm", {"dim": d, "eps": eps}, {"weight": tensor})

        layers, ignorable = [], []
        for i, layer in enumerate(c["layers"]):
            p, m, kind = f"l{i}", layer["mixer"], layer["type"]
            if kind == "attention":
                rot = m.get("rot") or {}
                size = (m.get("mask") or {}).get("size")
                names = ["q", "k", "v", "o", "q.b", "k.b", "v.b", "o.b", "q.norm", "k.norm", "lq1", "lk1", "lq2", "lk2"]
                mixer = PartSpec("differential_attention", {
                    "hidden": d, "heads": int(m["heads"]), "kv_heads": int(m["kv_heads"]), "dim": int(m["dim"]),
                    "vdim": int(m["vdim"]), "scale": float(m["scale"]), "diff": float(m["diff"]), "eps": eps,
                    "mask": ("blocks", int(size)) if size else None, "rot_dims": int(rot.get("dims", 0)),
                    "rot_base": float(rot.get("base", 1.0)), "rot_scaling": copy.deepcopy(rot.get("scaling")),
                    "bias": True, "qk_norm": "head",
                }, {k: f"{p}.mix.{k}" for k in names})
            elif kind == "latent_attention":
                names = ["q", "dkv", "dkv.norm", "uk", "uv", "sink", "o"]
                mixer = PartSpec("latent_attention", {
                    "hidden": d, "heads": int(m["heads"]), "dim": int(m["dim"]), "vdim": int(m["vdim"]),
                    "kv_rank": int(m["kv_rank"]), "rot_dim": 0, "window": None, "scale": float(m["scale"]), "eps": eps,
                    "gate": False, "sink": True,
                }, {k: f"{p}.mix.{k}" for k in names})
            else:
                ra, rg = self.ranks[i]
                names = ["q", "k", "v", "q.conv", "k.conv", "v.conv", "b", "A_log", "dt_bias", "a1", "a2", "g1", "g2",
                         "norm", "o"]
                mixer = PartSpec("gated_delta_rule", {
                    "hidden": d, "heads": int(m["heads"]), "kv_heads": int(m["kv_heads"]), "dim": int(m["dim"]),
                    "vdim": int(m["vdim"]), "conv": int(m["conv"]), "decay_rank": ra, "gate_rank": rg, "eps": eps,
                    "unit_eps": 1e-6, "q_scale": float(int(m["dim"])) ** -0.5,
                }, {k: f"{p}.mix.{k}" for k in names})
            parts = [("mixer_norm", "norm", norm(f"{p}.norm1")), ("mixer", "mixer", mixer)]
            f = layer.get("mlp")
            if f is None:
                ignorable.append(f"{p}.norm2")
            else:
                ffn = PartSpec("dense_mlp", {"hidden": d, "inner": int(f["ff"]), "act": "gelu", "bias": False},
                               {"up": f"{p}.mlp.up", "down": f"{p}.mlp.down"})
                parts += [("ffn_norm", "norm", norm(f"{p}.norm2")), ("ffn", "feed_forward", ffn)]
            layers.append(LayerSpec("prenorm_residual", tuple(parts)))

        e = c.get("embedding") or {}
        scale = float(e.get("scale", 1.0))
        big = e.get("bigram")
        if big is None:
            embedding = PartSpec("token_embedding", {"vocab": vocab, "dim": d, "scale": scale}, {"weight": "embed"})
        else:
            embedding = PartSpec("pair_embedding", {"vocab": vocab, "dim": d, "scale": scale, "buckets": int(big["buckets"]),
                                                    "mul_prev": int(big["mul_prev"]), "mul_cur": int(big["mul_cur"])},
                                 {"weight": "embed", "pairs": "bigram"})
        plan = ModelPlan(
            architecture="Sisadra", vocab_size=vocab, hidden_size=d, max_context=self.max_position_embeddings,
            embedding=embedding, layers=tuple(layers), order=tuple(OrderEntry(i) for i in range(len(layers))),
            final_norm=norm("final.norm"),
            head=PartSpec("lm_head", {"vocab": vocab, "dim": d, "softcap": float(c.get("logit_softcap") or 0.0)},
                          {"weight": "head"}),
            ignorable=tuple(ignorable),
        )
        plan.validate()
        return plan
