"""Configuration of the Selivik design and its plan.

Selivik is a decoder-only model whose config.json lists its layers one by one
(``layers``: ``type``, ``mixer``, ``mlp`` or null).  A layer has ONE norm, which
both of its sublayers read, and a residual sum with weights of its own:

    h = rmsnorm(x) * (1 + w);  x += residual_mult * (ls1 * mixer(h) + ls2 * ff(h))

(``ls1``, ``ls2``: a scale per channel; a layer whose ``mlp`` is null has the
first term only).  The norm's weight is stored around zero.  The embedded
tokens are multiplied by ``embedding.scale``; the model ends with a norm of the
same kind and the head.

Mixers (``type``):

``latent_attention``  keys and values of every head from one normed latent of
                      ``kv_rank`` entries per position plus one rotated key part
                      of ``rot_dim`` entries shared by the heads (neighbouring
                      entries turn together); the queries come through a normed
                      latent of ``q_rank`` entries; causal; ordinary softmax; a
                      sigmoid gate per output element in front of the output
                      projection.
``attention``         grouped-query attention with biases on q, k and v, a
                      rotation in halves of the first ``rot.dims`` entries whose
                      frequencies are divided by ``rot.scaling.factor``, every
                      head of q and k divided by its root mean square behind the
                      rotation, a soft cap on the scores, a sliding window of
                      ``mask.size`` positions beside the sequence's first
                      ``mask.keep_first`` ones, and a learned sink per head in
                      the softmax.

Feed-forwards (``mlp.kind``): ``dense``, W_down (gelu_tanh(W_gate h) * W_up h);
``moe``, ``router.experts`` units with silu of which a token uses ``router.top``:
the largest router logits (W_router h + b) win and the weights are the softmax
over the winners' logits.

Tensor names: ``embed``, ``final.norm``, ``head``; layer i's start with ``l<i>.``:
``norm1``, ``ls1``, ``ls2``, ``mix.*``, ``mlp.{gate,up,down}`` or
``mlp.router``, ``mlp.router.b``, ``mlp.e<j>.{gate,up,down}``.
"""
from __future__ import annotations

import copy
from dataclasses import dataclass

from .lfm2 import ConfigError
from .plan import LayerSpec, ModelPlan, OrderEntry, PartSpec

DEFAULT_CONTEXT = 131072          # config.json names no longest context; pools are sized by the engine's caller

MIXERS = ("latent_attention", "attention")
MLP_KINDS = ("dense", "moe")


def _need(d, key: str, where: str):
    if not isinstance(d, dict) or d.get(key) is None:
        raise ConfigError(f"config.json: {where} has no '{key}'")
    return d[key]


@dataclass(frozen=True)
class SelivikConfig:
    raw: dict

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
    def from_dict(cls, cfg: dict, tensor_names=None) -> "SelivikConfig":
        out = cls(copy.deepcopy(cfg))
        out.check()
        return out

    def check(self) -> None:
        c = self.raw
        for key in ("vocab", "width", "layers"):
            _need(c, key, "the model")
        _need(_need(c, "norm", "the model"), "eps", "norm")
        if not isinstance(c["layers"], list) or not c["layers"]:
            raise ConfigError("config.json: 'layers' is a non-empty list")
        for i, layer in enumerate(c["layers"]):
            where = f"layers[{i}]"
            kind = _need(layer, "type", where)
            if kind not in MIXERS:
                raise ConfigError(f"{where}: unknown mixer type '{kind}'; Selivik knows {list(MIXERS)}")
            m = _need(layer, "mixer", where)
            for k in ("heads", "dim", "vdim", "scale"):
                _need(m, k, where + ".mixer")
            if int(m["heads"]) < 1:
                raise ConfigError(f"{where}: {m['heads']} heads")
            rot = m.get("rot")
            if rot is not None:
                _need(rot, "base", where + ".mixer.rot"), _need(rot, "dims", where + ".mixer.rot")
            if kind == "attention":
                G = int(_need(m, "kv_heads", where + ".mixer"))
                if G < 1 or int(m["heads"]) % G:
                    raise ConfigError(f"{where}: {m['heads']} heads are not a multiple of {m['kv_heads']} kv heads")
                if rot is not None and (int(rot["dims"]) % 2 or not 0 <= int(rot["dims"]) <= int(m["dim"])):
                    raise ConfigError(f"{where}: {rot['dims']} rotated dimensions must be even and at most dim {m['dim']}")
                factor = ((rot or {}).get("scaling") or {}).get("factor")
                if factor is not None and float(factor) <= 0.0:
                    raise ConfigError(f"{where}: a rotation stretched by {factor}")
                mask = m.get("mask")
                if mask is not None:
                    if int(_need(mask, "size", where + ".mixer.mask")) < 1:
                        raise ConfigError(f"{where}: a window of {mask['size']} positions")
                    if int(mask.get("keep_first") or 0) < 0:
                        raise ConfigError(f"{where}: {mask['keep_first']} kept first positions")
            else:
                for k in ("kv_rank", "q_rank", "rot_dim"):
                    _need(m, k, where + ".mixer")
                dr = int(m["rot_dim"])
                dims = int((rot or {}).get("dims", 0))
                if dims % 2 or not 0 <= dims <= dr:
                    raise ConfigError(f"{where}: {dims} rotated dimensions must be even and at most rot_dim {dr}")
            f = layer.get("mlp")
            if f is not None:
                fk = _need(f, "kind", where + ".mlp")
                if fk not in MLP_KINDS:
                    raise ConfigError(f"{where}: unknown mlp kind '{fk}'; Selivik knows {list(MLP_KINDS)}")
                if fk == "dense":
                    _need(f, "ff", where + ".mlp")
                else:
                    _need(_need(f, "expert", where + ".mlp"), "ff", where + ".mlp.expert")
                    r = _need(f, "router", where + ".mlp")
                    E, top = int(_need(r, "experts", where + ".mlp.router")), int(_need(r, "top", where + ".mlp.router"))
                    if not 1 <= top <= E:
                        raise ConfigError(f"{where}: top {top} of {E} experts")

    def to_dict(self) -> dict:
        return copy.deepcopy(self.raw)

    def dump(self) -> dict:
        return self.to_dict()

    # -- plan ------------------------------------------------------------------------------
    def plan(self) -> ModelPlan:
        c = self.raw
        d, vocab, eps = self.hidden_size, self.vocab_size, self.norm_eps
        mult = float(c.get("residual_mult", 1.0))

        def norm(tensor):
            # (the stored weight is the gain's distance from one)
            return PartSpec("rmsnorm_rows", {"dim": d, "eps": eps, "gain_offset": 1.0}, {"weight": tensor})

        layers, ignorable = [], []
        for i, layer in enumerate(c["layers"]):
            p, m, kind = f"l{i}", layer["mixer"], layer["type"]
            rot = m.get("rot") or {}
            if kind == "attention":
                mask = m.get("mask") or {}
                names = ["q", "k", "v", "o", "q.b", "k.b", "v.b", "sink"]
                mixer = PartSpec("gated_attention", {
                    "hidden": d, "heads": int(m["heads"]), "kv_heads": int(m["kv_heads"]), "dim": int(m["dim"]),
                    "vdim": int(m["vdim"]), "scale": float(m["scale"]), "eps": eps,
                    "softcap": float(m.get("softcap") or 0.0),
                    "window": int(mask["size"]) if mask.get("size") else None,
                    "keep_first": int(mask.get("keep_first") or 0) if mask.get("size") else 0,
                    "rot_dims": int(rot.get("dims", 0)), "rot_base": float(rot.get("base", 1.0)), "rot_pairs": "halves",
                    "rot_factor": float((rot.get("scaling") or {}).get("factor", 1.0)),
                    "qk_norm": "head_after_rot", "bias": True, "sink": "learned", "gate": False,
                }, {k: f"{p}.mix.{k}" for k in names})
            else:
                names = ["dq", "dq.norm", "uq", "dkv", "dkv.norm", "uk", "uv", "g", "o"]
                mixer = PartSpec("latent_attention", {
                    "hidden": d, "heads": int(m["heads"]), "dim": int(m["dim"]), "vdim": int(m["vdim"]),
                    "kv_rank": int(m["kv_rank"]), "q_rank": int(m["q_rank"]), "rot_dim": int(m["rot_dim"]),
                    "rot_dims": int(rot.get("dims", 0)), "rot_base": float(rot.get("base", 1.0)), "window": None,
                    "scale": float(m["scale"]), "eps": eps, "gate": "outputs", "sink": False,
                }, {k: f"{p}.mix.{k}" for k in names})
            parts = [("norm", "norm", norm(f"{p}.norm1")), ("mixer", "mixer", mixer)]
            f = layer.get("mlp")
            if f is None:
                ignorable.append(f"{p}.ls2")
            elif f["kind"] == "dense":
                parts.append(("ffn", "feed_forward", PartSpec(
                    "gated_mlp", {"hidden": d, "inner": int(f["ff"]), "act": "gelu_tanh"},
                    {k: f"{p}.mlp.{k}" for k in ("gate", "up", "down")})))
            else:
                E, top = int(f["router"]["experts"]), int(f["router"]["top"])
                tensors = {"router": f"{p}.mlp.router", "router.b": f"{p}.mlp.router.b"}
                for e in range(E):
                    tensors.update({f"e{e}.{k}": f"{p}.mlp.e{e}.{k}" for k in ("gate", "up", "down")})
                parts.append(("ffn", "feed_forward", PartSpec("routed_glu", {
                    "hidden": d, "experts": E, "top": top, "expert_inner": int(f["expert"]["ff"]),
                    "scores": "logits", "normalise": "softmax", "router_bias": True, "weight_on": "output",
                    "alpha": 1.0, "up_add": 0.0, "expert_limit": None,        # silu(gate) * up
                }, tensors)))
            branches = ("mixer",) if f is None else ("mixer", "ffn")
            parts.append(("sum", "branch_sum", PartSpec(
                "scaled_sum", {"dim": d, "mult": mult, "branches": branches},
                {b: f"{p}.{n}" for b, n in zip(branches, ("ls1", "ls2"))})))
            layers.append(LayerSpec("parallel_residual", tuple(parts)))

        e = c.get("embedding") or {}
        plan = ModelPlan(
            architecture="Selivik", vocab_size=vocab, hidden_size=d, max_context=self.max_position_embeddings,
            embedding=PartSpec("token_embedding", {"vocab": vocab, "dim": d, "scale": float(e.get("scale", 1.0))},
                               {"weight": "embed"}),
            layers=tuple(layers), order=tuple(OrderEntry(i) for i in range(len(layers))),
            final_norm=norm("final.norm"),
            head=PartSpec("lm_head", {"vocab": vocab, "dim": d}, {"weight": "head"}),
            ignorable=tuple(ignorable),
            random_values=(("l*.norm1", 0.0), ("final.norm", 0.0), ("l*.ls[12]", 1.0)),
        )
        plan.validate()
        return plan
