"""Token embedding and the output head."""
from __future__ import annotations

import torch

from .. import ops
from ..ops import hybrid
from .runner import Eager, Planned, keep
from .base import Part, SlotState, TensorDecl, register_part
from .linear import Linear


class TokenEmbedding(Part):
    """x[t, :] = table[id_t, :] (MisterTK/gibbs arch/families/lfm2.json5:74), times ``scale`` for a
    design that has one (default 1: no scaling)."""
    category = "embedding"

    @classmethod
    def declare(cls, params):
        return {"weight": TensorDecl.of(params["vocab"], params["dim"])}

    def __init__(self, params, tensors, rt):
        super().__init__(params, tensors, rt)
        self.vocab, self.dim = int(params["vocab"]), int(params["dim"])
        self.table = tensors["weight"].contiguous()
        self.scale = float(params.get("scale", 1.0) or 1.0)

    def kernel_libraries(self):
        return ("core",) if self.scale == 1.0 else ("core", hybrid.LIBRARY)

    def _scaled(self, rn, ids: int, out: torch.Tensor) -> None:
        rn.op("embed_scaled", [keep(rn, self.table), ops.dtype_code(self.table.dtype), ids, out.data_ptr(), rn.N,
                               self.dim, self.vocab], [self.scale])

    def forward(self, ids: torch.Tensor) -> torch.Tensor:
        out = self.rt.empty(ids.numel(), self.dim, dtype=torch.float32)
        if self.scale == 1.0:
            return ops.embed(self.table, ids, out)
        hybrid.call("embed_scaled", [self.table.data_ptr(), ops.dtype_code(self.table.dtype), ids.data_ptr(),
                                     out.data_ptr(), ids.numel(), self.dim, self.vocab], [self.scale],
                    device=self.rt.device)
        return out

    def plan_ops(self, plan):
        if self.scale == 1.0:
            plan.embed(self.table)
        else:
            rn = Planned(plan)
            self._scaled(rn, rn.token_ids, plan.residual)


class PairEmbedding(TokenEmbedding):
    """x[t, :] = table[id_t, :] * scale + pairs[(id_(t-1) * mul_prev + id_t * mul_cur) mod buckets, :]; a
    sequence's first token takes row ``buckets`` (the last) of ``pairs``.  The id before a portion's first
    token is per-request state: one int32 in the request's slot, which the kernel reads and then replaces
    by the portion's last id."""

    @classmethod
    def declare(cls, params):
        return {"weight": TensorDecl.of(params["vocab"], params["dim"]),
                "pairs": TensorDecl.of(int(params["buckets"]) + 1, params["dim"])}

    def __init__(self, params, tensors, rt):
        super().__init__(params, tensors, rt)
        self.buckets, self.mul_prev, self.mul_cur = (int(params[k]) for k in ("buckets", "mul_prev", "mul_cur"))
        if self.buckets < 1:
            raise ValueError(f"a pair table of {self.buckets} buckets")
        self.pairs = tensors["pairs"].contiguous()
        if self.pairs.dtype != self.table.dtype:
            raise ValueError("the token table and the pair table are stored in different dtypes")

    def kernel_libraries(self):
        return ("core", hybrid.LIBRARY)

    def cache_needs(self):
        return [SlotState((1,), torch.int32)]

    def _run(self, rn, out: torch.Tensor, caches) -> None:
        last = caches[0]
        rn.op("embed_scaled", [keep(rn, self.table), ops.dtype_code(self.table.dtype), rn.token_ids, out.data_ptr(), rn.N,
                               self.dim, self.vocab, keep(rn, self.pairs), self.buckets, self.mul_prev, self.mul_cur,
                               rn.tok_req, rn.tok_pos, rn.q_start, rn.q_len, keep(rn, last.state), last.state.stride(0),
                               rn.slots(last)], [self.scale], label="embed_pairs")

    def forward(self, ids: torch.Tensor, step=None, caches=None) -> torch.Tensor:
        if step is None or not caches:
            raise ValueError("an embedding that looks at the token before needs the step and its state")
        out = self.rt.empty(ids.numel(), self.dim, dtype=torch.float32)
        self._run(Eager(self.rt, step), out, caches)
        return out

    def plan_ops(self, plan, caches=None):
        if not caches:
            raise ValueError("an embedding that looks at the token before needs its state")
        self._run(Planned(plan), plan.residual, caches)


class LMHead(Part):
    """logits = z W^T in 32-bit; with ``logit_scale`` they are divided by it, with
    ``softcap`` then passed through cap * tanh(x / cap)
    (MisterTK/gibbs arch/lib/transformer.json5:170-175; LFM2 has neither).  A
    tied head is given the embedding table's tensor and shares its memory."""
    category = "head"
    fuses_norm = True          # its input goes straight into a product (parts.linear.Linear)

    @classmethod
    def declare(cls, params):
        return {"weight": TensorDecl.of(params["vocab"], params["dim"])}

    def __init__(self, params, tensors, rt):
        super().__init__(params, tensors, rt)
        self.vocab = int(params["vocab"])
        self.proj = Linear(tensors["weight"], None, rt)
        self.logit_scale = float(params.get("logit_scale", 1.0) or 1.0)
        self.softcap = float(params.get("softcap", 0.0) or 0.0)

    def kernel_libraries(self):
        return self.proj.kernel_libraries()

    def forward(self, z: torch.Tensor) -> torch.Tensor:
        logits = self.proj(z, out_dtype=torch.float32)
        if self.logit_scale != 1.0 or self.softcap > 0.0:
            ops.scale_softcap(logits, 1.0 / self.logit_scale, self.softcap)
        return logits

    def plan_ops(self, plan, z, logits: int):
        """``logits``: the plan's symbol for where the step's float32 logits go."""
        plan.linear(z, self.proj.weight, self.proj.bias, logits, "plain", rows_symbol=plan.WANTED, role="lm_head")
        if self.logit_scale != 1.0 or self.softcap > 0.0:
            plan.scale_softcap(logits, self.vocab, plan.WANTED, 1.0 / self.logit_scale, self.softcap)


register_part("embedding", "token_embedding", TokenEmbedding)
register_part("embedding", "pair_embedding", PairEmbedding)
register_part("head", "lm_head", LMHead)
