"""Gated feed-forwards with clamps, dense and routed.

Dense (``clamped_glu``):

    g = min(W_gate h, limit),  u = clamp(W_up h, -limit, limit)
    out = W_down (g * sigmoid(alpha * g) * (u + up_add))

Routed (``routed_glu``): E such experts without biases, of which every token
uses ``top``.  Router logits z = W_router h and scores s = sigmoid(z) are 32-bit;
the ``top`` largest scores choose the experts; a chosen expert's weight is its
score (not renormalised) and multiplies the expert's INPUT: out = sum_e
expert_e(s_e * h).  An optional shared expert runs for every token and is added
times sigmoid(W_sg h), one number per token.  Tokens are ordered by expert on
the device (no host round trip), the experts' products run over the ragged row
ranges (csrc/moe.cu).

The router's rule is made of parameters, so that other designs can set it:
``scores`` "sigmoid" (default), "softmax" (over all router outputs) or "logits"
(the router's outputs as they are); ``normalise`` None (a chosen output's weight
is its score), "sum" (divided by the sum of the chosen scores) or "softmax" (the
softmax over the chosen scores alone); ``router_bias``: the logits are
W_router h + b (tensor ``router.b``);
``correction``: a vector added to the scores for the CHOICE only (the weights
use the scores without it); ``groups`` / ``groups_keep``: the router outputs
form that many equal groups of neighbours, a group's mark is its largest choice
score, and only outputs of the best ``groups_keep`` groups can be chosen;
``identity``: that many router outputs behind the experts' stand for experts
that return their input (they have no tensors; they count in the softmax and in
the groups); ``weight_on`` "input" (default: s_e multiplies the expert's input)
or "output" (out = sum_e s_e * expert_e(h)); ``limit`` 0 or absent: no clamp.
A routed unit whose weights are on the output can add its result straight
into the residual stream (``adds_in_place``).
"""
from __future__ import annotations

import ctypes
import math

import torch

from .. import ops
from ..ops import hybrid
from ..ops.library import library
from .base import FeedForward, TensorDecl, VECTOR, register_part, tensor_bytes
from .linear import can_fuse_swiglu, interleave_gate_up
from .runner import BranchPart, Runner, keep


class ClampedGLU(BranchPart, FeedForward):
    @classmethod
    def declare(cls, params):
        h, f = params["hidden"], params["inner"]
        return {"gate": TensorDecl.of(f, h), "up": TensorDecl.of(f, h), "down": TensorDecl.of(h, f)}

    def __init__(self, params, tensors, rt):
        super().__init__(params, tensors, rt)
        self.hidden, self.inner = int(params["hidden"]), int(params["inner"])
        self.limit = float(params["limit"])
        self.alpha, self.up_add = float(params.get("alpha", 1.702)), float(params.get("up_add", 1.0))
        if tensors["gate"].dtype != tensors["up"].dtype:
            raise ValueError("gate and up projections are stored in different dtypes")
        # in bfloat16 gate and up are one product whose epilogue applies the unit (as SwiGLU's does)
        self.fused = can_fuse_swiglu(tensors["gate"], rt)
        join = interleave_gate_up if self.fused else (lambda g, u: torch.cat([g, u], 0))
        self.gate_up = join(tensors["gate"], tensors["up"]).contiguous()
        self.down = tensors["down"].contiguous()

    def kernel_libraries(self):
        return tuple(set(ops.linear_libraries(self.gate_up.dtype, self.rt.dtype)) | {"core", hybrid.LIBRARY})

    def run(self, rn: Runner, h, out, caches=None):
        act = rn.buffer("glu_act", self.inner)
        if self.fused:
            rn.glu_linear(h, self.gate_up, act, (self.alpha, self.limit, self.up_add), role="glu_gate_up")
        else:
            gu = rn.buffer("glu_gate_up", 2 * self.inner, torch.float32)
            rn.linear(h, self.gate_up, None, gu, role="glu_gate_up")
            rn.op("clamped_glu", [gu.data_ptr(), gu.stride(0), act.data_ptr(), ops.dtype_code(act.dtype), act.stride(0),
                                  rn.N, self.inner], [self.alpha, self.limit, self.up_add])
        rn.linear(act, self.down, None, out, role="glu_down")


class RoutedGLU(BranchPart, FeedForward):
    @classmethod
    def declare(cls, params):
        h, E, f = params["hidden"], params["experts"], params["expert_inner"]
        d = {"router": TensorDecl.of(E + int(params.get("identity", 0) or 0), h)}
        if params.get("router_bias"):
            d["router.b"] = TensorDecl.of(E + int(params.get("identity", 0) or 0), role=VECTOR)
        if params.get("correction"):
            d["correction"] = TensorDecl.of(E + int(params.get("identity", 0) or 0), role=VECTOR)
        for e in range(E):
            d.update({f"e{e}.gate": TensorDecl.of(f, h), f"e{e}.up": TensorDecl.of(f, h), f"e{e}.down": TensorDecl.of(h, f)})
        if params.get("shared_inner"):
            s = params["shared_inner"]
            d.update({"shared.gate": TensorDecl.of(s, h), "shared.up": TensorDecl.of(s, h),
                      "shared.down": TensorDecl.of(h, s), "shared.sg": TensorDecl.of(1, h)})
        return d

    def __init__(self, params, tensors, rt):
        super().__init__(params, tensors, rt)
        p = params
        self.hidden, self.E, self.top, self.inner = int(p["hidden"]), int(p["experts"]), int(p["top"]), int(p["expert_inner"])
        self.limit = float(p.get("expert_limit") or 0.0) or math.inf
        self.alpha, self.up_add = float(p.get("alpha", 1.702)), float(p.get("up_add", 1.0))
        self.identity = int(p.get("identity", 0) or 0)
        self.n_out = self.E + self.identity                      # router outputs
        self.scores = {"sigmoid": 0, "softmax": 1, "logits": 2}[p.get("scores", "sigmoid")]
        self.normalise = {None: 0, "sum": 1, "softmax": 2}[p.get("normalise")]
        self.groups = int(p.get("groups", 1) or 1)
        self.groups_keep = int(p.get("groups_keep", self.groups) or self.groups)
        self.weight_on_output = {"input": False, "output": True}[p.get("weight_on", "input")]
        self.correction = tensors["correction"].to(torch.float32).contiguous() if p.get("correction") else None
        if self.n_out % self.groups or not 1 <= self.groups_keep <= self.groups:
            raise ValueError(f"{self.n_out} router outputs in {self.groups} groups of which {self.groups_keep} stay open")
        if not 1 <= self.top <= (self.n_out // self.groups) * self.groups_keep:
            raise ValueError(f"top {self.top} of {self.n_out} router outputs ({self.groups_keep} of {self.groups} groups open)")
        if self.identity and not self.weight_on_output:
            raise ValueError("identity experts come with weights on the experts' outputs")
        # the plain rule (sigmoid scores, the largest win) has a kernel of its own
        self.plain_rule = (self.scores == 0 and self.correction is None and self.groups == 1 and not self.identity
                           and not self.normalise)
        self.adds_in_place = self.weight_on_output
        E = self.E
        # gate and up rows of an expert side by side; in blocks of 64 features where the width allows, the
        # layout the tensor-core kernel's epilogue wants (csrc/moe_tc.cu)
        self.blocks64 = self.inner % 64 == 0
        join = interleave_gate_up if self.blocks64 else (lambda g, u: torch.cat([g, u], 0))
        self.w_gate_up = torch.stack([join(tensors[f"e{e}.gate"], tensors[f"e{e}.up"]) for e in range(E)]).contiguous()
        self.w_down = torch.stack([tensors[f"e{e}.down"] for e in range(E)]).contiguous()
        self.shared = None
        # (stored as the checkpoint has them: a product of two bfloat16 numbers is exact in the 32-bit
        # accumulator, so the logits are 32-bit sums of exact products on the tensor cores as well)
        rows = [tensors["router"]]
        if p.get("shared_inner"):
            self.shared = ClampedGLU({"hidden": self.hidden, "inner": int(p["shared_inner"]), "limit": float(p["shared_limit"]),
                                      "alpha": self.alpha, "up_add": self.up_add},
                                     {k: tensors["shared." + k] for k in ("gate", "up", "down")}, rt)
            rows.append(tensors["shared.sg"].reshape(1, self.hidden))
        # the router and the shared expert's gate in one small 32-bit product
        self.w_router = torch.cat(rows, 0).contiguous()
        self.router_bias = None
        if p.get("router_bias"):
            if p.get("shared_inner"):
                raise ValueError("a router with a bias has no shared expert's gate beside it")
            self.router_bias = tensors["router.b"].to(torch.float32).contiguous()

    def kernel_libraries(self):
        return tuple(set(ops.linear_libraries(self.w_down.dtype, self.rt.dtype)) | {"core", hybrid.LIBRARY})

    def step_weight_bytes(self, n_tokens: int, seen: set) -> int:
        """A step reads the router, the shared expert and the experts its tokens choose:
        at most n_tokens * top of them."""
        per_expert = (self.w_gate_up[0].numel() + self.w_down[0].numel()) * self.w_down.element_size()
        total = min(self.E, n_tokens * self.top) * per_expert + self.w_router.numel() * self.w_router.element_size()
        seen.update((self.w_gate_up.data_ptr(), self.w_down.data_ptr(), self.w_router.data_ptr()))
        if self.shared is not None:
            total += tensor_bytes(self.shared, seen)
        return total

    def run(self, rn: Runner, h, out, caches=None, accumulate: bool = False):
        E, top, d, f, n_out = self.E, self.top, self.hidden, self.inner, self.n_out
        shared = self.shared is not None
        if accumulate and not self.weight_on_output:
            raise ValueError("a routed unit with weights on the experts' inputs writes its output")
        logits = rn.buffer("moe_logits", n_out + (1 if shared else 0), torch.float32)
        rn.linear(h, self.w_router, self.router_bias, logits, role="router")
        idx = rn.buffer("moe_choice", top, torch.int32)
        wts = rn.buffer("moe_weight", top, torch.float32)
        sg = rn.buffer("moe_shared_gate", 1, torch.float32)
        if self.plain_rule:
            rn.op("moe_route", [logits.data_ptr(), logits.stride(0), rn.N, E, top, E, idx.data_ptr(), wts.data_ptr(),
                                sg.data_ptr() if shared else 0])
        else:
            if shared:
                raise ValueError("a shared expert's gate comes with the plain router rule")
            rn.op("moe_route_grouped", [logits.data_ptr(), logits.stride(0), rn.N, n_out, top, self.scores,
                                        keep(rn, self.correction), self.groups, self.groups_keep, idx.data_ptr(),
                                        wts.data_ptr(), self.normalise])
        # (identity outputs are sorted behind the experts: their rows lie beyond offsets[E] and no product reads them)
        offsets = rn.buffer("moe_offsets", n_out + 1, torch.int32, fixed_rows=1)
        row_pair = rn.buffer("moe_row_pair", top, torch.int32)
        pair_row = rn.buffer("moe_pair_row", top, torch.int32)
        rn.op("moe_sort", [idx.data_ptr(), rn.N, n_out, offsets.data_ptr(), row_pair.data_ptr(), pair_row.data_ptr(), top])
        rows = rn.buffer("moe_rows", d, per_token=top)
        rn.op("moe_gather", [h.data_ptr(), h.stride(0), ops.dtype_code(h.dtype), row_pair.data_ptr(),
                             0 if self.weight_on_output else wts.data_ptr(), rows.data_ptr(), rows.stride(0), rn.N, d, top])
        act = rn.buffer("moe_act", f, per_token=top)
        wdt = ops.dtype_code(self.w_down.dtype)
        eout = rn.buffer("moe_expert_out", d, torch.float32, per_token=top)
        lib = library(hybrid.LIBRARY)
        tc = self.rt.dtype == torch.bfloat16 and self.w_down.dtype == torch.bfloat16
        up_tc = tc and self.blocks64 and lib.gb_moe_experts_tc_supported(0, f, d, ctypes.c_longlong(rows.stride(0)), ctypes.c_longlong(d))
        down_tc = tc and lib.gb_moe_experts_tc_supported(1, d, f, ctypes.c_longlong(act.stride(0)), ctypes.c_longlong(f))
        if up_tc:
            rn.op("moe_experts_tc", [rows.data_ptr(), rows.stride(0), rows.shape[0], keep(rn, self.w_gate_up), 0,
                                     offsets.data_ptr(), E, act.data_ptr(), act.stride(0), rn.N, f, d, 0, top],
                  [self.alpha, self.limit, self.up_add], label="moe_experts:gate_up")
        else:
            rn.op("moe_experts", [rows.data_ptr(), rows.stride(0), ops.dtype_code(rows.dtype), keep(rn, self.w_gate_up),
                                  wdt, offsets.data_ptr(), E, act.data_ptr(), act.stride(0), rn.N, f, d, 0, top,
                                  int(self.blocks64)], [self.alpha, self.limit, self.up_add], label="moe_experts:gate_up")
        if down_tc:
            rn.op("moe_experts_tc", [act.data_ptr(), act.stride(0), act.shape[0], keep(rn, self.w_down), 0,
                                     offsets.data_ptr(), E, eout.data_ptr(), eout.stride(0), rn.N, d, f, 1, top],
                  label="moe_experts:down")
        else:
            rn.op("moe_experts", [act.data_ptr(), act.stride(0), ops.dtype_code(act.dtype), keep(rn, self.w_down), wdt,
                                  offsets.data_ptr(), E, eout.data_ptr(), eout.stride(0), rn.N, d, f, 1, top, 0],
                  label="moe_experts:down")
        if self.weight_on_output:
            if shared:
                raise ValueError("a shared expert comes with weights on the experts' inputs")
            rn.op("moe_combine_weighted", [eout.data_ptr(), eout.stride(0), pair_row.data_ptr(), idx.data_ptr(),
                                           wts.data_ptr(), h.data_ptr(), h.stride(0), ops.dtype_code(h.dtype),
                                           out.data_ptr(), out.stride(0), rn.N, d, top, E], flags=1 if accumulate else 0)
            return
        sh = None
        if shared:
            sh = rn.buffer("moe_shared_out", d, torch.float32)
            self.shared.run(rn, h, sh)
        rn.op("moe_combine", [eout.data_ptr(), eout.stride(0), pair_row.data_ptr(), sg.data_ptr() if shared else 0,
                              sh.data_ptr() if shared else 0, sh.stride(0) if shared else 0, out.data_ptr(),
                              out.stride(0), rn.N, d, top])


register_part("feed_forward", "clamped_glu", ClampedGLU)
register_part("feed_forward", "routed_glu", RoutedGLU)
