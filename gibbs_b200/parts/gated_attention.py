"""Grouped-query attention with a gate on its output and a sink in its softmax.

For a token with mixer input h (H query heads, G key/value heads, query/key
entries ``dim`` and value entries ``vdim`` per head, which may differ):

    q = W_q h,  k = W_k h,  v = W_v h                 no biases
    q <- rmsnorm(q) * gain_q,  k <- rmsnorm(k) * gain_k   over the WHOLE projection (``qk_norm``: "whole"), or not at all
    q, k <- rot(q), rot(k)                            first ``rot_dims`` entries of every head, adjacent pairs
    s_j = cap(scale * q_h . k_g,j),  g = h // (H / G),  cap(s) = c tanh(s / c) with ``softcap`` c > 0
    p_j = exp(s_j) / (sink + sum_i exp(s_i))          over the visible j: 0 <= pos - j < window (all j <= pos without one)
    o_h = sigmoid(W_g h)_h * sum_j p_j v_g,j          ``gate``: one gate per output element
    out = W_o [o_1 .. o_H]

``sink`` adds 1 to the softmax's denominator: a key of score 0 that has no
value; ``sink`` "learned": the sink's score is a number per head (tensor
``sink`` [H]), neither scaled nor capped, so exp(sink_h) joins the denominator.
More options: ``bias`` (q, k and v have biases ``q.b``, ``k.b``, ``v.b``, added
by the product); ``rot_pairs`` "halves" (entry i turns with entry i +
rot_dims / 2) instead of "adjacent"; ``rot_factor`` (every frequency is divided
by it: positions stretched linearly); ``qk_norm`` "head_after_rot": q and k are
turned first and every head is then divided by its root mean square over
``dim`` (no gain); ``keep_first`` n with a window: position i also sees every
j < n (at their true positions), and the pages of those positions stay.  With ``shares_kv`` the layer has no key/value projections and reads the
pages another entry of the model's order writes (keys as that entry stored
them: normed and rotated); its window is its own.  ``retain`` is what the pages
keep for the layers that read them (their widest window; None: everything).
Scores, weights, norms and angles are 32-bit in both compute dtypes; the fused
input product writes 32-bit values, pages hold the compute dtype.
"""
from __future__ import annotations

import os

import numpy as np
import torch

from .. import ops
from ..ops import hybrid
from .base import Mixer, PagedKV, Residual, TensorDecl, VECTOR, register_part
from .linear import Linear
from .runner import BranchPart, Eager, Planned, Runner, keep


def _workspace_rows() -> int:
    from ..ops.library import library
    return int(library(hybrid.LIBRARY).gb_sink_attention_workspace_rows())


def _tensor_cores_take(heads: int, kv_heads: int, dim: int, vdim: int) -> bool:
    from ..ops.library import library
    return bool(library(hybrid.LIBRARY).gb_sink_attention_tc_supported(heads, kv_heads, dim, vdim))


# GIBBS_B200_GATED_ATTN_TC=0: the generic kernel also where the tensor-core kernel would run (for comparison runs)
USE_TENSOR_CORES = os.environ.get("GIBBS_B200_GATED_ATTN_TC", "1") != "0"


class GatedAttention(Mixer):
    # (also usable where an arrangement wants a sublayer's output WRITTEN: ``run``, as ``parts.runner.BranchPart``)
    writes_branch = True
    adds_in_place = True

    @classmethod
    def declare(cls, params):
        d, H, G = params["hidden"], params["heads"], params["kv_heads"]
        dim, vdim = params["dim"], params["vdim"]
        shares, whole = params.get("shares_kv", False), params.get("qk_norm") == "whole"
        t = {"q": TensorDecl.of(H * dim, d), "o": TensorDecl.of(d, H * vdim)}
        if whole:
            t["q.norm"] = TensorDecl.of(H * dim, role=VECTOR)
        if params.get("gate", True):
            t["g"] = TensorDecl.of(H * vdim, d)
        if not shares:
            t["k"], t["v"] = TensorDecl.of(G * dim, d), TensorDecl.of(G * vdim, d)
            if whole:
                t["k.norm"] = TensorDecl.of(G * dim, role=VECTOR)
        if params.get("bias", False):
            t["q.b"] = TensorDecl.of(H * dim, role=VECTOR)
            if not shares:
                t["k.b"], t["v.b"] = TensorDecl.of(G * dim, role=VECTOR), TensorDecl.of(G * vdim, role=VECTOR)
        if params.get("sink") == "learned":
            t["sink"] = TensorDecl.of(H, role=VECTOR)
        return t

    def __init__(self, params, tensors, rt):
        super().__init__(params, tensors, rt)
        p = params
        self.hidden, self.heads, self.kv_heads = int(p["hidden"]), int(p["heads"]), int(p["kv_heads"])
        self.dim, self.vdim = int(p["dim"]), int(p["vdim"])
        if self.kv_heads < 1 or self.heads % self.kv_heads:
            raise ValueError(f"{self.heads} heads are not a multiple of {self.kv_heads} kv heads")
        self.scale, self.eps = float(p["scale"]), float(p.get("eps", 0.0))
        self.softcap = float(p.get("softcap") or 0.0)
        self.window = int(p["window"]) if p.get("window") else None
        self.retain = p.get("retain", self.window)
        self.sink, self.gated = bool(p.get("sink", False)), bool(p.get("gate", True))
        self.sink_scores = tensors["sink"].to(torch.float32).contiguous() if p.get("sink") == "learned" else None
        self.keep_first = int(p.get("keep_first") or 0) if self.window else 0
        if self.keep_first < 0:
            raise ValueError(f"{self.keep_first} kept first positions")
        self.whole_norm = p.get("qk_norm") == "whole"
        self.norm_after_rot = p.get("qk_norm") == "head_after_rot"
        if p.get("qk_norm") not in (None, "whole", "head_after_rot"):
            raise ValueError(f"qk_norm '{p.get('qk_norm')}': this mixer norms the whole projection, every head behind "
                             "the rotation, or nothing")
        self.rot_halves = {"adjacent": False, "halves": True}[p.get("rot_pairs", "adjacent")]
        self.shares_kv = bool(p.get("shares_kv", False))
        self.rot_dims = int(p.get("rot_dims", 0) or 0)
        if self.rot_dims % 2 or not 0 <= self.rot_dims <= self.dim:
            raise ValueError(f"{self.rot_dims} rotated dimensions must be even and at most the head's {self.dim}")
        H, G, dim, vdim = self.heads, self.kv_heads, self.dim, self.vdim
        # one product for [q | k | v | gate logits] (a layer that reads another's pages: [q | gate logits])
        names = ["q"] + ([] if self.shares_kv else ["k", "v"]) + (["g"] if self.gated else [])
        self.fused = torch.cat([tensors[n] for n in names], 0).contiguous()
        self.fused_bias = None
        if p.get("bias", False):
            zeros = lambda n: torch.zeros(tensors[n].shape[0], dtype=torch.float32, device=tensors[n].device)
            self.fused_bias = torch.cat([tensors[n + ".b"].to(torch.float32) if n != "g" else zeros(n)
                                         for n in names]).contiguous()
        self.k_col = H * dim
        self.v_col = self.k_col + G * dim
        self.gate_col = H * dim if self.shares_kv else self.v_col + G * vdim
        f32 = lambda n: tensors[n].to(torch.float32).contiguous() if n in tensors else None
        self.q_gain, self.k_gain = f32("q.norm"), f32("k.norm")
        self.out_proj = Linear(tensors["o"], None, rt)
        i = np.arange(self.rot_dims // 2, dtype=np.float64)
        inv = np.power(float(p.get("rot_base", 10000.0)), -2.0 * i / max(self.rot_dims, 1)) / float(p.get("rot_factor") or 1.0)
        self.inv_freq = torch.from_numpy(np.concatenate([inv, [0.0]]).astype(np.float32)).to(rt.device)

    def kernel_libraries(self):
        return tuple(set(ops.linear_libraries(self.fused.dtype, self.rt.dtype)) | {"core", hybrid.LIBRARY})

    def cache_needs(self):
        return [] if self.shares_kv else [PagedKV(self.kv_heads, self.dim, self.retain, self.vdim,
                                                  keep_first=self.keep_first if self.retain else 0)]

    def attention_flops(self, n_tokens: int) -> int:
        pairs = n_tokens * (n_tokens + 1) // 2
        if self.window and n_tokens > self.window:
            far = n_tokens - self.window                  # positions with keys in front of their window
            pairs -= far * (far + 1) // 2
            if self.keep_first:                           # ... of which they still see the first ones
                full = max(far - self.keep_first, 0)
                pairs += full * self.keep_first + (far - full) * (far - full + 1) // 2
        return 2 * self.heads * (self.dim + self.vdim) * pairs

    def _attend(self, rn: Runner, fused: torch.Tensor, kv) -> torch.Tensor:
        """Everything between the two products: fused [rows, q | k | v | gate] (float32) -> heads' outputs."""
        H, G, dim, vdim = self.heads, self.kv_heads, self.dim, self.vdim
        if not self.shares_kv and not kv.writable:
            raise RuntimeError("an attention layer with k/v projections was given a read-only cache")
        if self.window is not None and kv.window is not None and kv.window < self.window:
            raise RuntimeError(f"the pages keep {kv.window} positions; this layer's window is {self.window}")
        if self.window is None and kv.window is not None:
            raise RuntimeError(f"the pages keep {kv.window} positions; this layer sees every position")
        if self.keep_first and kv.window is not None and (getattr(kv, "keep_first", 0) or 0) < self.keep_first:
            raise RuntimeError(f"this layer sees the first {self.keep_first} positions; the pages do not keep them")
        kp, vp = kv.k_pages, kv.v_pages
        if tuple(kp.shape[1:]) != (G, kv.page_size, dim) or tuple(vp.shape[1:]) != (G, kv.page_size, vdim):
            raise RuntimeError(f"pages of {tuple(kp.shape[1:])} / {tuple(vp.shape[1:])} for {G} kv heads of {dim} / {vdim}")
        table, bt_stride = rn.table(kv)
        pages_bf16 = kp.dtype == torch.bfloat16
        # bfloat16 pages and sizes the tensor-core kernel is built for: queries in bfloat16 as well
        tc = pages_bf16 and self.rt.dtype == torch.bfloat16 and USE_TENSOR_CORES and _tensor_cores_take(H, G, dim, vdim)
        q = rn.buffer("ga_query", H * dim, torch.bfloat16 if tc else torch.float32)
        write = not self.shares_kv
        rn.op("qk_prep", [fused.data_ptr(), fused.stride(0), self.k_col, self.v_col, keep(rn, self.q_gain),
                          keep(rn, self.k_gain), keep(rn, self.inv_freq), self.rot_dims, rn.tok_req, rn.tok_pos, table,
                          bt_stride, kv.page_size, keep(rn, kp) if write else 0, keep(rn, vp) if write else 0,
                          kp.shape[0], rn.N, H, G, dim, vdim, q.data_ptr()], [self.eps],
              flags=(1 if self.whole_norm else 0) | (2 if tc else 0) | (4 if pages_bf16 else 0) |
                    (16 if self.rot_halves else 0) | (32 if self.norm_after_rot else 0))
        out = rn.buffer("ga_heads_out", H * vdim)
        ws = rn.buffer("ga_partial", vdim + 2, torch.float32, fixed_rows=_workspace_rows())
        gate = fused.data_ptr() + 4 * self.gate_col if self.gated else 0
        if tc:
            rn.op("sink_attention_tc", [q.data_ptr(), keep(rn, kp), keep(rn, vp), table, bt_stride, kv.page_size,
                                        kp.shape[0], rn.tok_req, rn.tok_pos, gate, fused.stride(0), out.data_ptr(),
                                        out.stride(0), rn.N, H, G, dim, vdim, self.window or 0, rn.max_context,
                                        ws.data_ptr(), rn.R, rn.q_start, keep(rn, self.sink_scores)],
                  [self.scale, self.softcap, self.keep_first], label="sink_attention", flags=1 if self.sink else 0)
            return out
        rn.op("sink_attention", [q.data_ptr(), keep(rn, kp), keep(rn, vp), table, bt_stride, kv.page_size, kp.shape[0],
                                 rn.tok_req, rn.tok_pos, gate, fused.stride(0), out.data_ptr(), out.stride(0), rn.N, H, G,
                                 dim, vdim, self.window or 0, rn.max_context, ws.data_ptr(), 1, keep(rn, self.sink_scores)],
              [self.scale, self.softcap, self.keep_first],
              flags=(1 if self.sink else 0) | (4 if pages_bf16 else 0) | (8 if out.dtype == torch.bfloat16 else 0))
        return out

    def run(self, rn: Runner, h, out, caches, accumulate: bool = False):
        """The mixer written once for both ways of running it; its output is written into ``out`` (32-bit), or
        added when ``out`` is the stream and ``accumulate`` is set."""
        fused = rn.buffer("ga_fused", self.fused.shape[0], torch.float32)
        rn.linear(h, self.fused, self.fused_bias, fused, role="qkvg")
        heads_out = self._attend(rn, fused, caches[0])
        (rn.add_linear if accumulate else rn.linear)(heads_out, self.out_proj.weight, None, out, role="out_proj")

    def forward(self, h, residual, step, caches):
        rn = Eager(self.rt, step)
        if not isinstance(residual, Residual):                 # an arrangement that takes the output as it is
            return self.run(rn, h, residual, caches)
        fused = rn.buffer("ga_fused", self.fused.shape[0], torch.float32)
        ops.linear(h, self.fused, self.fused_bias, fused)
        out = self._attend(rn, fused, caches[0])
        self.out_proj(out, out=residual, accumulate=True)

    def plan_ops(self, plan, h, caches, out=None):
        if out is not None:
            return self.run(Planned(plan), h, out, caches)
        fused = plan.linear(h, self.fused, self.fused_bias, plan.buffer("ga_fused", self.fused.shape[0], torch.float32),
                            "plain", role="qkvg")
        out = self._attend(Planned(plan), fused, caches[0])
        plan.linear(out, self.out_proj.weight, None, None, "residual", role="out_proj")


register_part("mixer", "gated_attention", GatedAttention)
