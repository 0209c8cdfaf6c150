"""Attention over a compressed key/value cache ("latent attention"), with an
optional output gate per head, an optional sliding window, an optional rotated
key part and an optional learned sink in the softmax.

For a token with mixer input h (H heads; per head ``dim`` unrotated and
``rot_dim`` rotated query/key entries, values of ``vdim``, latent of ``kv_rank``):

    q            = W_q h                      per head [unrotated | rotated]
    [l | kr]     = W_dkv h                    kv_rank + rot_dim entries
    c            = rmsnorm(l) * gain          the latent; kr is ONE rotated key part for all heads
    k_h          = [W_uk,h c | rot(kr)],  v_h = W_uv,h c
    o_h          = sigmoid(W_g h)_h * sum_j softmax_j(scale * q_h . k_h,j) v_h,j
    out          = W_o [o_1 .. o_H]

Only [c | rot(kr)] is cached, one row per position (``PagedRows``).  The kernels
use the absorbed form: W_uk,h is moved to the query side and W_uv,h behind the
weighted sum of latents, so that prompt portions and decoded tokens alike read
nothing but cache rows (csrc/latent_attention.cu).  Position i sees the
positions j with 0 <= i - j < window (all earlier ones without a window).  The
rotation turns the first ``rot_dims`` entries of a rotated part in adjacent
pairs by pos * base^(-2i / rot_dims).

Options: ``rot_dim`` 0: no rotated part at all (no positions: q has ``dim``
entries per head and the cache row is the latent alone); ``gate`` False: no
output gate (then no tensor ``g``); ``gate`` "outputs": one gate per output
element instead of one per head, o = sigmoid(W_g h) * [o_1 .. o_H] with W_g of
H * vdim rows (applied behind W_uv, where it no longer commutes with the head's
linear map); ``sink`` True: a learned score per head (tensor ``sink``) whose
exponential is added to the softmax's denominator; it has no key and no value
and is not scaled; ``q_rank`` r_q: the queries come through a latent of their
own, q = W_uq (rmsnorm(W_dq h) * gain_q), with tensors ``dq`` [r_q, hidden],
``dq.norm`` [r_q] and ``uq`` [H * (dim + rot_dim), r_q] in place of ``q``.
"""
from __future__ import annotations

import numpy as np
import torch

from .. import ops
from ..ops import hybrid
from .base import Mixer, PagedRows, TensorDecl, VECTOR, register_part
from .runner import BranchPart, Runner, keep


USE_TENSOR_CORES = True          # (the tests switch it off to compare the two kernels)


def _workspace_rows() -> int:
    from ..ops.library import library
    return int(library(hybrid.LIBRARY).gb_latent_attention_workspace_rows())


class LatentAttention(BranchPart, Mixer):
    @classmethod
    def declare(cls, params):
        d, H = params["hidden"], params["heads"]
        dn, dr, dv, r = params["dim"], params.get("rot_dim", 0), params["vdim"], params["kv_rank"]
        t = {"dkv": TensorDecl.of(r + dr, d),
             "dkv.norm": TensorDecl.of(r, role=VECTOR), "uk": TensorDecl.of(H * dn, r),
             "uv": TensorDecl.of(H * dv, r), "o": TensorDecl.of(d, H * dv)}
        if params.get("q_rank"):
            rq = int(params["q_rank"])
            t.update({"dq": TensorDecl.of(rq, d), "dq.norm": TensorDecl.of(rq, role=VECTOR),
                      "uq": TensorDecl.of(H * (dn + dr), rq)})
        else:
            t["q"] = TensorDecl.of(H * (dn + dr), d)
        if params.get("gate", True):
            t["g"] = TensorDecl.of(H * dv if params.get("gate") == "outputs" else H, d)
        if params.get("sink", False):
            t["sink"] = TensorDecl.of(H, role=VECTOR)
        return t

    def __init__(self, params, tensors, rt):
        super().__init__(params, tensors, rt)
        p = params
        self.hidden, self.heads = int(p["hidden"]), int(p["heads"])
        self.dn, self.dr, self.dv, self.r = int(p["dim"]), int(p.get("rot_dim", 0)), int(p["vdim"]), int(p["kv_rank"])
        self.window = int(p["window"]) if p.get("window") else None
        self.scale, self.eps = float(p["scale"]), float(p["eps"])
        self.rot_dims = int(p.get("rot_dims", self.dr))
        if self.rot_dims % 2 or not 0 <= self.rot_dims <= self.dr:
            raise ValueError(f"{self.rot_dims} rotated dimensions must be even and at most rot_dim {self.dr}")
        H = self.heads
        # one product for [q | latent, rotated key | gate logits]
        self.gated = bool(p.get("gate", True))
        self.gate_outputs = p.get("gate") == "outputs"
        if p.get("gate", True) not in (True, False, None, "outputs"):
            raise ValueError(f"gate {p.get('gate')!r}: True (one per head), 'outputs' (one per output element) or False")
        # one product for [q (or the queries' latent) | latent, rotated key | gate logits]
        self.q_rank = int(p.get("q_rank") or 0)
        first = tensors["dq"] if self.q_rank else tensors["q"]
        self.fused = torch.cat([first, tensors["dkv"]] + ([tensors["g"]] if self.gated else []), 0).contiguous()
        self.sink = tensors["sink"].to(torch.float32).contiguous() if p.get("sink", False) else None
        self.dkv_col = first.shape[0]
        self.gate_col = self.dkv_col + self.r + self.dr
        if self.q_rank:
            self.q_gain = tensors["dq.norm"].to(torch.float32).contiguous()
            self.uq = tensors["uq"].contiguous()
        # per head: W_uk,h^T as [kv_rank, dim] (applied to the query), W_uv,h as [vdim, kv_rank]
        self.uk_t = tensors["uk"].reshape(H, self.dn, self.r).transpose(1, 2).contiguous()
        self.uv = tensors["uv"].reshape(H, self.dv, self.r).contiguous()
        self.latent_gain = tensors["dkv.norm"].to(torch.float32).contiguous()
        self.o = tensors["o"].contiguous()
        i = np.arange(self.rot_dims // 2, dtype=np.float64)
        inv = np.power(float(p.get("rot_base", 1.0)), -2.0 * i / max(self.rot_dims, 1))
        self.inv_freq = torch.from_numpy(np.concatenate([inv, [0.0]]).astype(np.float32)).to(rt.device)

    def kernel_libraries(self):
        return tuple(set(ops.linear_libraries(self.fused.dtype, self.rt.dtype)) | {"core", hybrid.LIBRARY})

    def cache_needs(self):
        return [PagedRows(self.r + self.dr, self.window)]

    def attention_flops(self, n_tokens: int) -> int:
        pairs = n_tokens * (n_tokens + 1) // 2
        if self.window and n_tokens > self.window:
            pairs -= (n_tokens - self.window) * (n_tokens - self.window + 1) // 2
        return 2 * self.heads * (2 * self.r + self.dr) * pairs

    adds_in_place = True       # with ``accumulate`` the output projection adds into the stream

    def run(self, rn: Runner, h, out, caches, accumulate: bool = False):
        view = caches[0]
        if not view.writable:
            raise RuntimeError("latent attention writes the cache it reads")
        H, dn, dr, dv, r = self.heads, self.dn, self.dr, self.dv, self.r
        F, Dk = self.fused.shape[0], r + dr
        fused = rn.buffer("la_fused", F, torch.float32)
        rn.linear(h, self.fused, None, fused, role="latent_in")
        qp = rn.buffer("la_query", H * Dk, torch.float32)
        table, bt_stride = rn.table(view)
        pages = view.pages
        q, own_q = fused, []
        if self.q_rank:
            # the queries' latent is normed (32-bit statistics) and goes through a product of its own
            cq = rn.buffer("la_q_latent", self.q_rank)
            rn.op("row_norm", [fused.data_ptr(), fused.stride(0), keep(rn, self.q_gain), cq.data_ptr(),
                               ops.dtype_code(cq.dtype), 0, rn.N, self.q_rank, hybrid.NORM_RMS], [self.eps],
                  label="row_norm:q_latent")
            q = rn.buffer("la_q", H * (dn + dr), torch.float32)
            rn.linear(cq, self.uq, None, q, role="latent_q")
            own_q = [q.data_ptr(), q.stride(0)]
        rn.op("latent_prep", [fused.data_ptr(), fused.stride(0), self.dkv_col, keep(rn, self.latent_gain),
                              keep(rn, self.inv_freq), self.rot_dims, rn.tok_req, rn.tok_pos, table, bt_stride,
                              pages.shape[1], keep(rn, pages), pages.shape[0], ops.dtype_code(pages.dtype), rn.N, H,
                              dn, dr, r, qp.data_ptr()] + own_q, [self.eps])
        rn.op("head_linear", [q.data_ptr(), q.stride(0), dn + dr, keep(rn, self.uk_t),
                              ops.dtype_code(self.uk_t.dtype), qp.data_ptr(), ops.F32, qp.stride(0), Dk, rn.N, H, r, dn],
              label="head_linear:absorb", flags=0 if USE_TENSOR_CORES else 1)
        lat = rn.buffer("la_latent_out", H * r, torch.float32)
        ws = rn.buffer("la_partial", r + 2, torch.float32, fixed_rows=_workspace_rows())
        rn.op("latent_attention", [qp.data_ptr(), pages.data_ptr(), ops.dtype_code(pages.dtype), table, bt_stride,
                                   pages.shape[1], pages.shape[0], rn.tok_req, rn.tok_pos,
                                   fused.data_ptr() + 4 * self.gate_col if self.gated and not self.gate_outputs else 0,
                                   fused.stride(0),
                                   lat.data_ptr(), lat.stride(0), rn.N, H, r, dr, self.window or 0, rn.max_context,
                                   ws.data_ptr(), keep(rn, self.sink), rn.R if USE_TENSOR_CORES else 0,
                                   rn.q_start if USE_TENSOR_CORES else 0], [self.scale])
        o = rn.buffer("la_heads_out", H * dv)
        rn.op("head_linear", [lat.data_ptr(), lat.stride(0), r, keep(rn, self.uv), ops.dtype_code(self.uv.dtype),
                              o.data_ptr(), ops.dtype_code(o.dtype), o.stride(0), dv, rn.N, H, dv, r] +
              ([fused.data_ptr() + 4 * self.gate_col, fused.stride(0)] if self.gate_outputs else []),
              label="head_linear:values", flags=0 if USE_TENSOR_CORES else 1)
        (rn.add_linear if accumulate else rn.linear)(o, self.o, None, out, role="latent_out")


register_part("mixer", "latent_attention", LatentAttention)
