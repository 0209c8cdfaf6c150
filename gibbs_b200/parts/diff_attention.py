"""Differential attention: every head takes two softmax maps over the same
values and returns their difference.

For a token with mixer input h (H query heads, G key/value heads, ``dim``
query/key entries per map, ``vdim`` value entries per head):

    q = W_q h + b_q     H heads of [map 1 | map 2], each map ``dim`` entries
    k = W_k h + b_k     G heads of [map 1 | map 2]
    v = W_v h + b_v     G heads of ``vdim`` entries, shared by both maps
    q, k <- rmsnorm(q), rmsnorm(k)   per head AND map over ``dim``, one gain vector for all (``qk_norm``: "head")
    q, k <- rot(q), rot(k)           first ``rot_dims`` entries of every map; entry i pairs with i + rot_dims / 2
    a_m  = softmax_j(scale * q_m . k_m,j) v_j        m = 1, 2, over the visible j
    o    = rmsnorm(a_1 - lambda * a_2) * (1 - diff)  per head over ``vdim``, no gain
    out  = W_o [o_1 .. o_H] + b_o

lambda = exp(lq1 . lk1) - exp(lq2 . lk2) + diff is one number for the layer.
The rotation's frequencies are base^(-2i / rot_dims), optionally stretched for
long wavelengths (``parts.position.stretched_inv_freq``).  What position i
sees (``mask``): every j <= i; with ("window", n) the last n; with ("blocks", n)
the j <= i of i's own block of n positions, blocks counted from position 0 of
the sequence.  A key row of the pages holds both maps' keys side by side
(``PagedKV`` with keys of 2 * dim entries); pages of blocks a request has left
go back to the pool.  Norms, angles, scores, weights and the combination are
32-bit in both compute dtypes; the pages hold the compute dtype.
"""
from __future__ import annotations

import math

import torch

from .. import ops
from ..ops import hybrid
from .base import Mixer, PagedKV, TensorDecl, VECTOR, register_part
from .position import stretched_inv_freq
from .runner import BranchPart, Runner, keep

MAPS = 2
USE_TENSOR_CORES = True          # (the tests switch it off to compare the two kernels)


def _workspace_rows() -> int:
    from ..ops.library import library
    return int(library(hybrid.LIBRARY).gb_sink_attention_workspace_rows())


def _tensor_cores_take(heads: int, kv_heads: int, dim: int, vdim: int) -> bool:
    from ..ops.library import library
    return bool(library(hybrid.LIBRARY).gb_sink_attention_tc_supported(heads, kv_heads, dim, vdim))


class DifferentialAttention(BranchPart, Mixer):
    adds_in_place = True

    @classmethod
    def declare(cls, params):
        d, H, G, dim, vdim = (params[k] for k in ("hidden", "heads", "kv_heads", "dim", "vdim"))
        t = {"q": TensorDecl.of(H * MAPS * dim, d), "k": TensorDecl.of(G * MAPS * dim, d), "v": TensorDecl.of(G * vdim, d),
             "o": TensorDecl.of(d, H * vdim)}
        if params.get("bias", True):
            t.update({"q.b": TensorDecl.of(H * MAPS * dim, role=VECTOR), "k.b": TensorDecl.of(G * MAPS * dim, role=VECTOR),
                      "v.b": TensorDecl.of(G * vdim, role=VECTOR), "o.b": TensorDecl.of(d, role=VECTOR)})
        if params.get("qk_norm", "head") == "head":
            t.update({"q.norm": TensorDecl.of(dim, role=VECTOR), "k.norm": TensorDecl.of(dim, role=VECTOR)})
        for n in ("lq1", "lk1", "lq2", "lk2"):
            t[n] = TensorDecl.of(dim, role=VECTOR)
        return t

    def __init__(self, params, tensors, rt):
        super().__init__(params, tensors, rt)
        p = params
        self.hidden, self.heads, self.kv_heads = int(p["hidden"]), int(p["heads"]), int(p["kv_heads"])
        self.dim, self.vdim = int(p["dim"]), int(p["vdim"])
        if self.kv_heads < 1 or self.heads % self.kv_heads:
            raise ValueError(f"{self.heads} heads are not a multiple of {self.kv_heads} kv heads")
        self.scale, self.eps, self.diff = float(p["scale"]), float(p["eps"]), float(p["diff"])
        mask = p.get("mask")
        self.mask_kind, self.mask_size = (None, 0) if not mask else (str(mask[0]), int(mask[1]))
        if self.mask_kind not in (None, "window", "blocks") or (self.mask_kind and self.mask_size < 1):
            raise ValueError(f"mask {mask!r}: None, ('window', n) or ('blocks', n) with n >= 1")
        self.head_norm = p.get("qk_norm", "head") == "head"
        if p.get("qk_norm", "head") not in (None, "head"):
            raise ValueError(f"qk_norm '{p.get('qk_norm')}': this mixer norms every head and map or nothing")
        self.rot_dims = int(p.get("rot_dims", 0) or 0)
        if self.rot_dims % 2 or not 0 <= self.rot_dims <= self.dim:
            raise ValueError(f"{self.rot_dims} rotated dimensions must be even and at most the map's {self.dim}")
        H, G, dim, vdim = self.heads, self.kv_heads, self.dim, self.vdim
        biased = bool(p.get("bias", True))
        self.fused = torch.cat([tensors[n] for n in ("q", "k", "v")], 0).contiguous()
        self.fused_bias = torch.cat([tensors[n + ".b"].to(torch.float32) for n in ("q", "k", "v")]).contiguous() \
            if biased else None
        self.k_col, self.v_col = H * MAPS * dim, (H + G) * MAPS * dim
        f32 = lambda n: tensors[n].to(torch.float32).contiguous() if n in tensors else None
        self.q_gain, self.k_gain = f32("q.norm"), f32("k.norm")
        self.o, self.o_bias = tensors["o"].contiguous(), f32("o.b") if biased else None
        lam = [float((tensors[a].double() * tensors[b].double()).sum()) for a, b in (("lq1", "lk1"), ("lq2", "lk2"))]
        self.lam = math.exp(lam[0]) - math.exp(lam[1]) + self.diff
        inv = stretched_inv_freq(self.rot_dims, float(p.get("rot_base", 10000.0)), p.get("rot_scaling"))
        self.inv_freq = torch.cat([torch.from_numpy(inv), torch.zeros(1)]).to(torch.float32).to(rt.device)

    def kernel_libraries(self):
        return tuple(set(ops.linear_libraries(self.fused.dtype, self.rt.dtype)) | {"core", hybrid.LIBRARY})

    def cache_needs(self):
        return [PagedKV(self.kv_heads, MAPS * self.dim, self.mask_size if self.mask_kind == "window" else None, self.vdim,
                        block=self.mask_size if self.mask_kind == "blocks" else None)]

    def attention_flops(self, n_tokens: int) -> int:
        if self.mask_kind == "blocks":
            full, rest = divmod(n_tokens, self.mask_size)
            pairs = full * (self.mask_size * (self.mask_size + 1) // 2) + rest * (rest + 1) // 2
        else:
            pairs = n_tokens * (n_tokens + 1) // 2
            if self.mask_kind == "window" and n_tokens > self.mask_size:
                pairs -= (n_tokens - self.mask_size) * (n_tokens - self.mask_size + 1) // 2
        return 2 * self.heads * MAPS * (self.dim + self.vdim) * pairs

    def run(self, rn: Runner, h, out, caches, accumulate: bool = False):
        kv = caches[0]
        H, G, dim, vdim = self.heads, self.kv_heads, self.dim, self.vdim
        if not kv.writable:
            raise RuntimeError("differential attention writes the cache it reads")
        kp, vp = kv.k_pages, kv.v_pages
        if tuple(kp.shape[1:]) != (G, kv.page_size, MAPS * dim) or tuple(vp.shape[1:]) != (G, kv.page_size, vdim):
            raise RuntimeError(f"pages of {tuple(kp.shape[1:])} / {tuple(vp.shape[1:])} for {G} kv heads of "
                               f"{MAPS} x {dim} / {vdim}")
        fused = rn.buffer("da_fused", self.fused.shape[0], torch.float32)
        rn.linear(h, self.fused, self.fused_bias, fused, role="qkv")
        table, bt_stride = rn.table(kv)
        pages_bf16 = kp.dtype == torch.bfloat16
        # bfloat16 pages and sizes the tensor-core kernel is built for: queries in bfloat16 as well; the maps'
        # outputs stay 32-bit either way, for the combination behind them
        tc = pages_bf16 and self.rt.dtype == torch.bfloat16 and USE_TENSOR_CORES and _tensor_cores_take(H, G, dim, vdim)
        q = rn.buffer("da_query", H * MAPS * dim, torch.bfloat16 if tc else torch.float32)
        rn.op("qk_prep", [fused.data_ptr(), fused.stride(0), self.k_col, self.v_col, keep(rn, self.q_gain),
                          keep(rn, self.k_gain), keep(rn, self.inv_freq), self.rot_dims, rn.tok_req, rn.tok_pos, table,
                          bt_stride, kv.page_size, keep(rn, kp), keep(rn, vp), kp.shape[0], rn.N, H, G, dim, vdim,
                          q.data_ptr(), MAPS], [self.eps],
              flags=(8 if self.head_norm else 0) | 16 | (4 if pages_bf16 else 0) | (2 if tc else 0))
        maps_out = rn.buffer("da_maps_out", H * MAPS * vdim, torch.float32)
        ws = rn.buffer("ga_partial", vdim + 2, torch.float32, fixed_rows=_workspace_rows())
        if tc:
            rn.op("sink_attention_tc", [q.data_ptr(), keep(rn, kp), keep(rn, vp), table, bt_stride, kv.page_size,
                                        kp.shape[0], rn.tok_req, rn.tok_pos, 0, 0, maps_out.data_ptr(), maps_out.stride(0),
                                        rn.N, H, G, dim, vdim, self.mask_size, rn.max_context, ws.data_ptr(), rn.R,
                                        rn.q_start], [self.scale, 0.0], label="diff_attention",
                  flags=2 | (4 if self.mask_kind == "blocks" else 0) | (MAPS << 8))
        else:
            rn.op("sink_attention", [q.data_ptr(), keep(rn, kp), keep(rn, vp), table, bt_stride, kv.page_size, kp.shape[0],
                                     rn.tok_req, rn.tok_pos, 0, 0, maps_out.data_ptr(), maps_out.stride(0), rn.N, H, G, dim,
                                     vdim, self.mask_size, rn.max_context, ws.data_ptr(), MAPS], [self.scale, 0.0],
                  label="diff_attention", flags=(4 if pages_bf16 else 0) | (16 if self.mask_kind == "blocks" else 0))
        heads_out = rn.buffer("da_heads_out", H * vdim)
        rn.op("head_norm", [maps_out.data_ptr(), maps_out.stride(0), MAPS * vdim, maps_out.data_ptr() + 4 * vdim, 0, 0, 0,
                            heads_out.data_ptr(), ops.dtype_code(heads_out.dtype), heads_out.stride(0), rn.N, H, vdim],
              [self.eps, self.lam, 1.0 - self.diff], label="diff_combine")
        (rn.add_linear if accumulate else rn.linear)(heads_out, self.o, self.o_bias, out, role="out_proj")


register_part("mixer", "differential_attention", DifferentialAttention)
