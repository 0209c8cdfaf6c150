"""A gated delta rule mixer with one decay per head and key channel.

For a token with mixer input h (H heads of ``vdim`` values, G key heads of
``dim`` entries; head h uses the queries and keys of key head h // (H / G)):

    q, k, v = silu(conv(W_q h)), silu(conv(W_k h)), silu(conv(W_v h))   causal convolution per channel, ``conv`` taps
    q, k   <- q / sqrt(sum q^2 + unit_eps) * dim^-1/2,  k / sqrt(sum k^2 + unit_eps)      per key head
    beta    = sigmoid(W_b h)                                            one per head
    g       = exp(-exp(A_log_h) * softplus(W_a2 (W_a1 h) + dt_bias))    [H, dim]: one decay per key channel
    S      <- diag(g) S;  u = beta (v - S^T k);  S <- S + k u^T;  o = S^T q          S: [dim, vdim] per head
    o      <- rmsnorm(o) * gain * sigmoid(W_g2 (W_g1 h))                per head over ``vdim``; one gain vector
    out     = W_o [o_1 .. o_H]

Per request a slot holds the convolution's last conv - 1 inputs and S, both in
32-bit and zero for a new request.  Everything that enters the recurrence
behind the projections and the convolution (unit norms, beta, decays) and the
recurrence itself are 32-bit in every compute dtype (csrc/delta_rule.cu); the
ranks of the two low-rank projections are read from their tensors' shapes.
"""
from __future__ import annotations

import torch

from .. import ops
from ..ops import hybrid
from .base import Mixer, SlotState, TensorDecl, VECTOR, register_part
from .runner import BranchPart, Runner, keep

SPLIT_COLUMNS = True             # (the tests switch it off to compare the recurrence's two kernels)


class GatedDeltaRule(BranchPart, Mixer):
    adds_in_place = True

    @classmethod
    def declare(cls, params):
        d, H, G, dim, vdim, K = (params[k] for k in ("hidden", "heads", "kv_heads", "dim", "vdim", "conv"))
        ra, rg = params["decay_rank"], params["gate_rank"]
        return {"q": TensorDecl.of(G * dim, d), "k": TensorDecl.of(G * dim, d), "v": TensorDecl.of(H * vdim, d),
                "q.conv": TensorDecl.of(G * dim, K, role=VECTOR), "k.conv": TensorDecl.of(G * dim, K, role=VECTOR),
                "v.conv": TensorDecl.of(H * vdim, K, role=VECTOR), "b": TensorDecl.of(H, d),
                "A_log": TensorDecl.of(H, role=VECTOR), "dt_bias": TensorDecl.of(H * dim, role=VECTOR),
                "a1": TensorDecl.of(ra, d), "a2": TensorDecl.of(H * dim, ra), "g1": TensorDecl.of(rg, d),
                "g2": TensorDecl.of(H * vdim, rg), "norm": TensorDecl.of(vdim, role=VECTOR), "o": TensorDecl.of(d, H * vdim)}

    def __init__(self, params, tensors, rt):
        super().__init__(params, tensors, rt)
        p = params
        self.hidden, self.heads, self.kv_heads = int(p["hidden"]), int(p["heads"]), int(p["kv_heads"])
        self.dim, self.vdim, self.K = int(p["dim"]), int(p["vdim"]), int(p["conv"])
        self.eps, self.unit_eps = float(p["eps"]), float(p.get("unit_eps", 1e-6))
        self.q_scale = float(p.get("q_scale", self.dim ** -0.5))
        if self.kv_heads < 1 or self.heads % self.kv_heads or self.K < 1:
            raise ValueError(f"{self.heads} heads over {self.kv_heads} key heads, {self.K} taps")
        H, G, dim, vdim = self.heads, self.kv_heads, self.dim, self.vdim
        self.ra, self.rg = tensors["a1"].shape[0], tensors["g1"].shape[0]
        # one product for [q | k | v | beta logits | low-rank decay input | low-rank gate input]
        self.fused = torch.cat([tensors[n] for n in ("q", "k", "v", "b", "a1", "g1")], 0).contiguous()
        self.channels = 2 * G * dim + H * vdim
        self.b_col = self.channels
        self.a_col, self.g_col = self.b_col + H, self.b_col + H + self.ra
        self.a2, self.g2, self.o = (tensors[n].contiguous() for n in ("a2", "g2", "o"))
        f32 = lambda n: tensors[n].to(torch.float32).contiguous()
        self.taps = torch.cat([f32("q.conv"), f32("k.conv"), f32("v.conv")], 0).contiguous()
        self.dt_bias, self.a_log, self.gain = f32("dt_bias"), f32("A_log"), f32("norm")

    def kernel_libraries(self):
        return tuple(set(ops.linear_libraries(self.fused.dtype, self.rt.dtype)) | {"core", hybrid.LIBRARY})

    def cache_needs(self):
        # (a convolution of one tap has nothing to remember; its slot is one unused row)
        return [SlotState((max(self.K - 1, 1), self.channels), torch.float32),
                SlotState((self.heads, self.dim, self.vdim), torch.float32)]

    def run(self, rn: Runner, h, out, caches, accumulate: bool = False):
        conv, rec = caches[0], caches[1]
        H, G, dim, vdim, C = self.heads, self.kv_heads, self.dim, self.vdim, self.channels
        u = rn.buffer("dr_in", self.fused.shape[0], torch.float32)
        rn.linear(h, self.fused, None, u, role="delta_in")
        # the second halves of the two low-rank projections read the first halves as they are: 32-bit columns of u
        a = rn.buffer("dr_decay", H * dim, torch.float32)
        gate = rn.buffer("dr_gate", H * vdim, torch.float32)
        rn.linear(u[:, self.a_col:self.a_col + self.ra], self.a2, None, a, role="delta_decay")
        rn.linear(u[:, self.g_col:self.g_col + self.rg], self.g2, None, gate, role="delta_gate")
        qkv = rn.buffer("dr_conv", C, torch.float32)
        slots = rn.slots(conv)
        rn.op("causal_conv_silu", [u.data_ptr(), u.stride(0), keep(rn, self.taps), 0, keep(rn, conv.state),
                                   conv.state.stride(0), slots, rn.tok_req, rn.q_start, rn.q_len, qkv.data_ptr(),
                                   qkv.stride(0), rn.N, C, self.K, rn.R])
        beta = rn.buffer("dr_beta", H, torch.float32)
        rn.op("delta_prep", [qkv.data_ptr(), qkv.stride(0), G * dim, u.data_ptr() + 4 * self.b_col, u.stride(0),
                             a.data_ptr(), a.stride(0), keep(rn, self.dt_bias), keep(rn, self.a_log), beta.data_ptr(),
                             rn.N, H, G, dim], [self.unit_eps, self.q_scale])
        y = rn.buffer("dr_out", H * vdim, torch.float32)
        rn.op("delta_scan", [qkv.data_ptr(), qkv.stride(0), G * dim, 2 * G * dim, a.data_ptr(), a.stride(0),
                             beta.data_ptr(), keep(rn, rec.state), rec.state.stride(0), slots, rn.q_start, rn.q_len,
                             y.data_ptr(), y.stride(0), rn.R, H, G, dim, vdim], flags=0 if SPLIT_COLUMNS else 1)
        o = rn.buffer("dr_heads_out", H * vdim)
        rn.op("head_norm", [y.data_ptr(), y.stride(0), vdim, 0, keep(rn, self.gain), gate.data_ptr(), gate.stride(0),
                            o.data_ptr(), ops.dtype_code(o.dtype), o.stride(0), rn.N, H, vdim], [self.eps, 0.0, 1.0],
              label="delta_norm_gate")
        (rn.add_linear if accumulate else rn.linear)(o, self.o, None, out, role="delta_out")


register_part("mixer", "gated_delta_rule", GatedDeltaRule)
