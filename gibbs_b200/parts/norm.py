"""Norms over rows of the residual stream.

RMSNorm: x * (1/sqrt(mean(x^2) + eps)) * gain, statistics in 32-bit
(MisterTK/gibbs arch/lib/transformer.json5:9-11; src/model/simd.rs:73-111), with the
split-K and decode-product couplings of the core kernels.  RowNorm and its kinds (layer
norm, plain RMS norm): the same statistics on the hybrid library, usable in front of a
sublayer and behind one.

``gain_offset`` (every kind; default 0): the stored weight is the gain's distance from this number, so a
design that keeps its norm weights around zero sets 1 and the rows are multiplied by 1 + weight.  The sum is
taken once, in 32-bit, when the part is built."""
from __future__ import annotations

import torch

from .. import ops
from ..ops import hybrid
from .base import Norm, Residual, TensorDecl, VECTOR, register_part
from .runner import Planned, Runner, keep, stream_tensor


def stored_gain(weight: torch.Tensor, params: dict) -> torch.Tensor:
    """The 32-bit gain a norm multiplies by: the stored weight plus ``gain_offset``."""
    gain = weight.to(torch.float32)
    offset = float(params.get("gain_offset", 0.0) or 0.0)
    return (gain + offset if offset else gain).contiguous()


class RMSNorm(Norm):
    @classmethod
    def declare(cls, params):
        return {"weight": TensorDecl.of(params["dim"], role=VECTOR)}

    def __init__(self, params, tensors, rt):
        super().__init__(params, tensors, rt)
        self.dim, self.eps = int(params["dim"]), float(params["eps"])
        self.gain = stored_gain(tensors["weight"], params)

    def forward(self, x, out=None, rows=None):
        pending = None
        if isinstance(x, Residual):
            pending, x = x.take_pending(), x.x
        n = x.shape[0] if rows is None else rows.numel()
        if out is None:
            out = self.rt.empty(n, self.dim)
        return ops.rmsnorm(x, self.gain, self.eps, out, rows, pending)

    def lazy(self, x, rows=None):
        """Up to 16 rows of the stream in bfloat16: the product that reads them runs the
        norm itself (csrc/gemm_tc_decode.cu), with the sums of squares the product before
        left when there are some."""
        n = (x.shape[0] if rows is None else rows.numel())
        if (isinstance(x, Residual) and x.pending is None and ops.DECODE_PRODUCTS and ops.DECODE_NORM_INSIDE and self.rt.dtype == torch.bfloat16
                and n <= min(16, ops.DECODE_ROWS) and self.dim % 8 == 0 and x.x.stride(1) == 1 and x.x.stride(0) % 4 == 0
                and x.x.data_ptr() % 16 == 0):
            return ops.NormedRows(x.x, self.gain, self.eps, rows, x.ssq)
        return self.forward(x, rows=rows)

    def plan_ops(self, plan, wanted_rows: bool = False, lazy: bool = False):
        return plan.rmsnorm(self.gain, self.eps, wanted_rows, lazy=lazy)


register_part("norm", "rmsnorm", RMSNorm)


class RowNorm(Norm):
    """A norm over rows of the 32-bit stream with a gain and no bias, statistics in 32-bit,
    on the hybrid library's kernels.  ``KIND`` picks the rule.  Besides the norm in front of
    a sublayer (``forward``) it serves as the norm BEHIND one: ``add_normed`` adds
    norm(y) * gain into the stream."""
    KIND = hybrid.NORM_LAYER

    @classmethod
    def declare(cls, params):
        return {"weight": TensorDecl.of(params["dim"], role=VECTOR)}

    def __init__(self, params, tensors, rt):
        super().__init__(params, tensors, rt)
        self.dim, self.eps = int(params["dim"]), float(params["eps"])
        self.gain = stored_gain(tensors["weight"], params)

    def kernel_libraries(self):
        return ("core", hybrid.LIBRARY)

    def run(self, rn: Runner, x: torch.Tensor, wanted_rows: bool = False) -> torch.Tensor:
        out = rn.buffer("normed_wanted" if wanted_rows else "normed", self.dim)
        rn.op("row_norm", [x.data_ptr(), x.stride(0), keep(rn, self.gain), out.data_ptr(), ops.dtype_code(out.dtype),
                           rn.want_rows if wanted_rows else 0, rn.W if wanted_rows else rn.N, self.dim, self.KIND],
              [self.eps], label="row_norm", flags=hybrid.TAKES_PENDING)
        return out

    def add_normed(self, rn: Runner, x: torch.Tensor, y: torch.Tensor, copy: torch.Tensor = None, then=None):
        """x += norm(y) * gain, for x the stream and y a sublayer's output (both float32).  ``copy``
        (bfloat16 [rows, dim], contiguous) also receives the new rows, for a product that reads
        the stream next.  ``then`` (another RowNorm: the norm in front of the next sublayer) is taken
        of the new rows in the same kernel; its output is returned."""
        a = [x.data_ptr(), x.stride(0), y.data_ptr(), y.stride(0), keep(rn, self.gain), rn.N, self.dim, self.KIND,
             0 if copy is None else copy.data_ptr()]
        f = [self.eps]
        out = None
        if then is not None:
            out = rn.buffer("normed", then.dim)
            a += [keep(rn, then.gain), out.data_ptr(), ops.dtype_code(out.dtype), then.KIND]
            f += [then.eps]
        rn.op("norm_add", a, f, label="norm_add")
        return out

    def forward(self, x, out=None, rows=None):
        x = stream_tensor(x)
        n = x.shape[0] if rows is None else rows.numel()
        if out is None:
            out = self.rt.empty(n, self.dim)
        hybrid.call("row_norm", [x.data_ptr(), x.stride(0), self.gain.data_ptr(), out.data_ptr(),
                                 ops.dtype_code(out.dtype), 0 if rows is None else rows.data_ptr(), n, self.dim,
                                 self.KIND], [self.eps], device=self.rt.device)
        return out

    def plan_ops(self, plan, wanted_rows: bool = False, lazy: bool = False):
        return self.run(Planned(plan), plan.residual, wanted_rows)


class LayerNorm(RowNorm):
    """(x - mean) / sqrt(var + eps) * gain, var the mean of the squared deviations."""
    KIND = hybrid.NORM_LAYER


class PlainRMSNorm(RowNorm):
    """x / sqrt(mean(x^2) + eps) * gain."""
    KIND = hybrid.NORM_RMS


register_part("norm", "layernorm", LayerNorm)
register_part("norm", "rmsnorm_rows", PlainRMSNorm)
