"""Bindings of the "hybrid" kernel library (csrc/norms.cu, latent_attention.cu,
gated_attention.cu, gated_attention_tc.cu, ssm.cu, delta_rule.cu, moe.cu): layer norms, clamped gated units, latent
attention, gated attention with a sink, state-space and delta-rule recurrences and routed experts.

Every operation of that library has the signature of a step-plan operation,
``int op(ctx, a[24], f[3], flags)``.  So an operation is described ONCE, by
its operand list, and run in either of two ways: ``call`` launches it now, on
the current stream; ``plan_id`` registers it with the step walker, which then
calls the same function with the same operands for every step.  An operand is
an integer, a device address, or (in a plan) a symbol of the step.
"""
from __future__ import annotations

import ctypes

import torch

from . import _launched, _stream, device_status
from .library import check, library

LIBRARY = "hybrid"
OPERATIONS = ("row_norm", "norm_add", "clamped_glu", "gelu_mul_rows", "gated_group_norm", "causal_conv_silu",
              "ssm_scan", "latent_prep", "head_linear", "latent_attention", "moe_route", "moe_sort", "moe_gather",
              "moe_experts", "moe_experts_tc", "moe_combine", "moe_route_grouped", "moe_combine_weighted",
              "embed_scaled", "qk_prep", "sink_attention", "sink_attention_tc", "act_rows", "head_norm", "delta_prep",
              "delta_scan", "scaled_sum")

NORM_LAYER, NORM_RMS = 0, 1
TAKES_PENDING = 1 << 30          # a record's flag: the operation adds the sums a product left pending itself


class _Ctx(ctypes.Structure):
    _fields_ = [("stream", ctypes.c_void_p), ("status", ctypes.c_void_p), ("sym", ctypes.c_void_p),
                ("n_sym", ctypes.c_int), ("residual", ctypes.c_void_p), ("residual_ld", ctypes.c_longlong),
                ("pend", ctypes.c_void_p), ("pend_splits", ctypes.c_int), ("pend_bias", ctypes.c_void_p)]


_FN: dict = {}
_IDS: dict = {}


def _function(name: str):
    fn = _FN.get(name)
    if fn is None:
        if name not in OPERATIONS:
            raise KeyError(f"the hybrid library has no operation '{name}'; it has {OPERATIONS}")
        fn = _FN[name] = getattr(library(LIBRARY), "gb_op_" + name)
        fn.restype = ctypes.c_int
    return fn


def call(name: str, a, f=(), flags: int = 0, device=None) -> int:
    """Launch one operation now, on the current stream."""
    fn = _function(name)
    if len(a) > 24 or len(f) > 3:
        raise ValueError("an operation has 24 integer and 3 floating-point operands")
    if any(int(v) < 0 for v in a):
        raise ValueError(f"{name}: operands are non-negative numbers or addresses (a plan keeps bit 62 for symbols); got {list(a)}")
    ia = (ctypes.c_longlong * 24)(*[int(v) for v in a])
    fa = (ctypes.c_double * 3)(*[float(v) for v in f])
    status = device_status(device if device is not None else torch.device("cuda", torch.cuda.current_device()))
    stream = _stream()
    ctx = _Ctx(stream.value if isinstance(stream, ctypes.c_void_p) else stream, status.data_ptr(), None, 0, None, 0, None, 0,
               None)                # (called directly, nothing is ever pending)
    rc = fn(ctypes.byref(ctx), ia, fa, ctypes.c_int(flags))
    if rc < 0:
        check(library(LIBRARY), rc)
    _launched(rc)
    return rc


def plan_id(name: str) -> int:
    """The operation's id with the step walker (registered at first use)."""
    i = _IDS.get(name)
    if i is None:
        from ..engine.plan import register_op
        i = _IDS[name] = register_op("hybrid." + name, _function(name))
    return i
