"""Feed-forwards whose activation is named: without a gate, out = W_down act(W_up h)
(``dense_mlp``), and with one, out = W_down (act(W_gate h) * (W_up h)) (``gated_mlp``).

``act`` is one of "gelu" (the exact one, with erf), "gelu_tanh", "silu",
"relu".  The first product writes 32-bit values, the function (and the gate's
product with the up rows) is taken in 32-bit and rounded to the compute dtype
for the second product, which adds into the residual stream or writes for an
arrangement that takes the output as it is.
"""
from __future__ import annotations

import torch

from .. import ops
from ..ops import hybrid
from .base import FeedForward, TensorDecl, VECTOR, register_part
from .linear import can_fuse_swiglu, interleave_gate_up
from .runner import BranchPart, Runner

ACTIVATIONS = {"gelu": 0, "gelu_tanh": 1, "silu": 2, "relu": 3}
# act(g) = g * sigmoid(alpha * (g + cubic * g^3)) for the functions that have this form: (alpha, cubic).  The tanh form
# of gelu has it because 0.5 (1 + tanh y) = sigmoid(2 y), with y = sqrt(2 / pi) (g + 0.044715 g^3).
SIGMOID_FORMS = {"silu": (1.0, 0.0), "gelu_tanh": (1.5957691216057308, 0.044715)}
FUSE_GATED_UNIT = True             # (the tests switch it off to compare the two ways)


class DenseMLP(BranchPart, FeedForward):
    adds_in_place = True

    @classmethod
    def declare(cls, params):
        h, f = params["hidden"], params["inner"]
        d = {"up": TensorDecl.of(f, h), "down": TensorDecl.of(h, f)}
        if params.get("bias"):
            d.update({"up.b": TensorDecl.of(f, role=VECTOR), "down.b": TensorDecl.of(h, role=VECTOR)})
        return d

    def __init__(self, params, tensors, rt):
        super().__init__(params, tensors, rt)
        self.hidden, self.inner = int(params["hidden"]), int(params["inner"])
        act = params.get("act", "gelu")
        if act not in ACTIVATIONS:
            raise ValueError(f"unknown activation '{act}'; known: {sorted(ACTIVATIONS)}")
        self.act = ACTIVATIONS[act]
        self.up, self.down = tensors["up"].contiguous(), tensors["down"].contiguous()
        f32 = lambda n: tensors[n].to(torch.float32).contiguous() if params.get("bias") else None
        self.up_bias, self.down_bias = f32("up.b"), f32("down.b")

    def kernel_libraries(self):
        return tuple(set(ops.linear_libraries(self.up.dtype, self.rt.dtype)) | {"core", hybrid.LIBRARY})

    def run(self, rn: Runner, h, out, caches=None, accumulate: bool = False):
        z = rn.buffer("mlp_up", self.inner, torch.float32)
        rn.linear(h, self.up, self.up_bias, z, role="mlp_up")
        act = rn.buffer("mlp_act", self.inner)
        rn.op("act_rows", [z.data_ptr(), z.stride(0), act.data_ptr(), ops.dtype_code(act.dtype), act.stride(0), rn.N,
                           self.inner, self.act])
        (rn.add_linear if accumulate else rn.linear)(act, self.down, self.down_bias, out, role="mlp_down")


class GatedMLP(BranchPart, FeedForward):
    adds_in_place = True

    @classmethod
    def declare(cls, params):
        h, f = params["hidden"], params["inner"]
        return {"gate": TensorDecl.of(f, h), "up": TensorDecl.of(f, h), "down": TensorDecl.of(h, f)}

    def __init__(self, params, tensors, rt):
        super().__init__(params, tensors, rt)
        self.hidden, self.inner = int(params["hidden"]), int(params["inner"])
        act = params.get("act", "silu")
        if act not in ACTIVATIONS:
            raise ValueError(f"unknown activation '{act}'; known: {sorted(ACTIVATIONS)}")
        self.act = ACTIVATIONS[act]
        if tensors["gate"].dtype != tensors["up"].dtype:
            raise ValueError("gate and up projections are stored in different dtypes")
        # one product for gate and up; in bfloat16, for a function of the sigmoid form, its epilogue applies the unit
        # (gate and up rows then alternate in blocks of 64, as for SwiGLU)
        self.fused = FUSE_GATED_UNIT and act in SIGMOID_FORMS and can_fuse_swiglu(tensors["gate"], rt)
        join = interleave_gate_up if self.fused else (lambda g, u: torch.cat([g, u], 0))
        self.gate_up = join(tensors["gate"], tensors["up"]).contiguous()
        self.form = SIGMOID_FORMS.get(act)
        self.down = tensors["down"].contiguous()

    def kernel_libraries(self):
        return tuple(set(ops.linear_libraries(self.gate_up.dtype, self.rt.dtype)) | {"core", hybrid.LIBRARY})

    def run(self, rn: Runner, h, out, caches=None, accumulate: bool = False):
        act = rn.buffer("gmlp_act", self.inner)
        if self.fused:
            alpha, cubic = self.form
            rn.glu_linear(h, self.gate_up, act, (alpha, 0.0, 0.0, cubic), role="mlp_gate_up")
            (rn.add_linear if accumulate else rn.linear)(act, self.down, None, out, role="mlp_down")
            return
        gu = rn.buffer("gmlp_gate_up", 2 * self.inner, torch.float32)
        rn.linear(h, self.gate_up, None, gu, role="mlp_gate_up")
        rn.op("act_rows", [gu.data_ptr(), gu.stride(0), act.data_ptr(), ops.dtype_code(act.dtype), act.stride(0), rn.N,
                           self.inner, self.act, 1], label="act_rows:gated")
        (rn.add_linear if accumulate else rn.linear)(act, self.down, None, out, role="mlp_down")


register_part("feed_forward", "dense_mlp", DenseMLP)
register_part("feed_forward", "gated_mlp", GatedMLP)
