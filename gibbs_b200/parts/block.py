"""Arrangements of norm, mixer and feed-forward around the residual stream."""
from __future__ import annotations

import torch

from .. import ops
from .base import Block, Part, TensorDecl, VECTOR, plan_ops_of, register_part
from .norm import RowNorm
from .runner import Eager, Planned, stream_tensor


class PreNormResidual(Block):
    """x += mixer(norm(x)); x += ffn(norm(x))
    (MisterTK/gibbs arch/families/lfm2.json5:76-89)."""
    ROLES = (("mixer_norm", "norm"), ("mixer", "mixer"), ("ffn_norm", "norm"), ("ffn", "feed_forward"))
    OPTIONAL_ROLES = ("ffn_norm", "ffn")       # a layer may have no feed-forward (then neither its norm)

    # A mixer or feed-forward that says ``fuses_norm`` hands its input straight to a product
    # (``parts.linear.Linear``), which may then run the norm itself.

    def forward(self, x, step, caches):
        h = self.mixer_norm.lazy(x) if getattr(self.mixer, "fuses_norm", False) else self.mixer_norm.forward(x)
        self.mixer.forward(h, x, step, self.caches_of("mixer", caches))
        if "ffn" not in self.parts:
            return
        h = self.ffn_norm.lazy(x) if getattr(self.ffn, "fuses_norm", False) else self.ffn_norm.forward(x)
        self.ffn.forward(h, x, step)

    def plan_ops(self, plan, caches):
        h = self._norm_ops(plan, self.mixer_norm, self.mixer)
        plan_ops_of(self.mixer)(plan, h, self.caches_of("mixer", caches))
        if "ffn" not in self.parts:
            return
        h = self._norm_ops(plan, self.ffn_norm, self.ffn)
        plan_ops_of(self.ffn)(plan, h)

    @staticmethod
    def _norm_ops(plan, norm, consumer):
        if getattr(consumer, "fuses_norm", False) and getattr(norm, "lazy", None) is not None:
            try:
                return plan_ops_of(norm)(plan, lazy=True)
            except TypeError:            # a norm from outside whose plan_ops knows no such option
                pass
        return plan_ops_of(norm)(plan)


register_part("block", "prenorm_residual", PreNormResidual)


class SandwichResidual(Block):
    """A norm in front of AND behind every sublayer:

        x += post_norm(mixer(norm(x)));  x += post_norm(ffn(norm(x)));  token_input(x)

    The feed-forward (with its two norms) and the token input are optional.  Sublayers write
    their output for the norm behind them (``parts.runner.BranchPart``); the norms behind are
    ``RowNorm`` kinds, whose ``add_normed`` adds into the stream."""
    ROLES = (("mixer_norm", "norm"), ("mixer", "mixer"), ("mixer_post_norm", "norm"), ("ffn_norm", "norm"),
             ("ffn", "feed_forward"), ("ffn_post_norm", "norm"), ("token_input", "token_input"))
    OPTIONAL_ROLES = ("ffn_norm", "ffn", "ffn_post_norm", "token_input")

    def __init__(self, parts, rt, params=None):
        super().__init__(parts, rt, params)
        have = set(self.parts)
        if len(have & {"ffn_norm", "ffn", "ffn_post_norm"}) not in (0, 3):
            raise ValueError("a feed-forward comes with the norm in front of it and the norm behind it")
        for role in ("mixer", "ffn"):
            if role in have and not getattr(self.parts[role], "writes_branch", False):
                raise ValueError(f"the {role} of this arrangement must be able to write its output for the norm "
                                 f"behind it; {type(self.parts[role]).__name__} only adds into the stream")
        for role in ("mixer_post_norm", "ffn_post_norm"):
            if role in have and not hasattr(self.parts[role], "add_normed"):
                raise ValueError(f"the {role} must be a norm that can add into the stream (a RowNorm kind)")

    def _run(self, rn, x, caches, h_of):
        hidden = x.shape[1]
        y = rn.buffer("branch", hidden, torch.float32)
        # a token input reads the stream through a product: in bfloat16 the norm that completes the
        # stream also leaves the rows in that type
        copy = None
        if "token_input" in self.parts and self.rt.dtype == torch.bfloat16:
            copy = rn.buffer("stream_rows", hidden, torch.bfloat16)
        has_ffn = "ffn" in self.parts
        self.mixer.run(rn, h_of(self.mixer_norm), y, self.caches_of("mixer", caches))
        # the norm in front of the feed-forward is taken in the kernel that completes the stream behind the mixer
        fuse = has_ffn and isinstance(self.ffn_norm, RowNorm) and self.ffn_norm.dim == hidden
        h = self.mixer_post_norm.add_normed(rn, x, y, None if has_ffn else copy, self.ffn_norm if fuse else None)
        if has_ffn:
            self.ffn.run(rn, h if fuse else h_of(self.ffn_norm), y, None)
            self.ffn_post_norm.add_normed(rn, x, y, copy)
        if "token_input" in self.parts:
            self.token_input.run(rn, x, copy)

    def forward(self, x, step, caches):
        rn, xt = Eager(self.rt, step), stream_tensor(x)
        self._run(rn, xt, caches, lambda norm: norm.forward(xt))

    def plan_ops(self, plan, caches):
        self._run(Planned(plan), plan.residual, caches, lambda norm: plan_ops_of(norm)(plan))


register_part("block", "sandwich_residual", SandwichResidual)


class ScaledSum(Part):
    """The residual sum of sublayers that run side by side: x += mult * (s_1 * y_1 + s_2 * y_2 + ...), with one
    scale vector per sublayer (tensors named after the sublayers' roles, ``branches``) and one factor ``mult``
    on the whole; 32-bit throughout.  One kernel reads the stream and the outputs once."""
    category = "branch_sum"

    @classmethod
    def declare(cls, params):
        return {name: TensorDecl.of(params["dim"], role=VECTOR) for name in params["branches"]}

    def __init__(self, params, tensors, rt):
        super().__init__(params, tensors, rt)
        self.dim, self.mult = int(params["dim"]), float(params.get("mult", 1.0))
        self.branches = tuple(params["branches"])
        if not 1 <= len(self.branches) <= 2:
            raise ValueError(f"a sum of {len(self.branches)} sublayers; the kernel takes one or two")
        self.scales = [tensors[name].to(torch.float32).contiguous() for name in self.branches]

    def kernel_libraries(self):
        from ..ops import hybrid
        return ("core", hybrid.LIBRARY)

    def add(self, rn, x: torch.Tensor, outputs: list, then=None):
        """``outputs``: the sublayers' outputs (float32 [rows, dim]) in the order of ``branches``.  ``then`` (a
        RowNorm: the norm in front of the next layer) is taken of the new rows in the same kernel; its output is
        returned."""
        from .runner import keep
        if len(outputs) != len(self.branches):
            raise ValueError(f"{len(outputs)} outputs for the sublayers {self.branches}")
        y2 = outputs[1] if len(outputs) > 1 else None
        a = [x.data_ptr(), x.stride(0), outputs[0].data_ptr(), outputs[0].stride(0), keep(rn, self.scales[0]),
             0 if y2 is None else y2.data_ptr(), 0 if y2 is None else y2.stride(0),
             0 if y2 is None else keep(rn, self.scales[1]), rn.N, self.dim]
        f, out = [self.mult], None
        if then is not None:
            out = rn.buffer("normed", then.dim)
            a += [keep(rn, then.gain), out.data_ptr(), ops.dtype_code(out.dtype), then.KIND]
            f += [then.eps]
        rn.op("scaled_sum", a, f, label="scaled_sum")
        return out


register_part("branch_sum", "scaled_sum", ScaledSum)


FUSE_NEXT_NORM = True            # (the tests switch it off to compare the two ways)


class ParallelResidual(Block):
    """One norm, and both sublayers read its output:

        h = norm(x);  x += sum(mixer(h), ffn(h))

    where ``sum`` is a ``branch_sum`` part (scales per channel, a factor).  The feed-forward is optional.  The
    sublayers write their outputs (``parts.runner.BranchPart``, or any part with such a ``run``).

    When the layer that runs next is of this kind too, its norm is taken in the kernel of this layer's sum, of the
    new rows while they are in registers (``hands_over``, which the model calls for neighbours in its order)."""
    ROLES = (("norm", "norm"), ("mixer", "mixer"), ("ffn", "feed_forward"), ("sum", "branch_sum"))
    OPTIONAL_ROLES = ("ffn",)

    def __init__(self, parts, rt, params=None):
        super().__init__(parts, rt, params)
        for role in ("mixer", "ffn"):
            if role in self.parts and not getattr(self.parts[role], "writes_branch", False):
                raise ValueError(f"the {role} of this arrangement must be able to write its output for the sum behind "
                                 f"it; {type(self.parts[role]).__name__} only adds into the stream")
        want = ("mixer", "ffn") if "ffn" in self.parts else ("mixer",)
        if tuple(self.parts["sum"].branches) != want:
            raise ValueError(f"the sum is over {self.parts['sum'].branches}; the layer has {want}")
        self._next = None          # the block that runs next, when its norm is taken here
        self._handed = None        # the normed rows the block in front left for this one

    def hands_over(self, following) -> bool:
        """Called once when the model is put together: ``following`` runs right behind this block, and only there."""
        if (FUSE_NEXT_NORM and isinstance(following, ParallelResidual) and isinstance(following.norm, RowNorm)
                and following.norm.dim == self.sum.dim):
            self._next = following
            return True
        return False

    def _run(self, rn, x, caches, h):
        hidden = x.shape[1]
        outputs = [rn.buffer("branch", hidden, torch.float32)]
        self.mixer.run(rn, h, outputs[0], self.caches_of("mixer", caches))
        if "ffn" in self.parts:
            outputs.append(rn.buffer("branch_ffn", hidden, torch.float32))
            self.ffn.run(rn, h, outputs[1], None)
        if self._next is None:
            self.sum.add(rn, x, outputs)
        else:
            self._next._handed = self.sum.add(rn, x, outputs, then=self._next.norm)

    def _take_handed(self):
        h, self._handed = self._handed, None
        return h

    def forward(self, x, step, caches):
        xt = stream_tensor(x)
        h = self._take_handed()
        self._run(Eager(self.rt, step), xt, caches, self.norm.forward(xt) if h is None else h)

    def plan_ops(self, plan, caches):
        h = self._take_handed()
        self._run(Planned(plan), plan.residual, caches, plan_ops_of(self.norm)(plan) if h is None else h)


register_part("block", "parallel_residual", ParallelResidual)
