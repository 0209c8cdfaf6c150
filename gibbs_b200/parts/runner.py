"""Two ways to run the same list of operations.

A part whose kernels are operations of the hybrid library writes its work
once, against a ``Runner``: buffers, matrix products, operations with operand
lists.  ``Eager`` launches everything now (the parts' ``forward``); ``Planned``
appends the same operations to a step plan (``plan_ops``), where the numbers
and addresses that change from step to step are symbols.  Both therefore
compute the same bits.
"""
from __future__ import annotations

from typing import Optional

import torch

from .. import ops
from ..ops import hybrid
from .base import NotPlannable, Residual


class Runner:
    # rows in the step, requests, wanted rows; addresses of the step's metadata
    N = R = W = 0
    max_context = 0      # the longest context of the step after it (inside a CUDA graph: an upper bound)
    token_ids = tok_req = tok_pos = q_start = q_len = start_pos = want_rows = 0

    def buffer(self, name: str, width: int, dtype=None, per_token: int = 1, fixed_rows: Optional[int] = None):
        """A scratch tensor [rows, width]: one row per token of the step (times ``per_token``),
        or ``fixed_rows`` rows whatever the step."""
        raise NotImplementedError

    def linear(self, x, weight, bias, out, role: str = "") -> None:
        """out = x weight^T (+ bias); the kernel is chosen by the operand types.  ``role`` names
        the product in the timing table."""
        raise NotImplementedError

    def add_linear(self, x, weight, bias, out, role: str = "") -> None:
        """out += x weight^T (+ bias), for ``out`` the 32-bit residual stream: a sublayer's last product does
        the residual sum."""
        raise NotImplementedError

    def glu_linear(self, x, weight, out, glu, role: str = "") -> None:
        """out = unit(x weight^T) on the tensor cores, for a weight whose gate and up rows alternate in
        blocks of 64 (``parts.linear.interleave_gate_up``); ``glu`` = (alpha, limit, add)."""
        raise NotImplementedError

    def op(self, name: str, a, f=(), label: str = "", flags: int = 0) -> None:
        raise NotImplementedError

    def table(self, view):
        """(address of the step's block table for a paged view, its entries per request)."""
        raise NotImplementedError

    def slots(self, view):
        """Address of the step's slot ids."""
        raise NotImplementedError


class Eager(Runner):
    def __init__(self, rt, step):
        self.rt, self.step = rt, step
        self.N, self.R, self.W = step.n_tokens, step.n_requests, step.n_want
        self.max_context = max(int(step.max_ctx_len), 1)
        for k in ("token_ids", "tok_req", "tok_pos", "q_start", "q_len", "start_pos", "want_rows"):
            setattr(self, k, getattr(step, k).data_ptr())

    def buffer(self, name, width, dtype=None, per_token=1, fixed_rows=None):
        rows = fixed_rows if fixed_rows is not None else self.N * per_token
        return torch.empty(rows, int(width), dtype=dtype or self.rt.dtype, device=self.rt.device)

    def linear(self, x, weight, bias, out, role=""):
        ops.linear(x[:self.N] if x.shape[0] != self.N else x, weight, bias, out)

    def add_linear(self, x, weight, bias, out, role=""):
        ops.linear(x[:self.N] if x.shape[0] != self.N else x, weight, bias, out, True)

    def glu_linear(self, x, weight, out, glu, role=""):
        ops.linear_tc(x[:self.N] if x.shape[0] != self.N else x, weight, None, out, swiglu=True, glu=glu)

    def op(self, name, a, f=(), label="", flags=0):
        hybrid.call(name, a, f, flags=flags, device=self.rt.device)

    def table(self, view):
        bt = view.block_table
        return bt.data_ptr(), (bt.shape[1] if bt.dim() == 2 else 0)

    def slots(self, view):
        return view.slot_ids.data_ptr()


class Planned(Runner):
    def __init__(self, plan):
        from ..engine import plan as P
        self.plan, self.rt = plan, plan.rt
        self.N, self.R, self.W = P.sym(P.S_N), P.sym(P.S_R), P.sym(P.S_W)
        self.token_ids, self.tok_req, self.tok_pos = P.sym(P.S_TOKEN_IDS), P.sym(P.S_TOK_REQ), P.sym(P.S_TOK_POS)
        self.q_start, self.q_len, self.start_pos = P.sym(P.S_Q_START), P.sym(P.S_Q_LEN), P.sym(P.S_START_POS)
        self.want_rows = P.sym(P.S_WANT_ROWS)
        self.max_context = P.sym(P.S_MAXCTX)
        self._P = P

    def buffer(self, name, width, dtype=None, per_token=1, fixed_rows=None):
        rows = fixed_rows if fixed_rows is not None else self.plan.cap * per_token
        return self.plan.buffer(f"{name}[{rows}]", width, dtype, rows=rows)

    def linear(self, x, weight, bias, out, role=""):
        self.plan.linear(x, weight, bias, out, "plain", role=role or "plain")

    def add_linear(self, x, weight, bias, out, role=""):
        if out is not self.plan.residual:
            raise NotPlannable("a plan's products add into the plan's own residual stream")
        self.plan.linear(x, weight, bias, None, "residual", role=role or "residual")

    def glu_linear(self, x, weight, out, glu, role=""):
        self.plan.linear(x, weight, None, out, "swiglu", role=role or "glu", glu=glu)

    def op(self, name, a, f=(), label="", flags=0):
        self.plan.emit(hybrid.plan_id(name), list(a), list(f), flags=flags, label=label or name)

    def table(self, view):
        if not isinstance(view.block_table, self._P.TableRef):
            raise NotPlannable("a paged cache is read through the step's block tables")
        return self._P.sym(self._P.S_BLOCK_TABLE0 + view.block_table.group), self.plan.bt_stride

    def slots(self, view):
        if not isinstance(view.slot_ids, self._P.SlotRef):
            raise NotPlannable("state lives in the step's slots")
        return self._P.sym(self._P.S_SLOT_IDS)


def keep(rn: Runner, t: Optional[torch.Tensor]) -> int:
    """Address of a tensor an operation reads (0 for None); a plan keeps it alive."""
    if t is None:
        return 0
    if isinstance(rn, Planned):
        return rn.plan.keep(t)
    return t.data_ptr()


def stream_tensor(x) -> torch.Tensor:
    """The 32-bit residual stream as a tensor."""
    return x.tensor() if isinstance(x, Residual) else x


class BranchPart:
    """Mixin for mixers and feed-forwards written against a ``Runner``: ``run(rn, h, out,
    caches)`` WRITES the sublayer's output into ``out`` (float32 [rows, hidden]), so that an
    arrangement can put a norm between the sublayer and the residual sum.  In an arrangement
    that adds sublayers straight into the stream, ``forward`` adds ``out`` to it."""
    writes_branch = True
    # True for a part whose ``run`` takes ``accumulate=True`` and then ADDS its output into ``out``: in an
    # arrangement that sums sublayers straight into the stream its last kernel does the residual sum
    adds_in_place = False

    def forward(self, h, residual, step, caches=None):
        rn = Eager(self.rt, step)
        if isinstance(residual, Residual):
            if self.adds_in_place:
                self.run(rn, h, residual.tensor(), caches, accumulate=True)
                return
            y = rn.buffer("branch", residual.shape[1], torch.float32)
            self.run(rn, h, y, caches)
            ops.add_pending(residual.tensor(), y.unsqueeze(0), None)
        else:
            self.run(rn, h, residual, caches)

    def plan_ops(self, plan, h, caches=None, out=None):
        if out is None:
            if not self.adds_in_place:
                raise NotPlannable(f"{type(self).__name__} writes its output for a norm to add; a plan needs an "
                                   "arrangement that takes it")
            # (an operation of the hybrid library finds the stream whole: the walker adds what a product left)
            self.run(Planned(plan), h, plan.residual, caches, accumulate=True)
            return
        self.run(Planned(plan), h, out, caches)
