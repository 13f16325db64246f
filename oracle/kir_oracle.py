"""CPU oracle: a torch restatement of the reference's interpreter for kernel IR.

TEST INFRASTRUCTURE ONLY.  Nothing in ``mlc_compiler_b200`` imports this file;
it is the checker used by ``tests/``, by ``__graft_entry__.smoke()`` and by the
CPU-baseline legs of ``bench.py``.  It shares only the IR data classes
(``mlc_compiler_b200.kir``) with the product.

What it restates: the reference's torch backend, ``mlc/codegen/torch_backend.py``
-- ``run_pointwise`` (``:100-118``), ``run_reduction`` (``:128-248``: the
persistent walk ``:172-186`` and the streamed form ``:187-236`` with its 1024
column chunks, chunk-wise accumulation order and per-row online softmax
recurrence), ``eval_expr`` (``:65-83``), the fp16/bf16 -> fp32 widening of loads
(``:53-62``) -- together with the pass rules of
``mlc/codegen/reduction_schedule.py`` (what a pass recomputes stops at earlier
reductions ``:62-91``, online softmax detection ``:119-147``) and the executor's
buffer table and extern dispatch (``mlc/runtime/executor.py:107-162, 369-402``).
The arithmetic itself lives in torch (ATen CPU kernels), exactly as in the
reference; this file only decides which tensors meet which operator, in which
dtype and in which order.

It is organised differently from the reference: offsets come from the
``(size, out_stride, in_stride)`` terms rather than from ``eval`` of rendered
index text, and a reduction is evaluated on demand -- asking for a value over a
span of columns pulls in exactly the temporaries it depends on, stopping at
reduction results -- instead of from a precomputed list of passes.  A
persistent kernel is then the special case of a single span covering the row.

Parity pin: ``tests/golden/`` holds schedules, seeded inputs and the outputs of
the *reference's own* torch backend for them (written by
``tests/golden/make_golden.py`` with the reference importable);
``tests/test_oracle.py`` checks this file against those kernel by kernel, and
it reproduces them bit for bit on the machine that generated them.
"""

from __future__ import annotations

import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
from mlc_compiler_b200 import kir  # noqa: E402  (IR definitions only)

OPS = {
    "neg": lambda a: -a, "abs": torch.abs, "reciprocal": torch.reciprocal, "exp": torch.exp,
    "log": torch.log, "sqrt": torch.sqrt, "rsqrt": torch.rsqrt, "sin": torch.sin,
    "cos": torch.cos, "tanh": torch.tanh, "erf": torch.erf, "sigmoid": torch.sigmoid,
    "floor": torch.floor, "logical_not": torch.logical_not, "add": torch.add,
    "sub": torch.sub, "mul": torch.mul, "div": torch.div, "pow": torch.pow,
    "maximum": torch.maximum, "minimum": torch.minimum, "gt": torch.gt, "lt": torch.lt,
    "ge": torch.ge, "le": torch.le, "eq": torch.eq, "ne": torch.ne,
    "logical_and": torch.logical_and, "logical_or": torch.logical_or, "where": torch.where,
}
ROW_REDUCE = {"sum": torch.sum, "max": torch.amax, "min": torch.amin, "prod": torch.prod}
MERGE = {"sum": torch.add, "max": torch.maximum, "min": torch.minimum, "prod": torch.mul}
#: columns per step of a streamed reduction (``run_reduction(..., chunk=1024)``)
CHUNK = 1024


def widen(t: torch.Tensor) -> torch.Tensor:
    """Narrow floats are computed on as fp32."""
    return t.float() if t.dtype in (torch.float16, torch.bfloat16) else t


def offsets(m: kir.IndexMap, **var: torch.Tensor) -> torch.Tensor:
    """``base + sum ((v // out_stride) % size) * in_stride`` over broadcastable
    int64 tensors, one per iteration variable."""
    total = torch.zeros((), dtype=torch.int64)
    for axis in m.axes:
        v = var[axis.var]
        for size, ostride, istride in axis.terms:
            total = total + (torch.div(v, ostride, rounding_mode="floor") % size) * istride
    return total + m.base


def constant(c: kir.Const, like: torch.Tensor) -> torch.Tensor:
    # bool literals are materialised at full size, numbers as 0-dim tensors: the
    # difference decides torch's type promotion further up the expression
    if isinstance(c.value, bool):
        return torch.full_like(like, float(c.value), dtype=torch.bool)
    return torch.as_tensor(c.value, dtype=kir.torch_dtype(c.dtype) if c.dtype else None)


# --------------------------------------------------------------------------
# pointwise
# --------------------------------------------------------------------------

def run_pointwise(k: kir.PointwiseKernel, buffers: dict[str, torch.Tensor]) -> None:
    idx = torch.arange(k.numel, dtype=torch.int64)
    operands = [widen(buffers[a.buffer][offsets(a.index, idx=idx)]) for a in k.inputs]
    like = operands[0] if operands else idx
    temps: dict[str, torch.Tensor] = {}

    def value(e):
        if isinstance(e, kir.Load):
            return operands[e.slot]
        if isinstance(e, kir.Ref):
            return temps[e.name]
        if isinstance(e, kir.Const):
            return constant(e, like)
        if isinstance(e, kir.Cast):
            return value(e.x).to(kir.torch_dtype(e.dtype))
        return OPS[e.fn](*[value(a) for a in e.args])

    for name, e in k.body:
        temps[name] = value(e)
    for out in k.outputs:
        v = value(k.out_expr[out.name])
        dest = buffers[out.buffer]
        if v.numel() == 1:
            v = v.reshape(()).expand(k.numel)
        dest[offsets(out.index, idx=idx)] = v.reshape(-1).to(dest.dtype)


# --------------------------------------------------------------------------
# reductions
# --------------------------------------------------------------------------

class _Rows:
    """Demand-driven evaluation of one reduction kernel over all rows at once."""

    def __init__(self, k: kir.ReductionKernel, buffers: dict[str, torch.Tensor]):
        self.k, self.buffers = k, buffers
        self.row = torch.arange(k.n_rows, dtype=torch.int64).unsqueeze(1)
        self.steps = {s.name: s for s in k.steps}
        self.done: dict[str, torch.Tensor] = {}          # finished reductions, [rows, 1]

    def span(self, lo: int, hi: int) -> "_Span":
        return _Span(self, torch.arange(lo, hi, dtype=torch.int64).unsqueeze(0))

    def spans(self, width: int):
        for lo in range(0, self.k.n_cols, width):
            yield self.span(lo, min(lo + width, self.k.n_cols))

    def online_pair(self):
        """``(max step, sum step, maxed expression)`` when the kernel is a max
        followed by a sum of ``exp(x - max)`` over the same ``x``."""
        rs = self.k.reduces
        if len(rs) != 2 or (rs[0].kind, rs[1].kind) != ("max", "sum"):
            return None

        def through_binds(e):
            while isinstance(e, kir.Ref) and isinstance(self.steps.get(e.name), kir.Bind):
                e = self.steps[e.name].expr
            return e

        summed = through_binds(rs[1].expr)
        if not (isinstance(summed, kir.Call) and summed.fn == "exp"):
            return None
        shifted = through_binds(summed.args[0])
        if not (isinstance(shifted, kir.Call) and shifted.fn == "sub"):
            return None
        minuend, subtrahend = shifted.args
        if not (isinstance(subtrahend, kir.Ref) and subtrahend.name == rs[0].name):
            return None
        if through_binds(minuend) != through_binds(rs[0].expr):
            return None
        return rs[0], rs[1], rs[0].expr


class _Span:
    """Values of the kernel's expressions over a contiguous span of columns."""

    def __init__(self, rows: _Rows, col: torch.Tensor):
        self.rows, self.col = rows, col
        self.width = col.shape[1]
        self._operands: dict[int, torch.Tensor] = {}
        self._temps: dict[str, torch.Tensor] = {}

    def operand(self, slot: int) -> torch.Tensor:
        if slot not in self._operands:
            r = self.rows
            a = r.k.inputs[slot]
            row = r.row
            if a.via is not None:
                # row gather: the row of the table is the integer another operand
                # holds for this row (``aten.embedding`` folded into its consumer)
                slot, table_rows = a.via
                ids = r.k.inputs[slot]
                at = offsets(ids.index, row=r.row, col=torch.zeros((1, 1), dtype=torch.int64))
                row = r.buffers[ids.buffer][at.expand(r.k.n_rows, 1)].to(torch.int64)
                row = row.clamp(0, table_rows - 1)
            off = offsets(a.index, row=row, col=self.col)
            self._operands[slot] = widen(r.buffers[a.buffer][off.expand(r.k.n_rows, self.width)])
        return self._operands[slot]

    def _like(self) -> torch.Tensor:
        return self.operand(0) if self.rows.k.inputs else self.rows.row

    def value(self, e) -> torch.Tensor:
        if isinstance(e, kir.Load):
            return self.operand(e.slot)
        if isinstance(e, kir.Const):
            return constant(e, self._like())
        if isinstance(e, kir.Cast):
            return self.value(e.x).to(kir.torch_dtype(e.dtype))
        if isinstance(e, kir.Call):
            return OPS[e.fn](*[self.value(a) for a in e.args])
        # a reference: a finished reduction is a per-row scalar that outlives the
        # span that produced it; anything else is recomputed for this span
        if e.name in self.rows.done:
            return self.rows.done[e.name]
        if e.name not in self._temps:
            step = self.rows.steps[e.name]
            if isinstance(step, kir.Reduce):
                raise RuntimeError(f"{e.name} is read before it has been reduced")
            self._temps[e.name] = self.value(step.expr)
        return self._temps[e.name]

    def full(self, e) -> torch.Tensor:
        """``value`` broadcast to ``[rows, width]`` (what a reduction consumes)."""
        v = self.value(e)
        if v.dim() < 2 or v.shape[1] == 1:
            v = v.expand(self.rows.k.n_rows, self.width)
        return v

    def store(self, out: kir.Operand) -> None:
        r = self.rows
        v = self.value(r.k.out_expr[out.name])
        dest = r.buffers[out.buffer]
        shape = (r.k.n_rows, self.width)
        off = offsets(out.index, row=r.row, col=self.col).expand(shape).reshape(-1)
        dest[off] = v.expand(shape).reshape(-1).to(dest.dtype)


def run_reduction(k: kir.ReductionKernel, buffers: dict[str, torch.Tensor],
                  chunk: int = CHUNK) -> None:
    rows = _Rows(k, buffers)
    streamed = k.two_pass
    width = max(1, min(k.n_cols, chunk)) if streamed else max(1, k.n_cols)
    online = rows.online_pair() if streamed else None

    for step in k.steps:
        if not isinstance(step, kir.Reduce) or step.name in rows.done:
            continue
        if online is not None and step is online[0]:
            # one pass for both: m' = max(m, max(chunk)); l' = l e^(m - m') + sum e^(chunk - m')
            m = torch.full((k.n_rows, 1), -float("inf"))
            total = torch.zeros((k.n_rows, 1))
            for span in rows.spans(width):
                x = span.full(online[2])
                m_next = torch.maximum(m, x.amax(dim=1, keepdim=True))
                total = total * torch.exp(m - m_next) + torch.exp(x - m_next).sum(dim=1, keepdim=True)
                m = m_next
            rows.done[online[0].name], rows.done[online[1].name] = m, total
            continue
        acc = None
        for span in rows.spans(width):
            part = ROW_REDUCE[step.kind](span.full(step.expr), dim=1, keepdim=True)
            acc = part if acc is None else MERGE[step.kind](acc, part)
        rows.done[step.name] = acc

    for out in k.outputs:
        if out.name in k.row_outputs:
            continue
        for span in rows.spans(width):
            span.store(out)

    first = rows.span(0, 1)                # per-row values: any one column will do
    for out in k.outputs:
        if out.name not in k.row_outputs:
            continue
        v = first.value(k.out_expr[out.name])
        dest = buffers[out.buffer]
        if v.numel() == 1:
            v = v.reshape(1, 1).expand(k.n_rows, 1)
        off = offsets(out.index, row=rows.row, col=torch.zeros((1, 1), dtype=torch.int64))
        dest[off.reshape(-1)] = v.reshape(-1).to(dest.dtype)


# --------------------------------------------------------------------------
# extern kernels and whole schedules
# --------------------------------------------------------------------------

def run_extern(k: kir.ExternKernel, buffers: dict[str, torch.Tensor]) -> None:
    ns, op, *rest = k.op.split(".")
    target = getattr(getattr(getattr(torch.ops, ns), op), rest[0] if rest else "default")

    def tensor(a):
        if isinstance(a, kir.View):
            return a.as_torch(buffers[a.buffer])
        if isinstance(a, (list, tuple)):
            return type(a)(tensor(x) for x in a)
        if isinstance(a, dict) and "dtype" in a:
            return kir.torch_dtype(a["dtype"])
        return a

    got = target(*[tensor(a) for a in k.args], **{n: tensor(a) for n, a in k.kwargs.items()})
    for view, t in zip(k.outputs, got if isinstance(got, (list, tuple)) else [got]):
        view.as_torch(buffers[view.buffer]).copy_(t)


def run_kernel(k, buffers: dict[str, torch.Tensor]) -> None:
    if isinstance(k, kir.PointwiseKernel):
        run_pointwise(k, buffers)
    elif isinstance(k, kir.ReductionKernel):
        run_reduction(k, buffers)
    elif isinstance(k, kir.ExternKernel):
        run_extern(k, buffers)
    else:
        raise TypeError(type(k).__name__)


def tensor_table(params) -> dict[str, torch.Tensor]:
    if isinstance(params, torch.nn.Module):
        table = dict(params.named_parameters(remove_duplicate=False))
        table.update(dict(params.named_buffers(remove_duplicate=False)))
        return table
    return dict(params)


def allocate(schedule: kir.Schedule, params, inputs, fill: float | None = None
             ) -> dict[str, torch.Tensor]:
    """One flat CPU tensor per live buffer.  No arena: every buffer gets its own
    storage, so a mistake in a memory plan cannot hide an arithmetic one."""
    params = tensor_table(params)
    live = schedule.live_buffers()

    def flat(t, name):
        dt = kir.torch_dtype(schedule.buffers[name].dtype)
        return t.detach().to("cpu", dt).contiguous().reshape(-1).clone()

    buffers: dict[str, torch.Tensor] = {}
    for name, origin in schedule.params.items():
        if name in live:
            t = params.get(origin, params.get(name))
            if t is None:
                raise KeyError(f"no tensor for parameter {name} ({origin})")
            buffers[name] = flat(t, name)
    for view, t in zip(schedule.inputs, inputs):
        buffers[view.buffer] = flat(t, view.buffer)
    for name in live - set(buffers):
        spec = schedule.buffers[name]
        t = torch.empty(spec.numel, dtype=kir.torch_dtype(spec.dtype))
        if fill is not None:
            t.fill_(fill) if t.is_floating_point() else t.zero_()
        buffers[name] = t
    return buffers


def run_schedule(schedule: kir.Schedule, params, inputs, buffers=None, only=None):
    """Run the kernels in order on the CPU; returns ``(outputs, buffers)``."""
    if buffers is None:
        buffers = allocate(schedule, params, inputs)
    for k in schedule.kernels:
        if only is None or k.name in only:
            run_kernel(k, buffers)
    outs = [v.as_torch(buffers[v.buffer]) for v in schedule.outputs]
    return (outs[0] if len(outs) == 1 else tuple(outs)), buffers
