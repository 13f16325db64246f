"""Kernel IR: the input language of the CUDA backend.

This is a self-contained mirror of the data the reference hands its code
generator (reference: ``mlc/kernels.py:23-232`` for the kernel records,
``mlc/codegen/index.py:36-115`` for index maps, ``mlc/ir/scalar.py:30-75`` for
scalar expressions, ``mlc/ir/types.py:38-263`` for layouts and buffers, and
``mlc/passes/memory_planning.py:55-72`` for the arena plan).  The backend never
sees a graph, a fusion group or a torch.export program: only this.

Two ways in:

* :func:`from_reference` converts a live reference ``Schedule`` by attribute
  access alone (nothing from the reference is imported here), which is what the
  drop-in runtime adapter uses;
* :func:`load` / :func:`loads` read the JSON form written by :func:`dump`, which
  is how schedules travel to machines that do not have the reference frontend.

Offsets follow the reference's rule (``mlc/codegen/index.py:54-65``)::

    offset = base + sum over axes, sum over terms of
             ((var // out_stride) % size) * in_stride
"""

from __future__ import annotations

import gzip
import json
import math
from dataclasses import dataclass, field
from typing import Any, Iterator, Sequence

# --------------------------------------------------------------------------
# dtypes are carried as short strings so the IR does not need torch to exist
# --------------------------------------------------------------------------

ITEMSIZE = {
    "float32": 4, "float64": 8, "float16": 2, "bfloat16": 2,
    "int64": 8, "int32": 4, "int16": 2, "int8": 1, "uint8": 1, "bool": 1,
}
FLOAT_DTYPES = ("float16", "bfloat16", "float32", "float64")
NARROW_FLOATS = ("float16", "bfloat16")


def dtype_name(dt) -> str | None:
    """Normalise a torch dtype, a numpy-ish name or ``None`` to a short string."""
    if dt is None:
        return None
    s = str(dt)
    s = s.replace("torch.", "")
    if s == "half":
        s = "float16"
    if s not in ITEMSIZE:
        raise KeyError(f"dtype {dt!r} has no kernel form")
    return s


def torch_dtype(name: str):
    import torch

    return getattr(torch, name)


# --------------------------------------------------------------------------
# scalar expressions
# --------------------------------------------------------------------------

class Expr:
    __slots__ = ()


@dataclass(frozen=True)
class Load(Expr):
    slot: int


@dataclass(frozen=True)
class Ref(Expr):
    name: str


@dataclass(frozen=True)
class Const(Expr):
    value: Any
    dtype: str | None = None


@dataclass(frozen=True)
class Call(Expr):
    fn: str
    args: tuple[Expr, ...]


@dataclass(frozen=True)
class Cast(Expr):
    x: Expr
    dtype: str


#: name -> arity; the same thirty functions as ``mlc/ir/scalar.py:94-128``
FUNCTIONS: dict[str, int] = {
    "neg": 1, "abs": 1, "reciprocal": 1, "exp": 1, "log": 1, "sqrt": 1, "rsqrt": 1,
    "sin": 1, "cos": 1, "tanh": 1, "erf": 1, "sigmoid": 1, "floor": 1, "logical_not": 1,
    "add": 2, "sub": 2, "mul": 2, "div": 2, "pow": 2, "maximum": 2, "minimum": 2,
    "gt": 2, "lt": 2, "ge": 2, "le": 2, "eq": 2, "ne": 2,
    "logical_and": 2, "logical_or": 2,
    "where": 3,
}


def walk(e: Expr) -> Iterator[Expr]:
    """Every subexpression, children first."""
    if isinstance(e, Call):
        for a in e.args:
            yield from walk(a)
    elif isinstance(e, Cast):
        yield from walk(e.x)
    yield e


def expr_loads(e: Expr) -> set[int]:
    return {s.slot for s in walk(e) if isinstance(s, Load)}


def expr_refs(e: Expr) -> set[str]:
    return {s.name for s in walk(e) if isinstance(s, Ref)}


# --------------------------------------------------------------------------
# index maps
# --------------------------------------------------------------------------

@dataclass(frozen=True)
class Axis:
    """Contribution of one iteration variable (``idx``, ``row`` or ``col``)."""

    var: str
    numel: int
    #: (size, out_stride, in_stride), outermost first
    terms: tuple[tuple[int, int, int], ...] = ()

    @property
    def is_constant(self) -> bool:
        return not self.terms

    def offset_of(self, v: int) -> int:
        return sum(((v // o) % n) * i for n, o, i in self.terms)

    def max_offset(self) -> int:
        return sum((n - 1) * i for n, _, i in self.terms if i > 0)

    def min_offset(self) -> int:
        return sum((n - 1) * i for n, _, i in self.terms if i < 0)


@dataclass(frozen=True)
class IndexMap:
    axes: tuple[Axis, ...]
    base: int = 0

    def axis(self, var: str) -> Axis | None:
        for a in self.axes:
            if a.var == var:
                return a
        return None

    def varies_along(self, var: str) -> bool:
        a = self.axis(var)
        return a is not None and not a.is_constant

    def offset(self, **vars: int) -> int:
        return self.base + sum(a.offset_of(vars[a.var]) for a in self.axes)

    def bounds(self) -> tuple[int, int]:
        """Smallest and largest element offset the map can produce."""
        lo = self.base + sum(a.min_offset() for a in self.axes)
        hi = self.base + sum(a.max_offset() for a in self.axes)
        return lo, hi

    def distinct_elements(self) -> int:
        """Upper bound on distinct elements addressed (exact for injective maps)."""
        n = 1
        for a in self.axes:
            for size, _, _ in a.terms:
                n *= size
        return n


# --------------------------------------------------------------------------
# storage
# --------------------------------------------------------------------------

@dataclass
class BufferSpec:
    name: str
    shape: tuple[int, ...]
    dtype: str
    kind: str = "intermediate"  # input | param | intermediate | output | constant

    @property
    def numel(self) -> int:
        return math.prod(self.shape) if self.shape else 1

    @property
    def itemsize(self) -> int:
        return ITEMSIZE[self.dtype]

    @property
    def nbytes(self) -> int:
        return self.numel * self.itemsize

    @property
    def plannable(self) -> bool:
        return self.kind == "intermediate"


@dataclass(frozen=True)
class View:
    """A named strided window onto a buffer (the reference's Value + Layout)."""

    name: str
    buffer: str
    shape: tuple[int, ...]
    strides: tuple[int, ...]
    offset: int = 0

    @property
    def numel(self) -> int:
        return math.prod(self.shape) if self.shape else 1

    def as_torch(self, storage):
        """Same contract as ``Layout.as_torch`` (``mlc/ir/types.py:170-181``):
        the flat tensor's own storage offset is added, because arena slices are
        not at offset zero of their storage."""
        return storage.as_strided(self.shape, self.strides,
                                  self.offset + storage.storage_offset())


@dataclass
class Operand:
    """One tensor operand of a generated kernel and the map it is read by."""

    name: str
    buffer: str
    dtype: str
    index: IndexMap
    #: row gather (reduction inputs only; the reference has no such operand, its
    #: embeddings are separate library calls): ``(slot, rows)`` means the ``row``
    #: variable of ``index`` is not the kernel's row but the integer that input
    #: ``slot`` -- an operand indexed by row alone -- holds for this row, clamped
    #: to ``[0, rows)``; ``index``'s row axis then spans the table's ``rows``
    via: tuple[int, int] | None = None


# --------------------------------------------------------------------------
# kernels
# --------------------------------------------------------------------------

@dataclass
class PointwiseKernel:
    name: str
    space: tuple[int, ...]
    inputs: list[Operand]
    outputs: list[Operand]
    body: list[tuple[str, Expr]]
    out_expr: dict[str, Expr]
    ops: list[str] = field(default_factory=list)

    @property
    def numel(self) -> int:
        return math.prod(self.space) if self.space else 1

    def reads(self) -> list[str]:
        return [a.buffer for a in self.inputs]

    def writes(self) -> list[str]:
        return [a.buffer for a in self.outputs]

    def summary(self) -> str:
        return (f"{self.name}: pointwise{list(self.space)} {len(self.inputs)}in "
                f"{len(self.outputs)}out [{', '.join(self.ops)}]")


@dataclass
class Bind:
    name: str
    expr: Expr


@dataclass
class Reduce:
    name: str
    kind: str  # sum | max | min | prod
    expr: Expr


@dataclass
class ReductionKernel:
    name: str
    row_space: tuple[int, ...]
    reduce_space: tuple[int, ...]
    inputs: list[Operand]
    outputs: list[Operand]
    steps: list  # Bind | Reduce, ordered
    out_expr: dict[str, Expr]
    row_outputs: set[str] = field(default_factory=set)
    two_pass: bool = False
    ops: list[str] = field(default_factory=list)

    @property
    def n_rows(self) -> int:
        return math.prod(self.row_space) if self.row_space else 1

    @property
    def n_cols(self) -> int:
        return math.prod(self.reduce_space) if self.reduce_space else 1

    @property
    def reduces(self) -> list[Reduce]:
        return [s for s in self.steps if isinstance(s, Reduce)]

    def reads(self) -> list[str]:
        return [a.buffer for a in self.inputs]

    def writes(self) -> list[str]:
        return [a.buffer for a in self.outputs]

    def summary(self) -> str:
        kinds = "+".join(r.kind for r in self.reduces) or "none"
        mode = "streamed" if self.two_pass else "persistent"
        return (f"{self.name}: reduction {self.n_rows}x{self.n_cols} {kinds} ({mode}) "
                f"{len(self.inputs)}in {len(self.outputs)}out [{', '.join(self.ops)}]")


@dataclass
class ExternKernel:
    """An operator dispatched to ATen (matmuls land on cuBLAS), kept exactly as
    the reference dispatches it (``mlc/runtime/executor.py:369-402``)."""

    name: str
    op: str  # e.g. "aten.mm.default"
    args: list  # View | scalar | list of those
    kwargs: dict
    outputs: list[View]

    def _views(self) -> Iterator[View]:
        def go(a):
            if isinstance(a, View):
                yield a
            elif isinstance(a, (list, tuple)):
                for x in a:
                    yield from go(x)
        for a in self.args:
            yield from go(a)
        for a in self.kwargs.values():
            yield from go(a)

    def reads(self) -> list[str]:
        seen: list[str] = []
        for v in self._views():
            if v.buffer not in seen:
                seen.append(v.buffer)
        return seen

    def writes(self) -> list[str]:
        return [o.buffer for o in self.outputs]

    def summary(self) -> str:
        def show(v: View) -> str:
            dense, run = [], 1
            for n in reversed(v.shape):
                dense.append(run)
                run *= n
            text = str(list(v.shape))
            if tuple(reversed(dense)) != tuple(v.strides) or v.offset:
                # a strided window: say where it looks
                text += "@" + str(tuple(v.strides)) + (f"+{v.offset}" if v.offset else "")
            return text
        shapes = "x".join(show(v) for v in self._views())
        outs = [o for o in self.outputs if show(o) != str(list(o.shape))]
        tail = " -> " + ", ".join(show(o) for o in outs) if outs else ""
        return f"{self.name}: extern {self.op} {shapes}{tail}"


Kernel = PointwiseKernel | ReductionKernel | ExternKernel


@dataclass
class ArenaPlan:
    mode: str = "arena"  # arena | eager
    arena_bytes: int = 0
    offsets: dict[str, int] = field(default_factory=dict)
    peak_bytes: int = 0
    total_bytes: int = 0
    #: eager mode only: kernel index -> buffers to allocate before / free after
    alloc_at: dict[int, list[str]] = field(default_factory=dict)
    free_at: dict[int, list[str]] = field(default_factory=dict)

    def summary(self) -> str:
        if self.mode != "arena":
            return (f"memory: unplanned, peak {self.peak_bytes / 1024:.1f} KiB "
                    f"of {self.total_bytes / 1024:.1f} KiB total")
        eff = self.arena_bytes / self.peak_bytes if self.peak_bytes else 1.0
        return (f"memory: arena {self.arena_bytes / 1024:.1f} KiB, lower bound "
                f"{self.peak_bytes / 1024:.1f} KiB ({eff:.2f}x), unplanned would be "
                f"{self.total_bytes / 1024:.1f} KiB")


@dataclass
class Schedule:
    """Kernels in execution order plus everything the executor needs to bind
    them: buffers, graph boundary views, parameter origins and the arena plan."""

    name: str
    kernels: list = field(default_factory=list)
    buffers: dict[str, BufferSpec] = field(default_factory=dict)
    inputs: list[View] = field(default_factory=list)
    outputs: list[View] = field(default_factory=list)
    #: param buffer name -> state-dict key it came from
    params: dict[str, str] = field(default_factory=dict)
    plan: ArenaPlan = field(default_factory=ArenaPlan)
    meta: dict = field(default_factory=dict)

    @property
    def arena_bytes(self) -> int:
        return self.plan.arena_bytes

    def __iter__(self):
        return iter(self.kernels)

    def __len__(self) -> int:
        return len(self.kernels)

    def counts(self) -> dict[str, int]:
        out: dict[str, int] = {}
        for k in self.kernels:
            key = type(k).__name__.replace("Kernel", "").lower()
            out[key] = out.get(key, 0) + 1
        return out

    def kernel(self, name: str):
        for k in self.kernels:
            if k.name == name:
                return k
        raise KeyError(name)

    def generated(self) -> list:
        return [k for k in self.kernels if not isinstance(k, ExternKernel)]

    def live_buffers(self) -> set[str]:
        """Buffers some kernel touches plus the graph boundary
        (``mlc/runtime/executor.py:87-94``)."""
        live = {v.buffer for v in self.inputs} | {v.buffer for v in self.outputs}
        for k in self.kernels:
            live |= set(k.reads()) | set(k.writes())
        return live

    def format(self) -> str:
        lines = [f"schedule({len(self.kernels)} kernels, {self.counts()})"]
        lines += ["  " + k.summary() for k in self.kernels]
        lines.append("  " + self.plan.summary())
        return "\n".join(lines)


# --------------------------------------------------------------------------
# conversion from live reference objects (duck typed, no reference import)
# --------------------------------------------------------------------------

def _conv_expr(e) -> Expr:
    t = type(e).__name__
    if t == "Load":
        return Load(int(e.slot))
    if t == "Ref":
        return Ref(str(e.name))
    if t == "Const":
        return Const(e.value, dtype_name(e.dtype))
    if t == "Call":
        if e.fn not in FUNCTIONS:
            raise KeyError(f"no CUDA form for scalar function {e.fn!r}")
        return Call(e.fn, tuple(_conv_expr(a) for a in e.args))
    if t == "Cast":
        return Cast(_conv_expr(e.x), dtype_name(e.dtype))
    raise TypeError(f"cannot convert {t} to a kernel expression")


def _conv_index(m) -> IndexMap:
    return IndexMap(tuple(Axis(a.var, int(a.numel),
                               tuple((int(n), int(o), int(i)) for n, o, i in a.terms))
                          for a in m.axes), int(m.base))


def _conv_operand(a) -> Operand:
    return Operand(a.value.name, a.value.buffer.name, dtype_name(a.value.dtype),
                   _conv_index(a.index))


def _conv_view(v) -> View:
    lay = v.layout
    return View(v.name, v.buffer.name, tuple(lay.shape), tuple(lay.strides), int(lay.offset))


def _conv_arg(a):
    if hasattr(a, "buffer") and hasattr(a, "layout"):
        return _conv_view(a)
    if isinstance(a, (list, tuple)):
        return [_conv_arg(x) for x in a]
    if a is None or isinstance(a, (bool, int, float, str)):
        return a
    name = dtype_name(a) if str(a).startswith("torch.") and str(a)[6:] in ITEMSIZE else None
    if name is not None:
        return {"dtype": name}
    raise TypeError(f"extern argument {a!r} has no serialisable form")


def _op_names(nodes) -> list[str]:
    out = []
    for n in nodes or ():
        parts = n.op.split(".")
        out.append(parts[-2] if len(parts) >= 2 else n.op)
    return out


def from_reference(schedule) -> Schedule:
    """Convert a reference ``Schedule`` (``mlc/kernels.py:200-232``) and the graph
    it hangs off into this IR."""
    graph = schedule.graph
    out = Schedule(name=getattr(graph, "name", "graph"))
    for b in graph.buffers():
        out.buffers[b.name] = BufferSpec(b.name, tuple(b.shape), dtype_name(b.dtype), b.kind)
    out.inputs = [_conv_view(v) for v in graph.inputs]
    out.outputs = [_conv_view(v) for v in graph.outputs]
    for v in graph.params:
        out.params[v.buffer.name] = graph.param_origin.get(v.name, v.name)

    for k in schedule.kernels:
        t = type(k).__name__
        if t == "PointwiseKernel":
            out.kernels.append(PointwiseKernel(
                k.name, tuple(int(d) for d in k.space),
                [_conv_operand(a) for a in k.inputs], [_conv_operand(a) for a in k.outputs],
                [(nm, _conv_expr(e)) for nm, e in k.body],
                {nm: _conv_expr(e) for nm, e in k.out_expr.items()},
                _op_names(k.nodes)))
        elif t == "ReductionKernel":
            steps = []
            for s in k.steps:
                if type(s).__name__ == "Reduce":
                    steps.append(Reduce(s.name, s.kind, _conv_expr(s.expr)))
                else:
                    steps.append(Bind(s.name, _conv_expr(s.expr)))
            out.kernels.append(ReductionKernel(
                k.name, tuple(int(d) for d in k.row_space),
                tuple(int(d) for d in k.reduce_space),
                [_conv_operand(a) for a in k.inputs], [_conv_operand(a) for a in k.outputs],
                steps, {nm: _conv_expr(e) for nm, e in k.out_expr.items()},
                set(k.row_outputs), bool(k.two_pass), _op_names(k.nodes)))
        elif t == "ExternKernel":
            node = k.node
            out.kernels.append(ExternKernel(
                k.name, node.op, [_conv_arg(a) for a in node.args],
                {kk: _conv_arg(v) for kk, v in node.kwargs.items()},
                [_conv_view(o) for o in node.outputs]))
        else:
            raise TypeError(f"no CUDA emitter for {t}")

    p = schedule.plan
    if p is not None:
        out.plan = ArenaPlan(
            mode=p.mode, arena_bytes=int(p.arena_bytes), offsets=dict(p.offsets),
            peak_bytes=int(p.peak_bytes), total_bytes=int(p.total_bytes),
            alloc_at={int(i): [b.name for b in bs] for i, bs in p.alloc_at.items()},
            free_at={int(i): list(ns) for i, ns in p.free_at.items()})
    return out


# --------------------------------------------------------------------------
# JSON form
# --------------------------------------------------------------------------

def _enc_value(v):
    if isinstance(v, float):
        if v != v:
            return {"f": "nan"}
        if v in (math.inf, -math.inf):
            return {"f": "inf" if v > 0 else "-inf"}
        return {"f": repr(v)}
    return v  # bool / int


def _dec_value(v):
    if isinstance(v, dict):
        return float(v["f"])
    return v


def _enc_expr(e: Expr):
    if isinstance(e, Load):
        return ["L", e.slot]
    if isinstance(e, Ref):
        return ["R", e.name]
    if isinstance(e, Const):
        return ["K", _enc_value(e.value), e.dtype]
    if isinstance(e, Call):
        return ["C", e.fn, [_enc_expr(a) for a in e.args]]
    if isinstance(e, Cast):
        return ["T", _enc_expr(e.x), e.dtype]
    raise TypeError(type(e).__name__)


def _dec_expr(j) -> Expr:
    tag = j[0]
    if tag == "L":
        return Load(j[1])
    if tag == "R":
        return Ref(j[1])
    if tag == "K":
        return Const(_dec_value(j[1]), j[2])
    if tag == "C":
        return Call(j[1], tuple(_dec_expr(a) for a in j[2]))
    if tag == "T":
        return Cast(_dec_expr(j[1]), j[2])
    raise ValueError(f"bad expression tag {tag!r}")


def _enc_index(m: IndexMap):
    return {"base": m.base,
            "axes": [[a.var, a.numel, [list(t) for t in a.terms]] for a in m.axes]}


def _dec_index(j) -> IndexMap:
    return IndexMap(tuple(Axis(v, n, tuple(tuple(t) for t in terms))
                          for v, n, terms in j["axes"]), j["base"])


def _enc_operand(a: Operand):
    j = [a.name, a.buffer, a.dtype, _enc_index(a.index)]
    return j + [list(a.via)] if a.via is not None else j


def _dec_operand(j) -> Operand:
    return Operand(j[0], j[1], j[2], _dec_index(j[3]), tuple(j[4]) if len(j) > 4 else None)


def _enc_view(v: View):
    return {"view": [v.name, v.buffer, list(v.shape), list(v.strides), v.offset]}


def _dec_view(j) -> View:
    n, b, shape, strides, off = j["view"]
    return View(n, b, tuple(shape), tuple(strides), off)


def _enc_arg(a):
    if isinstance(a, View):
        return _enc_view(a)
    if isinstance(a, (list, tuple)):
        return [_enc_arg(x) for x in a]
    if isinstance(a, float):
        return _enc_value(a)
    return a


def _dec_arg(j):
    if isinstance(j, dict):
        if "view" in j:
            return _dec_view(j)
        if "f" in j:
            return _dec_value(j)
        return j  # {"dtype": ...}
    if isinstance(j, list):
        return [_dec_arg(x) for x in j]
    return j


def to_json(s: Schedule) -> dict:
    ks = []
    for k in s.kernels:
        if isinstance(k, PointwiseKernel):
            ks.append({"t": "pw", "name": k.name, "space": list(k.space),
                       "in": [_enc_operand(a) for a in k.inputs],
                       "out": [_enc_operand(a) for a in k.outputs],
                       "body": [[n, _enc_expr(e)] for n, e in k.body],
                       "out_expr": {n: _enc_expr(e) for n, e in k.out_expr.items()},
                       "ops": k.ops})
        elif isinstance(k, ReductionKernel):
            ks.append({"t": "red", "name": k.name, "row": list(k.row_space),
                       "col": list(k.reduce_space),
                       "in": [_enc_operand(a) for a in k.inputs],
                       "out": [_enc_operand(a) for a in k.outputs],
                       "steps": [["r" if isinstance(st, Reduce) else "b", st.name,
                                  getattr(st, "kind", None), _enc_expr(st.expr)]
                                 for st in k.steps],
                       "out_expr": {n: _enc_expr(e) for n, e in k.out_expr.items()},
                       "row_out": sorted(k.row_outputs), "two_pass": k.two_pass,
                       "ops": k.ops})
        else:
            ks.append({"t": "ext", "name": k.name, "op": k.op,
                       "args": [_enc_arg(a) for a in k.args],
                       "kwargs": {n: _enc_arg(a) for n, a in k.kwargs.items()},
                       "out": [_enc_view(o) for o in k.outputs]})
    p = s.plan
    return {
        "format": "mlcb-schedule-1", "name": s.name, "meta": s.meta,
        "buffers": [[b.name, list(b.shape), b.dtype, b.kind] for b in s.buffers.values()],
        "inputs": [_enc_view(v) for v in s.inputs],
        "outputs": [_enc_view(v) for v in s.outputs],
        "params": s.params,
        "plan": {"mode": p.mode, "arena_bytes": p.arena_bytes, "offsets": p.offsets,
                 "peak_bytes": p.peak_bytes, "total_bytes": p.total_bytes,
                 "alloc_at": {str(i): v for i, v in p.alloc_at.items()},
                 "free_at": {str(i): v for i, v in p.free_at.items()}},
        "kernels": ks,
    }


def from_json(j: dict) -> Schedule:
    if j.get("format") != "mlcb-schedule-1":
        raise ValueError(f"not a schedule file (format={j.get('format')!r})")
    s = Schedule(name=j["name"], meta=j.get("meta", {}))
    for n, shape, dt, kind in j["buffers"]:
        s.buffers[n] = BufferSpec(n, tuple(shape), dt, kind)
    s.inputs = [_dec_view(v) for v in j["inputs"]]
    s.outputs = [_dec_view(v) for v in j["outputs"]]
    s.params = dict(j["params"])
    p = j["plan"]
    s.plan = ArenaPlan(p["mode"], p["arena_bytes"], dict(p["offsets"]), p["peak_bytes"],
                       p["total_bytes"],
                       {int(i): v for i, v in p.get("alloc_at", {}).items()},
                       {int(i): v for i, v in p.get("free_at", {}).items()})
    for k in j["kernels"]:
        if k["t"] == "pw":
            s.kernels.append(PointwiseKernel(
                k["name"], tuple(k["space"]), [_dec_operand(a) for a in k["in"]],
                [_dec_operand(a) for a in k["out"]],
                [(n, _dec_expr(e)) for n, e in k["body"]],
                {n: _dec_expr(e) for n, e in k["out_expr"].items()}, k.get("ops", [])))
        elif k["t"] == "red":
            steps = [Reduce(n, kind, _dec_expr(e)) if tag == "r" else Bind(n, _dec_expr(e))
                     for tag, n, kind, e in k["steps"]]
            s.kernels.append(ReductionKernel(
                k["name"], tuple(k["row"]), tuple(k["col"]),
                [_dec_operand(a) for a in k["in"]], [_dec_operand(a) for a in k["out"]],
                steps, {n: _dec_expr(e) for n, e in k["out_expr"].items()},
                set(k["row_out"]), k["two_pass"], k.get("ops", [])))
        elif k["t"] == "ext":
            s.kernels.append(ExternKernel(
                k["name"], k["op"], [_dec_arg(a) for a in k["args"]],
                {n: _dec_arg(a) for n, a in k["kwargs"].items()},
                [_dec_view(o) for o in k["out"]]))
        else:
            raise ValueError(f"bad kernel tag {k['t']!r}")
    return s


def dumps(s: Schedule) -> str:
    return json.dumps(to_json(s), separators=(",", ":"))


def loads(text: str) -> Schedule:
    return from_json(json.loads(text))


def dump(s: Schedule, path) -> None:
    data = dumps(s).encode()
    if str(path).endswith(".gz"):
        with gzip.GzipFile(path, "wb", mtime=0) as f:
            f.write(data)
    else:
        with open(path, "wb") as f:
            f.write(data)


def load(path) -> Schedule:
    if str(path).endswith(".gz"):
        with gzip.open(path, "rb") as f:
            return loads(f.read().decode())
    with open(path, "rb") as f:
        return loads(f.read().decode())
