"""Scalar expressions -> CUDA C++, with the reference backend's typing rules.

The torch reference backend evaluates a kernel body with torch tensor ops
(``mlc/codegen/torch_backend.py:65-83``): fp16/bf16 loads are widened to fp32
(``:59-62``), a Python-number constant becomes a *0-dim* tensor (``:71-74``), a
bool constant becomes a full-size bool tensor, and every ``Call`` then follows
torch's type promotion -- where a 0-dim operand only matters if it is of a
higher *category* than the dimensioned ones.  Generated code has to land on the
same dtype at every node or a mid-body ``Cast`` (the GELU result rounded to
fp16 before a residual add, ``mlc/ir/ops.py:313-335``) rounds in the wrong
place.  Rather than restating the promotion lattice, result types are obtained
by applying the torch operator to one-element exemplars at emit time.

A value of IR dtype float16/bfloat16 lives in a ``float`` register holding an
exactly representable narrow value; every operation producing one rounds
explicitly.  This reproduces torch's "compute in fp32, round once" for narrow
float arithmetic on both CPU and CUDA.
"""

from __future__ import annotations

import functools
import math
from dataclasses import dataclass

import torch

from .. import kir
from ..kir import Call, Cast, Const, Expr, Load, Ref

#: storage type in global memory
STORAGE_T = {
    "float32": "float", "float64": "double", "float16": "__half", "bfloat16": "__nv_bfloat16",
    "int64": "i64", "int32": "int", "int16": "short", "int8": "signed char",
    "uint8": "unsigned char", "bool": "bool",
}
#: register type a value of this IR dtype is held in
REG_T = dict(STORAGE_T, float16="float", bfloat16="float")

_TORCH_FN = {
    "neg": lambda a: -a, "abs": torch.abs, "reciprocal": torch.reciprocal, "exp": torch.exp,
    "log": torch.log, "sqrt": torch.sqrt, "rsqrt": torch.rsqrt, "sin": torch.sin,
    "cos": torch.cos, "tanh": torch.tanh, "erf": torch.erf, "sigmoid": torch.sigmoid,
    "floor": torch.floor, "logical_not": torch.logical_not, "add": torch.add,
    "sub": torch.sub, "mul": torch.mul, "div": torch.div, "pow": torch.pow,
    "maximum": torch.maximum, "minimum": torch.minimum, "gt": torch.gt, "lt": torch.lt,
    "ge": torch.ge, "le": torch.le, "eq": torch.eq, "ne": torch.ne,
    "logical_and": torch.logical_and, "logical_or": torch.logical_or, "where": torch.where,
}

_COMPARE = {"gt": ">", "lt": "<", "ge": ">=", "le": "<=", "eq": "==", "ne": "!="}
_FAST_UNARY = {"exp": "mlcb_exp_fast", "log": "mlcb_log_fast", "tanh": "mlcb_tanh_fast",
               "erf": "mlcb_erf_fast", "sigmoid": "mlcb_sigmoid_fast", "rsqrt": "rsqrtf"}
_FLOAT_UNARY = {"exp": "exp", "log": "log", "sqrt": "sqrt", "sin": "sin", "cos": "cos",
                "tanh": "tanh", "erf": "erf"}


#: When set, float32 transcendentals and divisions use the SFU-based forms
#: (``ex2/rcp.approx.ftz`` and the closed forms in the device header), whose
#: error (~1e-6 relative, ~2e-7 absolute for erf/tanh) is four orders below the
#: half-precision rounding of the value that is finally stored.  The emitters
#: switch it on only for kernels all of whose outputs are fp16/bf16; kernels
#: with an fp32/fp64 output keep IEEE division and the full-precision libm.
_FAST = False


class math_mode:
    """``with math_mode(fast): ...`` around the rendering of one kernel."""

    def __init__(self, fast: bool):
        self.fast = bool(fast)

    def __enter__(self):
        global _FAST
        self.prev, _FAST = _FAST, self.fast
        return self

    def __exit__(self, *exc):
        global _FAST
        _FAST = self.prev


def wants_fast_math(k, cfg) -> bool:
    outs = list(k.outputs)
    return (bool(getattr(cfg, "narrow_fast_math", True)) and bool(outs)
            and all(a.dtype in kir.NARROW_FLOATS for a in outs))


@dataclass(frozen=True)
class Val:
    """A rendered value: C++ text, IR dtype, and whether torch would see it as a
    dimensioned tensor (True) or a 0-dim one (False)."""

    code: str
    dtype: str
    dim: bool = True
    #: varies along the column axis of a reduction kernel (unused by pointwise)
    varies: bool = False
    #: ``(fp32 code, narrow dtype)`` when ``code`` is that fp32 expression rounded
    #: to fp16/bf16 (possibly widened again): a store to the same narrow dtype
    #: can take the unrounded expression, because storing rounds identically
    unrounded: tuple[str, str] | None = None


def is_float(dt: str) -> bool:
    return dt in kir.FLOAT_DTYPES


def _exemplar(dtype: str, dim: bool) -> torch.Tensor:
    # ones, not zeros: reciprocal/log/div of zero would warn or trap in debug builds
    return torch.ones((1,) if dim else (), dtype=kir.torch_dtype(dtype))


@functools.lru_cache(maxsize=None)
def result_type(fn: str, sig: tuple[tuple[str, bool], ...]) -> tuple[str, bool]:
    """(dtype, dim) torch gives ``fn`` applied to operands of these types."""
    args = [_exemplar(dt, dim) for dt, dim in sig]
    out = _TORCH_FN[fn](*args)
    return kir.dtype_name(out.dtype), out.dim() > 0


@functools.lru_cache(maxsize=None)
def common_type(sig: tuple[tuple[str, bool], ...]) -> str:
    """The dtype torch's TensorIterator converts these operands to before it
    computes (``torch.result_type`` generalised to n operands)."""
    ts = [_exemplar(dt, dim) for dt, dim in sig]
    r = ts[0]
    for t in ts[1:]:
        dt = torch.result_type(r, t)
        r = torch.ones((1,) if (r.dim() or t.dim()) else (), dtype=dt)
    return kir.dtype_name(r.dtype)


@functools.lru_cache(maxsize=None)
def reduce_type(kind: str, dtype: str) -> str:
    fn = {"sum": torch.sum, "prod": torch.prod, "max": torch.amax, "min": torch.amin}[kind]
    return kir.dtype_name(fn(torch.ones((1, 1), dtype=kir.torch_dtype(dtype)),
                             dim=1, keepdim=True).dtype)


# --------------------------------------------------------------------------
# literals
# --------------------------------------------------------------------------

def float_literal(v: float, dtype: str) -> str:
    """A C++ literal holding ``v`` after rounding to ``dtype`` (exact: hex float)."""
    t = torch.tensor(v, dtype=torch.float64).to(kir.torch_dtype(dtype))
    if dtype == "float64":
        x = float(t)
        if x != x:
            return "MLCB_NAN_D"
        if math.isinf(x):
            return "MLCB_INF_D" if x > 0 else "MLCB_NINF_D"
        return f"({x.hex()})"
    x = float(t.to(torch.float32))
    if x != x:
        return "MLCB_NAN_F"
    if math.isinf(x):
        return "MLCB_INF_F" if x > 0 else "MLCB_NINF_F"
    return f"({x.hex()}f)"


def int_literal(v: int, dtype: str) -> str:
    if dtype == "int64":
        if v == -(1 << 63):
            return "((i64)(-9223372036854775807LL - 1))"
        return f"((i64){v}LL)"
    if dtype == "bool":
        return "true" if v else "false"
    return f"(({REG_T[dtype]}){v})"


def const_val(c: Const) -> Val:
    v = c.value
    if isinstance(v, bool):
        # the reference materialises bool constants as full bool tensors
        return Val("true" if v else "false", "bool", True)
    if isinstance(v, int):
        dt = c.dtype or "int64"
        if is_float(dt):
            return Val(float_literal(float(v), dt), dt, False)
        return Val(int_literal(v, dt), dt, False)
    if isinstance(v, float):
        dt = c.dtype or "float32"
        if not is_float(dt):
            if dt == "bool":
                return Val("true" if v != 0 else "false", "bool", False)
            return Val(int_literal(int(v), dt), dt, False)
        return Val(float_literal(v, dt), dt, False)
    raise TypeError(f"cannot emit constant {v!r}")


# --------------------------------------------------------------------------
# conversions
# --------------------------------------------------------------------------

def convert(code: str, src: str, dst: str) -> str:
    """C++ for ``tensor.to(dst)`` of a register value of IR dtype ``src``."""
    if src == dst:
        return code
    if dst == "bool":
        return f"({code} != 0)"
    if is_float(dst):
        if dst == "float64":
            return f"((double){code})"
        wide = code if REG_T[src] == "float" else f"((float){code})"
        if dst == "float32":
            return wide
        # narrow target: a narrower-or-equal source of the *same* format is exact,
        # anything else rounds to nearest even
        return f"mlcb_rn_{'f16' if dst == 'float16' else 'bf16'}({wide})"
    # integer target: C++ truncation is what torch does for in-range values
    return f"(({REG_T[dst]}){code})"


def _opmath(dt: str) -> str:
    return "double" if dt == "float64" else "float"


def _round_to(code: str, dt: str) -> str:
    if dt == "float16":
        return f"mlcb_rn_f16({code})"
    if dt == "bfloat16":
        return f"mlcb_rn_bf16({code})"
    return code


def _fname(base: str, dt: str) -> str:
    return base if dt == "float64" else base + "f"


def render_call(fn: str, args: list[Val]) -> Val:
    if fn not in kir.FUNCTIONS:
        raise KeyError(f"no CUDA form for scalar function {fn!r}")
    if len(args) != kir.FUNCTIONS[fn]:
        raise ValueError(f"{fn} takes {kir.FUNCTIONS[fn]} args, got {len(args)}")
    sig = tuple((a.dtype, a.dim) for a in args)
    rdt, rdim = result_type(fn, sig)
    varies = any(a.varies for a in args)

    def out(code: str) -> Val:
        return Val(code, rdt, rdim, varies)

    if fn in _COMPARE:
        ct = common_type(sig)
        a, b = (convert(x.code, x.dtype, ct) for x in args)
        return out(f"({a} {_COMPARE[fn]} {b})")
    if fn == "logical_not":
        return out(f"({args[0].code} == 0)")
    if fn in ("logical_and", "logical_or"):
        a, b = (convert(x.code, x.dtype, "bool") for x in args)
        return out(f"({a} {'&&' if fn == 'logical_and' else '||'} {b})")
    if fn == "where":
        ct = common_type(sig[1:])
        c = convert(args[0].code, args[0].dtype, "bool")
        a, b = (convert(x.code, x.dtype, ct) for x in args[1:])
        return out(f"({c} ? {a} : {b})")

    # arithmetic: operands go to the common dtype, math runs in its opmath type,
    # the result is rounded to the result dtype
    if is_float(rdt):
        ct = rdt
        xs = [convert(x.code, x.dtype, ct) for x in args]
        m = _opmath(ct)
        fast = _FAST and m == "float"
        if fast and fn in _FAST_UNARY:
            code = f"{_FAST_UNARY[fn]}({xs[0]})"
        elif fast and fn == "div":
            if args[0].varies and not args[1].varies:
                # divisor is a row statistic: one reciprocal per row, hoisted by the
                # compiler out of the unrolled element loop
                code = f"({xs[0]} * mlcb_rcp({xs[1]}))"
            else:
                code = f"mlcb_div_fast({xs[0]}, {xs[1]})"
        elif fast and fn == "reciprocal":
            code = f"mlcb_rcp_fast({xs[0]})"
        elif fn in _FLOAT_UNARY:
            code = f"{_fname(_FLOAT_UNARY[fn], ct)}({xs[0]})"
        elif fn == "neg":
            code = f"(-{xs[0]})"
        elif fn == "abs":
            code = f"{_fname('fabs', ct)}({xs[0]})"
        elif fn == "floor":
            code = f"{_fname('floor', ct)}({xs[0]})"
        elif fn == "reciprocal":
            code = f"(({m})1 / {xs[0]})"
        elif fn == "rsqrt":
            code = f"mlcb_rsqrt({xs[0]})"
        elif fn == "sigmoid":
            code = f"mlcb_sigmoid({xs[0]})"
        elif fn in ("add", "sub", "mul", "div"):
            op = {"add": "+", "sub": "-", "mul": "*", "div": "/"}[fn]
            code = f"({xs[0]} {op} {xs[1]})"
        elif fn == "pow":
            code = f"{_fname('pow', ct)}({xs[0]}, {xs[1]})"
        elif fn == "maximum":
            code = f"mlcb_max<{m}>({xs[0]}, {xs[1]})"
        elif fn == "minimum":
            code = f"mlcb_min<{m}>({xs[0]}, {xs[1]})"
        else:  # pragma: no cover - table and branches are kept in step
            raise KeyError(fn)
        return out(_round_to(code, rdt))

    if rdt == "bool":
        xs = [convert(x.code, x.dtype, "bool") for x in args]
        if fn in ("add", "maximum"):
            return out(f"({xs[0]} || {xs[1]})")
        if fn in ("mul", "minimum"):
            return out(f"({xs[0]} && {xs[1]})")
        if fn in ("abs", "floor"):
            return out(xs[0])
        raise TypeError(f"{fn} is not defined on bool operands")

    # integer result
    xs = [convert(x.code, x.dtype, rdt) for x in args]
    t = REG_T[rdt]
    if fn == "neg":
        code = f"(({t})(-{xs[0]}))"
    elif fn == "abs":
        code = f"mlcb_iabs<{t}>({xs[0]})"
    elif fn == "floor":
        code = xs[0]
    elif fn in ("add", "sub", "mul"):
        op = {"add": "+", "sub": "-", "mul": "*"}[fn]
        code = f"(({t})({xs[0]} {op} {xs[1]}))"
    elif fn == "pow":
        code = f"(({t})mlcb_ipow((i64){xs[0]}, (i64){xs[1]}))"
    elif fn == "maximum":
        code = f"mlcb_max<{t}>({xs[0]}, {xs[1]})"
    elif fn == "minimum":
        code = f"mlcb_min<{t}>({xs[0]}, {xs[1]})"
    else:
        raise TypeError(f"{fn} has no integer form")
    return out(code)


def render(e: Expr, loads: list[Val], refs: dict[str, Val]) -> Val:
    """Render ``e`` given rendered operands (``loads[slot]``) and bound temps."""
    if isinstance(e, Load):
        return loads[e.slot]
    if isinstance(e, Ref):
        return refs[e.name]
    if isinstance(e, Const):
        return const_val(e)
    if isinstance(e, Cast):
        x = render(e.x, loads, refs)
        unrounded = None
        if e.dtype in kir.NARROW_FLOATS and x.dtype == "float32":
            unrounded = (x.code, e.dtype)
        elif e.dtype == "float32" and x.dtype in kir.NARROW_FLOATS:
            unrounded = x.unrounded            # exact widening of a rounded value
        elif e.dtype == x.dtype:
            unrounded = x.unrounded
        return Val(convert(x.code, x.dtype, e.dtype), e.dtype, x.dim, x.varies, unrounded)
    if isinstance(e, Call):
        if e.fn == "div" and isinstance(e.args[1], Const) and _is_pow2(e.args[1].value):
            # x / 2^k == x * 2^-k in IEEE arithmetic, and a multiply is one
            # instruction where a correctly rounded divide is about ten
            c = e.args[1]
            recip = Const(1.0 / float(c.value), c.dtype if c.dtype in kir.FLOAT_DTYPES else None)
            num = render(e.args[0], loads, refs)
            if is_float(num.dtype):
                return render_call("mul", [num, const_val(recip)])
        return render_call(e.fn, [render(a, loads, refs) for a in e.args])
    raise TypeError(f"cannot emit {type(e).__name__}")


def _is_pow2(v) -> bool:
    if isinstance(v, bool) or not isinstance(v, (int, float)):
        return False
    f = float(v)
    if f == 0.0 or f != f or math.isinf(f):
        return False
    m, _ = math.frexp(abs(f))
    return m == 0.5 and 2.0 ** -100 < abs(f) < 2.0 ** 100


def promoted_load_dtype(dtype: str) -> str:
    """fp16/bf16 operands are computed on as fp32 (``torch_backend.py:53-62``)."""
    return "float32" if dtype in kir.NARROW_FLOATS else dtype


def store_only_casts(binds, out_expr: dict, outputs) -> set[str]:
    """Names of ``t = Cast(y, narrow)`` temps whose only readers are stores to
    buffers of that same narrow dtype.  The store converts fp32 -> fp16/bf16 with
    the same round-to-nearest-even, so rounding in the body as well would only
    repeat it; such a temp is carried in fp32 and rounded once, at the store."""
    uses: dict[str, int] = {}
    for _, e in binds:
        for sub in kir.walk(e):
            if isinstance(sub, Ref):
                uses[sub.name] = uses.get(sub.name, 0) + 1
    out_dtype = {a.name: a.dtype for a in outputs}
    store_uses: dict[str, list[str]] = {}
    for oname, e in out_expr.items():
        if isinstance(e, Ref):
            store_uses.setdefault(e.name, []).append(out_dtype.get(oname))
        else:
            for sub in kir.walk(e):
                if isinstance(sub, Ref):
                    uses[sub.name] = uses.get(sub.name, 0) + 1
    found = set()
    for name, e in binds:
        if (isinstance(e, Cast) and e.dtype in kir.NARROW_FLOATS and uses.get(name, 0) == 0
                and store_uses.get(name) and all(d == e.dtype for d in store_uses[name])):
            found.add(name)
    return found


def render_bind(name: str, e: Expr, loads, refs, elide: set[str]) -> Val:
    """Render one temp; a store-only narrowing cast of an fp32 value is carried
    unrounded (see :func:`store_only_casts`)."""
    if name in elide and isinstance(e, Cast):
        x = render(e.x, loads, refs)
        if x.dtype == "float32":
            return Val(x.code, e.dtype, x.dim, x.varies)
    return render(e, loads, refs)
