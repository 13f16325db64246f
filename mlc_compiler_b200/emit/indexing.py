"""Index maps -> integer arithmetic, and the proofs that let accesses be packed.

The reference renders ``((var // out_stride) % size) * in_stride`` per term into
Python text (``mlc/codegen/index.py:54-65``) and leaves vectorisation to Triton.
Here the terms themselves are analysed: for a run of W consecutive values of an
iteration variable starting at a multiple of W, an operand is

* ``contig``  -- the run maps to W consecutive, W-aligned elements (one packed
  access of W * itemsize bytes), or
* ``bcast``   -- the run maps to one element (one scalar access, reused), or
* neither     -- W falls back to 1 (a gather).

Every check is a divisibility statement over the (size, out_stride, in_stride)
triples and the base, so it is decided at emit time and the generated code
carries no runtime alignment test.  The same terms give the exact offset range
of a map, which is checked against the buffer size before any code is written
(an out-of-range map is a compile-time error, never a device fault).
"""

from __future__ import annotations

from dataclasses import dataclass

from ..kir import Axis, IndexMap


def pow2_floor(n: int) -> int:
    return 1 << (n.bit_length() - 1) if n > 0 else 1


def pow2_ceil(n: int) -> int:
    return 1 << max(0, (n - 1).bit_length())


def _pow2_divisor(n: int, cap: int) -> int:
    """Largest power of two <= cap dividing n (n == 0 counts as divisible)."""
    w = cap
    while w > 1 and n % w != 0:
        w //= 2
    return w


def render_axis(a: Axis, var: str) -> list[str]:
    parts = []
    for size, ostr, istr in a.terms:
        t = var
        if ostr != 1:
            t = f"({t} / {ostr})"
        if size * ostr != a.numel:
            t = f"({t} % {size})"
        if istr != 1:
            t = f"{t} * {istr}"
        parts.append(t)
    return parts


def render_offset(m: IndexMap, names: dict[str, str], skip: tuple[str, ...] = ()) -> str:
    """C++ for the element offset; ``names`` maps axis variables to C++ names.
    Axes listed in ``skip`` are left out (used to hoist the row part)."""
    parts: list[str] = []
    for a in m.axes:
        if a.var in skip:
            continue
        parts += render_axis(a, names[a.var])
    if m.base and "base" not in skip:
        parts.append(str(m.base))
    return " + ".join(parts) if parts else "0"


@dataclass(frozen=True)
class Access:
    mode: str  # "contig" | "bcast"
    width: int  # run length W (1 = per-element)


def classify(m: IndexMap, var: str, vmax: int, other_ok: bool = True) -> Access:
    """Best packed access for runs along ``var`` of length <= ``vmax``.

    Runs start at multiples of their length.  Terms of *other* axes and the base
    only matter for alignment of a contiguous run.
    """
    ax = m.axis(var)
    terms = ax.terms if ax is not None else ()
    if not terms:
        return Access("bcast", vmax)

    # broadcast along the run: no term changes inside an aligned run of W
    wb = vmax
    for _, ostr, _ in terms:
        wb = min(wb, _pow2_divisor(ostr, vmax))
    # contiguous: innermost term walks unit stride, everything else is W-aligned
    wc = 1
    size, ostr, istr = terms[-1]
    if ostr == 1 and istr == 1:
        wc = _pow2_divisor(size, vmax)
        for _, o, i in terms[:-1]:
            wc = min(wc, _pow2_divisor(o, vmax), _pow2_divisor(i, vmax))
        wc = min(wc, _pow2_divisor(m.base, vmax))
        for a in m.axes:
            if a.var != var:
                for _, _, i in a.terms:
                    wc = min(wc, _pow2_divisor(i, vmax))
    if wc >= wb and wc > 1:
        return Access("contig", wc)
    if wb > 1:
        return Access("bcast", wb)
    return Access("contig", 1)


def check_bounds(m: IndexMap, numel: int, what: str) -> None:
    lo, hi = m.bounds()
    if lo < 0 or hi >= numel:
        raise ValueError(f"{what}: index map addresses [{lo}, {hi}] outside a buffer "
                         f"of {numel} elements")


def needs_64bit(*extents: int) -> bool:
    return any(e >= (1 << 31) - 1 for e in extents)
