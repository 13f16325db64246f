"""Re-expressing strided index spaces after the elements of a buffer have moved.

Several rewrites ask the same question: *the elements of a buffer are going to
live somewhere else -- what do the index maps and views that address it look
like afterwards?*  "Somewhere else" is described by **digits**: the old offset
space is a mixed radix ``old = sum d_k * old_k`` (``0 <= d_k < size_k``), and
digit ``k`` weighs ``new_k`` in the new space.  A permutation of the logical
dimensions of a dense buffer is of that form (``[B, T, F] -> [T, B, F]``), and so
is the correspondence a pure copy kernel establishes between its source and its
destination.

``remap`` pushes one strided index space (a list of ``(size, stride)`` pieces
plus a base) through such a table.  A piece that runs across several digits is
split at the digit boundaries; the caller decides whether splits are acceptable
(index-map terms: yes, each sub-piece becomes a term of its own) or have to fuse
back into one stride (the dimensions of a view handed to a library call).
"""

from __future__ import annotations

from typing import Sequence

from . import kir

Digit = tuple[int, int, int]          # (size, old stride, new stride)


class NoRemap(Exception):
    """The index space does not decompose along the digits."""


def dense_digits(shape: Sequence[int], new_order: Sequence[int]) -> list[Digit]:
    """Digits for a dense row-major buffer of ``shape`` whose dimensions are
    re-ordered to ``new_order`` (a permutation of ``range(len(shape))``, outermost
    first) and stored dense again."""
    old = [1] * len(shape)
    for j in range(len(shape) - 2, -1, -1):
        old[j] = old[j + 1] * shape[j + 1]
    new = [0] * len(shape)
    run = 1
    for j in reversed(list(new_order)):
        new[j] = run
        run *= shape[j]
    return sorted(((shape[j], old[j], new[j]) for j in range(len(shape)) if shape[j] > 1),
                  key=lambda d: d[1])


def _check_digits(digits: Sequence[Digit]) -> None:
    reach = 1
    for size, old, _ in digits:
        if old < reach or size < 1:
            raise NoRemap("digits overlap")
        reach = old * size


def remap(pieces: Sequence[tuple[int, int]], base: int, digits: Sequence[Digit]
          ) -> tuple[list[list[tuple[int, int]]], int]:
    """New strides for ``offset = base + sum c_i * stride_i`` (``0 <= c_i < size_i``).

    Returns, for every piece, its sub-pieces ``(size, new_stride)`` *innermost
    first* (one sub-piece unless the piece crosses a digit boundary), and the new
    base.  Raises ``NoRemap`` when a stride is not aligned to the digit it falls
    in, a piece leaves a digit without filling it, or base plus coordinates can
    carry from one digit into the next."""
    _check_digits(digits)
    load = [0] * len(digits)                      # largest coordinate seen per digit
    rest, new_base = base, 0
    for k in range(len(digits) - 1, -1, -1):
        size, old, new = digits[k]
        q, rest = divmod(rest, old)
        if q >= size:
            raise NoRemap("base outside the digits")
        load[k] += q
        new_base += q * new
    if rest:
        raise NoRemap("base between digits")

    out: list[list[tuple[int, int]]] = []
    for n, s in pieces:
        if n == 1 or s == 0:
            out.append([(n, 0)])
            continue
        if s < 0:
            raise NoRemap("negative stride")
        subs: list[tuple[int, int]] = []
        while n > 1:
            k = next((i for i, (size, old, _) in enumerate(digits)
                      if old <= s < old * size), None)
            if k is None:
                raise NoRemap("stride outside the digits")
            size, old, new = digits[k]
            c, r = divmod(s, old)
            if r or size % c:
                raise NoRemap("stride not aligned to its digit")
            room = size // c
            if n <= room:
                subs.append((n, c * new))
                load[k] += (n - 1) * c
                n = 1
            else:
                if n % room:
                    raise NoRemap("piece leaves a digit without filling it")
                subs.append((room, c * new))
                load[k] += (room - 1) * c
                n //= room
                s = old * size
        out.append(subs)
    for k, (size, _, _) in enumerate(digits):
        if load[k] >= size:
            raise NoRemap("coordinates can carry into the next digit")
    return out, new_base


def remap_index(m: kir.IndexMap, digits: Sequence[Digit]) -> kir.IndexMap:
    """``m`` after the buffer it addresses has moved.  Terms that cross a digit
    boundary become several terms."""
    pieces = [(size, s) for a in m.axes for size, _, s in a.terms]
    subs, base = remap(pieces, m.base, digits)
    it = iter(subs)
    axes = []
    for a in m.axes:
        terms = []
        for size, o, _ in a.terms:
            weight = o
            fresh = []
            for n, s in next(it):                  # innermost first
                fresh.append((n, weight, s))
                weight *= n
            terms += [t for t in reversed(fresh) if t[2] != 0 and t[0] > 1]
        axes.append(kir.Axis(a.var, a.numel, tuple(terms)))
    return kir.IndexMap(tuple(axes), base)


def remap_view(v: kir.View, buffer: str, digits: Sequence[Digit]) -> kir.View:
    """``v`` re-addressed onto ``buffer``; every dimension has to come out with a
    single stride again (sub-pieces must be dense in one another)."""
    subs, base = remap(list(zip(v.shape, v.strides)), v.offset, digits)
    strides = []
    for (size, old_stride), parts in zip(zip(v.shape, v.strides), subs):
        if size == 1:
            strides.append(old_stride if old_stride > 0 else 1)
            continue
        stride, run = parts[0][1], parts[0][0]
        for n, s in parts[1:]:
            if s != stride * run:
                raise NoRemap("a view dimension would need two strides")
            run *= n
        strides.append(stride)
    return kir.View(v.name, buffer, v.shape, tuple(strides), base)


def copy_digits(src: kir.IndexMap, dst: kir.IndexMap, forward: bool) -> list[Digit]:
    """The correspondence a pure copy ``dst[dst_map(i)] = src[src_map(i)]``
    establishes, as digits.  ``forward``: old space = source offsets, new space =
    destination offsets (for an extern that is to write the destination
    directly); otherwise the other way round (an extern that is to read the
    source directly).  Both maps must be single-axis, bases zero."""
    if src.base or dst.base or len(src.axes) != 1 or len(dst.axes) != 1:
        raise NoRemap("copy maps with a base or several axes")
    numel = src.axes[0].numel
    # common refinement of the two maps' digits of the iteration index
    cuts = {1, numel}
    for m in (src, dst):
        covered = 1
        for size, o, _ in m.axes[0].terms:
            cuts.add(o)
            cuts.add(o * size)
            covered *= size
        if covered != numel:
            raise NoRemap("copy map does not cover its iteration space")
    edges = sorted(cuts)
    digits: list[Digit] = []
    for lo, hi in zip(edges, edges[1:]):
        if hi % lo:
            raise NoRemap("iteration digits do not nest")
        size = hi // lo

        def stride(m):
            for n, o, s in m.axes[0].terms:
                if o <= lo and lo * size <= o * n and lo % o == 0:
                    return s * (lo // o)
            raise NoRemap("iteration digit not addressed")

        a, b = stride(src), stride(dst)
        digits.append((size, a, b) if forward else (size, b, a))
    digits.sort(key=lambda d: d[1])
    _check_digits(digits)
    return digits
