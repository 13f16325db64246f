"""Index spaces pushed through a change of buffer layout, checked by enumeration."""

import itertools
import random

import pytest

from mlc_compiler_b200 import kir
from mlc_compiler_b200.layout import (NoRemap, copy_digits, dense_digits, remap, remap_index,
                                      remap_view)


def _moved(offset, digits):
    """Where the element at old ``offset`` lives afterwards."""
    new = 0
    for size, old, nw in sorted(digits, key=lambda d: -d[1]):
        q, offset = divmod(offset, old)
        assert q < size
        new += q * nw
    assert offset == 0
    return new


def _ax(var, numel, *terms):
    return kir.Axis(var, numel, tuple(terms))


def test_token_major_buffer_to_sequence_first():
    B, T, F = 3, 4, 6
    digits = dense_digits((B, T, F), (1, 0, 2))
    assert sorted(digits) == sorted([(F, 1, 1), (T, F, B * F), (B, T * F, F)])
    # the usual row-major access: one row term covering (b, t), one column term
    m = kir.IndexMap((_ax("row", B * T, (B * T, 1, F)), _ax("col", F, (F, 1, 1))))
    r = remap_index(m, digits)
    assert r.axes[0].terms == ((B, T, F), (T, 1, B * F))
    for row, col in itertools.product(range(B * T), range(F)):
        assert r.offset(row=row, col=col) == _moved(m.offset(row=row, col=col), digits)


def test_head_layout_views_fuse_back_to_one_stride_per_dimension():
    B, H, T, D = 2, 3, 4, 5
    # dense [B, H, T, D] stored as [T, B, H, D]
    digits = dense_digits((B, H, T, D), (2, 0, 1, 3))
    q = kir.View("q", "old", (B * H, T, D), (T * D, D, 1))
    r = remap_view(q, "new", digits)
    assert r.strides == (D, B * H * D, 1) and r.buffer == "new" and r.offset == 0
    # dense [B, H, D, T] (a transposed key) stored as [T, B, H, D]
    digits = dense_digits((B, H, D, T), (3, 0, 1, 2))
    k = kir.View("k", "old", (B * H, D, T), (D * T, T, 1))
    assert remap_view(k, "new", digits).strides == (D, 1, B * H * D)
    # a [B*T, F] matrix over [B, T, F] stored as [T, B, F] has no single row stride
    with pytest.raises(NoRemap):
        remap_view(kir.View("a", "x", (B * T, D), (D, 1)), "x", dense_digits((B, T, D), (1, 0, 2)))


def test_random_maps_and_views_by_enumeration():
    rng = random.Random(7)
    done = 0
    for _ in range(400):
        rank = rng.randint(2, 4)
        shape = [rng.choice((1, 2, 3, 4)) for _ in range(rank)]
        order = list(range(rank))
        rng.shuffle(order)
        digits = dense_digits(shape, order)
        numel = 1
        for n in shape:
            numel *= n
        # an index map that walks the buffer through a random regrouping of its dimensions
        dense = [1] * rank
        for j in range(rank - 2, -1, -1):
            dense[j] = dense[j + 1] * shape[j + 1]
        dims = [(shape[j], dense[j]) for j in range(rank) if shape[j] > 1]
        rng.shuffle(dims)
        merged, terms, weight = [], [], 1
        for size, stride in dims:
            terms.append((size, weight, stride))
            weight *= size
        m = kir.IndexMap((_ax("idx", weight, *reversed(terms)),))
        try:
            r = remap_index(m, digits)
        except NoRemap:
            continue
        for i in range(weight):
            assert r.offset(idx=i) == _moved(m.offset(idx=i), digits)
        done += 1
        # the same space as a view: either it fuses or it is refused, never wrong
        v = kir.View("v", "x", tuple(s for s, _ in dims), tuple(st for _, st in dims))
        try:
            w = remap_view(v, "y", digits)
        except NoRemap:
            continue
        for coord in itertools.product(*[range(s) for s in v.shape]):
            old = sum(c * st for c, st in zip(coord, v.strides))
            assert sum(c * st for c, st in zip(coord, w.strides)) == _moved(old, digits)
    assert done > 100


def test_pieces_that_do_not_follow_the_digits_are_refused():
    digits = dense_digits((4, 6), (1, 0))                    # [4, 6] stored transposed
    with pytest.raises(NoRemap):
        remap([(3, 4)], 0, digits)                           # stride 4 inside the digit of size 6
    with pytest.raises(NoRemap):
        remap([(3, 3)], 0, digits)                           # 3 steps of 3 leave the digit half way
    with pytest.raises(NoRemap):
        remap([(6, 1)], 3, digits)                           # base 3 + 5 carries into the next digit
    subs, base = remap([(3, 2)], 6, digits)                  # row 1, every other column
    assert subs == [[(3, 8)]] and base == 1


def test_copy_digits_in_both_directions():
    H, T, D = 3, 4, 2
    n = H * T * D
    src = kir.IndexMap((_ax("idx", n, (T, H * D, D), (H, D, T * D), (D, 1, 1)),))   # reads [H, T, D]
    dst = kir.IndexMap((_ax("idx", n, (n, 1, 1)),))                                 # writes [T, H, D]
    fwd = copy_digits(src, dst, forward=True)
    out = remap_view(kir.View("x", "x", (H, T, D), (T * D, D, 1)), "y", fwd)
    assert out.strides == (D, H * D, 1)
    back = copy_digits(src, dst, forward=False)
    # a [T, H*D] matrix over the destination is [T, (H, D)] over the source: H and D do not fuse
    with pytest.raises(NoRemap):
        remap_view(kir.View("y", "y", (T, H * D), (H * D, 1)), "x", back)
    seen = remap_view(kir.View("y", "y", (T, H, D), (H * D, D, 1)), "x", back)
    assert seen.strides == (D, T * D, 1)
    for i in range(n):
        assert _moved(src.offset(idx=i), fwd) == dst.offset(idx=i)
        assert _moved(dst.offset(idx=i), back) == src.offset(idx=i)
