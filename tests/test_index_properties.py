"""Property tests: the emit-time proofs about index maps hold by brute force.

``classify`` is what licenses a 128-bit access without any runtime check, and
``compose`` is what licenses folding a producer into a kernel that reads it at
another index, so both are checked exhaustively on random small maps.
"""

import math

from hypothesis import given, settings, strategies as st

from mlc_compiler_b200 import kir, rewrite
from mlc_compiler_b200.emit.indexing import classify


@st.composite
def index_maps(draw, max_dims=4):
    """A random strided view of a random contiguous iteration space, in the
    canonical term form the lowering produces (size-1 and stride-0 dims dropped)."""
    rank = draw(st.integers(1, max_dims))
    shape = [draw(st.sampled_from([1, 2, 3, 4, 6, 8, 16])) for _ in range(rank)]
    numel = math.prod(shape)
    out_strides = [math.prod(shape[i + 1:]) for i in range(rank)]
    # input strides: a permutation of a contiguous layout, with optional broadcast / padding
    perm = draw(st.permutations(range(rank)))
    pad = draw(st.sampled_from([1, 1, 2, 8]))
    in_strides = [0] * rank
    acc = 1
    for d in reversed(perm):
        if draw(st.integers(0, 5)) == 0:
            in_strides[d] = 0                      # broadcast dim
        else:
            in_strides[d] = acc * (pad if acc > 1 else 1)
            acc *= shape[d]
    base = draw(st.sampled_from([0, 0, 4, 8, 16, 3]))
    terms = tuple((shape[d], out_strides[d], in_strides[d]) for d in range(rank)
                  if shape[d] != 1 and in_strides[d] != 0)
    return kir.IndexMap((kir.Axis("idx", numel, terms),), base), numel


@settings(max_examples=300, deadline=None)
@given(index_maps(), st.sampled_from([2, 4, 8, 16]))
def test_classified_access_is_what_the_map_really_does(mn, vmax):
    m, numel = mn
    acc = classify(m, "idx", vmax)
    w = acc.width
    assert w >= 1 and vmax % w == 0
    if numel % w:
        return                                      # emitters only ask for widths dividing numel
    for start in range(0, numel, w):
        offs = [m.offset(idx=i) for i in range(start, start + w)]
        if acc.mode == "contig":
            assert offs == list(range(offs[0], offs[0] + w)), (m, acc, start)
            assert offs[0] % w == 0, (m, acc, start)
        else:
            assert len(set(offs)) == 1, (m, acc, start)


@st.composite
def producer_and_reader(draw):
    """A producer space [A, B, C] and a reader that walks a permuted (optionally
    sliced) view of it, plus a producer operand of broadcast / identity kind."""
    dims = [draw(st.sampled_from([2, 3, 4, 8])) for _ in range(3)]
    n = math.prod(dims)
    strides = [dims[1] * dims[2], dims[2], 1]
    perm = draw(st.permutations(range(3)))
    cut = draw(st.integers(0, 1))                   # optionally slice the first producer dim
    shape = [dims[d] for d in perm]
    lo = 0
    if cut and dims[0] > 2:
        lo = 1
        shape[perm.index(0)] = dims[0] - 1
    numel = math.prod(shape)
    out_strides = [math.prod(shape[i + 1:]) for i in range(3)]
    terms = tuple((shape[i], out_strides[i], strides[perm[i]]) for i in range(3) if shape[i] != 1)
    outer = kir.IndexMap((kir.Axis("idx", numel, terms),), lo * strides[0])
    kind = draw(st.sampled_from(["identity", "last", "middle", "first", "last_two"]))
    inner_terms = {
        "identity": ((n, 1, 1),),
        "last": ((dims[2], 1, 1),),
        "middle": ((dims[1], dims[2], 1),),
        "first": ((dims[0], dims[1] * dims[2], 1),),
        "last_two": ((dims[1] * dims[2], 1, 1),),
    }[kind]
    inner = kir.IndexMap((kir.Axis("idx", n, inner_terms),), draw(st.sampled_from([0, 5])))
    return outer, inner, n, numel


@settings(max_examples=300, deadline=None)
@given(producer_and_reader())
def test_composed_map_equals_the_composition(case):
    outer, inner, n, numel = case
    try:
        c = rewrite.compose(outer, inner, n)
    except rewrite._NoCompose:
        return                                      # refusing is always allowed
    for i in range(numel):
        assert c.offset(idx=i) == inner.offset(idx=outer.offset(idx=i)), (outer, inner, i)
