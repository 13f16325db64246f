"""Compiler configuration, field for field the reference's ``Config``
(``mlc/config.py:14-67``) so that code written against it keeps working, plus
the few knobs that only the CUDA backend reads.

The pass flags (``elementwise_fusion`` ... ``memory_planning``) are consumed by
the reference's frontend, which decides *which* kernels exist; this backend reads
``cuda_graphs``, ``pointwise_block``, ``max_persistent_row`` (already folded into
``ReductionKernel.two_pass`` upstream, ``mlc/codegen/reduction_lowering.py:258``)
and ``backend``.
"""

from __future__ import annotations

from dataclasses import dataclass
from dataclasses import replace as _replace


@dataclass
class Config:
    # -- passes (read by the frontend) --------------------------------------
    elementwise_fusion: bool = True
    recompute: bool = True
    reduction_fusion: bool = True
    memory_planning: bool = True
    cuda_graphs: bool = True

    # -- codegen -------------------------------------------------------------
    #: upper bound on elements one CTA of a pointwise kernel covers
    pointwise_block: int = 1024
    max_persistent_row: int = 16384
    fp32_accumulate: bool = True

    # -- cost model (read by the frontend) ----------------------------------
    flops_per_byte: float = 20.0
    launch_overhead_bytes: float = 4.5e6
    graph_launch_overhead_bytes: float = 1.1e6
    max_recompute_ops: int = 32

    # -- misc ------------------------------------------------------------------
    backend: str = "auto"  # "auto" | "cuda" | "torch"; "triton" is refused
    debug: bool = False

    # -- CUDA backend only -----------------------------------------------------
    #: packs of 128 bits each thread of a persistent row reduction aims to own
    reduction_packs_per_thread: int = 2
    #: a row goes to a whole CTA (shared-memory hop) only when a warp would need
    #: more than this many packs per lane
    reduction_max_packs: int = 8
    #: force the number of threads that share one row (0 = choose)
    reduction_group: int = 0
    #: force the rows one CTA of a sub-warp row reduction covers (0 = choose)
    reduction_rows_per_cta: int = 0
    #: CTAs of a row reduction the compiler must keep resident per SM (caps the
    #: registers per thread through ``__launch_bounds__``; 0 = 512 threads' worth)
    reduction_min_ctas: int = 0
    #: load operands that no kernel of the schedule writes (weights, biases, masks)
    #: and do all index arithmetic *before* the grid-dependency wait, so that under
    #: programmatic dependent launch they overlap the predecessor's tail; the values
    #: cross the wait as packed words (a quarter of the registers of the widened form).
    #: True: launches that are resident all at once; "all": every launch; False: none
    hoist_stable_loads: bool | str = True
    #: release the dependent launch right after the wait instead of after the
    #: kernel's own loads have been issued
    trigger_early: bool = False
    #: kernels whose every output is fp16/bf16 may use SFU-based exp/tanh/erf and
    #: division (error ~1e-6, below half-precision resolution); fp32 kernels never do
    narrow_fast_math: bool = True
    #: programmatic dependent launch of generated kernels: False, True (every
    #: launch), "chain" (only behind another generated kernel on the same stream) or
    #: "auto" (the executor captures the graph both ways, times them, keeps the faster)
    dependent_launch: bool | str = "auto"
    #: which kernels release their dependents at their top (``launch_dependents``):
    #: 0 none, 1 launches that fit the machine in one wave, 2 all.  Measured: 0 costs the
    #: small kernels 0.15-0.25 us per launch; 2 makes the 2.6-wave bias+GELU kernel 10 %
    #: slower; releasing from the last wave only is no better than 1 and slower in the models
    dependent_trigger: int = 1
    #: pointwise kernels that move at least this many bytes use 256-bit global
    #: accesses (sm_100 ``ld/st.global.v4.b64``) when every operand allows it; 0 = never
    wide_access_bytes: int = 8 << 20
    #: same for persistent row reductions (0 = never; measured no better than 128-bit)
    wide_reduction_bytes: int = 0
    #: fold a pointwise producer into the pointwise kernels that only re-read it at
    #: another index (bias add + head-layout copy at batch > 1); bit-identical
    forward_into_copies: bool = True
    #: let a matmul store straight into the layout a following pure copy would have
    #: produced (the context ``clone`` at batch 1); same op, same values, one launch fewer
    write_through_copies: bool = True
    #: at batch > 1 store the operands and result of the attention ``bmm`` calls
    #: sequence-first, which makes ``(batch, head)`` one strided dimension: the context
    #: ``clone`` disappears and the key copy stops transposing
    sequence_first: bool = True
    #: fetch embedding rows inside the row reduction that consumes them instead of
    #: through a separate library gather (same table entries, bit-identical)
    fold_embeddings: bool = True
    #: turn ``mm`` + leading bias add into ``addmm`` (cuBLASLt bias epilogue).  Off by
    #: default: it changes how the matmul is dispatched and rounds once instead of twice
    bias_epilogue: bool = False
    #: run independent pointwise kernels over the same iteration space as one launch
    #: (BERT's q/k/v bias adds: 36 launches -> 12); bit-identical.  Off by default
    fuse_siblings: bool = False
    #: streams the schedule is captured over.  1 reproduces the reference's single
    #: chain of graph nodes; more lets kernels with no dependency between them
    #: (physical byte ranges considered) run as parallel branches of the graph
    graph_streams: int = 4

    @property
    def effective_launch_bytes(self) -> float:
        return (self.graph_launch_overhead_bytes if self.cuda_graphs
                else self.launch_overhead_bytes)

    def replace(self, **kw) -> "Config":
        return _replace(self, **kw)

    def as_scheduled(self) -> "Config":
        """The same configuration with every executor-side rewrite off: the schedule
        runs kernel for kernel and library call for library call as the frontend
        produced it, on one stream."""
        return _replace(self, forward_into_copies=False, write_through_copies=False,
                        sequence_first=False, fold_embeddings=False, bias_epilogue=False,
                        fuse_siblings=False,
                        graph_streams=1, dependent_launch="chain")


NO_FUSION = Config(elementwise_fusion=False, recompute=False, reduction_fusion=False,
                   memory_planning=False, cuda_graphs=False)
ELEMENTWISE_ONLY = Config(reduction_fusion=False)
