"""Expert-parallel MoE layer on top of the grouped GEMMs: experts are partitioned across
ranks, tokens travel by all-to-all (NCCL over NVLink on GPUs), every rank runs its local
gate+up and down grouped GEMMs.  The reference has no distributed code; this package is the
multi-GPU form of its grouped-GEMM path."""

from .dispatch import DispatchPlan, combine, dispatch, make_plan  # noqa: F401
