"""Model families: hierarchical Swin with FuXi-style sampling blocks (``credit_hierarchical_swin``) and the
plain Swin reference (``swin_reference``), each in a sequential and a parallel build."""
from .hierarchical_swin import (ParallelHierarchicalSwin, ParallelSwinReference, SequentialHierarchicalSwin,
                                SequentialSwinReference)

__all__ = ["SequentialHierarchicalSwin", "ParallelHierarchicalSwin", "SequentialSwinReference",
           "ParallelSwinReference"]
