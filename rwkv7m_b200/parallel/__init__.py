"""Multi-GPU execution: process-group setup, data-parallel trainers, fused
collective kernels, distributed checkpoints, input pipeline, metrics and audits."""

from .dp import DataParallelTrainer

__all__ = ["DataParallelTrainer"]
