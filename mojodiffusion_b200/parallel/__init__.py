"""Parallel execution: process-group plumbing, data-parallel LoRA gradient sync, Ulysses sequence parallel,
tensor parallel and FSDP paths with their fused peer-memory kernels."""
from . import dist
from .dp import DataParallelGrads, FlatGradBuffer, broadcast_parameters
