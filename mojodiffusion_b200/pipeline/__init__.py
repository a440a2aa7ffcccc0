"""Pipelines: the public sampler entry points (denoise loops, CLIs)."""
from .flux import FluxPipeline
