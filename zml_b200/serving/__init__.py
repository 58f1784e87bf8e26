"""Serving: paged KV cache, scheduler, CUDA-graph decode."""
from .engine import Engine, GenerationStats, PagePool, Request  # noqa: F401
