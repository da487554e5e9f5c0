"""Sampling: per-request options, greedy / temperature / top-p kernels behind `Sampler`."""
from .params import SamplingParams, GenStats
from .sampler import Sampler, draw_rows, uniform_for, request_seed

__all__ = ["SamplingParams", "GenStats", "Sampler", "draw_rows", "uniform_for", "request_seed"]
