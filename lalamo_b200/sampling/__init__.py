"""Sampling: the reference's options and their device-side implementation."""

from .policy import GenerationConfig, SamplingPolicy
from .sampler import SampleRow, Sampler, pack_rows, request_key

__all__ = ["GenerationConfig", "SampleRow", "Sampler", "SamplingPolicy", "pack_rows", "request_key"]
