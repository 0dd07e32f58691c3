"""Sampling: settings, per-request state, the device draw."""
from .params import GREEDY, SamplingParams
from .sampler import RequestSampling, XorShift64, sample

__all__ = ["GREEDY", "SamplingParams", "RequestSampling", "XorShift64", "sample"]
