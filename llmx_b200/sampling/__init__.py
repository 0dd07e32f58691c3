"""Sampling: settings, per-request state, the device draw."""
from .params import GREEDY, SamplingParams
from .sampler import PendingSample, RequestSampling, XorShift64, sample, sample_async

__all__ = ["GREEDY", "SamplingParams", "PendingSample", "RequestSampling", "XorShift64", "sample", "sample_async"]
