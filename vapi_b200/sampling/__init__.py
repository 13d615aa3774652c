"""Sampling options and token selection."""
from .params import FinishReason, SamplingParams

__all__ = ["FinishReason", "SamplingParams"]
