from .sample import SamplingParams, sample

__all__ = ["SamplingParams", "sample"]
