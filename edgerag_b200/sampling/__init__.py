from .params import SamplingParams, rng_state

__all__ = ["SamplingParams", "rng_state"]
