from .sampler import DEFAULTS, NEUTRAL, PRESETS, Sampler, SamplingParams, Xoshiro256

__all__ = ["DEFAULTS", "NEUTRAL", "PRESETS", "Sampler", "SamplingParams", "Xoshiro256"]
