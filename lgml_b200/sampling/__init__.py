from .sampler import DEFAULTS, NEUTRAL, PRESETS, Sampler, SamplingParams, Xoshiro256, log_min_p

__all__ = ["DEFAULTS", "NEUTRAL", "PRESETS", "Sampler", "SamplingParams", "Xoshiro256", "log_min_p"]
