from .sampler import AllLogitsNaN, Sampler, SamplingParams
