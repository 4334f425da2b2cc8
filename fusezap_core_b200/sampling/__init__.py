from .params import SamplingParams
from .sampler import RequestSampler, repetition_penalty, top_k_filter, top_p_filter, softmax

__all__ = ["SamplingParams", "RequestSampler", "repetition_penalty", "top_k_filter", "top_p_filter", "softmax"]
