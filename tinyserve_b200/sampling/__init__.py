from .params import MAX_LOGPROBS, SamplingParams
from .sampler import Sampler, TokenLogprobs, derive_seed, token_logprobs

__all__ = ["MAX_LOGPROBS", "SamplingParams", "Sampler", "TokenLogprobs", "derive_seed", "token_logprobs"]
