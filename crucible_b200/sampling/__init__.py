from .params import (DEFAULT_MAX_TOKENS, DEFAULT_SEED, DEFAULT_TEMPERATURE, DEFAULT_TOP_K,
                     SamplingParams)
from .rng import Xorshift64Star
