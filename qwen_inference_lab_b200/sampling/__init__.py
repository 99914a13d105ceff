from .sampler import SLOT, NonFiniteLogits, Sampler
