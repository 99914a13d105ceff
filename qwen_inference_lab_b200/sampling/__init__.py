from .sampler import NonFiniteLogits, Sampler
