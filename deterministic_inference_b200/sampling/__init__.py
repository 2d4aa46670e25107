from .sampler import sample
