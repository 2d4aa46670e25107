from .sampler import keep_mask, sample
