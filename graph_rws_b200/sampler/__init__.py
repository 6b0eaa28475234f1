from .sampler import BCSRSampler  # noqa: F401
