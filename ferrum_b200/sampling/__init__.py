from .sampler import DeviceSampler

__all__ = ["DeviceSampler"]
