from .options import Sampler, Sampling
from .select import DeviceStepError, NonFiniteLogits, sample_rows

__all__ = ["Sampler", "Sampling", "DeviceStepError", "NonFiniteLogits", "sample_rows"]
