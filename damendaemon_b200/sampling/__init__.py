from .options import Sampler, Sampling
from .select import NonFiniteLogits, sample_rows

__all__ = ["Sampler", "Sampling", "NonFiniteLogits", "sample_rows"]
