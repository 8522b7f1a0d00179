from matricxon_b200.sampling.config import SamplingConfig

__all__ = ["SamplingConfig"]
