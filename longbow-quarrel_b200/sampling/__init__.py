from .params import HISTORY_WINDOW, SamplingParams
from .sampler import history_window, sample

__all__ = ["HISTORY_WINDOW", "SamplingParams", "history_window", "sample"]
