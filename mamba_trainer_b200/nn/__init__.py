"""Host mirrors of the reference's layers that sit directly on the scan's path."""
from .conv import CausalConv1d, causal_conv1d
from .mixer import MixerCache, MixerCore, MixerShape

__all__ = ["CausalConv1d", "causal_conv1d", "MixerCache", "MixerCore", "MixerShape"]
