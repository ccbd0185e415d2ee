"""terra_b200: a Blackwell (sm_100a) native hierarchical-parallel training runtime for
high-resolution Earth-forecast Swin transformers."""

__version__ = "0.1.0"
