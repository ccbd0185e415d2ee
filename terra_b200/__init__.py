"""terra_b200: a Blackwell (sm_100a) native hierarchical-parallel training runtime for
high-resolution Earth-forecast Swin transformers.

    from terra_b200 import Trainer, get_model, get_model_for_train

The names below are resolved on first use, so importing the package stays cheap."""

__version__ = "0.2.0"

_LAZY = {
    "Trainer": ("terra_b200.api", "Trainer"),
    "get_model": ("terra_b200.models.get_model", "get_model"),
    "get_model_for_train": ("terra_b200.models.get_model", "get_model_for_train"),
    "ParallelManager": ("terra_b200.parallel.rank_manager", "ParallelManager"),
    "init_distributed": ("terra_b200.distributed", "init_distributed"),
}
__all__ = sorted(_LAZY) + ["__version__"]


def __getattr__(name):
    if name in _LAZY:
        import importlib

        module, attr = _LAZY[name]
        value = getattr(importlib.import_module(module), attr)
        globals()[name] = value
        return value
    raise AttributeError(f"module 'terra_b200' has no attribute {name!r}")
