"""Makes the reference importable: ``baseline/_ref`` (the offline install) plus the ``timm`` shim on sys.path."""
import os
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
REF = os.path.join(HERE, "_ref")
SHIMS = os.path.join(HERE, "shims")


def available() -> bool:
    return os.path.isdir(os.path.join(REF, "models"))


def enable() -> None:
    if not available():
        raise RuntimeError("reference is not installed under baseline/_ref")
    for p in (SHIMS, REF):
        if p not in sys.path:
            sys.path.insert(0, p)
