"""Two-function stand-in for ``timm`` (not installed here), used only when the reference is imported."""
