"""Data path: real / synthetic GLORYS-shaped datasets, online padding + stripe split + patchify, task constants."""
