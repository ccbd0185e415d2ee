"""Harness around the unmodified reference installed under ``baseline/_ref`` (git-ignored)."""
