"""Architectures: each module turns one family's configuration into a model made
of parts and registers itself under its config.json name."""

from . import qwen3  # noqa: F401
