"""Architectures.  Importing this package registers the built-in ones."""

from mini_engine_b200.models import bevadra, bizurax, molotar, pimezen, qwen3  # noqa: F401
