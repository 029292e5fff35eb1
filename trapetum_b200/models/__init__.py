"""Architectures: each module turns a configuration into a ModelSpec and registers it."""
from . import divanex, fidepel, gemma2, lofirax  # noqa: F401
