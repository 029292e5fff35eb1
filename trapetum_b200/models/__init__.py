"""Architectures: each module turns a configuration into a ModelSpec and registers it."""
from . import divanex, fibelix, fidepel, gemma2, lofirax  # noqa: F401
