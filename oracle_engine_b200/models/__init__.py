"""Architectures: importing this package registers each one under its config.json name."""
from . import fovirax, fuvipel, llama, pusunex  # noqa: F401
