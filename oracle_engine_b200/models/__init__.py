"""Architectures: importing this package registers each one under its config.json name."""
from . import bogupel, fovirax, fuvipel, llama, pusunex  # noqa: F401
