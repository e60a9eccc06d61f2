"""Command-line front end: ``brain <verb> <arch> …`` ≡ ``brain <arch> <verb> …``."""
from .main import main  # noqa: F401
