"""Architectures.  Importing this package registers the built-in ones."""
from . import buborax, gpt2, lubavik, tukavik, zuretar  # noqa: F401
