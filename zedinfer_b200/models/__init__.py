"""Architectures that ship with the engine.  Importing this package registers them."""
from . import baselix, gibalorn, kevatar, qwen2, sumitar  # noqa: F401
