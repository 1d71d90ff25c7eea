"""Architectures.  Importing this package registers them."""
from . import kagatar, pitenex, qwen3, ranudra  # noqa: F401
from .kagatar import KagatarConfig
from .pitenex import PitenexConfig
from .qwen3 import Qwen3Config
from .ranudra import RanudraConfig

__all__ = ["KagatarConfig", "PitenexConfig", "Qwen3Config", "RanudraConfig"]
