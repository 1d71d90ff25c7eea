"""Architectures.  Importing this package registers them."""
from . import kagatar, pitenex, puratar, qwen3, ranudra  # noqa: F401
from .kagatar import KagatarConfig
from .pitenex import PitenexConfig
from .puratar import PuratarConfig
from .qwen3 import Qwen3Config
from .ranudra import RanudraConfig

__all__ = ["KagatarConfig", "PitenexConfig", "PuratarConfig", "Qwen3Config", "RanudraConfig"]
