from .base import LatticeConfig  # noqa: F401
