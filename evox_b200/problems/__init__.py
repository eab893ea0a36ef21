from . import numerical

__all__ = ["numerical"]
