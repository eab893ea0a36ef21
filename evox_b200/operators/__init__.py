from . import selection

__all__ = ["selection"]
