from . import selection, variation

__all__ = ["selection", "variation"]
