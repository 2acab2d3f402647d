from . import library

__all__ = ["library"]
