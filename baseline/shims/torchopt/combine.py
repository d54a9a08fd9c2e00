from .transform import chain

__all__ = ["chain"]
