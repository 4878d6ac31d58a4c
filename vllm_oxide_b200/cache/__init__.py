from .pools import CachePools

__all__ = ["CachePools"]
