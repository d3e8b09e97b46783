from .torch_dist import GlooBackend, NcclBackend

__all__ = ["GlooBackend", "NcclBackend"]
