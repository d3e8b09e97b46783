from .dense_mlp import DenseMLP

__all__ = ["DenseMLP"]
