from .kernel import fully_fused_mlp
from .module import FullyFusedMLP


__all__ = ["fully_fused_mlp", "FullyFusedMLP"]
