from .kernel import fully_fused_mlp, fully_fused_mlp_mse
from .module import FullyFusedMLP


__all__ = ["fully_fused_mlp", "fully_fused_mlp_mse", "FullyFusedMLP"]
