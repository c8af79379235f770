from .kernel import reversible_mlp, reversible_mlp_backward, reversible_mlp_forward
from .module import ReversibleMLP


__all__ = ["reversible_mlp", "reversible_mlp_forward", "reversible_mlp_backward", "ReversibleMLP"]
