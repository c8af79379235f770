from .kernel import HashEncodedMLP, field_backward, field_forward, hash_encoded_mlp

__all__ = ["HashEncodedMLP", "field_backward", "field_forward", "hash_encoded_mlp"]
