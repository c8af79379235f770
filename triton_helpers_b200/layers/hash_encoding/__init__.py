from .kernel import hash_encoding
from .module import HashEncoding


__all__ = ["hash_encoding", "HashEncoding"]
