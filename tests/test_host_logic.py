r"""Host-side logic of the Python layer that needs no GPU."""
import torch

from triton_helpers_b200.layers.hash_encoding.kernel import PI_1, PI_2, PI_3, host_primes


def test_host_primes_are_cached_per_tensor_and_version():
    pi = torch.tensor([PI_1, PI_2, PI_3], dtype=torch.int64)
    assert host_primes(pi, 3) == (PI_1, PI_2, PI_3)
    assert host_primes(pi, 2) == (PI_1, PI_2)  # a shorter prefix comes from the same cached read
    pi[1] = 7  # an in-place change bumps the tensor's version: the cache must not serve the old value
    assert host_primes(pi, 3) == (PI_1, 7, PI_3)
    other = torch.tensor([1, 3, 5, 9], dtype=torch.int64)  # longer than D, like a user-supplied `pi`
    assert host_primes(other, 3) == (1, 3, 5)
    assert host_primes((11, 13, 17), 2) == (11, 13)  # already extracted values pass through


def test_host_primes_forgets_dead_tensors():
    from triton_helpers_b200.layers.hash_encoding import kernel

    pi = torch.tensor([1, 2, 3], dtype=torch.int64)
    host_primes(pi, 3)
    key = id(pi)
    assert key in kernel._PRIMES_SEEN
    del pi
    import gc

    gc.collect()
    assert key not in kernel._PRIMES_SEEN
