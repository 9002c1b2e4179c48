"""Helpers shared by the GPU parity tests: numpy <-> torch device transfer for float and bit tensors."""
import numpy as np
import torch


def dev_f32(a):
    return torch.from_numpy(np.ascontiguousarray(a, dtype=np.float32)).cuda()


def dev_bits(a):
    return torch.from_numpy(np.ascontiguousarray(a, dtype=np.uint64).view(np.int64)).cuda()


def host_bits(t):
    return t.cpu().numpy().view(np.uint64)


def host(t):
    return t.cpu().numpy()


def same_bits(a, b):
    a, b = np.ascontiguousarray(a), np.ascontiguousarray(b)
    return a.shape == b.shape and a.tobytes() == b.tobytes()


def rand_bits(rng, shape):
    return rng.integers(0, 2**64, size=shape, dtype=np.uint64)
