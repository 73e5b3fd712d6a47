"""Helpers shared by the GPU parity tests."""
import numpy as np
import torch

import rptc_oracle as o


def rand_words(rng, m, n, K):
    return rng.integers(0, 2**32, (m, n * K // 32), dtype=np.uint64).astype(np.uint32)


def rand_lut(rng, code, L=16, S=8):
    if code == o.CODE_A:
        return rng.standard_normal(1 << L).astype(np.float16)
    return rng.standard_normal(2 << S).astype(np.float16)


def to_dev(a):
    a = np.ascontiguousarray(a)
    if a.dtype == np.uint32:
        a = a.view(np.int32)
    return torch.from_numpy(a).cuda()


def bits(a):
    if isinstance(a, torch.Tensor):
        a = a.cpu().numpy()
    return np.ascontiguousarray(a, dtype=np.float16).view(np.uint16)


def lut_for_oracle(lut, code, S):
    return lut.reshape(1 << S, 2) if code == o.CODE_C else lut
