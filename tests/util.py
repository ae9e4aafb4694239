"""Helpers shared by the GPU parity tests: device buffers via torch, raw pointers for the C ABI."""
import ctypes

import numpy as np


def torch_mod():
    import torch

    return torch


def to_dev(a):
    """numpy array -> CUDA tensor holding the same bytes."""
    torch = torch_mod()
    a = np.ascontiguousarray(a)
    if a.size == 0:
        return torch.empty(0, dtype=torch.uint8, device="cuda")
    t = torch.from_numpy(a.view(np.uint8).reshape(-1).copy()).cuda()
    return t


def dev_zeros(nbytes):
    torch = torch_mod()
    return torch.zeros(max(int(nbytes), 16), dtype=torch.uint8, device="cuda")


def dptr(t, offset=0):
    return ctypes.c_void_p(t.data_ptr() + offset)


def hptr(a):
    return a.ctypes.data_as(ctypes.c_void_p)


def to_host(t, dtype, count):
    torch = torch_mod()
    torch.cuda.synchronize()
    return t.cpu().numpy().view(np.uint8)[: count * np.dtype(dtype).itemsize].view(dtype).copy()
