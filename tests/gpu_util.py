"""Helpers for the GPU parity tests: numpy <-> CUDA tensors (bf16 travels as
int16 bit patterns) and comparison statistics."""
import numpy as np
import torch


def dev(a: np.ndarray) -> torch.Tensor:
    a = np.ascontiguousarray(a)
    if a.dtype == np.uint16:
        return torch.from_numpy(a.view(np.int16)).cuda()
    if a.dtype == np.uint32:
        return torch.from_numpy(a.view(np.int32)).cuda()
    return torch.from_numpy(a).cuda()


def host(t: torch.Tensor) -> np.ndarray:
    if t.dtype == torch.bfloat16:
        return t.view(torch.int16).cpu().numpy().view(np.uint16)
    a = t.cpu().numpy()
    if a.dtype == np.int16:
        return a.view(np.uint16)
    return a


def bf16_ulp_diff(a_u16: np.ndarray, b_u16: np.ndarray) -> np.ndarray:
    """Distance in bf16 units-in-the-last-place between two bit-pattern arrays."""
    def key(u):
        u = u.astype(np.int32)
        return np.where(u & 0x8000, -(u & 0x7FFF), u & 0x7FFF)
    return np.abs(key(a_u16) - key(b_u16))
