"""Comparison helpers shared by the parity tests."""
import numpy as np
import torch


def max_rel_rows(got, ref):
    """Worst row of max|got - ref| / max|ref| (the Stat::max_rel of the reference's tests/forward_verify.cpp:199-211)."""
    ref = np.asarray(ref)
    if ref.size == 0:
        return 0.0
    got = np.asarray(got, dtype=np.float64).reshape(ref.shape[0], -1) if ref.ndim > 1 else np.asarray(got, np.float64)[None]
    ref = np.asarray(ref, dtype=np.float64).reshape(got.shape)
    d = np.abs(got - ref).max(axis=1)
    m = np.abs(ref).max(axis=1)
    return float(np.where(m > 0, d / np.where(m > 0, m, 1), d).max())


def bf16_ulp_dist(a, b):
    """Distance in units of the last place between two arrays of bf16 bit patterns (monotone integer mapping)."""
    def key(u):
        u = np.asarray(u, dtype=np.uint16).astype(np.int32)
        return np.where(u & 0x8000, -(u & 0x7FFF), u)
    return np.abs(key(a) - key(b))


def dev(a, dtype=None):
    """numpy -> CUDA tensor. uint16 arrays are bf16 / fp16 bit patterns: pass dtype=torch.bfloat16 / float16."""
    if a is None:
        return None
    t = torch.from_numpy(np.ascontiguousarray(a))
    if dtype is not None and a.dtype == np.uint16:
        t = t.view(torch.int16).view(dtype)
    return t.cuda()


def host(t):
    """CUDA tensor -> numpy; 16-bit float tensors come back as uint16 bit patterns."""
    t = t.detach().cpu()
    if t.dtype in (torch.bfloat16, torch.float16):
        return t.view(torch.int16).numpy().view(np.uint16)
    return t.numpy()
