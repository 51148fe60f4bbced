"""Helpers shared by the GPU parity tests: host bits <-> device tensors, and one comparison of the
CUDA operator (through the C ABI) with the CPU oracle on identical stored bits."""
import numpy as np
import torch

F32, F16, BF16 = 0, 2, 14
TORCH_DTYPE = {F32: torch.float32, F16: torch.float16, BF16: torch.bfloat16}
# tolerances of the path: relative Frobenius error <= 1e-5 for Float32, <= 1e-2 for 16-bit inputs
TOL = {F32: 1e-5, F16: 1e-2, BF16: 1e-2}


def to_dev(bits: np.ndarray, dtype: int, device="cuda:0") -> torch.Tensor:
    """Stored bits (uint16 for 16-bit types) -> device tensor with the same shape and strides.
    The view is re-based on a fresh (256-byte aligned) allocation that spans exactly its elements."""
    t = torch.from_numpy(bits)
    if dtype != F32:
        t = t.view(TORCH_DTYPE[dtype])
    span = 1 + sum((n - 1) * s for n, s in zip(t.shape, t.stride())) if t.numel() else 0
    d = torch.as_strided(torch.zeros(span, dtype=t.dtype, device=device), t.shape, t.stride())
    d.copy_(t)
    return d


def from_dev(t: torch.Tensor, dtype: int) -> np.ndarray:
    t = t.detach().cpu()
    if dtype != F32:
        return t.contiguous().view(torch.uint16).numpy()
    return t.contiguous().numpy()


def random_bits(oracle, rng, shape, dtype, dist="uniform", scale=1.0):
    x = rng.standard_normal(shape) if dist == "normal" else rng.uniform(-scale, scale, shape)
    return oracle.encode(x.astype(np.float32), dtype)
