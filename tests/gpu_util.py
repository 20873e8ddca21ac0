"""Helpers shared by the GPU parity tests."""

import numpy as np
import torch

from oracle import nvfp4_oracle as O


def seeded_bf16(shape, seed, scale=1.0, device="cuda"):
    """bf16 tensor ~N(0, scale^2) generated on the CPU (same bits for oracle and GPU)."""
    g = torch.Generator().manual_seed(seed)
    x = (torch.randn(*shape, generator=g, dtype=torch.float32) * scale).to(torch.bfloat16)
    return x.to(device), x.float().numpy()


def np_u8(t: torch.Tensor) -> np.ndarray:
    return t.contiguous().view(torch.uint8).cpu().numpy()


def cos(a, b) -> float:
    return O.cosine(np.asarray(a, np.float64), np.asarray(b, np.float64))
