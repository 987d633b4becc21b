"""How parts bring loaded tensors onto the device for a compute path."""
from __future__ import annotations

import torch


def bind_matrix(t: torch.Tensor, rt) -> torch.Tensor:
    """Matrices take the compute dtype: bf16 widens exactly for the 32-bit
    path; a matrix stored in 32-bit is rounded to bf16 for the bf16 path,
    whose matrix products read bf16."""
    return t.to(device=rt.device, dtype=rt.dtype).contiguous()


def bind_vector(t: torch.Tensor, rt) -> torch.Tensor:
    """Vectors (norm weights) stay in 32-bit when stored so; bf16 vectors
    widen for the 32-bit path and stay bf16 for the bf16 path."""
    if t.dtype == torch.float32 or rt.dtype == torch.float32:
        return t.to(device=rt.device, dtype=torch.float32).contiguous()
    return t.to(device=rt.device, dtype=rt.dtype).contiguous()
