"""Host-side helpers around the edge rotation; the rotation itself is computed by the
``zp_wigner_forward`` kernel.  Mirrors the public names of the reference's blocks/wigner.py
that callers of the block use."""

from __future__ import annotations

import torch


def gamma_harmonics(gamma: torch.Tensor, lmax: int) -> tuple[torch.Tensor, torch.Tensor]:
    """cos(k gamma), sin(k gamma) for k = 0..lmax as [E, lmax+1] (blocks/wigner.py:203-213)."""
    k = torch.arange(lmax + 1, device=gamma.device, dtype=gamma.dtype)
    kg = gamma.unsqueeze(1) * k.unsqueeze(0)
    return torch.cos(kg), torch.sin(kg)
