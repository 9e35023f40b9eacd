"""Shared helpers of the test-suite: golden loading, input hashing, layout conversions."""

from __future__ import annotations

import hashlib
from pathlib import Path

import numpy as np
import torch

GOLDEN = Path(__file__).resolve().parent / "golden"


def load_golden(name: str) -> dict:
    with np.load(GOLDEN / name, allow_pickle=False) as z:
        return {k: z[k] for k in z.files}


def t(a: np.ndarray, dtype=None) -> torch.Tensor:
    out = torch.from_numpy(np.ascontiguousarray(a))
    if dtype is torch.bfloat16:
        return out.view(torch.bfloat16)
    return out if dtype is None else out.to(dtype)


def sha(x: torch.Tensor) -> str:
    return hashlib.sha256(x.detach().cpu().contiguous().view(torch.uint8).numpy().tobytes()).hexdigest()


def atoms_to_rows(atoms: torch.Tensor, mtile: int, atoms_per_tile: int, nrows: int, ncols: int) -> torch.Tensor:
    """Scale bytes of one 128-row tile, stored as a chain of 512-byte atoms, -> [nrows, ncols]."""
    a = atoms.reshape(-1)[mtile * atoms_per_tile * 512:(mtile + 1) * atoms_per_tile * 512]
    a = a.reshape(atoms_per_tile, 32, 4, 4)          # [col/4][row%32][row/32][col%4]
    full = a.permute(2, 1, 0, 3).reshape(128, atoms_per_tile * 4)
    return full[:nrows, :ncols]
