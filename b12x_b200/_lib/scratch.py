"""Caller-owned scratch: a plan names ONE contiguous uint8 buffer, the caller allocates it, ``bind``
only takes views of it.  The public names and the accepted container forms are the contract of the
reference's ``b12x/_lib/scratch.py:12-77`` (a tensor, a mapping by spec name, or a one-element
sequence); the checking itself is this library's."""

from __future__ import annotations

from collections.abc import Mapping, Sequence
from dataclasses import dataclass
from math import prod

import torch


@dataclass(frozen=True, kw_only=True)
class ScratchBufferSpec:
    name: str
    shape: tuple[int, ...]
    dtype: torch.dtype
    device: torch.device

    @property
    def nbytes(self) -> int:
        return prod(int(d) for d in self.shape) * torch.empty((), dtype=self.dtype).element_size()


def scratch_buffer_spec(name: str, *, nbytes: int, device: torch.device) -> ScratchBufferSpec:
    """Spec of an opaque byte buffer (never empty: a zero-byte plan still names one byte)."""
    return ScratchBufferSpec(name=name, shape=(max(int(nbytes), 1),), dtype=torch.uint8, device=device)


def _pick(scratch, name: str) -> torch.Tensor:
    """The tensor the caller meant, out of the three accepted container forms."""
    if isinstance(scratch, torch.Tensor):
        return scratch
    if isinstance(scratch, Mapping):
        try:
            return scratch[name]
        except KeyError:
            raise KeyError(f"scratch mapping has no entry {name!r}") from None
    if isinstance(scratch, Sequence):
        if len(scratch) == 1:
            return scratch[0]
        raise ValueError(f"a scratch sequence holds exactly one tensor, got {len(scratch)}")
    raise TypeError(f"scratch must be a tensor, a mapping or a sequence of tensors, not {type(scratch).__name__}")


def scratch_tensor(scratch, specs: tuple[ScratchBufferSpec, ...], *, owner: str) -> torch.Tensor:
    """Resolve and check the caller's buffer against ``specs``; returns it flattened.  Nothing is
    allocated or copied."""
    if len(specs) != 1:
        raise RuntimeError(f"{owner} plans use exactly one scratch buffer, this one names {len(specs)}")
    (spec,) = specs
    buf = _pick(scratch, spec.name)
    problems = []
    if buf.dtype != spec.dtype:
        raise TypeError(f"{owner} scratch {spec.name!r} has dtype {buf.dtype}, the plan needs {spec.dtype}")
    if buf.device != spec.device:
        problems.append(f"is on {buf.device}, the plan is for {spec.device}")
    needed = int(spec.shape[0])
    if buf.numel() < needed:
        problems.append(f"holds {buf.numel()} bytes, the plan needs {needed}")
    if not buf.is_contiguous():
        problems.append("is not contiguous")
    if problems:
        raise ValueError(f"{owner} scratch {spec.name!r} " + "; ".join(problems))
    return buf.reshape(-1)
