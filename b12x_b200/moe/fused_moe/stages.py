"""Stage-level access to the C ABI for callers that compose the layer themselves (the
expert-parallel wrapper sorts by destination rank, packs rows for the dispatch and combines the
returned rows with the same kernels the single-GPU path uses)."""

from __future__ import annotations

import ctypes as C

import torch

from ..._lib import ext


class StageArena:
    """A scratch arena plus its layout, for ``num_groups`` sort keys and ``hidden`` wide rows."""

    def __init__(self, max_tokens: int, num_topk: int, num_groups: int, hidden: int, device: torch.device):
        self.layout = ext.scratch_layout(max_tokens, num_topk, num_groups, hidden, 32, "w4a16", "silu")
        self.scratch = torch.empty(int(self.layout.total_nbytes), dtype=torch.uint8, device=device)
        self.max_tokens, self.num_topk, self.num_groups, self.hidden = max_tokens, num_topk, num_groups, hidden
        self.device = device
        self._lp = C.pointer(self.layout)

    def _view(self, name: str, count: int, dtype: torch.dtype) -> torch.Tensor:
        off = int(getattr(self.layout, name))
        nbytes = count * torch.empty((), dtype=dtype).element_size()
        return self.scratch.narrow(0, off, nbytes).view(dtype)

    @property
    def group_counts(self) -> torch.Tensor:
        return self._view("expert_counts", self.num_groups, torch.int32)

    @property
    def group_offsets(self) -> torch.Tensor:
        return self._view("expert_offsets", self.num_groups + 1, torch.int32)

    @property
    def inv_perm(self) -> torch.Tensor:
        return self._view("inv_perm", self.max_tokens * self.num_topk, torch.int32)

    @property
    def sorted_route_ids(self) -> torch.Tensor:
        return self._view("sorted_route_ids", self.max_tokens * self.num_topk, torch.int32)

    @property
    def routed(self) -> torch.Tensor:
        rows = self.max_tokens * self.num_topk
        return self._view("routed", rows * self.hidden, torch.float32).view(rows, self.hidden)

    def _stream(self) -> int:
        return torch.cuda.current_stream(self.device).cuda_stream

    def sort(self, topk_ids: torch.Tensor, group_map: torch.Tensor | None = None) -> None:
        tokens = topk_ids.shape[0]
        args = ext.SortArgs(topk_ids.data_ptr(), None if group_map is None else group_map.data_ptr(),
                            self.scratch.data_ptr(), self._lp, tokens, self.num_topk, self.num_groups,
                            0 if group_map is None else int(group_map.numel()))
        ext.check(ext.load().b200moe_expert_sort(C.byref(args), self._stream()), "expert_sort")

    def gather_rows(self, x: torch.Tensor, topk_ids: torch.Tensor, out_rows: torch.Tensor,
                    out_ids: torch.Tensor, local_modulus: int) -> None:
        args = ext.GatherArgs(x.data_ptr(), topk_ids.data_ptr(), out_rows.data_ptr(), out_ids.data_ptr(),
                              self.scratch.data_ptr(), self._lp, x.stride(0), x.shape[0], self.num_topk,
                              self.num_groups, self.hidden, int(local_modulus), 0)
        ext.check(ext.load().b200moe_gather_rows(C.byref(args), self._stream()), "gather_rows")

    def combine(self, topk_weights: torch.Tensor, out: torch.Tensor, *, output_scale: float = 1.0) -> None:
        tokens = topk_weights.shape[0]
        args = ext.CombineArgs(topk_weights.data_ptr(), out.data_ptr(), self.scratch.data_ptr(), self._lp,
                               out.stride(0), tokens, self.num_topk, self.hidden,
                               1 if out.dtype == torch.float32 else 0, float(output_scale), 0)
        ext.check(ext.load().b200moe_combine(C.byref(args), self._stream()), "combine")
