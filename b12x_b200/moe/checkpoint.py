"""On-disk side of ``prepare_weights``: ModelOpt NVFP4 expert weights from safetensors files.

The reference consumes expert tensors that its serving host has already stacked, fused and
swizzled (``prepare_b12x_fp4_moe_weights``, b12x/moe/fused_moe/_impl.py:5045-5365; its vLLM glue
hands over ``w13_weight`` / ``w13_weight_scale`` / ``w13_weight_scale_2`` / ``w13_input_scale``,
b12x/integration/vllm/plugin.py).  This module does that host's part for a ModelOpt HF export, so
that a layer can be brought up from the checkpoint alone:

* per expert and projection the export holds ``<proj>.weight`` (uint8, two E2M1 per byte,
  ``[out, in/2]``), ``<proj>.weight_scale`` (E4M3 per 16 inputs, plain ``[out, in/16]``),
  ``<proj>.weight_scale_2`` (f32 scalar, the weight's global de-quantisation factor) and
  ``<proj>.input_scale`` (f32 scalar, the activation's);
* gate and up are fused into one FC1 matrix in the plan's ``w13_layout`` ("w13" = ``[up; gate]``,
  "w31" = ``[gate; up]``), block scales are re-laid into 128x4 atoms, ``a*_gscale`` become the
  RECIPROCAL input scales the reference's contract wants (_impl.py:4955-4989);
* expert parallelism loads a contiguous expert range, tensor parallelism a slice of the
  intermediate dimension (rows of gate / up, columns of down).

Tensors are read one expert at a time into pre-allocated destination tensors (no second
model-sized copy on the host).
"""

from __future__ import annotations

import json
import warnings
from pathlib import Path
from typing import Iterable, Sequence

import torch

from b12x_b200.moe.fused_moe import _impl

HF_PROJ_NAMES = ("gate_proj", "up_proj", "down_proj")
MIXTRAL_PROJ_NAMES = ("w1", "w3", "w2")


class CheckpointIndex:
    """Tensor name -> file, over one file, a list of files, or a directory (with or without a
    ``*.safetensors.index.json``).  Files are opened lazily and kept open until :meth:`close`."""

    def __init__(self, source: str | Path | Iterable[str | Path]):
        try:
            import safetensors  # noqa: F401
        except ImportError as exc:  # pragma: no cover - the image ships safetensors
            raise RuntimeError("the safetensors package is required to read checkpoints") from exc
        self._handles: dict[Path, object] = {}
        self._where: dict[str, Path] = {}
        if isinstance(source, (str, Path)):
            root = Path(source)
            if root.is_dir():
                idx = sorted(root.glob("*.safetensors.index.json"))
                if idx:
                    wm = json.loads(idx[0].read_text())["weight_map"]
                    self._where = {k: root / v for k, v in wm.items()}
                    return
                files = sorted(root.glob("*.safetensors"))
            else:
                files = [root]
        else:
            files = [Path(f) for f in source]
        if not files:
            raise FileNotFoundError(f"no safetensors files under {source}")
        for f in files:
            for key in self._open(f).keys():
                self._where[key] = f

    def _open(self, path: Path):
        h = self._handles.get(path)
        if h is None:
            from safetensors import safe_open

            h = safe_open(str(path), framework="pt", device="cpu")
            self._handles[path] = h
        return h

    def __contains__(self, name: str) -> bool:
        return name in self._where

    def keys(self):
        return self._where.keys()

    def get(self, name: str) -> torch.Tensor:
        try:
            path = self._where[name]
        except KeyError:
            raise KeyError(f"tensor {name!r} is not in the checkpoint") from None
        return self._open(path).get_tensor(name)

    def close(self) -> None:
        self._handles.clear()

    def __enter__(self):
        return self

    def __exit__(self, *exc):
        self.close()


def _scalar(t: torch.Tensor, name: str) -> float:
    if t.numel() != 1:
        raise ValueError(f"{name} must be a scalar, got shape {tuple(t.shape)}")
    return float(t.reshape(()).to(torch.float32))


def load_modelopt_nvfp4_experts(
    source,
    *,
    layer_prefix: str,
    num_experts: int,
    activation: str = "silu",
    quant_modes: str | Sequence[str] = "nvfp4",
    w13_layout: str = "w13",
    device: torch.device | str = "cuda",
    params_dtype: torch.dtype = torch.bfloat16,
    proj_names: Sequence[str] = HF_PROJ_NAMES,
    expert_range: tuple[int, int] | None = None,
    intermediate_shard: tuple[int, int] | None = None,
    shared_input_scale: bool = False,
) -> _impl.B12XFP4ExpertWeights:
    """Read the experts ``<layer_prefix>.<e>.<proj>.*`` and return prepared weights.

    ``layer_prefix`` is everything before the expert number, e.g.
    ``"model.layers.3.mlp.experts"``.  ``expert_range=(lo, hi)`` keeps experts ``lo..hi-1`` (the
    result's expert dimension is ``hi - lo``).  ``intermediate_shard=(rank, world)`` keeps the
    rank-th of ``world`` equal slices of the intermediate dimension.  ``shared_input_scale`` uses
    the largest input scale over the loaded experts for all of them (what hosts do that quantise
    the activations once, before routing); the default keeps the checkpoint's per-expert scales.

    A non-gated activation (``relu2``) reads only ``proj_names[1]`` (up) and ``proj_names[2]``."""
    gate_name, up_name, down_name = proj_names
    lo, hi = expert_range if expert_range is not None else (0, int(num_experts))
    if not (0 <= lo < hi <= int(num_experts)):
        raise ValueError(f"expert_range {expert_range} is outside 0..{num_experts}")
    e_loc = hi - lo
    own = not isinstance(source, CheckpointIndex)
    ck = CheckpointIndex(source) if own else source
    try:
        gated = _impl.is_gated_moe_activation(activation)
        first = ck.get(f"{layer_prefix}.{lo}.{up_name}.weight")
        i_full, k = int(first.shape[0]), int(first.shape[1]) * 2
        if first.dtype != torch.uint8:
            raise TypeError(f"{up_name}.weight must be packed uint8 FP4, got {first.dtype}")
        rank, world = intermediate_shard if intermediate_shard is not None else (0, 1)
        if not (0 <= rank < world) or i_full % world != 0 or (i_full // world) % 64 != 0:
            raise ValueError(f"intermediate size {i_full} does not split into {world} shards of a "
                             "multiple of 64")
        i = i_full // world
        r0 = rank * i
        plan = _impl.plan_b12x_fp4_moe_weights(
            quant_modes=quant_modes, source_format="modelopt_nvfp4", activation=activation,
            params_dtype=params_dtype, num_experts=e_loc, hidden_size=k, intermediate_size=i,
            w13_layout=w13_layout)
        w1_rows = plan.w1_rows
        dev = torch.device(device)
        w1 = torch.empty((e_loc, w1_rows, k // 2), dtype=torch.uint8, device=dev)
        w2 = torch.empty((e_loc, k, i // 2), dtype=torch.uint8, device=dev)
        s1 = torch.empty((e_loc, w1_rows, k // 16), dtype=torch.uint8, device=dev)
        s2 = torch.empty((e_loc, k, i // 16), dtype=torch.uint8, device=dev)
        g1 = torch.empty(e_loc, dtype=torch.float32)
        g2 = torch.empty(e_loc, dtype=torch.float32)
        in1 = torch.empty(e_loc, dtype=torch.float32)
        in2 = torch.empty(e_loc, dtype=torch.float32)
        # row ranges of the fused FC1 matrix
        if gated:
            up_at, gate_at = (0, i) if plan.w13_layout == "w13" else (i, 0)
        else:
            up_at, gate_at = 0, None

        def rows_of(name: str, what: str) -> torch.Tensor:
            t = ck.get(f"{name}.{what}")
            if what == "weight_scale":
                t = t.view(torch.uint8)
            return t[r0:r0 + i]

        for j, e in enumerate(range(lo, hi)):
            base = f"{layer_prefix}.{e}"
            w1[j, up_at:up_at + i].copy_(rows_of(f"{base}.{up_name}", "weight"))
            s1[j, up_at:up_at + i].copy_(rows_of(f"{base}.{up_name}", "weight_scale"))
            up_g = _scalar(ck.get(f"{base}.{up_name}.weight_scale_2"), "weight_scale_2")
            up_in = _scalar(ck.get(f"{base}.{up_name}.input_scale"), "input_scale")
            if gated:
                w1[j, gate_at:gate_at + i].copy_(rows_of(f"{base}.{gate_name}", "weight"))
                s1[j, gate_at:gate_at + i].copy_(rows_of(f"{base}.{gate_name}", "weight_scale"))
                gate_g = _scalar(ck.get(f"{base}.{gate_name}.weight_scale_2"), "weight_scale_2")
                gate_in = _scalar(ck.get(f"{base}.{gate_name}.input_scale"), "input_scale")
                if gate_g != up_g:
                    # one FC1 matrix has one global factor; the block scales cannot absorb the
                    # ratio exactly, so the gate's is used and the caller is told
                    warnings.warn(f"{base}: gate and up weight_scale_2 differ ({gate_g} vs {up_g}); "
                                  "using the gate's for the fused FC1 matrix", stacklevel=2)
                    up_g = gate_g
                up_in = max(up_in, gate_in)
            g1[j], in1[j] = up_g, up_in
            dw = ck.get(f"{base}.{down_name}.weight")
            ds = ck.get(f"{base}.{down_name}.weight_scale").view(torch.uint8)
            w2[j].copy_(dw[:, r0 // 2:(r0 + i) // 2])
            s2[j].copy_(ds[:, r0 // 16:(r0 + i) // 16])
            g2[j] = _scalar(ck.get(f"{base}.{down_name}.weight_scale_2"), "weight_scale_2")
            in2[j] = _scalar(ck.get(f"{base}.{down_name}.input_scale"), "input_scale")
        if shared_input_scale:
            in1 = in1.max().expand(e_loc).contiguous()
            in2 = in2.max().expand(e_loc).contiguous()
        return _impl.prepare_b12x_fp4_moe_weights(
            plan=plan, params_dtype=params_dtype, w1_fp4=w1, w2_fp4=w2,
            w1_blockscale=_impl._swizzle_scale_grid(s1), w2_blockscale=_impl._swizzle_scale_grid(s2),
            w1_global_scale=g1.to(dev), w2_global_scale=g2.to(dev),
            a1_gscale=torch.reciprocal(in1).to(dev), a2_gscale=torch.reciprocal(in2).to(dev))
    finally:
        if own:
            ck.close()
