"""Top-k router: argument checks of the reference's ``route_topk``
(b12x/moe/_shared/routing.py:62-134) in front of the ``b200moe_route_topk`` kernel."""

from __future__ import annotations

import ctypes as C

import torch

from ..._lib import ext


def route_topk(
    router_logits: torch.Tensor,
    topk_logits: torch.Tensor,
    topk_ids: torch.Tensor,
    topk_weights: torch.Tensor,
    *,
    renormalize: bool,
    score_func: str = "softmax",
    selection_bias: torch.Tensor | None = None,
    route_scale: float = 1.0,
) -> None:
    """Fill ``topk_logits`` / ``topk_ids`` / ``topk_weights`` in place.

    ``score_func="softmax"``: top-k on the raw logits (ties to the larger expert index), weights =
    softmax over the k selected logits when ``renormalize`` else the logits themselves.
    ``score_func="sigmoid"``: scores = sigmoid(logits), selection on scores + ``selection_bias``,
    weights = selected scores (divided by their sum when ``renormalize``) times ``route_scale``."""
    outs = {"topk_logits": (topk_logits, torch.float32), "topk_ids": (topk_ids, torch.int32),
            "topk_weights": (topk_weights, torch.float32)}
    if router_logits.ndim != 2:
        raise ValueError(f"expected router_logits with rank 2, got shape {tuple(router_logits.shape)}")
    shapes = {tuple(t.shape) for t, _ in outs.values()}
    if any(t.ndim != 2 for t, _ in outs.values()) or len(shapes) != 1:
        raise ValueError("topk_logits, topk_ids and topk_weights must be rank-2 tensors of one shape, got "
                         + ", ".join(f"{n}{tuple(t.shape)}" for n, (t, _) in outs.items()))
    if topk_ids.shape[0] != router_logits.shape[0]:
        raise ValueError(f"router_logits batch mismatch: expected {router_logits.shape[0]}, got {topk_ids.shape[0]}")
    for name, (t, dt) in outs.items():
        if t.dtype != dt:
            raise ValueError(f"expected {name} dtype {str(dt).removeprefix('torch.')}, got {t.dtype}")
        if not t.is_contiguous():
            raise ValueError(f"{name} must be contiguous")
    if not router_logits.is_cuda:
        raise ValueError("route_topk requires CUDA tensors")
    if router_logits.dtype not in (torch.float32, torch.bfloat16):
        raise ValueError(f"router_logits must be float32 or bfloat16, got {router_logits.dtype}")
    if router_logits.stride(-1) != 1:
        raise ValueError("router_logits must be contiguous in the expert dimension")
    if router_logits.shape[1] > 1024:
        raise ValueError(f"route_topk currently supports up to 1024 experts, got {router_logits.shape[1]}")
    num_tokens, num_experts = router_logits.shape
    top_k = topk_logits.shape[1]
    if top_k <= 0:
        raise ValueError("top_k must be positive")
    if top_k > num_experts:
        raise ValueError(f"top_k={top_k} exceeds num_experts={num_experts}")
    if top_k > 32:
        raise ValueError(f"route_topk supports top_k <= 32, got {top_k}")
    if score_func == "softmax":
        mode = "softmax_topk" if renormalize else "raw"
    elif score_func == "sigmoid":
        mode = "sigmoid"
    else:
        raise ValueError(f"unsupported score_func {score_func!r}")
    bias_ptr = None
    if selection_bias is not None:
        if mode != "sigmoid":
            raise ValueError("selection_bias is only used with score_func='sigmoid'")
        if selection_bias.dtype != torch.float32 or selection_bias.numel() != num_experts:
            raise ValueError("selection_bias must be float32 [experts]")
        bias_ptr = selection_bias.contiguous().data_ptr()
    args = ext.RouteArgs(
        router_logits.data_ptr(), bias_ptr, topk_logits.data_ptr(), topk_ids.data_ptr(),
        topk_weights.data_ptr(), router_logits.stride(0), num_tokens, num_experts, top_k,
        0 if router_logits.dtype == torch.float32 else 1, ext.ROUTE_MODES[mode],
        1 if renormalize else 0, float(route_scale), 0)
    stream = torch.cuda.current_stream(router_logits.device).cuda_stream
    ext.check(ext.load().b200moe_route_topk(C.byref(args), stream), "route_topk")
