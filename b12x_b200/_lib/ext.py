"""ctypes binding of ``libb200moe.so`` (C ABI declared in ``include/b200moe.h``).

There is no fallback: if the shared library is missing or fails to load, every operator that
needs it raises.  Build it with ``python -m b12x_b200._build`` (needs nvcc).
"""

from __future__ import annotations

import ctypes as C
from pathlib import Path

_LIB_PATH = Path(__file__).resolve().parents[1] / "csrc" / "libb200moe.so"
_lib = None

RECIPES = {"nvfp4": 0, "w4a8_mx": 1, "w4a16": 2}
ACTIVATIONS = {"silu": 0, "relu2": 1, "swigluoai": 2, "situ": 3}
ROUTE_MODES = {"softmax_topk": 0, "raw": 1, "sigmoid": 2}

OK, EINVAL, ECAPACITY, ECUDA, EUNSUPPORTED, EALIGN = 0, -1, -2, -3, -4, -5


class DeviceInfo(C.Structure):
    _fields_ = [("sm_major", C.c_int32), ("sm_minor", C.c_int32), ("num_sms", C.c_int32),
                ("max_smem_optin", C.c_int32), ("total_mem", C.c_int64)]


class CapsC(C.Structure):
    _fields_ = [("max_tokens", C.c_int32), ("num_topk", C.c_int32), ("num_experts", C.c_int32),
                ("hidden_size", C.c_int32), ("intermediate", C.c_int32), ("recipe", C.c_int32),
                ("activation", C.c_int32), ("tile_rows", C.c_int32)]


class ScratchLayout(C.Structure):
    _fields_ = [(n, C.c_int64) for n in (
        "total_nbytes", "status", "expert_counts", "expert_offsets", "tile_base", "mtile_expert",
        "mtile_row0", "mtile_rows", "sorted_route_ids", "inv_perm", "act_q", "act_sf", "mid_q",
        "mid_sf", "routed", "sort_tmp")] + [("rows", C.c_int32), ("mtile_cap", C.c_int32),
                                    ("tile_rows", C.c_int32), ("reserved", C.c_int32)]


class RouteArgs(C.Structure):
    _fields_ = [("logits", C.c_void_p), ("bias", C.c_void_p), ("topk_logits", C.c_void_p),
                ("topk_ids", C.c_void_p), ("topk_weights", C.c_void_p),
                ("logits_row_stride", C.c_int64),
                ("num_tokens", C.c_int32), ("num_experts", C.c_int32), ("num_topk", C.c_int32),
                ("logits_dtype", C.c_int32), ("mode", C.c_int32), ("renormalize", C.c_int32),
                ("route_scale", C.c_float), ("reserved", C.c_int32)]


class GateRouteArgs(C.Structure):
    _fields_ = [("hidden", C.c_void_p), ("gate_weight", C.c_void_p), ("gate_bias", C.c_void_p),
                ("logits_out", C.c_void_p), ("tile_counters", C.c_void_p), ("selection_bias", C.c_void_p),
                ("topk_logits", C.c_void_p), ("topk_ids", C.c_void_p), ("topk_weights", C.c_void_p),
                ("status", C.c_void_p), ("hidden_row_stride", C.c_int64),
                ("num_tokens", C.c_int32), ("num_experts", C.c_int32), ("hidden_size", C.c_int32),
                ("num_topk", C.c_int32), ("hidden_dtype", C.c_int32), ("weight_dtype", C.c_int32),
                ("bias_dtype", C.c_int32), ("mode", C.c_int32), ("renormalize", C.c_int32),
                ("route_scale", C.c_float), ("kernel", C.c_int32), ("reserved", C.c_int32)]


GATE_KERNELS = {"auto": 0, "simt": 1, "tc": 2}


class SortArgs(C.Structure):
    _fields_ = [("topk_ids", C.c_void_p), ("expert_map", C.c_void_p), ("scratch", C.c_void_p),
                ("layout", C.POINTER(ScratchLayout)),
                ("num_tokens", C.c_int32), ("num_topk", C.c_int32), ("num_experts", C.c_int32),
                ("expert_map_len", C.c_int32), ("wait_flags", C.c_void_p), ("wait_epoch_dev", C.c_void_p),
                ("wait_status", C.c_void_p), ("wait_world", C.c_int32), ("wait_timeout_ms", C.c_int32)]


class QuantArgs(C.Structure):
    _fields_ = [("x", C.c_void_p), ("a1_gscale", C.c_void_p), ("scratch", C.c_void_p),
                ("layout", C.POINTER(ScratchLayout)), ("x_row_stride", C.c_int64),
                ("num_tokens", C.c_int32), ("num_topk", C.c_int32), ("num_experts", C.c_int32),
                ("hidden_size", C.c_int32), ("gscale_len", C.c_int32), ("reserved", C.c_int32)]


class GatherArgs(C.Structure):
    _fields_ = [("x", C.c_void_p), ("topk_ids", C.c_void_p), ("out_rows", C.c_void_p),
                ("out_ids", C.c_void_p), ("scratch", C.c_void_p), ("layout", C.POINTER(ScratchLayout)),
                ("x_row_stride", C.c_int64),
                ("num_tokens", C.c_int32), ("num_topk", C.c_int32), ("num_groups", C.c_int32),
                ("hidden_size", C.c_int32), ("local_modulus", C.c_int32), ("reserved", C.c_int32)]


class GemmArgs(C.Structure):
    _fields_ = [("w13", C.c_void_p), ("w13_sf", C.c_void_p), ("w13_sf_rows", C.c_void_p),
                ("w1_alphas", C.c_void_p),
                ("w2", C.c_void_p), ("w2_sf", C.c_void_p), ("w2_alphas", C.c_void_p),
                ("a2_gscale", C.c_void_p), ("x", C.c_void_p), ("scratch", C.c_void_p),
                ("layout", C.POINTER(ScratchLayout)), ("fc1_tap", C.c_void_p),
                ("x_row_stride", C.c_int64),
                ("num_tokens", C.c_int32), ("num_topk", C.c_int32), ("num_experts", C.c_int32),
                ("hidden_size", C.c_int32), ("intermediate", C.c_int32),
                ("recipe", C.c_int32), ("activation", C.c_int32), ("gate_first", C.c_int32),
                ("gscale_len", C.c_int32), ("swiglu_limit", C.c_float),
                ("swiglu_alpha", C.c_float), ("swiglu_beta", C.c_float),
                ("num_sms", C.c_int32), ("sf_e8m0", C.c_int32), ("fc1_route_weights", C.c_void_p)]


class AmaxArgs(C.Structure):
    _fields_ = [("scratch", C.c_void_p), ("layout", C.POINTER(ScratchLayout)), ("amax", C.c_void_p),
                ("num_rows", C.c_int32), ("num_experts", C.c_int32), ("hidden_size", C.c_int32),
                ("intermediate", C.c_int32), ("layer_idx", C.c_int32), ("recipe", C.c_int32)]


class CombineArgs(C.Structure):
    _fields_ = [("topk_weights", C.c_void_p), ("out", C.c_void_p), ("scratch", C.c_void_p),
                ("layout", C.POINTER(ScratchLayout)), ("out_row_stride", C.c_int64),
                ("num_tokens", C.c_int32), ("num_topk", C.c_int32), ("hidden_size", C.c_int32),
                ("out_f32", C.c_int32), ("output_scale", C.c_float), ("unit_weights", C.c_int32)]


MAX_RANKS = 16
PeerArray = C.c_void_p * MAX_RANKS


class EpDispatchArgs(C.Structure):
    _fields_ = [("x", C.c_void_p), ("topk_ids", C.c_void_p), ("peer_rows", PeerArray),
                ("peer_ids", PeerArray), ("peer_flags", PeerArray), ("done_counter", C.c_void_p),
                ("epoch_dev", C.c_void_p), ("scratch", C.c_void_p), ("layout", C.POINTER(ScratchLayout)), ("x_row_stride", C.c_int64),
                ("num_tokens", C.c_int32), ("num_topk", C.c_int32), ("world", C.c_int32), ("rank", C.c_int32),
                ("hidden_size", C.c_int32), ("local_modulus", C.c_int32), ("cap_rows", C.c_int32),
                ("epoch", C.c_int32), ("payload", C.c_int32), ("sf_row_stride", C.c_int32),
                ("gscale_len", C.c_int32), ("reserved", C.c_int32), ("peer_sf", PeerArray),
                ("a1_gscale", C.c_void_p), ("status", C.c_void_p), ("local_ids", C.c_void_p)]


EP_PAYLOADS = {"bf16": 0, "nvfp4": 1, "mxfp8": 2}


class PackedArgs(C.Structure):
    _fields_ = [("q_rows", C.c_void_p), ("sf_rows", C.c_void_p), ("scratch", C.c_void_p),
                ("layout", C.POINTER(ScratchLayout)), ("num_rows", C.c_int32), ("num_experts", C.c_int32),
                ("hidden_size", C.c_int32), ("payload", C.c_int32), ("sf_row_stride", C.c_int32),
                ("reserved", C.c_int32)]


class EpCombineArgs(C.Structure):
    _fields_ = [("topk_weights", C.c_void_p), ("out", C.c_void_p), ("peer_scratch", PeerArray),
                ("scratch", C.c_void_p), ("layout", C.POINTER(ScratchLayout)),
                ("peer_inv_perm_off", C.c_int64), ("peer_routed_off", C.c_int64), ("out_row_stride", C.c_int64),
                ("num_tokens", C.c_int32), ("num_topk", C.c_int32), ("world", C.c_int32), ("rank", C.c_int32),
                ("hidden_size", C.c_int32), ("cap_rows", C.c_int32), ("output_scale", C.c_float),
                ("timeout_ms", C.c_int32), ("signal_flags", PeerArray), ("wait_flags", C.c_void_p),
                ("epoch_dev", C.c_void_p), ("status", C.c_void_p)]


def peer_array(ptrs) -> PeerArray:
    arr = PeerArray()
    for i, p in enumerate(ptrs):
        arr[i] = int(p)
    return arr


# every symbol include/b200moe.h declares, with its argument types
EXPORTS = {
    "b200moe_abi_version": ([], C.c_int),
    "b200moe_strerror": ([C.c_int], C.c_char_p),
    "b200moe_query_device": ([C.c_int, C.POINTER(DeviceInfo)], C.c_int),
    "b200moe_scratch_nbytes": ([C.POINTER(CapsC), C.POINTER(ScratchLayout)], C.c_int),
    "b200moe_route_topk": ([C.POINTER(RouteArgs), C.c_void_p], C.c_int),
    "b200moe_gate_route": ([C.POINTER(GateRouteArgs), C.c_void_p], C.c_int),
    "b200moe_expert_sort": ([C.POINTER(SortArgs), C.c_void_p], C.c_int),
    "b200moe_expert_sort_static": ([C.c_void_p, C.c_void_p, C.c_int32, C.c_int32, C.c_int32, C.c_int32,
                                    C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p], C.c_int),
    "b200moe_permute_quant_nvfp4": ([C.POINTER(QuantArgs), C.c_void_p], C.c_int),
    "b200moe_permute_quant_mxfp8": ([C.POINTER(QuantArgs), C.c_void_p], C.c_int),
    "b200moe_gather_rows": ([C.POINTER(GatherArgs), C.c_void_p], C.c_int),
    "b200moe_grouped_gemm1_act": ([C.POINTER(GemmArgs), C.c_void_p], C.c_int),
    "b200moe_grouped_gemm2": ([C.POINTER(GemmArgs), C.c_void_p], C.c_int),
    "b200moe_combine": ([C.POINTER(CombineArgs), C.c_void_p], C.c_int),
    "b200moe_ep_dispatch": ([C.POINTER(EpDispatchArgs), C.c_void_p], C.c_int),
    "b200moe_permute_packed": ([C.POINTER(PackedArgs), C.c_void_p], C.c_int),
    "b200moe_activation_amax": ([C.POINTER(AmaxArgs), C.c_void_p], C.c_int),
    "b200moe_round_rows_bf16": ([C.c_void_p, C.c_void_p, C.c_int64, C.c_void_p], C.c_int),
    "b200moe_ep_place_routes": ([C.c_void_p, C.c_int32, C.c_int32, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p,
                                 C.c_void_p], C.c_int),
    "b200moe_ep_signal": ([C.POINTER(C.c_void_p), C.c_int32, C.c_int32, C.c_int32, C.c_void_p, C.c_void_p], C.c_int),
    "b200moe_ep_wait": ([C.c_void_p, C.c_int32, C.c_int32, C.c_void_p, C.c_void_p, C.c_int32, C.c_void_p], C.c_int),
    "b200moe_ep_combine": ([C.POINTER(EpCombineArgs), C.c_void_p], C.c_int),
    "b200moe_quantize_rows_nvfp4": ([C.c_void_p, C.c_int64, C.c_int32, C.c_int32, C.c_void_p, C.c_void_p,
                                     C.c_void_p, C.c_void_p], C.c_int),
    "b200moe_quantize_rows_mxfp8": ([C.c_void_p, C.c_int64, C.c_int32, C.c_int32, C.c_void_p, C.c_void_p,
                                     C.c_void_p, C.c_void_p], C.c_int),
}


def lib_path() -> Path:
    return _LIB_PATH


def load():
    """Load the extension (once).  Raises RuntimeError if it is not built."""
    global _lib
    if _lib is not None:
        return _lib
    if not _LIB_PATH.exists():
        raise RuntimeError(
            f"{_LIB_PATH} is missing: the sm_100a extension is not built and there is no other "
            "implementation of this operator (run `python -m b12x_b200._build`)")
    lib = C.CDLL(str(_LIB_PATH))
    for name, (argtypes, restype) in EXPORTS.items():
        fn = getattr(lib, name)
        fn.argtypes = argtypes
        fn.restype = restype
    if lib.b200moe_abi_version() != 4:
        raise RuntimeError("libb200moe.so ABI version mismatch; rebuild it")
    _lib = lib
    return lib


def is_loaded() -> bool:
    return _lib is not None


def strerror(code: int) -> str:
    return load().b200moe_strerror(code).decode()


def check(code: int, what: str) -> None:
    """Map a negative status to the exception type the reference raises for that situation."""
    if code == OK:
        return
    msg = f"{what}: {strerror(code)} (status {code})"
    if code in (EINVAL, EALIGN):
        raise ValueError(msg)
    if code == EUNSUPPORTED:
        raise NotImplementedError(msg)
    raise RuntimeError(msg)


def scratch_layout(max_tokens: int, num_topk: int, num_experts: int, hidden: int, intermediate: int,
                   recipe: str, activation: str, tile_rows: int = 0) -> ScratchLayout:
    caps = CapsC(max_tokens, num_topk, num_experts, hidden, intermediate, RECIPES[recipe],
                 ACTIVATIONS[activation], int(tile_rows))
    out = ScratchLayout()
    check(load().b200moe_scratch_nbytes(C.byref(caps), C.byref(out)), "scratch layout")
    return out
