"""CPU checks of the boundary: the shared library loads, exports every symbol the header declares,
host-only entry points answer, and the planner mirrors the reference's contracts."""

import ctypes as C
import re
from pathlib import Path

import pytest
import torch

from b12x_b200._lib import ext
from b12x_b200.moe import fused_moe

ROOT = Path(__file__).resolve().parents[1]


@pytest.fixture(scope="module")
def lib():
    from b12x_b200 import _build
    _build.build()
    return ext.load()


def test_every_declared_symbol_is_exported(lib):
    header = (ROOT / "include" / "b200moe.h").read_text()
    declared = set(re.findall(r"\b(b200moe_[a-z0-9_]+)\s*\(", header))
    assert declared == set(ext.EXPORTS), declared ^ set(ext.EXPORTS)
    for name in declared:
        assert hasattr(lib, name), name
    assert lib.b200moe_abi_version() == 4
    assert lib.b200moe_strerror(-2).decode().startswith("problem exceeds")


def test_struct_sizes_match_header_layout():
    # pointer-first layouts with explicit int32 padding: sizes are multiples of 8
    for st in (ext.RouteArgs, ext.SortArgs, ext.QuantArgs, ext.GatherArgs, ext.GemmArgs, ext.CombineArgs,
               ext.ScratchLayout, ext.CapsC):
        assert C.sizeof(st) % 8 == 0, st
    assert C.sizeof(ext.ScratchLayout) == 16 * 8 + 16
    assert C.sizeof(ext.GemmArgs) == 14 * 8 + 14 * 4


def test_scratch_layout_is_monotone_and_aligned(lib):
    L = ext.scratch_layout(64, 8, 256, 7168, 2048, "nvfp4", "silu")
    names = ["status", "expert_counts", "expert_offsets", "tile_base", "mtile_expert", "mtile_row0",
             "mtile_rows", "sorted_route_ids", "inv_perm", "act_q", "act_sf", "mid_q", "mid_sf", "routed"]
    offs = [int(getattr(L, n)) for n in names]
    assert offs == sorted(offs) and all(o % 1024 == 0 for o in offs)
    # 512 routed rows over 256 experts: a small-batch plan, experts cut into 64-row tiles
    assert L.rows == 512 and L.tile_rows == 64 and L.mtile_cap == 8 + 256
    wide = ext.scratch_layout(64, 8, 256, 7168, 2048, "nvfp4", "silu", tile_rows=128)
    assert wide.tile_rows == 128 and wide.mtile_cap == 4 + 256
    # 16384 routed rows over 8 experts: 128-row tiles; other recipes have no small-batch kernel
    assert ext.scratch_layout(8192, 2, 8, 4096, 14336, "nvfp4", "silu").tile_rows == 128
    assert ext.scratch_layout(64, 8, 256, 7168, 2048, "w4a8_mx", "silu").tile_rows == 128
    assert ext.scratch_layout(64, 8, 256, 7168, 2048, "w4a8_mx", "silu", tile_rows=64).tile_rows == 128
    with pytest.raises(ValueError):
        ext.scratch_layout(64, 8, 256, 7168, 2048, "nvfp4", "silu", tile_rows=32)
    assert L.total_nbytes >= offs[-1] + 512 * 7168 * 4
    with pytest.raises(ValueError):
        ext.scratch_layout(64, 8, 256, 7170, 2048, "nvfp4", "silu")
    with pytest.raises(ValueError):
        ext.scratch_layout(64, 8, 2000, 7168, 2048, "nvfp4", "silu")


def test_host_side_argument_errors_need_no_gpu(lib):
    assert lib.b200moe_route_topk(None, None) == ext.EINVAL
    assert lib.b200moe_expert_sort(None, None) == ext.EINVAL
    assert lib.b200moe_combine(None, None) == ext.EINVAL
    assert lib.b200moe_grouped_gemm1_act(None, None) == ext.EINVAL
    a = ext.RouteArgs()
    a.logits = a.topk_ids = a.topk_weights = 16
    a.num_experts, a.num_topk, a.num_tokens = 2000, 2, 1
    assert lib.b200moe_route_topk(C.byref(a), None) == ext.EINVAL   # > 1024 experts
    # the sort's optional wait needs its epoch pointer and a sane rank count
    L = ext.scratch_layout(8, 2, 4, 256, 128, "nvfp4", "silu")
    s = ext.SortArgs(16, None, 16, C.pointer(L), 8, 2, 4, 0, 16, None, None, 2, 0)
    assert lib.b200moe_expert_sort(C.byref(s), None) == ext.EINVAL
    s = ext.SortArgs(16, None, 16, C.pointer(L), 8, 2, 4, 0, 16, 16, None, 64, 0)
    assert lib.b200moe_expert_sort(C.byref(s), None) == ext.EINVAL
    # standalone quantisers and the peer-memory entry points validate before they launch
    assert lib.b200moe_quantize_rows_nvfp4(None, 0, 1, 16, None, None, None, None) == ext.EINVAL
    assert lib.b200moe_quantize_rows_nvfp4(16, 8, 4, 24, 16, 16, 16, None) == ext.EINVAL      # K % 16
    assert lib.b200moe_quantize_rows_mxfp8(16, 8, 4, 48, 16, None, None, None) == ext.EINVAL  # K % 32
    assert lib.b200moe_quantize_rows_mxfp8(24, 8, 4, 64, 16, None, None, None) == ext.EALIGN
    assert lib.b200moe_ep_wait(None, 2, 1, None, None, 0, None) == ext.EINVAL
    assert lib.b200moe_ep_wait(16, 2, 1, None, None, 20000, None) == ext.EINVAL               # timeout too long
    assert lib.b200moe_ep_dispatch(None, None) == ext.EINVAL
    assert lib.b200moe_ep_combine(None, None) == ext.EINVAL
    assert lib.b200moe_permute_packed(None, None) == ext.EINVAL
    assert lib.b200moe_round_rows_bf16(None, None, 8, None) == ext.EINVAL
    assert lib.b200moe_round_rows_bf16(16, 16, 7, None) == ext.EINVAL                          # count % 8
    assert lib.b200moe_round_rows_bf16(20, 16, 8, None) == ext.EALIGN
    assert lib.b200moe_ep_place_routes(None, 4, 8, None, None, None, None, None) == ext.EINVAL


def _wplan(**kw):
    args = dict(quant_modes="nvfp4", source_format="modelopt_nvfp4", activation="silu",
                params_dtype=torch.bfloat16, num_experts=8, hidden_size=1024, intermediate_size=512)
    args.update(kw)
    return fused_moe.plan_weights(**args)


def test_weight_plan_contracts():
    wp = _wplan()
    assert wp.quant_modes == frozenset({"nvfp4"}) and wp.w1_rows == 1024 and wp.w13_layout == "w13"
    assert _wplan(activation="relu2").w1_rows == 512
    assert _wplan(activation="swigluoai_uninterleave").w13_layout == "w31"
    with pytest.raises(ValueError):
        _wplan(source_format="fp4_e8m0_k32")                     # nvfp4 needs a ModelOpt source
    with pytest.raises(ValueError):
        _wplan(activation="gelu")
    assert _wplan(activation="situ").w1_rows == 1024 and _wplan(activation="situ").w13_layout == "w13"
    with pytest.raises(NotImplementedError):
        _wplan(activation="situ", quant_modes="w4a16")          # no W4A16 oracle for situ
    with pytest.raises(ValueError):
        fused_moe.Caps(max_tokens=4, num_topk=1, device="cpu", quant_mode="nvfp4",
                       weight_plan=_wplan(activation="situ"), swiglu_limit=7.0)
    with pytest.raises(ValueError):
        _wplan(hidden_size=1000)
    with pytest.raises(TypeError):
        _wplan(params_dtype=torch.float16)
    mx = _wplan(quant_modes="w4a8_mx", source_format="fp4_e8m0_k32", hidden_size=2880, intermediate_size=2880)
    assert mx.source_format == "fp4_e8m0_k32"


def test_caps_plan_and_required_nbytes_agree(lib):
    wp = _wplan()
    caps = fused_moe.Caps(max_tokens=16, num_topk=2, device="cpu", weight_plan=wp, quant_mode="NVFP4")
    assert caps.quant_mode == "nvfp4" and caps.k == 1024 and caps.n == 512 and caps.weight_E == 8
    plan = fused_moe.plan(caps)
    (spec,) = plan.scratch_specs()
    assert spec.dtype == torch.uint8 and spec.shape == (fused_moe.required_nbytes(caps),)
    assert plan.shapes_and_dtypes() == ((spec.shape, torch.uint8),)
    assert plan.launch_plan.max_m_tiles == 1 + 8
    ep = fused_moe.plan_execution(num_tokens=3, num_topk=caps.num_topk, device="cpu", weight_plan=caps.weight_plan,
                                  quant_mode=caps.quant_mode)
    assert ep.routed_rows == 6 and ep.execution.regime.value == ep.implementation
    with pytest.raises(ValueError):
        fused_moe.Caps(max_tokens=16, num_topk=2, device="cpu", weight_plan=wp, quant_mode="w4a16")
    with pytest.raises(ValueError):
        fused_moe.Caps(max_tokens=16, num_topk=2, device="cpu", weight_plan=wp, quant_mode="nvfp4", swiglu_alpha=2.0)
    oai = fused_moe.Caps(max_tokens=4, num_topk=1, device="cpu", quant_mode="nvfp4",
                         weight_plan=_wplan(activation="swigluoai_uninterleave"))
    assert (oai.swiglu_limit, oai.swiglu_alpha, oai.swiglu_beta) == (7.0, 1.702, 1.0)


def _cpu_experts(wp):
    e, k, i = wp.num_experts, wp.hidden_size, wp.intermediate_size
    return fused_moe.prepare_weights(
        plan=wp, params_dtype=torch.bfloat16,
        w1_fp4=torch.zeros(e, wp.w1_rows, k // 2, dtype=torch.uint8), w2_fp4=torch.zeros(e, k, i // 2, dtype=torch.uint8),
        w1_blockscale=torch.zeros(e, wp.w1_rows, k // 16, dtype=torch.uint8),
        w2_blockscale=torch.zeros(e, k, i // 16, dtype=torch.uint8),
        w1_global_scale=torch.full((e,), 2.0), w2_global_scale=torch.full((e,), 3.0),
        a1_gscale=torch.full((e,), 4.0), a2_gscale=torch.tensor(6.0))


def test_prepare_weights_alphas_and_bind_validation(lib):
    wp = _wplan()
    ex = _cpu_experts(wp)
    assert torch.equal(ex.w1_alphas, torch.full((8,), 0.5)) and torch.equal(ex.w2_alphas, torch.full((8,), 0.5))
    assert ex.w1_fp4.data_ptr() == ex.w1_fp4.data_ptr() and ex.a2_gscale.numel() == 8
    caps = fused_moe.Caps(max_tokens=16, num_topk=2, device="cpu", weight_plan=wp, quant_mode="nvfp4")
    plan = fused_moe.plan(caps)
    scratch = torch.empty(plan.scratch_specs()[0].shape, dtype=torch.uint8)
    x = torch.zeros(16, 1024, dtype=torch.bfloat16)
    ids = torch.zeros(16, 2, dtype=torch.int32)
    w = torch.zeros(16, 2)
    b = fused_moe.bind(plan, scratch=scratch, a=x, experts=ex, topk_weights=w, topk_ids=ids)
    assert b.kernel_workspace.data_ptr() == scratch.data_ptr()         # views only
    assert b.status.data_ptr() == scratch.data_ptr() + int(b.core_layout.status)
    with pytest.raises(RuntimeError):
        fused_moe.run(binding=b)                                         # no CPU path
    with pytest.raises(ValueError):
        fused_moe.bind(plan, scratch=scratch, a=torch.zeros(17, 1024, dtype=torch.bfloat16), experts=ex,
                       topk_weights=torch.zeros(17, 2), topk_ids=torch.zeros(17, 2, dtype=torch.int32))
    with pytest.raises(ValueError):
        fused_moe.bind(plan, scratch=scratch, a=torch.zeros(16, 512, dtype=torch.bfloat16), experts=ex,
                       topk_weights=w, topk_ids=ids)
    with pytest.raises(ValueError):
        fused_moe.bind(plan, scratch=scratch, a=x, experts=ex, topk_weights=torch.zeros(16, 3),
                       topk_ids=torch.zeros(16, 3, dtype=torch.int32))
    with pytest.raises(TypeError):
        fused_moe.bind(plan, scratch=scratch, a=x, experts=ex, topk_weights=w, topk_ids=ids.long())
    with pytest.raises(TypeError):
        fused_moe.bind(plan, scratch=scratch.float(), a=x, experts=ex, topk_weights=w, topk_ids=ids)
    with pytest.raises(ValueError):
        fused_moe.bind(plan, scratch=scratch[:100], a=x, experts=ex, topk_weights=w, topk_ids=ids)
    other = _cpu_experts(_wplan(num_experts=4))
    with pytest.raises(ValueError):
        fused_moe.bind(plan, scratch=scratch, a=x, experts=other, topk_weights=w, topk_ids=ids)
    with pytest.raises(TypeError):
        fused_moe.bind(plan, scratch=scratch, a=x, experts=object(), topk_weights=w, topk_ids=ids)


def test_route_topk_argument_checks():
    lg = torch.zeros(4, 8)
    out = (torch.zeros(4, 2), torch.zeros(4, 2, dtype=torch.int32), torch.zeros(4, 2))
    with pytest.raises(ValueError, match="CUDA"):
        fused_moe.route_topk(lg, *out, renormalize=True)
    with pytest.raises(ValueError, match="int32"):
        fused_moe.route_topk(lg, out[0], out[1].long(), out[2], renormalize=True)
    with pytest.raises(ValueError, match="rank 2"):
        fused_moe.route_topk(lg[0], *out, renormalize=True)
