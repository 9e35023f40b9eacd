"""-m gpu: the step in front of the layer -- ``route`` (gate projection + top-k in one launch) and
``run_sparse`` (gate -> top-k -> experts) -- against the reference's known answers
(tests/moe/test_sparse_moe_api.py:152-236, run here on CUDA tensors), against fixtures computed by
the reference's own functions (``tests/golden/routing_gate.npz``) and against the CPU oracle."""

import pytest
import torch

from b12x_b200 import synth
from b12x_b200.moe import fused_moe
from oracle import moe_oracle as O
from tests.gpu_utils import oracle_layer, prepare_experts
from tests.helpers import load_golden, t

pytestmark = pytest.mark.gpu
DEV = torch.device("cuda")


def _bf16_ulp(x: torch.Tensor) -> torch.Tensor:
    return torch.clamp(x.abs().float(), min=2.0 ** -120) * 2.0 ** -7


# ---- the reference's known-answer tests, on the GPU -------------------------------------------
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_route_from_gate_weight_renormalizes(dtype):
    hs = torch.tensor([[1.0, 0.0], [0.0, 1.0]], dtype=dtype, device=DEV)
    gw = torch.tensor([[10.0, 0.0], [0.0, 10.0], [-1.0, -1.0]], dtype=dtype, device=DEV)
    r = fused_moe.route(binding=fused_moe.bind_route(hidden_states=hs, top_k=2, gate_weight=gw))
    assert r.router_logits is not None and r.router_logits.dtype == dtype
    assert r.topk_ids.dtype == torch.int32
    assert r.topk_ids.tolist() == [[0, 1], [1, 0]]
    expected = torch.softmax(torch.tensor([[10.0, 0.0], [10.0, 0.0]]), dim=-1)
    torch.testing.assert_close(r.topk_weights.cpu(), expected)
    assert torch.equal(r.flat_ids, r.topk_ids.view(-1)) and torch.equal(r.flat_weights, r.topk_weights.view(-1))


def test_route_without_renormalize_returns_topk_logits():
    hs = torch.tensor([[1.0, 2.0]], device=DEV)
    lg = torch.tensor([[0.5, 3.0, -4.0]], device=DEV)
    r = fused_moe.route(binding=fused_moe.bind_route(hidden_states=hs, top_k=2, router_logits=lg, renormalize=False))
    assert r.topk_ids.tolist() == [[1, 0]]
    torch.testing.assert_close(r.topk_weights.cpu(), torch.tensor([[3.0, 0.5]]))


def test_route_applies_gate_bias():
    hs = torch.tensor([[1.0, 0.0]], device=DEV)
    gw = torch.tensor([[0.0, 0.0], [1.0, 0.0]], device=DEV)
    gb = torch.tensor([5.0, 0.0], device=DEV)
    r = fused_moe.route(binding=fused_moe.bind_route(hidden_states=hs, top_k=1, gate_weight=gw, gate_bias=gb))
    assert r.topk_ids.tolist() == [[0]]
    torch.testing.assert_close(r.router_logits.cpu(), torch.tensor([[5.0, 1.0]]))


def test_route_argument_errors():
    hs = torch.zeros(2, 4, device=DEV)
    with pytest.raises(ValueError, match="either router_logits or gate_weight"):
        fused_moe.bind_route(hidden_states=hs, top_k=1, gate_weight=torch.zeros(3, 4, device=DEV),
                             router_logits=torch.zeros(2, 3, device=DEV))
    with pytest.raises(ValueError, match="expected router_logits or gate_weight"):
        fused_moe.bind_route(hidden_states=hs, top_k=1)
    with pytest.raises(ValueError, match="top_k must be positive"):
        fused_moe.bind_route(hidden_states=hs, top_k=0, router_logits=torch.zeros(2, 3, device=DEV))
    with pytest.raises(TypeError, match="scratch must be"):
        fused_moe.bind_route(scratch=torch.zeros(8), hidden_states=hs, top_k=1, router_logits=torch.zeros(2, 3))
    with pytest.raises(ValueError, match="hidden-size mismatch"):
        fused_moe.route(binding=fused_moe.bind_route(hidden_states=hs, top_k=1, gate_weight=torch.zeros(3, 5, device=DEV)))
    with pytest.raises(ValueError, match="exceeds num_experts"):
        fused_moe.route(binding=fused_moe.bind_route(hidden_states=hs, top_k=4, gate_weight=torch.zeros(3, 4, device=DEV)))
    with pytest.raises(ValueError, match="CUDA"):
        fused_moe.route(binding=fused_moe.bind_route(hidden_states=hs.cpu(), top_k=1, router_logits=torch.zeros(2, 3)))
    with pytest.raises(TypeError):
        fused_moe.route(binding=object())


# ---- fixtures computed by the reference's own routing functions --------------------------------
@pytest.mark.parametrize("kernel", ["simt", "tc"])
@pytest.mark.parametrize("tag", ["f32", "bf16"])
@pytest.mark.parametrize("bias", [False, True])
@pytest.mark.parametrize("renorm", [True, False])
def test_gate_route_matches_reference_fixture(tag, bias, renorm, kernel):
    if kernel == "tc" and tag != "bf16":
        pytest.skip("the tensor-core gate kernel takes bf16 operands")
    g = load_golden("routing_gate.npz")
    dt = torch.float32 if tag == "f32" else torch.bfloat16
    hs, gw, gb = (t(g[f"gate_{tag}_{n}"], dt).to(DEV) for n in ("hidden", "weight", "gbias"))
    key = f"gate_{tag}{'_bias' if bias else ''}{'' if renorm else '_raw'}"
    ref_logits = t(g[key + "_logits"], dt).float()
    r = fused_moe.route(binding=fused_moe.bind_route(hidden_states=hs, top_k=6, gate_weight=gw,
                                                     gate_bias=gb if bias else None, renormalize=renorm,
                                                     gate_kernel=kernel))
    got = r.router_logits.float().cpu()
    if tag == "f32":
        torch.testing.assert_close(got, ref_logits, rtol=2e-5, atol=2e-5)
    else:
        # bf16 logits: the fixture rounds the biased sum once (the reference's CPU path), the GPU path
        # of the reference and this kernel round the product, then the biased sum; and the fp32 sums
        # differ in order: an ulp of the larger of the two magnitudes
        mag = ref_logits.abs() + (2.0 * gb.float().abs().cpu() if bias else 0.0)
        assert bool(((got - ref_logits).abs() <= mag * 2.0 ** -7 + 1e-3).all())
    # the router on the logits this call stored is exactly the oracle's router
    mode = "softmax_topk" if renorm else "raw"
    _, ids, w = O.route_topk(got, 6, mode=mode)
    assert torch.equal(r.topk_ids.cpu(), ids)
    torch.testing.assert_close(r.topk_weights.cpu(), w, rtol=1e-5, atol=1e-6)
    # and agrees with the reference's selection (torch.topk on the CPU) on every row whose seven
    # largest reference logits are further apart than the two sets of logits differ (bf16 logits
    # tie often; ties go to the larger index here, as in the reference's GPU router, while
    # torch.topk does not promise an order)
    top7 = torch.sort(ref_logits, dim=1, descending=True).values[:, :7]
    gap = (top7[:, :-1] - top7[:, 1:]).min(dim=1).values
    rows = gap > 2.0 * (got - ref_logits).abs().max(dim=1).values
    assert int(rows.sum()) >= (15 if tag == "f32" else 5), int(rows.sum())
    ref_ids = t(g[key + "_ids"])
    assert torch.equal(r.topk_ids.cpu()[rows], ref_ids[rows])


@pytest.mark.parametrize("kernel", ["auto", "simt"])
def test_sigmoid_gate_router_matches_reference_benchmark_function(kernel):
    g = load_golden("routing_gate.npz")
    x, gw, bias = t(g["sig_x"]).to(DEV), t(g["sig_gate"]).to(DEV), t(g["sig_bias"]).to(DEV)
    r = fused_moe.route(binding=fused_moe.bind_route(hidden_states=x, top_k=4, gate_weight=gw, score_func="sigmoid",
                                                     selection_bias=bias, renormalize=True, route_scale=2.5,
                                                     gate_kernel=kernel))
    torch.testing.assert_close(r.router_logits.cpu(), t(g["sig_scores_logits"]), rtol=2e-5, atol=2e-5)
    assert torch.equal(r.topk_ids.cpu(), t(g["sig_ids"]))
    torch.testing.assert_close(r.topk_weights.cpu(), t(g["sig_weights"]), rtol=2e-5, atol=1e-6)


# ---- larger shapes, both kernels, against the oracle's router on torch's own projection ---------
@pytest.mark.parametrize("tokens,hidden,experts,topk,kernel", [
    (300, 2880, 128, 4, "tc"),      # GPT-OSS-shaped gate, 45 k-blocks, ragged last token tile
    (1024, 200, 64, 8, "tc"),       # K tail: 200 = 3 x 64 + 8
    (129, 512, 256, 8, "tc"),       # 256 experts: the widest MMA
    (64, 7168, 256, 8, "simt"),     # DeepSeek-V3-shaped decode gate
    (7, 520, 40, 3, "simt"),        # nothing divides anything
    (1, 7168, 256, 8, "auto"),
])
def test_gate_route_large(tokens, hidden, experts, topk, kernel):
    gen = torch.Generator().manual_seed(tokens + hidden)
    hs = torch.randn(tokens, hidden, generator=gen).to(torch.bfloat16)
    gw = (torch.randn(experts, hidden, generator=gen) * 0.05).to(torch.bfloat16)
    r = fused_moe.route(binding=fused_moe.bind_route(hidden_states=hs.to(DEV), top_k=topk, gate_weight=gw.to(DEV),
                                                     gate_kernel=kernel))
    ref = torch.nn.functional.linear(hs.float(), gw.float())
    got = r.router_logits.float().cpu()
    # half a bf16 ulp for the one rounding, plus the accumulation error of the fp32 sum (the tensor
    # cores' fp32 accumulation is a few 1e-6 of the partial sums' magnitude away from the CPU's)
    ulp = torch.exp2(torch.floor(torch.log2(ref.abs().clamp(min=1e-30))) - 7)
    assert bool(((got - ref).abs() <= 0.51 * ulp + 3e-5 * ref.abs() + 3e-4).all()), (got - ref).abs().max()
    _, ids, w = O.route_topk(got, topk)
    assert torch.equal(r.topk_ids.cpu(), ids)
    torch.testing.assert_close(r.topk_weights.cpu(), w, rtol=1e-5, atol=1e-6)


# ---- scratch-carved buffers, the sparse block, graph capture ------------------------------------
def _sparse_setup(tokens=24, route_in_scratch=True, seed=9):
    shp = synth.shape("c1", name="sparse", tokens=tokens, hidden=256, intermediate=128, experts=8, topk=2)
    inp = synth.make_inputs(shp, seed=seed)
    ex = prepare_experts(inp, DEV)
    caps = fused_moe.Caps(max_tokens=32, num_topk=2, device=DEV, weight_plan=ex.plan, quant_mode="nvfp4",
                          route_num_experts=8 if route_in_scratch else None, route_logits_dtype=torch.bfloat16)
    plan = fused_moe.plan(caps)
    ws = fused_moe.Workspace.allocate(plan)
    gen = torch.Generator().manual_seed(seed)
    gate = (torch.randn(8, 256, generator=gen) * 0.1).to(torch.bfloat16).to(DEV)
    return shp, inp, ex, plan, ws, gate


def test_route_buffers_are_views_of_the_scratch_and_nothing_is_allocated():
    shp, inp, ex, plan, ws, gate = _sparse_setup()
    x = inp.x.to(DEV)
    rb = fused_moe.bind_route(scratch=ws, hidden_states=x, top_k=2, gate_weight=gate)
    fused_moe.route(binding=rb)          # first call loads kernels
    torch.cuda.synchronize()
    before = torch.cuda.memory_allocated()
    r = fused_moe.route(binding=rb)
    torch.cuda.synchronize()
    assert torch.cuda.memory_allocated() == before
    lo, hi = ws.storage.data_ptr(), ws.storage.data_ptr() + plan.layout.route_workspace_nbytes
    for buf in (r.router_logits, r.topk_ids, r.topk_weights):
        assert lo <= buf.data_ptr() < hi
    assert plan.layout.route_workspace_nbytes > 0 and plan.layout.total_nbytes == fused_moe.required_nbytes(plan.caps)


def test_run_sparse_equals_route_bind_run_and_the_oracle():
    shp, inp, ex, plan, ws, gate = _sparse_setup()
    x = inp.x.to(DEV)
    out_sparse, routing = fused_moe.run_sparse(binding=fused_moe.bind_sparse(
        scratch=ws, hidden_states=x, experts=ex, top_k=2, gate_weight=gate, return_routing=True))
    out_sparse = out_sparse.clone()
    ids, w = routing.topk_ids.clone(), routing.topk_weights.clone()
    b = fused_moe.bind(plan, scratch=ws.storage, a=x, experts=ex, topk_weights=w, topk_ids=ids)
    out_run = fused_moe.run(binding=b)
    assert torch.equal(out_sparse, out_run)
    ref, taps = oracle_layer(inp, ids.cpu(), w.cpu())
    rms = taps.out_f32.square().mean().sqrt().item()
    assert (out_sparse.float().cpu() - taps.out_f32).abs().max().item() <= 1e-2 * rms + 2.0 ** -8 * taps.out_f32.abs().max().item()
    # precomputed routing, and the scaling factor (applied to the rounded output, as the
    # reference's in-place multiply does)
    scaled = fused_moe.run_sparse(binding=fused_moe.bind_sparse(
        scratch=ws, hidden_states=x, experts=ex, routing=fused_moe.Routing(topk_weights=w, topk_ids=ids),
        routed_scaling_factor=2.5))
    assert torch.equal(scaled, (out_run.float() * 2.5).to(torch.bfloat16))
    with pytest.raises(ValueError, match="mutually exclusive"):
        fused_moe.bind_sparse(scratch=ws, hidden_states=x, experts=ex, top_k=2,
                              routing=fused_moe.Routing(topk_weights=w, topk_ids=ids))
    with pytest.raises(ValueError, match="top_k is required"):
        fused_moe.bind_sparse(scratch=ws, hidden_states=x, experts=ex, gate_weight=gate)
    with pytest.raises(TypeError, match="scratch must be"):
        fused_moe.bind_sparse(scratch=ws.storage, hidden_states=x, experts=ex, top_k=2, gate_weight=gate)


def test_run_sparse_is_captured_in_a_cuda_graph():
    shp, inp, ex, plan, ws, gate = _sparse_setup()
    x = inp.x.to(DEV).clone()
    out = torch.empty(x.shape[0], 256, dtype=torch.bfloat16, device=DEV)
    sb = fused_moe.bind_sparse(scratch=ws, hidden_states=x, experts=ex, top_k=2, gate_weight=gate, output=out)
    eager = fused_moe.run_sparse(binding=sb).clone()
    torch.cuda.synchronize()
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g):
        fused_moe.run_sparse(binding=sb)
    out.zero_()
    g.replay()
    torch.cuda.synchronize()
    assert torch.equal(out, eager)
    # new tokens in the same buffers
    x.copy_(synth.make_inputs(shp, seed=77).x.to(DEV))
    g.replay()
    torch.cuda.synchronize()
    replayed = out.clone()
    again = fused_moe.run_sparse(binding=sb)
    torch.cuda.synchronize()
    assert torch.equal(replayed, again)


def test_route_without_priced_route_buffers_allocates_but_refuses_under_capture(monkeypatch):
    shp, inp, ex, plan, ws, gate = _sparse_setup(route_in_scratch=False)
    x = inp.x.to(DEV)
    assert plan.layout.route_workspace_nbytes == 0
    rb = fused_moe.bind_route(scratch=ws, hidden_states=x, top_k=2, gate_weight=gate)
    r = fused_moe.route(binding=rb)
    assert r.topk_ids.shape == (x.shape[0], 2)
    # while a graph is being captured there is nowhere to allocate from (the capture state is faked:
    # an exception inside a real capture would leave the stream invalidated for the tests after this)
    monkeypatch.setattr(torch.cuda, "is_current_stream_capturing", lambda: True)
    with pytest.raises(RuntimeError, match="caller-owned scratch"):
        fused_moe.route(binding=rb)
