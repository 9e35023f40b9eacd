"""moe.ep_moe (replicated-input expert parallelism): map validation on CPU, and on a GPU the
identity the reference tests (tests/moe/test_ep_moe.py:60-108): the rank-local partials of two
interleaved expert placements sum to the full layer's output."""

import pytest
import torch

from b12x_b200 import synth
from b12x_b200.moe import ep_moe


def test_expert_map_validation_matches_reference_rules():
    good = torch.tensor([0, -1, 1, -1, 2], dtype=torch.int32)
    m = ep_moe.prepare_expert_map(good, local_num_experts=3, global_num_experts=5)
    assert (m.global_num_experts, m.local_num_experts) == (5, 3)
    m.validate_static()
    with pytest.raises(TypeError):
        ep_moe.prepare_expert_map(good.long(), local_num_experts=3)
    with pytest.raises(ValueError):
        ep_moe.prepare_expert_map(good, local_num_experts=3, global_num_experts=6)
    with pytest.raises(ValueError):      # local id 2 missing
        ep_moe.prepare_expert_map(torch.tensor([0, 1, 1, -1], dtype=torch.int32), local_num_experts=3)
    with pytest.raises(ValueError):      # id out of range
        ep_moe.prepare_expert_map(torch.tensor([0, 3, 1, 2], dtype=torch.int32), local_num_experts=3)
    with pytest.raises(ValueError):
        ep_moe.prepare_expert_map(torch.tensor([0, 1], dtype=torch.int32), local_num_experts=3)
    good[1] = 0                          # mutation after preparation is detected
    with pytest.raises(RuntimeError):
        m.validate_static()


@pytest.mark.gpu
@pytest.mark.parametrize("recipe", ["nvfp4", "w4a16"])
def test_rank_partials_sum_to_the_full_layer(recipe):
    from b12x_b200.moe import fused_moe
    from b12x_b200.moe.distributed import prepare_experts
    from tests.gpu_utils import run_layer

    dev = torch.device("cuda")
    shp = synth.shape("c1", name="epf", tokens=24, hidden=256, intermediate=128, experts=7, topk=3, recipe=recipe)
    full = synth.make_inputs(shp, seed=630)
    ref = run_layer(full, want_fc1=False)
    total = torch.zeros(shp.tokens, shp.hidden, device=dev)
    for rank in range(2):
        gids = list(range(rank, shp.experts, 2))          # interleaved placement
        local = synth.MoEInputs(shp, full.x, full.router_logits, None, full.w1_fp4[gids], full.w1_blockscale[gids],
                                full.w1_global_scale[gids], full.w2_fp4[gids], full.w2_blockscale[gids],
                                full.w2_global_scale[gids], full.a1_gscale[gids], full.a2_gscale[gids])
        ex = prepare_experts(local, dev)
        emap = torch.full((shp.experts,), -1, dtype=torch.int32, device=dev)
        emap[torch.tensor(gids, device=dev)] = torch.arange(len(gids), dtype=torch.int32, device=dev)
        prepared = ep_moe.prepare_expert_map(emap, local_num_experts=len(gids), global_num_experts=shp.experts)
        plan = ep_moe.plan(ep_moe.Caps(max_tokens=shp.tokens, num_topk=shp.topk, global_num_experts=shp.experts,
                                       device=dev, weight_plan=ex.plan))
        spec = plan.scratch_specs()[0]
        scratch = torch.empty(spec.shape, dtype=spec.dtype, device=dev)
        f32 = torch.zeros(shp.tokens, shp.hidden, device=dev)
        b = ep_moe.bind(plan, scratch=scratch, a=full.x.to(dev), experts=ex, topk_weights=ref.topk_weights.to(dev),
                        topk_ids=ref.topk_ids.to(dev), expert_map=prepared, output_f32=f32)
        out = ep_moe.run(binding=b)
        torch.cuda.synchronize()
        fused_moe.check_device_status(b.inner)
        assert out.shape == (shp.tokens, shp.hidden) and out.dtype == torch.bfloat16
        total += f32
    # fp32 partials: the two partial sums differ from the full sum only by fp32 summation order
    scale = ref.out_f32.abs().max().item()
    assert (total.cpu() - ref.out_f32).abs().max().item() <= 1e-5 * scale
