"""Expert-parallel MoE for REPLICATED inputs (reference ``b12x/moe/ep_moe/__init__.py``,
``_impl.py:1-14``): every rank receives the same activations and the same global top-k routes,
``expert_map`` maps global expert ids to this rank's local weight ids (-1 = not held here), the
layer produces the zero-filled rank-local partial output, and the CALLER sums the partials over the
EP group.  No collective is issued here.  (For the dispatching form, where every rank brings its own
tokens, see ``b12x_b200.moe.ep_peer``.)

    from b12x_b200.moe import ep_moe

    emap    = ep_moe.prepare_expert_map(expert_map_i32, local_num_experts=E_local)
    plan    = ep_moe.plan(ep_moe.Caps(max_tokens=T, num_topk=k, global_num_experts=E, device="cuda",
                                      weight_plan=wplan))
    scratch = torch.empty(plan.scratch_specs()[0].shape, dtype=torch.uint8, device="cuda")
    binding = ep_moe.bind(plan, scratch=scratch, a=x, experts=experts, topk_weights=tw, topk_ids=ti,
                          expert_map=emap, output=out)
    partial = ep_moe.run(binding=binding)
"""

from .api import Binding, Caps, ExpertMap, Plan, bind, is_supported, plan, prepare_expert_map, run

__all__ = ["Caps", "Plan", "Binding", "ExpertMap", "plan", "bind", "run", "prepare_expert_map", "is_supported"]
