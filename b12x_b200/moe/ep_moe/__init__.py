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

from ..._lib.meta import OpMeta, Provenance, install_lazy_api

META = OpMeta(
    name="ep_moe",
    group="moe",
    api_style="planned",
    entry_points=("Caps", "Plan", "Binding", "ExpertMap", "plan", "bind", "run", "prepare_expert_map",
                  "is_supported"),
    archs=("sm100a",),
    dtypes=("bf16",),
    recipes=("nvfp4", "w4a8_mx", "w4a16"),
    provenance=Provenance(
        repo="https://github.com/lukealonso/b12x",
        commit="6627d342",
        paths=("b12x/moe/ep_moe/",),
    ),
    test_path="tests/test_ep_moe_facade.py",
)

install_lazy_api(globals(), META)
