"""The safetensors loader for ModelOpt NVFP4 experts against direct ``prepare_weights``: a
synthetic checkpoint is written in the export's per-expert naming and read back whole, as an
expert range and as an intermediate shard.  CPU only (the loader is host code)."""

import json

import pytest
import torch

from b12x_b200 import synth
from b12x_b200.moe import checkpoint, fused_moe
from oracle import moe_oracle as O

safetensors_torch = pytest.importorskip("safetensors.torch")

E, K, I = 4, 256, 128
PREFIX = "model.layers.3.mlp.experts"


def _inputs(act="silu"):
    return synth.make_inputs(synth.shape("c1", name="ck", tokens=4, hidden=K, intermediate=I, experts=E,
                                         topk=2, activation=act), seed=21)


def _write(tmp_path, inp, *, gated=True, split=True):
    """The layer as a ModelOpt export: plain (unswizzled) E4M3 scale grids, scalar global and
    input scales per projection, FC1 split into gate and up (synth fuses [up; gate])."""
    tensors = {}
    for e in range(E):
        s1 = O.unswizzle_block_scale(inp.w1_blockscale[e], inp.w1_fp4.shape[1], K // 16)
        s2 = O.unswizzle_block_scale(inp.w2_blockscale[e], K, I // 16)
        parts = {"up_proj": (inp.w1_fp4[e, :I], s1[:I])}
        if gated:
            parts["gate_proj"] = (inp.w1_fp4[e, I:], s1[I:])
        for name, (w, s) in parts.items():
            tensors[f"{PREFIX}.{e}.{name}.weight"] = w.clone()
            tensors[f"{PREFIX}.{e}.{name}.weight_scale"] = s.clone().view(torch.float8_e4m3fn)
            tensors[f"{PREFIX}.{e}.{name}.weight_scale_2"] = inp.w1_global_scale[e].reshape(()).clone()
            tensors[f"{PREFIX}.{e}.{name}.input_scale"] = (1.0 / inp.a1_gscale[e]).reshape(()).clone()
        tensors[f"{PREFIX}.{e}.down_proj.weight"] = inp.w2_fp4[e].clone()
        tensors[f"{PREFIX}.{e}.down_proj.weight_scale"] = s2.clone().view(torch.float8_e4m3fn)
        tensors[f"{PREFIX}.{e}.down_proj.weight_scale_2"] = inp.w2_global_scale[e].reshape(()).clone()
        tensors[f"{PREFIX}.{e}.down_proj.input_scale"] = (1.0 / inp.a2_gscale[e]).reshape(()).clone()
    if not split:
        safetensors_torch.save_file(tensors, str(tmp_path / "model.safetensors"))
        return
    names = sorted(tensors)
    half = len(names) // 2
    wm = {}
    for fi, chunk in enumerate((names[:half], names[half:])):
        fn = f"model-{fi + 1:05d}-of-00002.safetensors"
        safetensors_torch.save_file({n: tensors[n] for n in chunk}, str(tmp_path / fn))
        wm.update({n: fn for n in chunk})
    (tmp_path / "model.safetensors.index.json").write_text(json.dumps({"weight_map": wm}))


def _direct(inp, act="silu", sl=slice(None)):
    e = len(range(E)[sl])
    wp = fused_moe.plan_weights(quant_modes="nvfp4", source_format="modelopt_nvfp4", activation=act,
                                params_dtype=torch.bfloat16, num_experts=e, hidden_size=K, intermediate_size=I)
    return fused_moe.prepare_weights(
        plan=wp, params_dtype=torch.bfloat16, w1_fp4=inp.w1_fp4[sl].contiguous(), w2_fp4=inp.w2_fp4[sl].contiguous(),
        w1_blockscale=inp.w1_blockscale[sl].contiguous(), w2_blockscale=inp.w2_blockscale[sl].contiguous(),
        w1_global_scale=inp.w1_global_scale[sl], w2_global_scale=inp.w2_global_scale[sl],
        a1_gscale=inp.a1_gscale[sl], a2_gscale=inp.a2_gscale[sl])


def _same(a, b):
    for name in ("w1_fp4", "w2_fp4", "w1_blockscale", "w2_blockscale", "w1_blockscale_rows"):
        x, y = getattr(a, name), getattr(b, name)
        assert (x is None) == (y is None), name
        if x is not None:
            assert torch.equal(x.view(torch.uint8).reshape(-1), y.view(torch.uint8).reshape(-1)), name
    for name in ("w1_alphas", "w2_alphas", "a1_gscale", "a2_gscale"):
        assert torch.allclose(getattr(a, name), getattr(b, name), rtol=3e-7, atol=0), name


@pytest.mark.parametrize("split", [False, True])
def test_whole_layer(tmp_path, split):
    inp = _inputs()
    _write(tmp_path, inp, split=split)
    got = checkpoint.load_modelopt_nvfp4_experts(tmp_path, layer_prefix=PREFIX, num_experts=E, device="cpu")
    _same(got, _direct(inp))


def test_expert_range_and_relu2(tmp_path):
    inp = _inputs("relu2")
    _write(tmp_path, inp, gated=False)
    got = checkpoint.load_modelopt_nvfp4_experts(tmp_path, layer_prefix=PREFIX, num_experts=E, device="cpu",
                                                 activation="relu2", expert_range=(1, 3))
    _same(got, _direct(inp, "relu2", slice(1, 3)))
    with pytest.raises(ValueError):
        checkpoint.load_modelopt_nvfp4_experts(tmp_path, layer_prefix=PREFIX, num_experts=E, device="cpu",
                                               activation="relu2", expert_range=(3, 5))


def test_w31_layout_puts_gate_first(tmp_path):
    inp = _inputs()
    _write(tmp_path, inp)
    got = checkpoint.load_modelopt_nvfp4_experts(tmp_path, layer_prefix=PREFIX, num_experts=E, device="cpu",
                                                 w13_layout="w31")
    assert torch.equal(got.w1_fp4[:, :I], inp.w1_fp4[:, I:]) and torch.equal(got.w1_fp4[:, I:], inp.w1_fp4[:, :I])
    # the pair-atom scale tensor does not depend on the order the halves are stored in
    assert torch.equal(got.w1_blockscale, _direct(inp).w1_blockscale)


def test_intermediate_shard(tmp_path):
    inp = _inputs()
    _write(tmp_path, inp)
    half = I // 2
    for rank in (0, 1):
        got = checkpoint.load_modelopt_nvfp4_experts(tmp_path, layer_prefix=PREFIX, num_experts=E, device="cpu",
                                                     intermediate_shard=(rank, 2))
        r = slice(rank * half, (rank + 1) * half)
        assert got.plan.intermediate_size == half
        assert torch.equal(got.w1_fp4[:, :half], inp.w1_fp4[:, :I][:, r])
        assert torch.equal(got.w1_fp4[:, half:], inp.w1_fp4[:, I:][:, r])
        assert torch.equal(got.w2_fp4, inp.w2_fp4[:, :, rank * half // 2:(rank + 1) * half // 2])
        s2 = torch.stack([O.unswizzle_block_scale(inp.w2_blockscale[e], K, I // 16) for e in range(E)])
        got_s2 = torch.stack([O.unswizzle_block_scale(got.w2_blockscale[e], K, half // 16) for e in range(E)])
        assert torch.equal(got_s2, s2[:, :, rank * half // 16:(rank + 1) * half // 16])
    with pytest.raises(ValueError):
        checkpoint.load_modelopt_nvfp4_experts(tmp_path, layer_prefix=PREFIX, num_experts=E, device="cpu",
                                               intermediate_shard=(0, 4))     # 32-wide shards


def test_shared_input_scale_and_missing_tensor(tmp_path):
    inp = _inputs()
    _write(tmp_path, inp)
    got = checkpoint.load_modelopt_nvfp4_experts(tmp_path, layer_prefix=PREFIX, num_experts=E, device="cpu",
                                                 shared_input_scale=True)
    assert torch.allclose(got.a1_gscale, inp.a1_gscale.min().expand(E), rtol=3e-7, atol=0)
    with pytest.raises(KeyError):
        checkpoint.load_modelopt_nvfp4_experts(tmp_path, layer_prefix="model.layers.4.mlp.experts",
                                               num_experts=E, device="cpu")


@pytest.mark.gpu
def test_loaded_layer_runs_like_directly_prepared_weights(tmp_path):
    inp = _inputs()
    _write(tmp_path, inp)
    dev = torch.device("cuda")
    ex = checkpoint.load_modelopt_nvfp4_experts(tmp_path, layer_prefix=PREFIX, num_experts=E, device=dev)
    from tests.gpu_utils import run_layer

    ref = run_layer(inp)
    p = fused_moe.plan(fused_moe.Caps(max_tokens=4, num_topk=2, device=dev, weight_plan=ex.plan, quant_mode="nvfp4"))
    spec = p.scratch_specs()[0]
    scratch = torch.zeros(spec.shape, dtype=spec.dtype, device=dev)
    out = torch.empty(4, K, dtype=torch.bfloat16, device=dev)
    b = fused_moe.bind(p, scratch=scratch, a=inp.x.to(dev), experts=ex, topk_weights=ref.topk_weights.to(dev),
                       topk_ids=ref.topk_ids.to(dev), output=out)
    fused_moe.run(binding=b)
    torch.cuda.synchronize()
    assert torch.equal(out.cpu(), ref.out)
