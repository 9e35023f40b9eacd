"""-m gpu: one layer step (routing included) recorded into a CUDA graph gives the eager step's
result bit for bit, on new inputs too (the reference requires its ``run`` to be capture-safe:
README.md:97-100, tests/moe/test_fused_moe.py:85-132)."""

import pytest
import torch

from b12x_b200 import synth
from b12x_b200.moe.distributed import ExpertParallelMoE

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("tokens", [1, 48])
def test_captured_step_equals_eager(tokens):
    dev = torch.device("cuda")
    shp = synth.shape("c2", name="graph", tokens=tokens, hidden=512, intermediate=256, experts=16, topk=4)
    layer = ExpertParallelMoE.from_synthetic(shp, dev, 0, 1)
    assert layer.can_capture
    x, lg = layer.inputs.x.to(dev), layer.inputs.router_logits.to(dev)
    eager = layer.forward(x, lg).clone()
    layer.capture()
    g = torch.Generator().manual_seed(7)
    x2 = torch.randn(x.shape, generator=g).to(torch.bfloat16).to(dev)
    lg2 = torch.randn(lg.shape, generator=g).to(dev)
    eager2 = layer.forward(x2, lg2).clone()
    for xi, li, want in ((x, lg, eager), (x2, lg2, eager2), (x, lg, eager)):
        layer.x_stage.copy_(xi)
        layer.lg_stage.copy_(li)
        layer.out.fill_(float("nan"))
        layer.graph.replay()
        torch.cuda.synchronize()
        assert torch.equal(layer.out, want)
    layer.check_status()
    assert eager.float().abs().max().item() > 0
