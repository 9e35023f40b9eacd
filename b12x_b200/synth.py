"""Seeded synthetic inputs for the five benchmark shapes of the fused MoE layer.

Real checkpoints are not needed to exercise the layer: activations and router logits are
N(0, 1), weights are N(0, 0.02) quantised on the spot with the quantisers the reference library
uses for its own synthetic tests (NVFP4: tests/moe/test_tp_moe_relu2_reference.py:21-41 and
tests/_reference/helpers.py:366-369; MXFP4: benchmarks/benchmark_ds4_moe.py:36-62).  Everything
here is plain torch and runs on whichever device is asked for, so full-size weights can be
produced directly in GPU memory.
"""

from __future__ import annotations

import math
from dataclasses import dataclass, replace

import torch

FP4_MAX = 6.0
E4M3_MAX = 448.0


@dataclass(frozen=True)
class MoEShape:
    name: str
    tokens: int
    hidden: int            # K
    intermediate: int      # I (per expert)
    experts: int
    topk: int
    recipe: str            # "nvfp4" | "w4a16" | "w4a8_mx"
    activation: str = "silu"
    router: str = "softmax_topk"   # "softmax_topk" | "sigmoid"
    route_scale: float = 1.0
    zipf_s: float = 0.0            # > 0: per-expert logit bias so that load follows Zipf(s)
    parallelism: str = "ep"

    @property
    def rows(self) -> int:
        return self.tokens * self.topk

    @property
    def flops(self) -> float:
        """2*K*2I + 2*I*K per routed row (benchmarks/benchmark_ds4_moe.py:102-104)."""
        per_row = 6.0 if self.activation != "relu2" else 4.0
        return per_row * self.hidden * self.intermediate * self.rows

    def expert_weight_bytes(self) -> float:
        """Codes plus block scales of one expert (both projections)."""
        g = 32 if self.recipe == "w4a8_mx" else 16
        n = 3 if self.activation != "relu2" else 2
        return n * self.hidden * self.intermediate * (0.5 + 1.0 / g)


SHAPES = {
    "c1": MoEShape("c1_tiny_nvfp4", 16, 1024, 512, 8, 2, "nvfp4"),
    "c2": MoEShape("c2_dsv3_decode_nvfp4", 64, 7168, 2048, 256, 8, "nvfp4", router="sigmoid", route_scale=2.5),
    "c3": MoEShape("c3_qwen3_prefill_w4a16", 4096, 4096, 1536, 128, 8, "w4a16", parallelism="tp"),
    "c4": MoEShape("c4_mixtral_skew_nvfp4", 8192, 4096, 14336, 8, 2, "nvfp4", zipf_s=1.2),
    "c5": MoEShape("c5_gptoss_w4a8_mx", 16384, 2880, 2880, 128, 4, "w4a8_mx", activation="swigluoai"),
}


SHAPES_RECIPES = ("nvfp4", "w4a16", "w4a8_mx")


def shape(key: str, **overrides) -> MoEShape:
    return replace(SHAPES[key], **overrides)


# ---------------------------------------------------------------------------------------------
# quantisers (device-agnostic torch)
# ---------------------------------------------------------------------------------------------
def _fp4_round(x: torch.Tensor) -> torch.Tensor:
    a = x.abs()
    q = torch.zeros_like(a)
    q = torch.where(a > 0.25, torch.full_like(a, 0.5), q)
    q = torch.where(a >= 0.75, torch.full_like(a, 1.0), q)
    q = torch.where(a > 1.25, torch.full_like(a, 1.5), q)
    q = torch.where(a >= 1.75, torch.full_like(a, 2.0), q)
    q = torch.where(a > 2.5, torch.full_like(a, 3.0), q)
    q = torch.where(a >= 3.5, torch.full_like(a, 4.0), q)
    q = torch.where(a > 5.0, torch.full_like(a, 6.0), q)
    return q * torch.sign(x)


def _fp4_pack(q: torch.Tensor) -> torch.Tensor:
    mag = q.abs()
    code = torch.zeros_like(mag, dtype=torch.uint8)
    for c, m in enumerate((0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0)):
        code = torch.where(mag == m, torch.full_like(code, c), code)
    code = code | ((q < 0).to(torch.uint8) << 3)
    pair = code.reshape(*q.shape[:-1], q.shape[-1] // 2, 2)
    return (pair[..., 0] | (pair[..., 1] << 4)).contiguous()


def swizzle_block_scale(scale: torch.Tensor) -> torch.Tensor:
    """[rows, cols] bytes -> 128x4-swizzled [pad128(rows), pad4(cols)] (b12x/_lib/intrinsics.py:62-82)."""
    rows, cols = scale.shape
    rp, cp = (rows + 127) // 128 * 128, (cols + 3) // 4 * 4
    padded = torch.zeros((rp, cp), dtype=scale.dtype, device=scale.device)
    padded[:rows, :cols] = scale
    return padded.reshape(rp // 128, 4, 32, cp // 4, 4).permute(0, 3, 2, 1, 4).contiguous().reshape(rp, cp)


def quantize_nvfp4_matrix(w: torch.Tensor):
    """One expert matrix [rows, cols] -> (codes u8 [rows, cols/2], swizzled E4M3 bytes, 1/global_scale).

    The global scale is 448*6/amax and every 16-block scale is E4M3(global * amax_block / 6)."""
    rows, cols = w.shape
    w = w.float()
    amax = w.abs().amax()
    g = torch.where(amax > 0, (E4M3_MAX * FP4_MAX) / amax, torch.ones_like(amax))
    blocks = w.view(rows, cols // 16, 16)
    bmax = blocks.abs().amax(dim=-1, keepdim=True)
    scale = (g * (bmax / FP4_MAX)).to(torch.float8_e4m3fn).to(torch.float32)
    out_scale = 1.0 / (scale * (1.0 / g))
    clipped = torch.nan_to_num(torch.clamp(blocks * out_scale, -FP4_MAX, FP4_MAX), nan=0.0)
    codes = _fp4_pack(_fp4_round(clipped.view(rows, cols)))
    sf = swizzle_block_scale(scale.squeeze(-1).to(torch.float8_e4m3fn).view(torch.uint8))
    return codes, sf, (1.0 / g).to(torch.float32)


def quantize_mxfp4_matrix(w: torch.Tensor):
    """One expert matrix -> (codes u8 [rows, cols/2], E8M0 bytes u8 [rows, cols/32])."""
    rows, cols = w.shape
    blocks = w.float().view(rows, cols // 32, 32)
    bmax = blocks.abs().amax(dim=-1, keepdim=True)
    safe = torch.where(bmax > 0, bmax / 6.0, torch.ones_like(bmax))
    exponent = torch.ceil(torch.log2(safe)).clamp(-127, 127)
    byte = torch.where(bmax > 0, exponent + 127, torch.zeros_like(exponent)).to(torch.uint8).squeeze(-1)
    scale = torch.where(bmax > 0, torch.exp2(exponent), torch.zeros_like(exponent))
    q = _fp4_round(torch.where(scale > 0, blocks / scale.clamp(min=1e-30), torch.zeros_like(blocks)))
    return _fp4_pack(q.view(rows, cols)), byte.contiguous()


# ---------------------------------------------------------------------------------------------
# inputs
# ---------------------------------------------------------------------------------------------
@dataclass
class MoEInputs:
    shape: MoEShape
    x: torch.Tensor                  # bf16 [T, K]
    router_logits: torch.Tensor      # f32 [T, E]
    router_bias: torch.Tensor | None
    w1_fp4: torch.Tensor             # u8 [E, w1_rows, K/2]
    w1_blockscale: torch.Tensor      # nvfp4/w4a16: swizzled E4M3 [E, pad128(w1_rows), pad4(K/16)]; mx: E8M0 [E, w1_rows, K/32]
    w1_global_scale: torch.Tensor    # f32 [E]
    w2_fp4: torch.Tensor             # u8 [E, K, I/2]
    w2_blockscale: torch.Tensor
    w2_global_scale: torch.Tensor
    a1_gscale: torch.Tensor          # f32 [E] reciprocal input scales
    a2_gscale: torch.Tensor


def zipf_logit_bias(experts: int, topk: int, s: float, *, seed: int = 1234) -> torch.Tensor:
    """Per-expert bias lam*log(p_e), p_e ~ rank^-s, with lam chosen on a fixed host sample so that
    the realised top-k load shares are closest (L1) to p."""
    p = torch.arange(1, experts + 1, dtype=torch.float64).pow(-s)
    p = p / p.sum()
    g = torch.Generator().manual_seed(seed)
    z = torch.randn(8192, experts, generator=g, dtype=torch.float64)
    best_lam, best_err = 1.0, float("inf")
    for step in range(8, 81):
        lam = step / 16.0
        ids = torch.topk(z + lam * p.log(), topk, dim=-1).indices.reshape(-1)
        share = torch.bincount(ids, minlength=experts).double() / ids.numel()
        err = (share - p).abs().sum().item()
        if err < best_err:
            best_lam, best_err = lam, err
    return (best_lam * p.log()).to(torch.float32)


def make_inputs(shp: MoEShape, *, seed: int = 0, device: str | torch.device = "cpu",
                experts: int | None = None) -> MoEInputs:
    """Seeded inputs for ``shp``.  ``experts`` limits how many experts' weights are built (a rank of
    an expert-parallel group only holds its own)."""
    dev = torch.device(device)
    gen = torch.Generator(device=dev).manual_seed(seed)
    t, k, i, e_all = shp.tokens, shp.hidden, shp.intermediate, shp.experts
    e = e_all if experts is None else experts
    x = torch.randn(t, k, generator=gen, device=dev, dtype=torch.float32).to(torch.bfloat16)
    logits = torch.randn(t, e_all, generator=gen, device=dev, dtype=torch.float32)
    bias = None
    if shp.zipf_s > 0:
        logits = logits + zipf_logit_bias(e_all, shp.topk, shp.zipf_s).to(dev)
    w1_rows = i if shp.activation == "relu2" else 2 * i
    mx = shp.recipe == "w4a8_mx"
    w1 = torch.empty((e, w1_rows, k // 2), dtype=torch.uint8, device=dev)
    w2 = torch.empty((e, k, i // 2), dtype=torch.uint8, device=dev)
    if mx:
        s1 = torch.empty((e, w1_rows, k // 32), dtype=torch.uint8, device=dev)
        s2 = torch.empty((e, k, i // 32), dtype=torch.uint8, device=dev)
    else:
        s1 = torch.empty((e, (w1_rows + 127) // 128 * 128, (k // 16 + 3) // 4 * 4), dtype=torch.uint8, device=dev)
        s2 = torch.empty((e, (k + 127) // 128 * 128, (i // 16 + 3) // 4 * 4), dtype=torch.uint8, device=dev)
    g1 = torch.ones(e, dtype=torch.float32, device=dev)
    g2 = torch.ones(e, dtype=torch.float32, device=dev)
    for ei in range(e):
        wa = torch.randn(w1_rows, k, generator=gen, device=dev, dtype=torch.float32) * 0.02
        wb = torch.randn(k, i, generator=gen, device=dev, dtype=torch.float32) * 0.02
        if mx:
            w1[ei], s1[ei] = quantize_mxfp4_matrix(wa)
            w2[ei], s2[ei] = quantize_mxfp4_matrix(wb)
        else:
            w1[ei], s1[ei], g1[ei] = quantize_nvfp4_matrix(wa)
            w2[ei], s2[ei], g2[ei] = quantize_nvfp4_matrix(wb)
        del wa, wb
    if shp.recipe == "nvfp4":
        # reciprocal input scales: 448*6/amax; x ~ N(0,1) and the intermediate is about
        # silu(g)*u with g,u ~ N(0, 0.02^2 K): both are taken from these analytic amax estimates
        per_e = 1.0 + 0.01 * torch.arange(e, dtype=torch.float32, device=dev)
        a1 = (E4M3_MAX * FP4_MAX / 5.0) * per_e
        sigma = 0.02 * math.sqrt(k)
        a2 = (E4M3_MAX * FP4_MAX / max((4.0 * sigma) ** 2, 1e-3)) * per_e
    else:
        a1 = torch.ones(e, dtype=torch.float32, device=dev)
        a2 = torch.ones(e, dtype=torch.float32, device=dev)
    return MoEInputs(shp, x, logits, bias, w1, s1, g1, w2, s2, g2, a1, a2)


# ---------------------------------------------------------------------------------------------
# sharding of a global problem (what a model loader does for expert / tensor parallelism)
# ---------------------------------------------------------------------------------------------
def unswizzle_block_scale(sw: torch.Tensor, rows: int, cols: int) -> torch.Tensor:
    rp, cp = (rows + 127) // 128 * 128, (cols + 3) // 4 * 4
    u = sw.reshape(-1)[: rp * cp].reshape(rp // 128, cp // 4, 32, 4, 4).permute(0, 3, 2, 1, 4)
    return u.contiguous().reshape(rp, cp)[:rows, :cols]


def slice_experts(inp: MoEInputs, lo: int, hi: int) -> MoEInputs:
    """The experts [lo, hi) of ``inp`` (an expert-parallel rank's share); tokens unchanged."""
    return replace(inp, w1_fp4=inp.w1_fp4[lo:hi].contiguous(), w1_blockscale=inp.w1_blockscale[lo:hi].contiguous(),
                   w1_global_scale=inp.w1_global_scale[lo:hi].contiguous(), w2_fp4=inp.w2_fp4[lo:hi].contiguous(),
                   w2_blockscale=inp.w2_blockscale[lo:hi].contiguous(),
                   w2_global_scale=inp.w2_global_scale[lo:hi].contiguous(),
                   a1_gscale=inp.a1_gscale[lo:hi].contiguous(), a2_gscale=inp.a2_gscale[lo:hi].contiguous())


def slice_intermediate(inp: MoEInputs, rank: int, world: int) -> MoEInputs:
    """Tensor-parallel shard ``rank`` of ``world``: FC1 rows [r*I/n, (r+1)*I/n) of both halves and the
    matching FC2 columns, block scales re-laid for the shard (b12x/moe/__init__.py:3-8)."""
    shp = inp.shape
    i, k = shp.intermediate, shp.hidden
    il = i // world
    lo, hi = rank * il, (rank + 1) * il
    gated = shp.activation != "relu2"
    mx = shp.recipe == "w4a8_mx"
    g = 32 if mx else 16
    e = inp.w1_fp4.shape[0]
    rows1 = [slice(lo, hi), slice(i + lo, i + hi)] if gated else [slice(lo, hi)]
    w1 = torch.cat([inp.w1_fp4[:, r] for r in rows1], dim=1).contiguous()
    w2 = inp.w2_fp4[:, :, lo // 2: hi // 2].contiguous()
    if mx:
        s1 = torch.cat([inp.w1_blockscale[:, r] for r in rows1], dim=1).contiguous()
        s2 = inp.w2_blockscale[:, :, lo // g: hi // g].contiguous()
    else:
        w1_rows = inp.w1_fp4.shape[1]
        s1l, s2l = [], []
        for ei in range(e):
            u1 = unswizzle_block_scale(inp.w1_blockscale[ei], w1_rows, k // g)
            s1l.append(swizzle_block_scale(torch.cat([u1[r] for r in rows1], dim=0).contiguous()))
            u2 = unswizzle_block_scale(inp.w2_blockscale[ei], k, i // g)
            s2l.append(swizzle_block_scale(u2[:, lo // g: hi // g].contiguous()))
        s1, s2 = torch.stack(s1l), torch.stack(s2l)
    return replace(inp, shape=replace(shp, intermediate=il), w1_fp4=w1, w1_blockscale=s1, w2_fp4=w2, w2_blockscale=s2)
