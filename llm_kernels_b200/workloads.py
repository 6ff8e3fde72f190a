"""Seeded synthetic workloads with the shapes and value distributions of the
benchmark configurations (no dataset is involved anywhere in this path).

Inputs are drawn with a torch.Generator seeded by (seed + 1000 * rank).  With
device="cpu" the tensors can be fed to the CPU oracle and copied to the GPU, so
both see identical bits; large benchmark weights are drawn directly on the GPU.
"""
from __future__ import annotations

import math
from dataclasses import dataclass

import torch

from .moe.config import Config


@dataclass
class LayerShape:
    name: str
    tokens: int
    hidden: int
    inter: int
    experts: int
    top_k: int
    n_group: int
    topk_group: int
    scoring: str
    scaling: float
    seed: int
    zipf_bias: float = 0.0       # strength of the popularity bias (0 = none)
    method: str = "fp8_block"    # expert quantization (Config.quantize_method)


# configs[0]: 512 tokens, H 1024, 8 experts top-2 softmax, SwiGLU 2048, fp8 blockwise
CONFIG0 = LayerShape("cfg0_fp8_small", 512, 1024, 2048, 8, 2, 1, 1, "softmax", 1.0, 0)
# configs[3]: DeepSeek-V3 shape, 256 experts top-8 (8 groups, 4 kept), 4096 tokens per rank,
# Zipf(1.1)-skewed expert popularity
CONFIG3 = LayerShape("cfg3_dsv3_fp8", 4096, 7168, 2048, 256, 8, 8, 4, "sigmoid", 2.5, 3, zipf_bias=1.0)


# configs[3] cut down for profiler captures and quick runs: same hidden/intermediate sizes (same
# tiles and K loop), 1/8 of the experts and of the slots -> 1.4 GB of weights (still far above L2)
CONFIG3_SMALL = LayerShape("cfg3_small", 1024, 7168, 2048, 32, 4, 4, 2, "sigmoid", 2.5, 3, zipf_bias=1.0)


# configs[2]: Mixtral shape, 8 experts top-2 softmax, hidden 4096, SwiGLU 14336, w4a16, 8192 tokens/rank
CONFIG2 = LayerShape("cfg2_mixtral_w4a16", 8192, 4096, 14336, 8, 2, 1, 1, "softmax", 1.0, 2, method="w4a16")
# configs[4]: decode regime, 64 tokens/rank, 256 experts top-8, hidden 7168, SwiGLU 2048, w4a8,
# routing uniform over the experts (zero bias, plain top-8 of the sigmoid scores)
CONFIG4 = LayerShape("cfg4_decode_w4a8", 64, 7168, 2048, 256, 8, 1, 1, "sigmoid", 2.5, 4, method="w4a8")


def make_config(shape: LayerShape, ep_size: int = 1) -> Config:
    c = Config()
    c.hidden_size, c.moe_intermediate_size = shape.hidden, shape.inter
    c.n_routed_experts, c.num_experts_per_tok = shape.experts, shape.top_k
    c.n_group, c.topk_group = shape.n_group, shape.topk_group
    c.scoring_func, c.routed_scaling_factor = shape.scoring, shape.scaling
    c.norm_topk_prob, c.n_shared_experts, c.ep_size = True, 0, ep_size
    c.quantize_method = shape.method
    return c


def zipf_bias(shape: LayerShape, gen: torch.Generator) -> torch.Tensor:
    """e_score_correction_bias that skews expert popularity towards Zipf(s=1.1).

    The expert with popularity rank r (0 = most popular) gets
    bias = zipf_bias * 0.08 * (log p_r - log p_last) with p_r ~ (r+1)^-1.1, so the bias is
    non-negative (selection scores stay positive, which keeps the reference's masked_fill(0.0)
    from competing) and the least popular expert gets 0.

    Placement: popularity ranks are dealt in serpentine order over 8 blocks of E/8 consecutive experts
    (the block a rank owns at EP = 8; EP = 2 and 4 own whole blocks), in a seeded random order
    inside each block.  Per-expert load stays Zipf-skewed (ragged groups, hot experts) while the
    blocks carry near-equal totals, as an expert placement balanced across ranks would."""
    E = shape.experts
    blocks = 8 if E % 8 == 0 else 1
    per = E // blocks
    slot = torch.stack([torch.randperm(per, generator=gen) for _ in range(blocks)])   # [block, position]
    r = torch.arange(E)
    blk = torch.where((r // blocks) % 2 == 0, r % blocks, blocks - 1 - r % blocks)
    expert_of_rank = blk * per + slot[blk, r // blocks]
    logp = -1.1 * torch.log(r.float() + 1.0)
    bias = torch.empty(E)
    bias[expert_of_rank] = shape.zipf_bias * 0.08 * (logp - logp.min())
    return bias.float()


def router_params(shape: LayerShape, device="cpu"):
    """Router weight ~N(0, 0.02) [E,H] f32 and the popularity bias (same on every rank)."""
    g = torch.Generator().manual_seed(shape.seed)
    W = torch.randn(shape.experts, shape.hidden, generator=g) * 0.02
    bias = zipf_bias(shape, g) if shape.zipf_bias else torch.zeros(shape.experts)
    return W.to(device), bias.to(device)


def tokens(shape: LayerShape, rank: int = 0, n: int | None = None, device="cpu") -> torch.Tensor:
    """bf16 activations ~N(0,1) [T,H] of one rank."""
    n = shape.tokens if n is None else n
    if torch.device(device).type == "cuda":
        g = torch.Generator(device=device).manual_seed(shape.seed + 1000 * rank + 7)
        return torch.randn(n, shape.hidden, generator=g, device=device, dtype=torch.float32).to(torch.bfloat16)
    g = torch.Generator().manual_seed(shape.seed + 1000 * rank + 7)
    return torch.randn(n, shape.hidden, generator=g).to(torch.bfloat16)


def expert_weights_cpu(shape: LayerShape, expert: int):
    """gate, up [I,H] and down [H,I] ~N(0, 0.02) f32 for one global expert id (CPU)."""
    g = torch.Generator().manual_seed(shape.seed * 100003 + expert + 1)
    gate = torch.randn(shape.inter, shape.hidden, generator=g) * 0.02
    up = torch.randn(shape.inter, shape.hidden, generator=g) * 0.02
    down = torch.randn(shape.hidden, shape.inter, generator=g) * 0.02
    return gate, up, down


def fill_layer_cpu_seeded(layer, shape: LayerShape):
    """Loads CPU-seeded weights into a DeepseekV3MoE (small shapes: parity tests)."""
    W, bias = router_params(shape)
    dev = layer._dev
    layer.gate.weight.data.copy_(W.to(dev))
    layer.gate.e_score_correction_bias.data.copy_(bias.to(dev))
    for le in range(layer.experts_per_rank):
        e = layer.ep_rank * layer.experts_per_rank + le
        g, u, d = expert_weights_cpu(shape, e)
        layer.load_expert(le, g.to(dev), u.to(dev), d.to(dev))


def fill_layer_gpu(layer, shape: LayerShape):
    """Draws ~N(0, 0.02) expert weights on the GPU, expert by expert (benchmark sizes)."""
    W, bias = router_params(shape)
    dev = layer._dev
    layer.gate.weight.data.copy_(W.to(dev))
    layer.gate.e_score_correction_bias.data.copy_(bias.to(dev))
    for le in range(layer.experts_per_rank):
        e = layer.ep_rank * layer.experts_per_rank + le
        g = torch.Generator(device=dev).manual_seed(shape.seed * 100003 + e + 1)
        gu = torch.randn(2 * shape.inter, shape.hidden, generator=g, device=dev) * 0.02
        dn = torch.randn(shape.hidden, shape.inter, generator=g, device=dev) * 0.02
        layer.load_expert(le, gu[: shape.inter], gu[shape.inter:], dn)


def layer_flops(shape: LayerShape, slots: int) -> float:
    """Algorithmic GEMM flops of the expert FFNs for `slots` (token, expert) pairs: 6*H*I*S."""
    return 6.0 * shape.hidden * shape.inter * slots
