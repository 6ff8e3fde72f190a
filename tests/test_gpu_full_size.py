"""Parity at the benchmark configurations' FULL sizes (single GPU) against the CPU oracle.

The layer runs at full size on the GPU; the CPU oracle is evaluated on a token subsample, which is exact
because a token's output depends on no other token (routing, quantization and the expert FFNs are all
per token).  Routing is compared on every token.  The weights the oracle uses are the layer's own
quantized tensors copied to the host, restricted to the experts the subsample reaches.
"""
from dataclasses import replace

import pytest
import torch

from oracle import restate as R

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def _routing_exact(layer, shape, x_cpu):
    """CUDA router against the oracle on all tokens (tokens whose deciding gap in fp64 is below f32
    summation noise are skipped; at least 99 % must be comparable).  Returns the layer's (idx, w) on the
    host and the mask of compared tokens."""
    from llm_kernels_b200 import workloads as WL
    W, bias = WL.router_params(shape)
    b = bias if shape.scoring == "sigmoid" else None
    kw = dict(top_k=shape.top_k, n_group=shape.n_group, topk_group=shape.topk_group, scoring_func=shape.scoring)
    ok = R.gate_margins_fp64(x_cpu, W, b, **kw) > 1e-5
    assert ok.float().mean() > 0.99
    oi, ow = R.gate_forward(x_cpu, W, b, routed_scaling_factor=shape.scaling, **kw)
    gi, gw = layer.gate(x_cpu.to(DEV).view(1, *x_cpu.shape))
    gi, gw = gi.cpu(), gw.cpu()
    ci, cw = R.canonical_rows(oi, ow)
    ki, kw_ = R.canonical_rows(gi, gw)
    assert torch.equal(ki[ok], ci[ok]), "top-k index sets must be bit-exact"
    # weights: two f32 summation orders of a 4096..7168-term dot product differ by ~1e-6 in the logit, which
    # reaches the normalised weight as a few 1e-6 relative
    torch.testing.assert_close(kw_[ok], cw[ok], rtol=1e-5, atol=1e-6)
    # per-expert counts and offsets of the full batch, bit-exact against the oracle's stable sort
    from llm_kernels_b200.moe import group_gemm_kernel as G
    _, s2d, seg = G.run_moe_ep_preproess(gi.to(DEV), shape.experts)
    _, s2d_o, seg_o = R.run_moe_ep_preproess(gi, shape.experts)
    assert torch.equal(seg.cpu(), seg_o) and torch.equal(s2d.cpu(), s2d_o)
    return gi, gw, ok


def _compact(idx_sub):
    """Experts the subsample reaches, and its indices renumbered 0..U-1 (order preserved)."""
    used = torch.unique(idx_sub)
    remap = torch.full((int(used.max()) + 1,), -1, dtype=torch.long)
    remap[used] = torch.arange(used.numel())
    return used, remap[idx_sub]


def test_cfg3_full_size_layer_matches_oracle_on_subsample():
    """configs[3] as benchmarked: 256 experts, top-8 of 4 of 8 groups, 4096 tokens, H 7168, I 2048, e4m3 weights
    with 128x128 scales, Zipf-skewed routing.  Routing, counts and permutation bit-exact on all 4096 tokens;
    output of every 64th token within relative Frobenius error 1e-2 of the oracle."""
    from llm_kernels_b200 import workloads as WL
    from llm_kernels_b200.moe.all2all_moe import DeepseekV3MoE
    shape = WL.CONFIG3
    layer = DeepseekV3MoE(WL.make_config(shape), device=torch.device(DEV)).eval()
    WL.fill_layer_gpu(layer, shape)
    x = WL.tokens(shape)
    gi, gw, ok = _routing_exact(layer, shape, x)
    y = layer(x.to(DEV).view(1, *x.shape)).view(shape.tokens, -1)
    layer.check_status()
    sub = torch.arange(0, shape.tokens, 64)
    used, idx_c = _compact(gi[sub])
    w13 = layer.w13_weight[used.to(DEV)].cpu(); w13s = layer.w13_weight_scale[used.to(DEV)].cpu()
    w2 = layer.w2_weight[used.to(DEV)].cpu(); w2s = layer.w2_weight_scale[used.to(DEV)].cpu()
    y_ref = R.moe_layer_fp8(x[sub], idx_c, gw[sub], w13, w13s, w2, w2s)
    err = R.rel_fro(y[sub.to(DEV)].cpu().float(), y_ref.float())
    assert err < 1e-2, err
    # rows conserve: every (token, expert) slot landed in exactly one group
    assert int(layer.last_recv_rows) == shape.tokens * shape.top_k


def test_cfg2_full_width_w4a16_layer_matches_oracle_on_subsample():
    """configs[2] at its full width on one GPU: 8 experts top-2 softmax, H 4096, I 14336, asymmetric int4 g128,
    8192 tokens.  Routing bit-exact on all tokens; every 256th token within 3e-3 of the oracle."""
    from llm_kernels_b200 import workloads as WL
    from llm_kernels_b200.moe.all2all_moe import DeepseekV3MoE
    shape = WL.CONFIG2
    layer = DeepseekV3MoE(WL.make_config(shape), device=torch.device(DEV)).eval()
    WL.fill_layer_gpu(layer, shape)
    x = WL.tokens(shape)
    gi, gw, ok = _routing_exact(layer, shape, x)
    y = layer(x.to(DEV).view(1, *x.shape)).view(shape.tokens, -1)
    layer.check_status()
    sub = torch.arange(0, shape.tokens, 256)
    H, I = shape.hidden, shape.inter
    unpack = lambda p, cols: R.unpack_over_cols(p.cpu(), 4, cols)
    q13 = torch.stack([unpack(layer.w13_qweight[e], H) for e in range(shape.experts)])
    q2 = torch.stack([unpack(layer.w2_qweight[e], I) for e in range(shape.experts)])
    y_ref = R.moe_layer_w4a16(x[sub], gi[sub], gw[sub], q13, layer.w13_scale.cpu(), layer.w13_zero.cpu(),
                              q2, layer.w2_scale.cpu(), layer.w2_zero.cpu())
    err = R.rel_fro(y[sub.to(DEV)].cpu().float(), y_ref.float())
    assert err < 3e-3, err


def test_cfg4_full_size_w4a8_layer_matches_oracle():
    """configs[4] whole: 64 tokens, 256 experts top-8, H 7168, I 2048, two-level int4 weights, int8 activations.
    Routing bit-exact; output of all 64 tokens within 1e-2 of the oracle."""
    from llm_kernels_b200 import workloads as WL
    from llm_kernels_b200.moe.all2all_moe import DeepseekV3MoE
    shape = WL.CONFIG4
    layer = DeepseekV3MoE(WL.make_config(shape), device=torch.device(DEV)).eval()
    WL.fill_layer_gpu(layer, shape)
    x = WL.tokens(shape)
    gi, gw, ok = _routing_exact(layer, shape, x)
    y = layer(x.to(DEV).view(1, *x.shape)).view(shape.tokens, -1)
    layer.check_status()
    used, idx_c = _compact(gi)
    pick = lambda name, e: getattr(layer, name)[e].cpu()
    w13 = [(pick("w13_qweight", e), pick("w13_weight_scale", e).to(torch.float16), pick("w13_s4", e), pick("w13_z4", e))
           for e in used.tolist()]
    w2 = [(pick("w2_qweight", e), pick("w2_weight_scale", e).to(torch.float16), pick("w2_s4", e), pick("w2_z4", e))
          for e in used.tolist()]
    y_ref = R.moe_layer_w4a8(x, idx_c, gw, w13, w2)
    err = R.rel_fro(y.cpu().float(), y_ref.float())
    assert err < 1e-2, err


@pytest.mark.parametrize("M", [16, 128, 1024, 4096])
def test_cfg1_dense_fp8_gemm_full_shape(M):
    """configs[1]: dense fp8 blockwise GEMM, N = K = 7168, bf16 output, A ~N(0,1) quantized 1x128, B ~N(0,0.02)
    quantized 128x128 (both by the library's own quantizers, which are bit-exact against the oracle's).  The
    oracle evaluates a 128-row x 512-column slice of the product from the same quantized operands; rel. Frobenius
    error below 1e-2 (measured: bf16 output rounding, ~2e-3)."""
    from llm_kernels_b200.quantization import fp8_kernel
    N_, K = 7168, 7168
    g = torch.Generator(device=DEV).manual_seed(1)
    a = torch.randn(M, K, generator=g, device=DEV).to(torch.bfloat16)
    b = torch.randn(N_, K, generator=g, device=DEV) * 0.02
    aq, a_s = fp8_kernel.act_quant(a)
    bq, b_s = fp8_kernel.weight_quant(b)
    old = torch.get_default_dtype()
    try:
        torch.set_default_dtype(torch.bfloat16)
        c = fp8_kernel.fp8_gemm(aq, a_s, bq, b_s)
    finally:
        torch.set_default_dtype(old)
    assert c.shape == (M, N_) and c.dtype == torch.bfloat16
    rows = torch.arange(0, M, max(1, M // 128))[:128]
    for c0 in (0, 3584, N_ - 512):
        ref = R.fp8_gemm(aq[rows.to(DEV)].cpu(), a_s[rows.to(DEV)].cpu(), bq[c0:c0 + 512].cpu(),
                         b_s[c0 // 128:c0 // 128 + 4].cpu(), out_dtype=torch.float32)
        err = R.rel_fro(c[rows.to(DEV), c0:c0 + 512].cpu().float(), ref)
        assert err < 1e-2, (M, c0, err)
