"""End-to-end parity of the fused MoE layer (single GPU) against the CPU oracle."""
import pytest
import torch

from oracle import restate as R

pytestmark = pytest.mark.gpu


def _oracle_layer(shape, x, ep_size=1, hidden_act="silu"):
    from llm_kernels_b200 import workloads as WL
    W, bias = WL.router_params(shape)
    kw = dict(top_k=shape.top_k, n_group=shape.n_group, topk_group=shape.topk_group,
              scoring_func=shape.scoring)
    b = bias if shape.scoring == "sigmoid" else None
    assert R.gate_margin_fp64(x, W, b, **kw) > 1e-6
    idx, w = R.gate_forward(x, W, b, routed_scaling_factor=shape.scaling, **kw)
    q13, q2 = [], []
    for e in range(shape.experts):
        g, u, d = WL.expert_weights_cpu(shape, e)
        q13.append(R.weight_quant_fp8(torch.cat([g, u], 0)))
        q2.append(R.weight_quant_fp8(d))
    w13 = torch.stack([a for a, _ in q13]); w13s = torch.stack([s for _, s in q13])
    w2 = torch.stack([a for a, _ in q2]); w2s = torch.stack([s for _, s in q2])
    y = R.moe_layer_fp8(x, idx, w, w13, w13s, w2, w2s, ep_size=ep_size, hidden_act=hidden_act)
    return idx, w, y, (w13, w13s, w2, w2s)


def _build_layer(shape, dev, hidden_act="silu"):
    from llm_kernels_b200 import workloads as WL
    from llm_kernels_b200.moe.all2all_moe import DeepseekV3MoE
    cfg = WL.make_config(shape)
    cfg.hidden_act = hidden_act
    layer = DeepseekV3MoE(cfg, device=dev).eval()
    WL.fill_layer_cpu_seeded(layer, shape)
    return layer


def test_layer_config0_matches_oracle():
    """configs[0]: 512 tokens, H 1024, 8 experts, softmax top-2, SwiGLU 2048, fp8 blockwise.
    Routing bit-exact; output within relative Frobenius error 1e-2."""
    from llm_kernels_b200 import workloads as WL
    dev = torch.device("cuda:0")
    shape = WL.CONFIG0
    x = WL.tokens(shape)
    idx, w, y_ref, (w13, w13s, _, _) = _oracle_layer(shape, x)
    layer = _build_layer(shape, dev)
    assert torch.equal(layer.w13_weight.cpu().view(torch.uint8), w13.view(torch.uint8))
    assert torch.equal(layer.w13_weight_scale.cpu(), w13s)
    gi, gw = layer.gate(x.to(dev).view(1, *x.shape))
    ci, cw = R.canonical_rows(idx, w)
    ki, kw = R.canonical_rows(gi.cpu(), gw.cpu())
    assert torch.equal(ki, ci)
    torch.testing.assert_close(kw, cw, rtol=1e-5, atol=1e-6)   # f32 logits summed in another order than the oracle
    y = layer(x.to(dev).view(2, 256, -1))
    layer.check_status()
    assert y.shape == (2, 256, shape.hidden) and y.dtype == torch.bfloat16
    err = R.rel_fro(y.cpu().view(-1, shape.hidden).float(), y_ref.float())
    assert err < 1e-2, err


def test_layer_gelu_activation_matches_oracle():
    """config.hidden_act = "gelu" (the activation switch of reference
    moe/sglang_moe_all_gather_all_reduce.py:374-397): the tanh-GELU of gelu_and_mul_triton_kernel fused into the
    GEMM-1 epilogue, fp8 and w4a16 paths, against the oracle with the same activation."""
    from llm_kernels_b200 import workloads as WL
    from dataclasses import replace
    dev = torch.device("cuda:0")
    shape = replace(WL.CONFIG0, tokens=160, hidden=512, inter=256, seed=61)
    x = WL.tokens(shape)
    _, _, y_ref, _ = _oracle_layer(shape, x, hidden_act="gelu")
    _, _, y_silu, _ = _oracle_layer(shape, x)
    assert R.rel_fro(y_ref.float(), y_silu.float()) > 0.05          # the two activations differ visibly here
    layer = _build_layer(shape, dev, hidden_act="gelu")
    y = layer(x.to(dev).view(1, shape.tokens, -1))
    layer.check_status()
    assert R.rel_fro(y.cpu().view(shape.tokens, -1).float(), y_ref.float()) < 1e-2
    # w4a16 path (bf16 GEMM-1 with the GELU epilogue)
    shape2 = replace(WL.CONFIG2, tokens=120, hidden=512, inter=256)
    x2, idx, w = _seeded_router_and_tokens(shape2)
    qs = [[], [], [], [], [], []]
    for e in range(shape2.experts):
        g, u, d = WL.expert_weights_cpu(shape2, e)
        q, s_, z = R.w4a16_quantize_asym(torch.cat([g, u], 0))
        qs[0].append(q); qs[1].append(s_); qs[2].append(z)
        q, s_, z = R.w4a16_quantize_asym(d)
        qs[3].append(q); qs[4].append(s_); qs[5].append(z)
    y_ref2 = R.moe_layer_w4a16(x2, idx, w, *[torch.stack(v) for v in qs], hidden_act="gelu")
    layer2 = _build_layer(shape2, dev, hidden_act="gelu")
    y2 = layer2.triton_group_gemm_moe_infer(x2.to(dev), idx.to(dev), w.to(dev))
    layer2.check_status()
    assert R.rel_fro(y2.cpu().float(), y_ref2.float()) < 3e-3


@pytest.mark.parametrize("T", [1, 3, 127, 129])
def test_layer_small_token_counts(T):
    """Ragged sizes: most experts get zero or a handful of rows."""
    from llm_kernels_b200 import workloads as WL
    from dataclasses import replace
    dev = torch.device("cuda:0")
    shape = replace(WL.CONFIG0, tokens=T, hidden=256, inter=256, seed=40 + T)
    x = WL.tokens(shape)
    _, _, y_ref, _ = _oracle_layer(shape, x)
    layer = _build_layer(shape, dev)
    y = layer(x.to(dev).view(1, T, -1))
    layer.check_status()
    assert R.rel_fro(y.cpu().view(T, -1).float(), y_ref.float()) < 1e-2


def test_layer_dsv3_routing_shape_reduced():
    """configs[3] routing (256 experts, 8 groups keep 4, top-8, popularity bias) at reduced H/I
    so the CPU oracle finishes in seconds."""
    from llm_kernels_b200 import workloads as WL
    from dataclasses import replace
    dev = torch.device("cuda:0")
    shape = replace(WL.CONFIG3, tokens=192, hidden=512, inter=256)
    x = WL.tokens(shape)
    idx, w, y_ref, _ = _oracle_layer(shape, x)
    layer = _build_layer(shape, dev)
    gi, _ = layer.gate(x.to(dev).view(1, *x.shape))
    assert torch.equal(R.canonical_rows(gi.cpu(), w)[0], R.canonical_rows(idx, w)[0])
    y = layer(x.to(dev).view(1, 192, -1))
    layer.check_status()
    assert R.rel_fro(y.cpu().view(192, -1).float(), y_ref.float()) < 1e-2


def test_layer_full_size_properties():
    """configs[3] at full single-GPU width (H 7168, I 2048) with fewer experts: properties that
    need no CPU oracle -- row counts conserve, linearity in the routing weights, and agreement
    with the same formulas evaluated by torch on the device."""
    from llm_kernels_b200 import workloads as WL
    from dataclasses import replace
    dev = torch.device("cuda:0")
    shape = replace(WL.CONFIG3, tokens=1024, experts=32, n_group=4, topk_group=2, top_k=4)
    layer_cfg = WL.make_config(shape)
    from llm_kernels_b200.moe.all2all_moe import DeepseekV3MoE
    layer = DeepseekV3MoE(layer_cfg, device=dev).eval()
    WL.fill_layer_gpu(layer, shape)
    x = WL.tokens(shape, device=dev)
    idx, w = layer.gate(x.view(1, *x.shape))
    y1 = layer.triton_group_gemm_moe_infer(x, idx, w)
    y2 = layer.triton_group_gemm_moe_infer(x, idx, w * 2.0)
    layer.check_status()
    torch.testing.assert_close(y2.float(), 2 * y1.float(), rtol=1e-2, atol=1e-3)   # bf16 rounding only
    # device-side evaluation of the oracle formulas on the same quantized weights
    y_ref = R.moe_layer_fp8(x, idx, w, layer.w13_weight, layer.w13_weight_scale, layer.w2_weight,
                            layer.w2_weight_scale)
    assert R.rel_fro(y1.float(), y_ref.float()) < 1e-2


def _seeded_router_and_tokens(shape):
    from llm_kernels_b200 import workloads as WL
    W, bias = WL.router_params(shape)
    b = bias if shape.scoring == "sigmoid" else None
    x = WL.tokens(shape)
    idx, w = R.gate_forward(x, W, b, top_k=shape.top_k, n_group=shape.n_group, topk_group=shape.topk_group,
                            scoring_func=shape.scoring, routed_scaling_factor=shape.scaling)
    return x, idx, w


def test_layer_w4a16_mixtral_shape_reduced():
    """configs[2] (Mixtral-shape w4a16: 8 experts, softmax top-2, asymmetric int4 g128 with bf16
    scale/zero) at reduced H/I/T.  Output within relative Frobenius error 3e-3."""
    from llm_kernels_b200 import workloads as WL
    from dataclasses import replace
    dev = torch.device("cuda:0")
    shape = replace(WL.CONFIG2, tokens=300, hidden=512, inter=768)
    x, idx, w = _seeded_router_and_tokens(shape)
    qs = [[], [], [], [], [], []]
    for e in range(shape.experts):
        g, u, d = WL.expert_weights_cpu(shape, e)
        q, s, z = R.w4a16_quantize_asym(torch.cat([g, u], 0))
        qs[0].append(q); qs[1].append(s); qs[2].append(z)
        q, s, z = R.w4a16_quantize_asym(d)
        qs[3].append(q); qs[4].append(s); qs[5].append(z)
    y_ref = R.moe_layer_w4a16(x, idx, w, *[torch.stack(v) for v in qs])
    layer = _build_layer(shape, dev)
    assert torch.equal(layer.w13_scale.cpu(), torch.stack(qs[1]))
    y = layer.triton_group_gemm_moe_infer(x.to(dev), idx.to(dev), w.to(dev))
    layer.check_status()
    err = R.rel_fro(y.cpu().float(), y_ref.float())
    assert err < 3e-3, err
    y_full = layer(x.to(dev).view(1, *x.shape))          # through the CUDA router as well
    assert R.rel_fro(y_full.cpu().view(-1, shape.hidden).float(), y_ref.float()) < 3e-3


def test_layer_w4a8_decode_shape_reduced():
    """configs[4] (decode-regime w4a8: 64 tokens, 256 experts top-8, two-level int4 weights, int8
    activations) at reduced H/I.  Output within relative Frobenius error 1e-2."""
    from llm_kernels_b200 import workloads as WL
    from dataclasses import replace
    dev = torch.device("cuda:0")
    shape = replace(WL.CONFIG4, hidden=512, inter=256)
    x, idx, w = _seeded_router_and_tokens(shape)
    w13, w2 = [], []
    for e in range(shape.experts):
        g, u, d = WL.expert_weights_cpu(shape, e)
        w13.append(R.w4a8_weight_quant(torch.cat([g, u], 0)))
        w2.append(R.w4a8_weight_quant(d))
    y_ref = R.moe_layer_w4a8(x, idx, w, w13, w2)
    layer = _build_layer(shape, dev)
    assert torch.equal(layer.w13_qweight.cpu(), torch.stack([a[0] for a in w13]))
    y = layer.triton_group_gemm_moe_infer(x.to(dev), idx.to(dev), w.to(dev))
    layer.check_status()
    err = R.rel_fro(y.cpu().float(), y_ref.float())
    assert err < 1e-2, err


def test_layer_w4a8_out_of_range_scales_take_the_expanded_path():
    """The fused w4a8 GEMM is only exact while (q - z4) * s4 fits int8; a weight whose second-level scales break that
    (none from the reference quantizer does) must be served by the expansion path, whose int8 wrap-around is the
    reference's (quantization/w4a8_kernel.py:362-380: the product is cast to int8)."""
    from llm_kernels_b200 import workloads as WL
    from dataclasses import replace
    dev = torch.device("cuda:0")
    shape = replace(WL.CONFIG4, hidden=512, inter=256)
    x, idx, w = _seeded_router_and_tokens(shape)
    layer = _build_layer(shape, dev)
    assert layer._raw_nibbles_ok("w13") and layer._raw_nibbles_ok("w2")
    y0 = layer.triton_group_gemm_moe_infer(x.to(dev), idx.to(dev), w.to(dev)).clone()
    layer.w4_fused_rows_per_group = 0                       # force expansion: the two paths agree bit for bit
    y1 = layer.triton_group_gemm_moe_infer(x.to(dev), idx.to(dev), w.to(dev)).clone()
    assert torch.equal(y0, y1)
    layer.w4_fused_rows_per_group = 64
    layer.w13_s4[0, 0, 0] = 127                             # (q - z) * 127 leaves int8 for q - z >= 2
    layer.w13_z4[0, 0, 0] = 0
    layer.w13_qweight[0, 0, 0] |= 0xF                       # make sure such a nibble is present
    assert not layer._raw_nibbles_ok("w13")
    y2 = layer.triton_group_gemm_moe_infer(x.to(dev), idx.to(dev), w.to(dev)).clone()
    layer.w4_fused_rows_per_group = 0
    y3 = layer.triton_group_gemm_moe_infer(x.to(dev), idx.to(dev), w.to(dev))
    layer.check_status()
    assert torch.equal(y2, y3)


@pytest.mark.parametrize("n_shared", [1, 2])
def test_layer_with_shared_experts(n_shared):
    """config.n_shared_experts (reference moe/all2all_moe.py:161-165, 182-183): an unquantized bf16
    DeepseekV3MLP of width n_shared * I on every token, added to the routed output in bf16."""
    from llm_kernels_b200 import workloads as WL
    from llm_kernels_b200.moe.all2all_moe import DeepseekV3MoE
    from dataclasses import replace
    dev = torch.device("cuda:0")
    shape = replace(WL.CONFIG0, tokens=200, hidden=512, inter=256, seed=77)
    x = WL.tokens(shape)
    _, _, y_routed, _ = _oracle_layer(shape, x)
    g = torch.Generator().manual_seed(5)
    Is = shape.inter * n_shared
    gw = (torch.randn(Is, shape.hidden, generator=g) * 0.05).to(torch.bfloat16)
    uw = (torch.randn(Is, shape.hidden, generator=g) * 0.05).to(torch.bfloat16)
    dw = (torch.randn(shape.hidden, Is, generator=g) * 0.05).to(torch.bfloat16)
    y_ref = y_routed + R.expert_mlp(x, gw, uw, dw)            # bf16 module arithmetic, as the reference
    cfg = WL.make_config(shape)
    cfg.n_shared_experts = n_shared
    layer = DeepseekV3MoE(cfg, device=dev).eval()
    WL.fill_layer_cpu_seeded(layer, shape)
    layer.load_shared_experts(gw.to(dev), uw.to(dev), dw.to(dev))
    for _ in range(2):
        y = layer(x.to(dev).view(1, shape.tokens, -1))
    layer.check_status()
    shared_only = R.expert_mlp(x, gw, uw, dw).float()
    assert shared_only.norm() > 0.2 * y_routed.float().norm()         # the shared term is not negligible here
    assert R.rel_fro(y.cpu().view(shape.tokens, -1).float(), y_ref.float()) < 1e-2


def test_grouped_gemm_bf16_accumulate_epilogue():
    """epilogue 3: c = bf16(c + bf16(a @ b^T)), bit-exact against the same sum formed by torch."""
    from llm_kernels_b200.moe import group_gemm_kernel as G
    dev = torch.device("cuda:0")
    g = torch.Generator().manual_seed(3)
    M, N, K = 200, 256, 192
    a = torch.randn(M, K, generator=g).to(torch.bfloat16).to(dev)
    b = (torch.randn(1, N, K, generator=g) * 0.1).to(torch.bfloat16).to(dev)
    c0 = torch.randn(M, N, generator=g).to(torch.bfloat16).to(dev)
    seg = torch.tensor([0, M], dtype=torch.int64, device=dev)
    plain = torch.empty(M, N, dtype=torch.bfloat16, device=dev)
    G.grouped_gemm_bf16(a, b, seg, None, plain, epilogue=0)
    c = c0.clone()
    G.grouped_gemm_bf16(a, b, seg, None, c, epilogue=3)
    torch.cuda.synchronize()
    assert torch.equal(c, c0 + plain)


@pytest.mark.parametrize("T,n_shared", [(64, 0), (200, 1)])
def test_layer_cuda_graph_replay_matches_eager(T, n_shared):
    """make_graphed: the captured launch sequence replayed on new inputs gives the eager result bit for bit."""
    from llm_kernels_b200 import workloads as WL
    from llm_kernels_b200.moe.all2all_moe import DeepseekV3MoE
    from dataclasses import replace
    dev = torch.device("cuda:0")
    shape = replace(WL.CONFIG0, tokens=T, hidden=512, inter=256, seed=90 + T)
    cfg = WL.make_config(shape)
    cfg.n_shared_experts = n_shared
    layer = DeepseekV3MoE(cfg, device=dev).eval()
    WL.fill_layer_cpu_seeded(layer, shape)
    if n_shared:
        g = torch.Generator().manual_seed(6)
        Is = shape.inter * n_shared
        layer.load_shared_experts(*[(torch.randn(*s, generator=g) * 0.05).to(torch.bfloat16).to(dev)
                                    for s in ((Is, shape.hidden), (Is, shape.hidden), (shape.hidden, Is))])
    xs = [WL.tokens(shape, rank=i).to(dev).view(1, T, -1) for i in range(3)]
    run = layer.make_graphed(xs[0])
    for x in xs[::-1]:
        y_graph = run(x).clone()
        y_eager = layer(x)
        torch.cuda.synchronize()
        assert torch.equal(y_graph, y_eager)
    layer.check_status()


def test_deepseek_v3_mlp_matches_torch_module():
    """DeepseekV3MLP (reference moe/all2all_moe.py:13-29) as a bf16 module: same parameters, output within
    bf16 rounding of the torch module evaluated on the CPU."""
    from llm_kernels_b200.moe.all2all_moe import DeepseekV3MLP
    from llm_kernels_b200.moe.config import Config
    dev = torch.device("cuda:0")
    cfg = Config()
    torch.manual_seed(11)
    mlp = DeepseekV3MLP(cfg, hidden_size=512, intermediate_size=384).to(torch.bfloat16)
    x = torch.randn(3, 50, 512).to(torch.bfloat16)
    want = R.expert_mlp(x.view(-1, 512), mlp.gate_proj.weight.detach(), mlp.up_proj.weight.detach(),
                        mlp.down_proj.weight.detach())
    got = mlp.to(dev)(x.to(dev))
    assert got.shape == (3, 50, 512) and got.dtype == torch.bfloat16
    assert R.rel_fro(got.cpu().view(-1, 512).float(), want.float()) < 3e-3
