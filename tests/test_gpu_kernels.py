"""Parity of the CUDA kernels (called through the C ABI) against the CPU oracle.
Integer/byte/index results must be bit-exact; floating-point results carry the tolerance
stated at each check."""
import numpy as np
import pytest
import torch

from oracle import restate as R

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def dev():
    assert torch.cuda.is_available(), "GPU tests need a CUDA device"
    import llm_kernels_b200._native as N
    N.lib()
    return torch.device("cuda:0")


def t(a, dtype=None):
    x = torch.from_numpy(np.ascontiguousarray(a))
    return x if dtype is None else x.to(dtype)


# ---------------------------------------------------------------- quantizers
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16, torch.float32])
@pytest.mark.parametrize("shape", [(1, 128), (7, 384), (3, 5, 256), (300, 7168)])
def test_act_quant_fp8_bit_exact(dev, dtype, shape):
    from llm_kernels_b200.quantization import fp8_kernel
    g = torch.Generator().manual_seed(1)
    x = (torch.randn(*shape, generator=g) * 3).to(dtype)
    x.view(-1)[:128] = 0          # an all-zero group: s = 0, y = NaN like the reference
    y, s = fp8_kernel.act_quant(x.to(dev))
    yo, so = R.act_quant_fp8(x)
    assert y.dtype == torch.float8_e4m3fn and s.dtype == torch.float32
    assert torch.equal(s.cpu(), so)
    # 0/0: the sign of the NaN is the platform's (x86 makes 0xff, the GPU 0x7f) -> fold it
    canon = lambda b: torch.where((b & 0x7F) == 0x7F, torch.full_like(b, 0x7F), b)
    assert torch.equal(canon(y.cpu().view(torch.uint8)), canon(yo.view(torch.uint8)))
    assert torch.isnan(y.cpu().float().view(-1)[:128]).all()


def test_act_quant_fp8_rejects_bad_input(dev):
    from llm_kernels_b200.quantization import fp8_kernel
    with pytest.raises(AssertionError):
        fp8_kernel.act_quant(torch.zeros(4, 100, device=dev))
    with pytest.raises(AssertionError):
        fp8_kernel.act_quant(torch.zeros(256, 4, device=dev).t())
    with pytest.raises(RuntimeError):
        fp8_kernel.act_quant(torch.zeros(4, 128))


@pytest.mark.parametrize("shape", [(128, 128), (200, 300), (512, 1024)])
def test_weight_quant_dequant_fp8(dev, shape):
    from llm_kernels_b200.quantization import fp8_kernel
    g = torch.Generator().manual_seed(2)
    w = torch.randn(*shape, generator=g) * 0.02
    q, s = fp8_kernel.weight_quant(w.to(dev))
    qo, so = R.weight_quant_fp8(w)
    assert torch.equal(s.cpu(), so)
    assert torch.equal(q.cpu().view(torch.uint8), qo.view(torch.uint8))
    old = torch.get_default_dtype()
    try:
        torch.set_default_dtype(torch.float32)
        d = fp8_kernel.weight_dequant(q, s)
    finally:
        torch.set_default_dtype(old)
    assert torch.equal(d.cpu(), R.weight_dequant_fp8(qo, so))


@pytest.mark.parametrize("shape", [(128, 128), (200, 300), (512, 1024), (7168, 256)])
@pytest.mark.parametrize("dtype", [torch.float32, torch.float16])
def test_weight_quant_dequant_int8_bit_exact(dev, shape, dtype):
    """int8_kernel.weight_quant / weight_dequant (reference quantization/int8_kernel.py:91-113, 145-170):
    int8 payload, f16 scales and the dequantized weight must equal the oracle bit for bit, edge blocks
    and a half-way value included."""
    from llm_kernels_b200.quantization import int8_kernel
    g = torch.Generator().manual_seed(7)
    w = (torch.randn(*shape, generator=g) * 0.01).to(dtype)
    w[0, 0] = w[:128, :128].abs().max() * (2.5 / 127.0)          # lands on a rounding tie
    q, s = int8_kernel.weight_quant(w.to(dev))
    qo, so = R.weight_quant_int8(w)
    assert s.dtype == torch.float16 and s.shape == so.shape and torch.equal(s.cpu(), so)
    assert q.dtype == torch.int8 and torch.equal(q.cpu(), qo)
    old = torch.get_default_dtype()
    try:
        torch.set_default_dtype(torch.float32)
        d = int8_kernel.weight_dequant(q, s)
    finally:
        torch.set_default_dtype(old)
    assert torch.equal(d.cpu(), R.weight_dequant_int8(qo, so))


@pytest.mark.parametrize("rounding", ["half_away", "floor_half"])
def test_act_quant_int8_bit_exact(dev, rounding):
    from llm_kernels_b200.quantization import int8_kernel
    g = torch.Generator().manual_seed(3)
    x = torch.randn(33, 512, generator=g)
    x[0, :4] = torch.tensor([0.5, -0.5, 1.5, -1.5]) * x[0, :128].abs().max() / 127.0
    y, s = int8_kernel.act_quant(x.to(dev), rounding=rounding)
    yo, so = R.act_quant_int8(x, rounding=rounding)
    assert torch.equal(s.cpu(), so)
    assert torch.equal(y.cpu(), yo)


def test_w4a8_act_quant_matches_reference_vector(dev, golden):
    from llm_kernels_b200.quantization import int8_kernel
    c = golden.case("w4a8")
    y, s = int8_kernel.act_quant(t(c["x"]).to(dev), rounding="floor_half")
    assert torch.equal(y.cpu(), t(c["a8"]))
    assert torch.equal(s.cpu(), t(c["a8s"], torch.float16))


# ---------------------------------------------------------------- bit packing
@pytest.mark.parametrize("nbits,width", [(4, 32), (4, 8), (2, 16), (8, 32), (1, 8)])
def test_bitpack_matches_reference_vectors(dev, golden, nbits, width):
    from llm_kernels_b200.quantization import bitpack
    c = golden.case(f"bitpack_{nbits}_{width}")
    W = t(c["W"]).to(dev)
    pr, e = bitpack.pack_weights_over_rows(W, nbits, width, False)
    pc, _ = bitpack.pack_weights_over_cols(W, nbits, width, False)
    assert e == int(c["e"])
    assert pr.dtype == t(c["rows"]).dtype
    assert torch.equal(pr.cpu(), t(c["rows"])) and torch.equal(pc.cpu(), t(c["cols"]))
    assert torch.equal(bitpack.unpack_over_rows(pr, nbits, W.shape[0]), W)
    assert torch.equal(bitpack.unpack_over_cols(pc, nbits, W.shape[1]), W)


# ---------------------------------------------------------------- router
def _check_router(dev, x, W, bias, k, ng, tg, scoring, scale, ref=None):
    from llm_kernels_b200.moe.all2all_moe import MoEGate
    from llm_kernels_b200.moe.config import Config
    cfg = Config()
    cfg.hidden_size, cfg.n_routed_experts, cfg.num_experts_per_tok = x.shape[1], W.shape[0], k
    cfg.n_group, cfg.topk_group, cfg.routed_scaling_factor, cfg.scoring_func = ng, tg, scale, scoring
    gate = MoEGate(cfg).to(dev).eval()
    gate.weight.data.copy_(W)
    gate.e_score_correction_bias.data.copy_(bias if bias is not None else torch.zeros(W.shape[0]))
    kw = dict(top_k=k, n_group=ng, topk_group=tg, scoring_func=scoring)
    # tokens whose deciding gap (in fp64) is below f32 summation noise are not comparable
    ok = R.gate_margins_fp64(x, W, bias, **kw) > 1e-5
    assert ok.float().mean() > 0.99, "seeded input has too many near-ties; pick another seed"
    idx, w = gate(x.to(dev).unsqueeze(0))
    oi, ow = R.gate_forward(x, W, bias, routed_scaling_factor=scale, **kw)
    assert idx.dtype == torch.int64 and w.dtype == torch.float32
    gi, gw = R.canonical_rows(idx.cpu(), w.cpu())
    ci, cw = R.canonical_rows(oi, ow)
    assert torch.equal(gi[ok], ci[ok]), "top-k index sets must be bit-exact"
    # weights: the logits are f32 sums of up to 7168 exact products taken in another order than the oracle's (here
    # in up to 16 partial sums of tensor-core accumulations); the difference reaches the normalised weight as a few
    # 1e-6 relative (measured: at most 6.2e-6 over the benchmark configurations)
    torch.testing.assert_close(gw[ok], cw[ok], rtol=1e-5, atol=1e-6)
    if ref is not None:
        ri, rw = R.canonical_rows(*ref)
        assert torch.equal(gi[ok], ri[ok])
        torch.testing.assert_close(gw[ok], rw[ok], rtol=1e-5, atol=1e-6)


@pytest.mark.parametrize("case", ["gate_small", "gate_v3", "gate_flat"])
def test_router_matches_reference_vectors(dev, golden, case):
    c = golden.case(case)
    k, ng, tg = (int(v) for v in c["params"])
    _check_router(dev, t(c["x"], torch.bfloat16), t(c["W"]), t(c["bias"]), k, ng, tg, "sigmoid",
                  float(c["scale"]), ref=(t(c["topk_idx"]), t(c["topk_weight"])))


@pytest.mark.parametrize("T,H,E,k,ng,tg,scoring,seed", [
    (512, 1024, 8, 2, 1, 1, "softmax", 0),        # configs[0] router
    (300, 4096, 8, 2, 1, 1, "softmax", 2),        # configs[2] router shape
    (257, 7168, 256, 8, 8, 4, "sigmoid", 3),      # configs[3] router shape (tensor-core path)
    (4096, 7168, 256, 8, 8, 4, "sigmoid", 13),    # configs[3] router at its full token count
    (640, 1024, 128, 6, 4, 2, "softmax", 14),     # tensor-core path, E = 128
    (300, 4096, 8, 2, 1, 1, "softmax", 15),
    (64, 7168, 256, 8, 1, 1, "sigmoid", 4),
    (1, 128, 32, 4, 4, 2, "sigmoid", 5),
    (33, 256, 64, 6, 1, 1, "softmax", 6),
])
def test_router_bit_exact_selection(dev, T, H, E, k, ng, tg, scoring, seed):
    g = torch.Generator().manual_seed(seed)
    x = torch.randn(T, H, generator=g).to(torch.bfloat16)
    W = torch.randn(E, H, generator=g) * 0.02
    bias = torch.rand(E, generator=g) * 0.1 if scoring == "sigmoid" else None
    _check_router(dev, x, W, bias, k, ng, tg, scoring, 2.5 if scoring == "sigmoid" else 1.0)


# ---------------------------------------------------------------- permutation metadata
def _check_prep(dev, ids, E):
    from llm_kernels_b200.moe.group_gemm_kernel import run_moe_ep_preproess
    r, s2d, seg = run_moe_ep_preproess(ids.to(dev), E)
    ro, so, go = R.run_moe_ep_preproess(ids, E)
    assert r.dtype == torch.int64 and s2d.dtype == torch.int32 and seg.dtype == torch.int64
    assert torch.equal(seg.cpu(), go)
    assert torch.equal(s2d.cpu(), so)
    assert torch.equal(r.cpu(), ro)


@pytest.mark.parametrize("case", ["prep_small", "prep_skew", "prep_empty_experts"])
def test_preprocess_matches_reference_vectors(dev, golden, case):
    c = golden.case(case)
    _check_prep(dev, t(c["topk_ids"]), int(c["num_experts"]))


@pytest.mark.parametrize("T,k,E,seed", [(1, 1, 1, 0), (1, 8, 256, 1), (127, 2, 8, 2), (129, 8, 256, 3),
                                        (4096, 8, 256, 4), (8192, 2, 8, 5), (5000, 6, 1000, 6)])
def test_preprocess_bit_exact_random(dev, T, k, E, seed):
    g = torch.Generator().manual_seed(seed)
    ids = torch.rand(T, E, generator=g).topk(k, dim=-1)[1]
    _check_prep(dev, ids, E)


def test_preprocess_all_tokens_one_expert_and_empty(dev):
    _check_prep(dev, torch.full((3000, 1), 5, dtype=torch.int64), 8)
    from llm_kernels_b200.moe.group_gemm_kernel import run_moe_ep_preproess
    r, s2d, seg = run_moe_ep_preproess(torch.zeros((0, 2), dtype=torch.int64, device=dev), 4)
    assert r.numel() == 0 and s2d.numel() == 0 and torch.equal(seg.cpu(), torch.zeros(5, dtype=torch.int64))


# ---------------------------------------------------------------- reorder / activation / combine
@pytest.mark.parametrize("name", ["all", "part"])
def test_reorder_kernels_match_reference_vectors(dev, golden, name):
    from llm_kernels_b200.moe import group_gemm_kernel as G
    c = golden.case(f"reorder_{name}")
    lo, hi = (int(v) for v in c["lohi"])
    ids, s2d = t(c["topk_ids"]).to(dev), t(c["src2dst"]).to(dev)
    x = t(c["x"], torch.float16).to(dev)
    T, k = ids.shape
    H = x.shape[1]
    pre = torch.zeros(T * k, H, dtype=torch.float16, device=dev)
    G.pre_reorder_triton_kernel[(T,)](x, pre, s2d, ids, None, lo, hi, k, H, BLOCK_SIZE=512)
    assert torch.equal(pre.cpu(), t(c["pre"], torch.float16))          # a copy: bit-exact
    gu = t(c["gateup"], torch.float16).to(dev)
    rids = t(c["reorder_topk_ids"]).to(dev)
    for kern, key in ((G.silu_and_mul_triton_kernel, "silu"), (G.gelu_and_mul_triton_kernel, "gelu")):
        out = torch.zeros(gu.shape[0], gu.shape[1] // 2, dtype=torch.float16, device=dev)
        kern[(gu.shape[0],)](gu, out, gu.shape[1], rids, None, lo, hi, BLOCK_SIZE=512)
        # f16 results; exp() differs by an ulp between libraries -> 1 f16 ulp
        torch.testing.assert_close(out.cpu(), t(c[key], torch.float16), rtol=2e-3, atol=1e-4)
    down = t(c["down"], torch.float16).to(dev)
    o = torch.full((T, H), 7.0, dtype=torch.float16, device=dev)
    G.post_reorder_triton_kernel[(T,)](down, o, s2d, ids, t(c["topk_weights"]).to(dev), lo, hi, k, H, BLOCK_SIZE=512)
    # the reference accumulates in f16, the kernel in f32: a few f16 ulps
    torch.testing.assert_close(o.cpu(), t(c["post"], torch.float16), rtol=2e-3, atol=2e-3)
    local = ((ids >= lo) & (ids <= hi)).any(dim=1).cpu()
    assert torch.all(o.cpu()[~local] == 0)


def test_pre_reorder_with_expert_scales_to_fp8(dev):
    from llm_kernels_b200.moe import group_gemm_kernel as G
    g = torch.Generator().manual_seed(7)
    T, k, E, H = 50, 4, 16, 256
    x = torch.randn(T, H, generator=g).to(torch.bfloat16)
    ids = torch.rand(T, E, generator=g).topk(k, dim=-1)[1]
    sc = torch.rand(8, generator=g) * 0.05 + 0.01
    _, s2d, _ = R.run_moe_ep_preproess(ids, E)
    out = torch.zeros(T * k, H, dtype=torch.float8_e4m3fn, device=dev)
    G.pre_reorder_triton_kernel[(T,)](x.to(dev), out, s2d.to(dev), ids.to(dev), sc.to(dev), 4, 11, k, H, BLOCK_SIZE=512)
    oo = R.pre_reorder(x, s2d, ids, sc, 4, 11, torch.zeros(T * k, H, dtype=torch.float8_e4m3fn))
    assert torch.equal(out.cpu().view(torch.uint8), oo.view(torch.uint8))


@pytest.mark.parametrize("T,k,E,H,lo,hi", [(64, 2, 8, 1024, 0, 7), (100, 8, 256, 7168, 0, 255),
                                           (37, 4, 16, 384, 4, 11), (5, 1, 4, 128, 0, 3)])
def test_permute_quant_fp8_bit_exact(dev, T, k, E, H, lo, hi):
    from llm_kernels_b200.moe import group_gemm_kernel as G
    g = torch.Generator().manual_seed(11)
    x = torch.randn(T, H, generator=g).to(torch.bfloat16)
    ids = torch.rand(T, E, generator=g).topk(k, dim=-1)[1]
    _, s2d, _ = R.run_moe_ep_preproess(ids, E)
    rec = (H + H // 32 + 15) // 16 * 16
    buf = torch.full((T * k, rec), 0xAB, dtype=torch.uint8, device=dev)
    q, s = buf[:, :H], buf[:, H:H + H // 32].view(torch.float32)
    G.permute_quant_fp8(x.to(dev), s2d.to(dev), ids.to(dev), lo, hi, q, s)
    xq, xs = R.act_quant_fp8(x)
    local = ((ids >= lo) & (ids <= hi)).reshape(-1)
    tok = torch.arange(T * k) // k
    rows = s2d.long()[local]
    assert torch.equal(q.cpu()[rows], xq.view(torch.uint8)[tok[local]])
    assert torch.equal(s.cpu()[rows], xs[tok[local]])
    untouched = torch.ones(T * k, dtype=torch.bool)
    untouched[rows] = False
    assert torch.all(buf.cpu()[untouched] == 0xAB), "non-local rows must not be written"


# ---------------------------------------------------------------- fp8 blockwise GEMM (tcgen05)
def _quant_ab(M, N, K, seed):
    g = torch.Generator().manual_seed(seed)
    a = torch.randn(M, K, generator=g).to(torch.bfloat16)
    b = torch.randn(N, K, generator=g) * 0.02
    aq, a_s = R.act_quant_fp8(a)
    bq, b_s = R.weight_quant_fp8(b)
    return aq, a_s, bq, b_s


@pytest.mark.parametrize("M,N,K", [(128, 256, 128), (128, 256, 512), (16, 256, 256), (1, 128, 128),
                                   (300, 384, 1024), (130, 1024, 7168), (1024, 512, 2048)])
@pytest.mark.parametrize("out_dtype", [torch.bfloat16])
def test_fp8_gemm_dense(dev, M, N, K, out_dtype):
    from llm_kernels_b200.quantization import fp8_kernel
    aq, a_s, bq, b_s = _quant_ab(M, N, K, 1)
    c = fp8_kernel.fp8_gemm(aq.to(dev), a_s.to(dev), bq.to(dev), b_s.to(dev), out_dtype=out_dtype)
    torch.cuda.synchronize()
    ref = R.fp8_gemm(aq, a_s, bq, b_s, out_dtype=torch.float32)
    # same quantized operands, f32 accumulation in a different order, bf16 output rounding
    assert R.rel_fro(c.cpu().float(), ref) < 3e-3
    torch.testing.assert_close(c.cpu().float(), ref, rtol=2e-2, atol=2e-2 * float(ref.abs().max()))


@pytest.mark.parametrize("M,N,K,ks", [(16, 512, 2048, 8), (128, 1024, 7168, 5), (100, 256, 1024, 3)])
def test_fp8_gemm_split_k(dev, M, N, K, ks):
    """Small-M products split the K loop over several sets of tiles (f32 partials added in split order):
    same result as the unsplit kernel up to f32 summation order."""
    from llm_kernels_b200.quantization import fp8_kernel
    aq, a_s, bq, b_s = _quant_ab(M, N, K, 3)
    d = [x.to(dev) for x in (aq, a_s, bq, b_s)]
    one = fp8_kernel.fp8_gemm(*d, out_dtype=torch.float32, ksplits=1)
    split = fp8_kernel.fp8_gemm(*d, out_dtype=torch.float32, ksplits=ks)
    auto = fp8_kernel.fp8_gemm(*d, out_dtype=torch.bfloat16)
    torch.cuda.synchronize()
    ref = R.fp8_gemm(aq, a_s, bq, b_s, out_dtype=torch.float32)
    assert R.rel_fro(split.cpu(), one.cpu()) < 1e-6
    assert R.rel_fro(split.cpu(), ref) < 1e-5
    assert R.rel_fro(auto.cpu().float(), ref) < 3e-3
    with pytest.raises(AssertionError):
        fp8_kernel.fp8_gemm(*d, out_dtype=torch.float32, ksplits=K // 128 + 1)     # an empty split


@pytest.mark.parametrize("out_dtype", [torch.float32, torch.float16])
def test_fp8_gemm_dense_out_dtypes(dev, out_dtype):
    from llm_kernels_b200.quantization import fp8_kernel
    aq, a_s, bq, b_s = _quant_ab(200, 256, 384, 2)
    c = fp8_kernel.fp8_gemm(aq.to(dev), a_s.to(dev), bq.to(dev), b_s.to(dev), out_dtype=out_dtype)
    ref = R.fp8_gemm(aq, a_s, bq, b_s, out_dtype=torch.float32)
    tol = 1e-5 if out_dtype == torch.float32 else 1e-3
    assert R.rel_fro(c.cpu().float(), ref) < tol


def test_fp8_gemm_matches_reference_vector(dev, golden):
    from llm_kernels_b200.quantization import fp8_kernel
    c = golden.case("fp8_gemm")
    a = t(c["a"]).view(torch.float8_e4m3fn).to(dev)
    b = t(c["b"]).view(torch.float8_e4m3fn).to(dev)
    out = fp8_kernel.fp8_gemm(a, t(c["a_s"]).to(dev), b, t(c["b_s"]).to(dev), out_dtype=torch.float32)
    assert R.rel_fro(out.cpu(), t(c["c"])) < 1e-5


def _grouped_case(seed, counts, N, K, W, widx=None):
    g = torch.Generator().manual_seed(seed)
    M = int(sum(counts))
    a = torch.randn(max(M, 1), K, generator=g).to(torch.bfloat16)[:M]
    b = torch.randn(W, N, K, generator=g) * 0.02
    aq, a_s = R.act_quant_fp8(a.contiguous()) if M else (torch.zeros(0, K).to(torch.float8_e4m3fn), torch.zeros(0, K // 128))
    qs = [R.weight_quant_fp8(b[i]) for i in range(W)]
    bq = torch.stack([q for q, _ in qs]); b_s = torch.stack([s for _, s in qs])
    seg = torch.zeros(len(counts) + 1, dtype=torch.int64)
    seg[1:] = torch.cumsum(torch.tensor(counts), 0)
    widx = torch.arange(len(counts), dtype=torch.int64) if widx is None else torch.tensor(widx, dtype=torch.int64)
    return aq, a_s, bq, b_s, seg, widx


@pytest.mark.parametrize("counts,N,K,W,widx", [
    ([5, 0, 65, 27], 256, 256, 4, [2, 0, 3, 1]),
    ([128, 128], 256, 128, 2, None),
    ([1, 300, 0, 0, 129, 7], 512, 1024, 6, None),
    ([40] * 16, 384, 512, 4, [i % 4 for i in range(16)]),     # (source rank, expert) runs share weights
])
def test_grouped_gemm_fp8_plain(dev, counts, N, K, W, widx):
    from llm_kernels_b200.moe import group_gemm_kernel as G
    aq, a_s, bq, b_s, seg, wi = _grouped_case(21, counts, N, K, W, widx)
    M = aq.shape[0]
    c = torch.full((M, N), float("nan"), dtype=torch.bfloat16, device=dev)
    status = torch.zeros(1, dtype=torch.int32, device=dev)
    G.grouped_gemm_fp8(aq.to(dev), a_s.to(dev), bq.to(dev), b_s.to(dev), seg.to(dev), wi.to(dev), c,
                       epilogue=0, status_word=status)
    torch.cuda.synchronize()
    assert int(status.item()) == 0
    ref = R.grouped_gemm_blockwise(aq, a_s, bq, b_s, seg, wi, out_dtype=torch.float32)
    assert not torch.isnan(c).any()
    assert R.rel_fro(c.cpu().float(), ref) < 3e-3


def test_grouped_gemm_triton_surface(dev):
    """The reference entry point: unquantized `a` is quantized 1x128 inside the call."""
    from llm_kernels_b200.moe.group_gemm_kernel import grouped_gemm_triton
    g = torch.Generator().manual_seed(5)
    counts = [70, 3, 0, 55]
    M, N, K = sum(counts), 256, 384
    a = torch.randn(M, K, generator=g).to(torch.bfloat16)
    b = torch.randn(4, N, K, generator=g) * 0.02
    qs = [R.weight_quant_fp8(b[i]) for i in range(4)]
    bq = torch.stack([q for q, _ in qs]); b_s = torch.stack([s for _, s in qs])
    seg = torch.tensor([0, 70, 73, 73, 128], dtype=torch.int64)
    widx = torch.arange(4, dtype=torch.int64)
    c = torch.zeros(M, N, dtype=torch.bfloat16, device=dev)
    grouped_gemm_triton(a.to(dev), bq.to(dev), c, 4, True, seg.to(dev), widx.to(dev), False, None,
                        b_s.to(dev), block_shape=[128, 128])
    aq, a_s = R.act_quant_fp8(a)
    ref = R.grouped_gemm_blockwise(aq, a_s, bq, b_s, seg, widx, out_dtype=torch.float32)
    assert R.rel_fro(c.cpu().float(), ref) < 3e-3


def test_grouped_gemm_runner_surface(dev):
    """GroupedGemmRunner(device).forward(...) (reference moe/sglang_moe_all_gather_all_reduce.py:25-55) gives what
    grouped_gemm_triton gives for the same arguments."""
    from llm_kernels_b200.moe.sglang_moe_all_gather_all_reduce import GroupedGemmRunner
    from llm_kernels_b200.moe.group_gemm_kernel import grouped_gemm_triton
    g = torch.Generator().manual_seed(9)
    a = torch.randn(100, 256, generator=g).to(torch.float16).to(dev)
    b = (torch.randn(3, 128, 256, generator=g) * 0.05).to(torch.float16).to(dev)
    seg = torch.tensor([0, 40, 40, 100], dtype=torch.int64, device=dev)
    widx = torch.arange(3, dtype=torch.int64, device=dev)
    c1 = torch.zeros(100, 128, dtype=torch.float16, device=dev)
    c2 = torch.zeros_like(c1)
    out = GroupedGemmRunner(dev)(a, b, c1, 3, True, seg, widx)
    grouped_gemm_triton(a, b, c2, 3, True, seg, widx)
    assert out is c1 and torch.equal(c1, c2)
    ref = R.grouped_gemm_plain(a.cpu(), b.cpu(), seg.cpu(), widx.cpu(), out_dtype=torch.float32)
    assert R.rel_fro(c1.cpu().float(), ref) < 2e-3


@pytest.mark.parametrize("act", ["silu", "gelu"])
@pytest.mark.parametrize("counts,I,K,W", [([5, 0, 65, 27], 128, 256, 4), ([200, 130], 256, 512, 2),
                                          ([33] * 8, 384, 1024, 8)])
def test_grouped_gemm_fp8_swiglu_epilogue(dev, counts, I, K, W, act):
    from llm_kernels_b200.moe import group_gemm_kernel as G
    aq, a_s, bq, b_s, seg, wi = _grouped_case(31, counts, 2 * I, K, W)
    M = aq.shape[0]
    hq = torch.zeros(M, I, dtype=torch.uint8, device=dev)
    hs = torch.zeros(M, I // 128, dtype=torch.float32, device=dev)
    G.grouped_gemm_fp8(aq.to(dev), a_s.to(dev), bq.to(dev), b_s.to(dev), seg.to(dev), wi.to(dev), hq, hs,
                       epilogue=1 if act == "silu" else 4)
    torch.cuda.synchronize()
    gu = R.grouped_gemm_blockwise(aq, a_s, bq, b_s, seg, wi, out_dtype=torch.bfloat16)
    h = torch.empty(M, I, dtype=torch.bfloat16)
    (R.silu_and_mul if act == "silu" else R.gelu_and_mul)(gu, torch.zeros(M, dtype=torch.long), None, 0, 0, h)
    ho, so = R.act_quant_fp8(h)
    got = hq.cpu().view(torch.float8_e4m3fn).float() * hs.cpu().repeat_interleave(128, 1)
    want = ho.float() * so.repeat_interleave(128, 1)
    # e4m3 outputs: a different f32 summation order can flip a bf16 rounding and then an
    # e4m3 rounding for a handful of elements -> compare dequantized values (rel. Frobenius)
    assert R.rel_fro(got, want) < 5e-3
    torch.testing.assert_close(hs.cpu(), so, rtol=1e-2, atol=0)
    assert float((hq.cpu() != ho.view(torch.uint8)).float().mean()) < 0.01


@pytest.mark.parametrize("kind", ["fp8", "int8"])
def test_quantized_allreduce_kernels_emulated_ranks(dev, kind):
    """The device pieces of the quantized all-reduce (reference quant_communication/quant_all2all_allreduce.py:52-99)
    with 4 ranks emulated on one GPU: quantize every rank's tensor, dequantize + sum each rank's chunk
    (b200moe_dequant_sum), re-quantize, dequantize.  Bit-exact against the oracle's simulation of the scheme,
    all-zero rows included; the int8 result also passes the reference's own allclose(rtol 1e-2, atol 1e-1)."""
    from llm_kernels_b200.moe import group_gemm_kernel as G
    from llm_kernels_b200.quantization import fp8_kernel, w4a8_kernel
    ep, T, H = 4, 40, 512
    g = torch.Generator().manual_seed(77)
    xs = [torch.randn(T, H, generator=g).to(torch.bfloat16) for _ in range(ep)]
    xs[2][5] = 0
    xs[0][17, 128:256] = 0
    quant = fp8_kernel.act_quant if kind == "fp8" else w4a8_kernel.act_quant
    R_ = T // ep
    qs = [quant(x.to(dev)) for x in xs]
    for (q, s_), x in zip(qs, xs):                       # the quantizers themselves against the oracle
        qo, so = R.comm_quant(x, kind)
        assert torch.equal(s_.cpu(), so)
        live = so.repeat_interleave(128, dim=-1) != 0        # all-zero groups: 0/0 payload, decoded as zero anyway
        assert torch.equal(q.cpu().view(torch.uint8)[live], qo.view(torch.uint8)[live])
    chunks = []
    for r in range(ep):
        q = torch.stack([qs[s_][0][r * R_:(r + 1) * R_] for s_ in range(ep)])
        sc = torch.stack([qs[s_][1][r * R_:(r + 1) * R_] for s_ in range(ep)])
        out = torch.empty(R_, H, dtype=torch.bfloat16, device=dev)
        G.dequant_sum(q.contiguous(), sc.contiguous(), out)
        q2, s2 = quant(out)
        fin = torch.empty(R_, H, dtype=torch.bfloat16, device=dev)
        G.dequant_sum(q2.unsqueeze(0), s2.unsqueeze(0), fin)
        chunks.append(fin)
    got = torch.cat(chunks).cpu()
    want = R.quant_allreduce(xs, kind)
    assert torch.equal(got, want)
    exact = sum(x.float() for x in xs)
    if kind == "int8":
        assert torch.allclose(got.float(), exact, rtol=1e-2, atol=1e-1)
    else:
        assert R.rel_fro(got.float(), exact) < 6e-2


# ---------------------------------------------------------------- int4 weight paths
def test_w4a8_weight_quant_expand_and_gemm_match_reference_vectors(dev, golden):
    from llm_kernels_b200.quantization import w4a8_kernel
    c = golden.case("w4a8")
    packed, s, s4, z4 = w4a8_kernel.weight_quant(t(c["w"]).to(dev))
    assert torch.equal(packed.cpu(), t(c["packed"]))
    assert torch.equal(s.cpu(), t(c["s"], torch.float16))
    assert torch.equal(s4.cpu(), t(c["s4"])) and torch.equal(z4.cpu(), t(c["z4"]))
    w8 = w4a8_kernel.expand_int8(packed, s4, z4)
    assert torch.equal(w8.cpu(), R.w4a8_weight_int8(t(c["packed"]), t(c["s4"]), t(c["z4"])))
    deq = w4a8_kernel.weight_dequant(packed, s, s4, z4)
    assert torch.equal(deq.cpu(), t(c["dequant"], torch.float16))
    a8, a8s = w4a8_kernel.act_quant(t(c["x"]).to(dev))
    out = w4a8_kernel.w4a8_gemm(a8, a8s, packed, s, s4, z4, out_dtype=torch.float32)
    # int8 dots are exact; only the f32 accumulation order of the K blocks differs
    assert R.rel_fro(out.cpu(), t(c["c"])) < 1e-6


def _w4a8_case(seed, counts, N, K, W, dev):
    g = torch.Generator().manual_seed(seed)
    M = sum(counts)
    w = [torch.randn(N, K, generator=g) * 0.02 for _ in range(W)]
    qz = [R.w4a8_weight_quant(x) for x in w]                       # (packed, s f16, s4, z4)
    packed = torch.stack([t_[0] for t_ in qz]).to(dev)
    b_s = torch.stack([t_[1].float() for t_ in qz]).to(dev)
    s4 = torch.stack([t_[2] for t_ in qz]).to(dev)
    z4 = torch.stack([t_[3] for t_ in qz]).to(dev)
    x = torch.randn(M, K, generator=g).to(torch.bfloat16)
    a, a_s = R.act_quant_int8(x, rounding="floor_half")
    seg = torch.zeros(len(counts) + 1, dtype=torch.int64); seg[1:] = torch.cumsum(torch.tensor(counts), 0)
    return qz, packed, b_s, s4, z4, a.to(dev), a_s.float().to(dev), seg.to(dev), M


@pytest.mark.parametrize("counts,N,K,W,widx", [([5, 0, 65, 27], 256, 256, 4, None), ([300, 129, 1], 384, 1024, 3, [2, 0, 1]),
                                               ([16] * 12, 512, 2048, 12, None)])
def test_grouped_gemm_w4a8_fused_dequant_plain(dev, counts, N, K, W, widx):
    """The GEMM that converts int4 -> int8 inside the kernel must equal, bit for bit, the expansion kernel followed
    by the int8 grouped GEMM (same int8 operands, same per-K-block f32 promotion), and agree with the oracle's
    w4a8_gemm (reference quantization/w4a8_kernel.py:317-448)."""
    from llm_kernels_b200.moe import group_gemm_kernel as G
    from llm_kernels_b200.quantization import w4a8_kernel
    qz, packed, b_s, s4, z4, a, a_s, seg, M = _w4a8_case(51, counts, N, K, W, dev)
    wi = None if widx is None else torch.tensor(widx, dtype=torch.int64, device=dev)
    for dt in (torch.float32, torch.bfloat16):
        c1 = torch.full((M, N), float("nan"), dtype=dt, device=dev)
        G.grouped_gemm_w4a8(a, a_s, packed, G.pair_scales_t(s4, z4), b_s, seg, wi, c1)
        c2 = torch.full((M, N), float("nan"), dtype=dt, device=dev)
        G.grouped_gemm_i8(a, a_s, w4a8_kernel.expand_int8(packed, s4, z4), b_s, seg, wi, c2)
        torch.cuda.synchronize()
        assert torch.equal(c1, c2)
    segl = seg.tolist()
    for gi in range(len(counts)):
        m0, m1 = segl[gi], segl[gi + 1]
        if m1 > m0:
            e = gi if widx is None else widx[gi]
            ref = R.w4a8_gemm(a[m0:m1].cpu(), a_s[m0:m1].cpu().to(torch.float16), *qz[e], out_dtype=torch.float32)
            assert R.rel_fro(c1[m0:m1].cpu().float(), ref) < 3e-3          # c1 is the bf16 result here


@pytest.mark.parametrize("act", ["silu", "gelu"])
@pytest.mark.parametrize("counts,I,K,W", [([5, 0, 65, 27], 128, 256, 4), ([33] * 8, 256, 1024, 8), ([140, 3], 128, 512, 2)])
def test_grouped_gemm_w4a8_fused_epilogue(dev, counts, I, K, W, act):
    """Fused act(gate)*up + int8 re-quantization epilogue: int8 rows and scales identical to the unfused chain
    (int8 GEMM to bf16, silu/gelu_and_mul, act_quant with floor(v + 0.5))."""
    from llm_kernels_b200.moe import group_gemm_kernel as G
    from llm_kernels_b200.quantization import w4a8_kernel
    qz, packed, b_s, s4, z4, a, a_s, seg, M = _w4a8_case(53, counts, 2 * I, K, W, dev)
    hq = torch.full((M, I), 77, dtype=torch.int8, device=dev)
    hs = torch.full((M, I // 128), -1.0, dtype=torch.float32, device=dev)
    G.grouped_gemm_w4a8(a, a_s, packed, G.pair_scales_t(s4, z4), b_s, seg, None, hq, hs,
                        epilogue=1 if act == "silu" else 4)
    gu = torch.zeros(M, 2 * I, dtype=torch.bfloat16, device=dev)
    G.grouped_gemm_i8(a, a_s, w4a8_kernel.expand_int8(packed, s4, z4), b_s, seg, None, gu)
    h = torch.empty(M, I, dtype=torch.bfloat16, device=dev)
    (G.silu_and_mul_triton_kernel if act == "silu" else G.gelu_and_mul_triton_kernel)[(M,)](gu, h, 2 * I, None, None, 0, 0)
    q, sc = w4a8_kernel.act_quant(h)
    torch.cuda.synchronize()
    # the standalone activation kernel uses expf and an IEEE division, the fused epilogue the fast intrinsics: a bf16
    # rounding can flip for a handful of values
    assert float((hq != q).float().mean()) < 2e-3
    torch.testing.assert_close(hs, sc.float(), rtol=1e-2, atol=0)
    got = hq.float() * hs.repeat_interleave(128, 1)
    want = q.float() * sc.float().repeat_interleave(128, 1)
    assert R.rel_fro(got.cpu(), want.cpu()) < 5e-3


@pytest.mark.parametrize("counts,N,K,W", [([5, 0, 65, 27], 256, 256, 4), ([300, 129], 384, 1024, 2)])
def test_grouped_gemm_i8(dev, counts, N, K, W):
    from llm_kernels_b200.moe import group_gemm_kernel as G
    g = torch.Generator().manual_seed(41)
    M = sum(counts)
    a = torch.randint(-127, 128, (M, K), generator=g, dtype=torch.int32).to(torch.int8)
    b = torch.randint(-119, 120, (W, N, K), generator=g, dtype=torch.int32).to(torch.int8)
    a_s = torch.rand(M, K // 128, generator=g) * 0.01 + 1e-3
    b_s = torch.rand(W, N // 128, K // 128, generator=g) * 0.01 + 1e-3
    seg = torch.zeros(len(counts) + 1, dtype=torch.int64); seg[1:] = torch.cumsum(torch.tensor(counts), 0)
    c = torch.full((M, N), float("nan"), dtype=torch.float32, device=dev)
    G.grouped_gemm_i8(a.to(dev), a_s.to(dev), b.to(dev), b_s.to(dev), seg.to(dev), None, c)
    ref = torch.zeros(M, N)
    for gi in range(len(counts)):
        m0, m1 = int(seg[gi]), int(seg[gi + 1])
        for kb in range(K // 128):
            ks = slice(kb * 128, (kb + 1) * 128)
            d = (a[m0:m1, ks].double() @ b[gi][:, ks].double().t()).float()
            ref[m0:m1] += d * a_s[m0:m1, kb:kb + 1] * b_s[gi].repeat_interleave(128, 0)[:, kb].unsqueeze(0)
    assert R.rel_fro(c.cpu(), ref) < 1e-6


def test_w4a16_quant_expand_and_gemm(dev):
    from llm_kernels_b200.quantization import w4a16_kernel
    g = torch.Generator().manual_seed(43)
    w = torch.randn(384, 512, generator=g) * 0.02
    packed, sc, z = w4a16_kernel.weight_quant(w.to(dev))
    qo, so, zo = R.w4a16_quantize_asym(w)
    assert torch.equal(sc.cpu(), so) and torch.equal(z.cpu(), zo)
    assert torch.equal(packed.cpu(), R.pack_weights_over_cols(qo, 4, 32)[0])
    wd = w4a16_kernel.expand_bf16(packed, sc, z)
    assert torch.equal(wd.cpu(), R.w4a16_dequant(qo, so, zo))           # bit-exact bf16
    a = torch.randn(200, 512, generator=g).to(torch.bfloat16)
    c = w4a16_kernel.w4a16_gemm(a.to(dev), packed, sc, z, out_dtype=torch.float32)
    ref = a.float() @ R.w4a16_dequant(qo, so, zo).float().t()
    # same bf16 operands, f32 accumulation: tolerance of the w4a16 path (3e-3) with a wide margin
    assert R.rel_fro(c.cpu(), ref) < 1e-5


@pytest.mark.parametrize("counts,I,K,W,widx", [([5, 0, 65, 27], 128, 256, 4, None), ([16] * 6, 256, 1024, 6, None),
                                               ([140, 3, 40], 128, 512, 3, [1, 2, 0])])
def test_grouped_gemm_w4a16_fused_dequant(dev, counts, I, K, W, widx):
    """The w4a16 GEMM that dequantizes inside the kernel must equal, bit for bit, the expansion kernel followed by the
    bf16 grouped GEMM, for the plain epilogue and for SiLU(gate)*up / GELU(gate)*up, and agree with the oracle."""
    from llm_kernels_b200.moe import group_gemm_kernel as G
    from llm_kernels_b200.quantization import w4a16_kernel
    g = torch.Generator().manual_seed(59)
    M = sum(counts)
    w = torch.randn(W, 2 * I, K, generator=g) * 0.02
    qs = [w4a16_kernel.weight_quant(w[i].to(dev)) for i in range(W)]
    packed = torch.stack([q[0] for q in qs]); sc = torch.stack([q[1] for q in qs]); zp = torch.stack([q[2] for q in qs])
    pairs = G.pair_scales_t(sc, zp)
    a = torch.randn(M, K, generator=g).to(torch.bfloat16).to(dev)
    seg = torch.zeros(len(counts) + 1, dtype=torch.int64); seg[1:] = torch.cumsum(torch.tensor(counts), 0)
    seg = seg.to(dev)
    wi = None if widx is None else torch.tensor(widx, dtype=torch.int64, device=dev)
    full = w4a16_kernel.expand_bf16(packed, sc, zp)
    for epi, cols, dt in ((0, 2 * I, torch.float32), (0, 2 * I, torch.bfloat16), (2, I, torch.bfloat16), (5, I, torch.bfloat16)):
        c1 = torch.full((M, cols), float("nan"), dtype=dt, device=dev)
        c2 = torch.full((M, cols), float("nan"), dtype=dt, device=dev)
        G.grouped_gemm_w4a16(a, packed, pairs, seg, wi, c1, epilogue=epi)
        G.grouped_gemm_bf16(a, full, seg, wi, c2, epilogue=epi)
        torch.cuda.synchronize()
        assert torch.equal(c1, c2), epi
    ref = R.grouped_gemm_plain(a.cpu(), full.cpu(), seg.cpu(), torch.arange(W) if widx is None else torch.tensor(widx),
                               out_dtype=torch.float32)
    c = torch.zeros(M, 2 * I, dtype=torch.float32, device=dev)
    G.grouped_gemm_w4a16(a, packed, pairs, seg, wi, c)
    assert R.rel_fro(c.cpu(), ref) < 1e-5


@pytest.mark.parametrize("counts,I,K,W", [([5, 0, 65, 27], 128, 256, 4), ([200, 130], 256, 512, 2)])
def test_grouped_gemm_bf16_plain_and_swiglu(dev, counts, I, K, W):
    from llm_kernels_b200.moe import group_gemm_kernel as G
    g = torch.Generator().manual_seed(47)
    M = sum(counts)
    a = torch.randn(M, K, generator=g).to(torch.bfloat16)
    b = (torch.randn(W, 2 * I, K, generator=g) * 0.05).to(torch.bfloat16)
    seg = torch.zeros(len(counts) + 1, dtype=torch.int64); seg[1:] = torch.cumsum(torch.tensor(counts), 0)
    widx = torch.arange(W, dtype=torch.int64)
    ref = R.grouped_gemm_plain(a, b, seg, widx, out_dtype=torch.float32)
    c = torch.zeros(M, 2 * I, dtype=torch.bfloat16, device=dev)
    G.grouped_gemm_bf16(a.to(dev), b.to(dev), seg.to(dev), None, c, epilogue=0)
    assert R.rel_fro(c.cpu().float(), ref) < 3e-3                      # bf16 output rounding
    h = torch.zeros(M, I, dtype=torch.bfloat16, device=dev)
    G.grouped_gemm_bf16(a.to(dev), b.to(dev), seg.to(dev), None, h, epilogue=2)
    want = torch.empty(M, I, dtype=torch.bfloat16)
    R.silu_and_mul(ref.to(torch.bfloat16), torch.zeros(M, dtype=torch.long), None, 0, 0, want)
    assert R.rel_fro(h.cpu().float(), want.float()) < 3e-3
    G.grouped_gemm_bf16(a.to(dev), b.to(dev), seg.to(dev), None, h, epilogue=5)       # GELU(gate) * up
    R.gelu_and_mul(ref.to(torch.bfloat16), torch.zeros(M, dtype=torch.long), None, 0, 0, want)
    assert R.rel_fro(h.cpu().float(), want.float()) < 3e-3
