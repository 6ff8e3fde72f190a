"""The symmetric int4 `mul` surface (reference: fast_dequant/simple_marlin/test.py) and the f16
scale-free grouped GEMM against the reference's vectors and the CPU oracle."""
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


@pytest.mark.parametrize("tag,gs", [("marlin_g128", 128), ("marlin_g-1", -1)])
def test_quantutils_and_expand_match_reference_vectors(dev, golden, tag, gs):
    """fake_quantize and pack run on the GPU must equal the reference's tensors bit for bit, and the
    expansion kernel must reproduce the reference's dequantized weight exactly (f16 product)."""
    from llm_kernels_b200.fast_dequant.simple_marlin import QuantUtils
    from llm_kernels_b200.fast_dequant.simple_marlin.marlin_cuda import expand
    c = golden.case(tag)
    w = t(c["w"], torch.float16).to(dev)
    ref, q, sc = QuantUtils.fake_quantize(w, gs)
    assert torch.equal(ref.cpu(), t(c["ref"], torch.float16))
    assert torch.equal(q.cpu(), t(c["q"]).int())
    assert torch.equal(sc.cpu(), t(c["scale"], torch.float16))
    pk, ps = QuantUtils.pack(q, sc, gs)
    assert torch.equal(pk.cpu(), t(c["packed"]).int())
    assert torch.equal(ps.cpu(), t(c["packed_scale"], torch.float16))
    K, Nn = w.shape
    full = expand(pk, ps, K, Nn, gs)
    assert torch.equal(full.cpu(), t(c["ref"], torch.float16).t().contiguous())


# (M, N, K, groupsize): the shapes of the reference's own test (test.py:138-157) that keep this
# file's run time short, plus one-group and ragged-M cases
CASES = [(16, 64, 128, 128), (16, 128, 128, 128), (16, 64, 512, 128), (16, 64, 1024, 128),
         (256, 512, 1024, 128), (512, 256, 1024, 128), (1024, 1024, 512, 128), (128, 2048, 1024, 128),
         (256, 512, 1024, 64), (256, 512, 1024, 256), (512, 512, 512, 512), (48, 192, 320, -1)]


@pytest.mark.parametrize("M,N,K,gs", CASES)
def test_mul_matches_dequantized_product(dev, M, N, K, gs):
    from llm_kernels_b200.fast_dequant.simple_marlin import QuantUtils, mul
    g = torch.Generator().manual_seed(M * 7 + N * 3 + K)
    A = (torch.randn(M, K, generator=g) * 0.1).half()
    W = (torch.randn(K, N, generator=g) * 0.1).half()
    ref, q, sc = R.w4a16_fake_quantize_sym(W, gs)
    pk, ps = R.marlin_pack(q, sc, gs)
    pk2, ps2 = QuantUtils.pack(q.to(dev), sc.to(dev), gs)
    assert torch.equal(pk2.cpu(), pk) and torch.equal(ps2.cpu(), ps)
    C = torch.zeros(M, N, dtype=torch.half, device=dev)
    ws = torch.zeros(max(N // 128, 1) * 16, dtype=torch.int32, device=dev)
    if gs == -1:
        ps2 = ps2.view(-1)                     # 1-D scales: the binding's "no groups" form (:70-88)
    mul(A.to(dev), pk2, C, ps2, ws)
    mul(A.to(dev), pk2, C, ps2, ws)            # second call takes the cached expansion
    want = (A.double() @ ref.double())
    got = C.cpu().double()
    # f32 accumulation of exact f16 products, one rounding to f16 at the end
    assert (got - want).abs().max() <= 2.0 ** -11 * want.abs().max() + 1e-6
    # the reference's own acceptance bar (test.py:108, threshold 0.05 on every element)
    assert (got - (A.to(dev) @ ref.to(dev)).cpu().double()).abs().max() < 0.05


def test_mul_rejects_what_the_reference_rejects(dev):
    from llm_kernels_b200.fast_dequant.simple_marlin import mul
    A = torch.zeros(16, 128, dtype=torch.half, device=dev)
    B = torch.zeros(8, 128, dtype=torch.int32, device=dev)
    C = torch.zeros(16, 64, dtype=torch.half, device=dev)
    s = torch.ones(1, 64, dtype=torch.half, device=dev)
    with pytest.raises(RuntimeError, match="divisible by 16"):
        mul(A[:15], B, C[:15], s, None)
    with pytest.raises(RuntimeError, match="torch.float16"):
        mul(A.float(), B, C, s, None)
    with pytest.raises(RuntimeError, match="Scale tensor must be"):
        mul(A, B, C, s.float(), None)
    with pytest.raises(RuntimeError, match="packed INT4"):
        mul(A, B.long(), C, s, None)
    with pytest.raises(RuntimeError, match="N dimension mismatch"):
        mul(A, B, C, torch.ones(1, 32, dtype=torch.half, device=dev), None)
    with pytest.raises(RuntimeError, match="same CUDA device"):
        mul(A, B.cpu(), C, s, None)
    mul(A, B, C, s, None)
    assert torch.equal(C, torch.zeros_like(C))          # q = 0 -> -8 * 1 * 0


def test_grouped_gemm_triton_f16_matches_reference_vector(dev, golden):
    """The reference's f16 scale-free grouped GEMM (moe/group_gemm_kernel.py:442-513 with
    use_fp8_w8a8=False).  Its N = 96 is padded to the 128-column tile of the tcgen05 kernel with
    zero weight rows; the first 96 output columns are compared."""
    from llm_kernels_b200.moe.group_gemm_kernel import grouped_gemm_triton
    c = golden.case("ggemm_fp16")
    a = t(c["a"], torch.float16).to(dev)
    b = t(c["b"], torch.float16)
    bp = torch.zeros(b.shape[0], 128, b.shape[2], dtype=torch.float16)
    bp[:, :96] = b
    seg, widx = t(c["seg_indptr"]).to(dev), t(c["weight_indices"]).to(dev)
    out = torch.zeros(a.shape[0], 128, dtype=torch.float16, device=dev)
    grouped_gemm_triton(a, bp.to(dev), out, b.shape[0], True, seg, widx)
    got = out[:, :96].cpu()
    torch.testing.assert_close(got, t(c["c_triton"], torch.float16), rtol=2e-3, atol=2e-3)
    torch.testing.assert_close(got, R.grouped_gemm_plain(t(c["a"], torch.float16), b, t(c["seg_indptr"]),
                                                         t(c["weight_indices"])), rtol=2e-3, atol=2e-3)
    assert torch.equal(out[:, 96:], torch.zeros_like(out[:, 96:]))
