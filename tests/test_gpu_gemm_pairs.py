"""The grouped GEMMs with CTA pairs forced on (256-row tiles shared by two SMs) must give the same
results as with single-CTA tiles, for every operand kind and epilogue, on ragged groups whose last
tile leaves the second CTA of a pair with few or no rows."""
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


@pytest.fixture
def modes(dev):
    from llm_kernels_b200.moe import group_gemm_kernel as G

    def run(fn):
        outs = []
        for mode in (0, 1):
            with G.gemm_options(pair_mode=mode):
                outs.append(fn())
                torch.cuda.synchronize()
        return outs
    return run


def _case(seed, counts, N, K, W):
    g = torch.Generator().manual_seed(seed)
    M = int(sum(counts))
    a = torch.randn(M, K, generator=g).to(torch.bfloat16)
    b = torch.randn(W, N, K, generator=g) * 0.02
    aq, a_s = R.act_quant_fp8(a.contiguous())
    qs = [R.weight_quant_fp8(b[i]) for i in range(W)]
    bq = torch.stack([q for q, _ in qs]); b_s = torch.stack([s for _, s in qs])
    seg = torch.zeros(len(counts) + 1, dtype=torch.int64)
    seg[1:] = torch.cumsum(torch.tensor(counts), 0)
    return a, b, aq, a_s, bq, b_s, seg


COUNTS = [[300, 0, 129, 7, 256, 1, 640], [128, 128, 257], [1000, 24]]


@pytest.mark.parametrize("counts", COUNTS)
@pytest.mark.parametrize("N,K", [(256, 512), (768, 1024)])
def test_fp8_plain_pairs_equal_single(dev, modes, counts, N, K):
    from llm_kernels_b200.moe import group_gemm_kernel as G
    W = len(counts)
    _, _, aq, a_s, bq, b_s, seg = _case(3, counts, N, K, W)
    M = aq.shape[0]
    d = [t.to(dev) for t in (aq, a_s, bq, b_s, seg)]
    rmap = torch.randperm(M, generator=torch.Generator().manual_seed(1)).to(torch.int32).to(dev)

    def run():
        c = torch.full((M, N), float("nan"), dtype=torch.bfloat16, device=dev)
        st = torch.zeros(1, dtype=torch.int32, device=dev)
        G.grouped_gemm_fp8(d[0], d[1], d[2], d[3], d[4], None, c, epilogue=0, status_word=st, c_row_map=rmap)
        assert int(st.item()) == 0
        return c
    single, pair = modes(run)
    assert not torch.isnan(pair).any()
    assert torch.equal(single, pair)
    ref = R.grouped_gemm_blockwise(aq, a_s, bq, b_s, seg, torch.arange(W), out_dtype=torch.float32)
    back = torch.empty_like(ref)
    back[rmap.cpu().long()] = ref
    assert R.rel_fro(pair.cpu().float(), back) < 3e-3


@pytest.mark.parametrize("counts", COUNTS)
def test_fp8_swiglu_pairs_equal_single(dev, modes, counts):
    from llm_kernels_b200.moe import group_gemm_kernel as G
    I, K, W = 256, 512, len(counts)
    _, _, aq, a_s, bq, b_s, seg = _case(4, counts, 2 * I, K, W)
    M = aq.shape[0]
    d = [t.to(dev) for t in (aq, a_s, bq, b_s, seg)]

    def run():
        hq = torch.zeros(M, I, dtype=torch.uint8, device=dev)
        hs = torch.zeros(M, I // 128, dtype=torch.float32, device=dev)
        G.grouped_gemm_fp8(d[0], d[1], d[2], d[3], d[4], None, hq, hs, epilogue=1)
        return hq, hs
    (q0, s0), (q1, s1) = modes(run)
    assert torch.equal(q0, q1) and torch.equal(s0, s1)
    assert s1.abs().sum() > 0


@pytest.mark.parametrize("counts", COUNTS[:2])
def test_i8_and_16bit_pairs_equal_single(dev, modes, counts):
    from llm_kernels_b200.moe import group_gemm_kernel as G
    N, K, W = 256, 512, len(counts)
    a, b, *_ , seg = _case(5, counts, N, K, W)
    M = a.shape[0]
    g = torch.Generator().manual_seed(9)
    ai = torch.randint(-127, 128, (M, K), generator=g, dtype=torch.int8).to(dev)
    bi = torch.randint(-127, 128, (W, N, K), generator=g, dtype=torch.int8).to(dev)
    a_s = (torch.rand(M, K // 128, generator=g) + 0.5).to(dev)
    b_s = (torch.rand(W, N // 128, K // 128, generator=g) + 0.5).to(dev)
    segd = seg.to(dev)

    def run_i8():
        c = torch.full((M, N), float("nan"), dtype=torch.bfloat16, device=dev)
        G.grouped_gemm_i8(ai, a_s, bi, b_s, segd, None, c)
        return c
    s, p = modes(run_i8)
    assert torch.equal(s, p) and not torch.isnan(p).any()

    for dt in (torch.bfloat16, torch.float16):
        ad, bd = a.to(dt).to(dev), b.to(dt).to(dev)

        def run_16():
            c = torch.full((M, N), float("nan"), dtype=dt, device=dev)
            G.grouped_gemm_bf16(ad, bd, segd, None, c)
            return c
        s, p = modes(run_16)
        assert torch.equal(s, p) and not torch.isnan(p).any()
        ref = R.grouped_gemm_plain(a.to(dt), b.to(dt), seg, torch.arange(W))
        assert R.rel_fro(p.cpu().float(), ref.float()) < 3e-3
