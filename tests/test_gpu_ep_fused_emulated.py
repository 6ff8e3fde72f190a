"""The exchange that is folded into the kernels (ep_plan, permute_quant_fp8_push, grouped_gemm_fp8 with
c_row_addr), with the ranks of an expert-parallel group emulated on ONE GPU: every "peer buffer" is an
ordinary local tensor, the ranks' kernels run one after the other.  Records and results must be
bit-identical to the unfused path (permute_quant_fp8 + a grouped GEMM over all experts)."""
import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def dev():
    assert torch.cuda.is_available(), "GPU tests need a CUDA device"
    import llm_kernels_b200._native as N
    N.lib()
    return torch.device("cuda:0")


def _route(T, k, E, seed, dev, skew):
    g = torch.Generator().manual_seed(seed)
    p = torch.rand(E, generator=g) ** skew + 1e-3
    rows = [torch.multinomial(p, k, replacement=False, generator=g) for _ in range(T)]
    ids = torch.stack(rows) if rows else torch.zeros(0, k, dtype=torch.int64)
    return ids.to(torch.int64).to(dev)


@pytest.mark.parametrize("ep,E,tokens,cap_factor", [(2, 8, [37, 50], 2.0), (4, 32, [64, 1, 0, 129], 2.0),
                                                    (8, 32, [40] * 8, 1.5), (2, 8, [64, 64], 0.55)])
def test_fused_exchange_emulated(dev, ep, E, tokens, cap_factor):
    from llm_kernels_b200.moe import group_gemm_kernel as G
    H, Nout, k = 256, 256, 4
    El = E // ep
    rec = (H + (H // 128) * 4 + 15) // 16 * 16
    slots = max(max(tokens) * k, 1)
    cap = int(cap_factor * slots)
    g = torch.Generator().manual_seed(7)
    w = (torch.randn(E, Nout, H, generator=g) * 0.05).to(torch.float8_e4m3fn).to(dev)
    w_s = (torch.rand(E, Nout // 128, H // 128, generator=g) + 0.5).to(dev)
    xs = [torch.randn(t, H, generator=g).to(torch.bfloat16).to(dev) for t in tokens]
    ids = [_route(t, k, E, 100 + r, dev, 3.0) for r, t in enumerate(tokens)]
    meta = [G.run_moe_ep_preproess(i, E) for i in ids]                     # (reorder_ids, src2dst, seg)
    recv = [torch.zeros(cap, rec, dtype=torch.uint8, device=dev) for _ in range(ep)]
    back = [torch.full((slots, Nout), float("nan"), dtype=torch.bfloat16, device=dev) for _ in range(ep)]
    recv_base = torch.tensor([t.data_ptr() for t in recv], dtype=torch.int64, device=dev)
    back_base = torch.tensor([t.data_ptr() for t in back], dtype=torch.int64, device=dev)
    counts_all = torch.stack([m[2][1:] - m[2][:-1] for m in meta]).contiguous()          # [ep, E]
    plans = [G.ep_plan(counts_all.view(-1), r, ep, cap, recv_base, rec, back_base, Nout * 2) for r in range(ep)]

    # ---- the plan against a host computation.  Capacity rule on both sides: block (expert, source) is accepted
    # iff it fits whole; accepted blocks are a prefix of the owner's buffer
    c = counts_all.cpu()
    overflow = False
    valid = []                                             # rows each owner computes
    rejected = torch.zeros(ep, E, dtype=torch.bool)        # [source, expert]
    for d in range(ep):
        run, first_bad = 0, None
        for el in range(El):
            for s_ in range(ep):
                cnt = int(c[s_, d * El + el])
                if cnt > 0 and run + cnt > cap:
                    rejected[s_, d * El + el] = True
                    first_bad = run if first_bad is None else first_bad
                run += cnt
        valid.append(run if first_bad is None else min(first_bad, cap))
        overflow |= first_bad is not None
    for r in range(ep):
        dst_base, local_seg, back_addr, info = [t.cpu() for t in plans[r]]
        tot = c[:, r * El:(r + 1) * El].sum(0)
        seg = torch.zeros(El + 1, dtype=torch.int64)
        seg[1:] = torch.cumsum(tot, 0)
        assert torch.equal(local_seg, seg.clamp(max=valid[r]))
        assert int(info[0]) == valid[r]
        assert bool(info[1]) == bool(valid[r] < int(seg[-1]) or rejected[r].any())
        assert torch.equal((dst_base == 0) & (c[r] > 0), rejected[r])
    if cap_factor < 1.0:
        assert overflow and any(int(p[3][1].item()) for p in plans), "the overflow case must be flagged"

    # ---- dispatch: every rank pushes; the owners' buffers against the unfused records
    sends = []
    for r in range(ep):
        send = torch.zeros(max(tokens[r] * k, 1), rec, dtype=torch.uint8, device=dev)
        G.permute_quant_fp8(xs[r], meta[r][1], ids[r], 0, E - 1, send[:, :H], send[:, H:H + (H // 128) * 4].view(torch.float32))
        sends.append(send)
        G.permute_quant_fp8_push(xs[r], meta[r][1], ids[r], meta[r][2], plans[r][0], rec, back_local=back[r])
    torch.cuda.synchronize()
    segs = [m[2].cpu() for m in meta]
    for d in range(ep):
        want = [sends[s][int(segs[s][d * El + el]):int(segs[s][d * El + el + 1])] for el in range(El) for s in range(ep)]
        want = torch.cat(want) if want else recv[d][:0]
        rows = valid[d]
        assert rows == int(plans[d][3][0].item()) and rows <= want.shape[0]
        used = H + (H // 128) * 4
        assert torch.equal(recv[d][:rows, :used], want[:rows, :used])

    # ---- compute on the owners, results stored at their sources; against one GEMM per source rank.  Slots whose
    # block was rejected get zeros back (cleared by the push kernel), never stale data
    for d in range(ep):
        a_q, a_s = recv[d][:, :H], recv[d][:, H:H + (H // 128) * 4].view(torch.float32)
        G.grouped_gemm_fp8(a_q, a_s, w[d * El:(d + 1) * El].contiguous(), w_s[d * El:(d + 1) * El].contiguous(),
                           plans[d][1], None, back[d], None, epilogue=0, c_row_addr=plans[d][2])
    torch.cuda.synchronize()
    for s in range(ep):
        n = tokens[s] * k
        if n == 0:
            continue
        ref = torch.empty(n, Nout, dtype=torch.bfloat16, device=dev)
        G.grouped_gemm_fp8(sends[s][:n, :H], sends[s][:n, H:H + (H // 128) * 4].view(torch.float32), w, w_s,
                           meta[s][2], None, ref, None, epilogue=0)
        torch.cuda.synchronize()
        dropped = rejected[s][meta[s][0].cpu()].to(dev)            # per sorted slot: its expert's block was rejected
        ref[dropped] = 0
        assert torch.equal(back[s][:n], ref)
        assert overflow or not bool(dropped.any())
