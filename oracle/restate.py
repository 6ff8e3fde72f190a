"""CPU restatement of the reference's expert-parallel quantized MoE path.

TEST INFRASTRUCTURE ONLY.  Nothing in the product package imports this module;
it is the checker used by tests/, by __graft_entry__.smoke() and by the
cpu_baseline / reference arm of bench.py.  Every function is plain torch and
device-agnostic (tests run it on CPU for small cases and may run the same
formulas on device tensors for full-size property checks).

Parity pin: the functions below are checked against outputs of the reference
itself (imported from the reference checkout) by tests/golden/make_golden.py,
which writes the fixtures that tests/test_oracle_golden.py re-checks.

Each function cites the reference file:line it follows (paths are relative to
the reference project root).
"""
from __future__ import annotations

import math
from typing import List, Optional, Sequence, Tuple

import torch
import torch.nn.functional as F

FP8_MAX = 448.0
FP8 = torch.float8_e4m3fn


def _div_const(t: torch.Tensor, c: float) -> torch.Tensor:
    """t / c as a true IEEE division on every device.  (torch's CUDA kernels turn a
    division by a Python scalar into a multiplication by its reciprocal, which is
    off by one ulp about half the time; tensor / tensor divides.)"""
    return t / torch.full_like(t, c)


# --------------------------------------------------------------------------
# Router  (moe/all2all_moe.py:60-118)
# --------------------------------------------------------------------------
def _topk_canonical(values: torch.Tensor, k: int) -> torch.Tensor:
    """Indices of the k largest entries per row; ties go to the lower index.

    torch.topk leaves tie order implementation-defined, so the canonical rule
    is expressed with a stable descending sort.
    """
    order = torch.sort(values, dim=-1, descending=True, stable=True)[1]
    return order[..., :k]


def gate_scores(x: torch.Tensor, weight: torch.Tensor, scoring_func: str,
                dtype=torch.float32) -> torch.Tensor:
    """logits = x.float() @ W.float()^T, then sigmoid (moe/all2all_moe.py:64-68)
    or softmax over experts (the extension BASELINE configs [0] and [2] need)."""
    logits = F.linear(x.to(dtype), weight.to(dtype), None)
    if scoring_func == "sigmoid":
        return logits.sigmoid()
    if scoring_func == "softmax":
        return logits.softmax(dim=-1)
    raise NotImplementedError(
        f"insupportable scoring function for MoE gating: {scoring_func}")


def gate_select(scores: torch.Tensor, bias: Optional[torch.Tensor], top_k: int,
                n_group: int, topk_group: int):
    """Group-limited top-k of moe/all2all_moe.py:75-106 on given scores.

    Returns (topk_idx [T,k] in descending choice-score order, margin [T]) where
    margin is, per token, the smallest gap that decided a selection (group cut
    and expert cut)."""
    T, E = scores.shape
    sfc = scores if bias is None else scores + bias.unsqueeze(0).to(scores.dtype)
    margin = torch.full((T,), float("inf"), dtype=scores.dtype, device=scores.device)
    if n_group > 1:
        grouped = sfc.view(T, n_group, E // n_group)
        group_scores = grouped.topk(2, dim=-1)[0].sum(dim=-1)          # :80-82
        gsorted = torch.sort(group_scores, dim=-1, descending=True, stable=True)
        group_idx = gsorted[1][:, :topk_group]                         # :84-85
        if topk_group < n_group:
            margin = torch.minimum(margin, gsorted[0][:, topk_group - 1] - gsorted[0][:, topk_group])
        group_mask = torch.zeros_like(group_scores)
        group_mask.scatter_(1, group_idx, 1)                           # :88-89
        score_mask = group_mask.unsqueeze(-1).expand(T, n_group, E // n_group).reshape(T, E)
        tmp = sfc.masked_fill(~score_mask.bool(), 0.0)                 # :101
    else:
        tmp = sfc
    ssorted = torch.sort(tmp, dim=-1, descending=True, stable=True)
    topk_idx = ssorted[1][:, :top_k]                                   # :104-106
    if top_k < E:
        margin = torch.minimum(margin, ssorted[0][:, top_k - 1] - ssorted[0][:, top_k])
    return topk_idx, margin


def gate_forward(x: torch.Tensor, weight: torch.Tensor, bias: Optional[torch.Tensor], *,
                 top_k: int, n_group: int = 1, topk_group: int = 1,
                 scoring_func: str = "sigmoid", norm_topk_prob: bool = True,
                 routed_scaling_factor: float = 1.0):
    """MoEGate.forward (moe/all2all_moe.py:60-118) on flattened tokens x [T,H].

    Returns (topk_idx int64 [T,k], topk_weight fp32 [T,k]).  Selection uses the
    biased scores; the returned weights gather the UNBIASED scores (:107),
    are renormalised with +1e-20 (:114-116) and scaled (:117)."""
    scores = gate_scores(x, weight, scoring_func)
    topk_idx, _ = gate_select(scores, bias, top_k, n_group, topk_group)
    topk_weight = scores.gather(1, topk_idx)
    if top_k > 1 and norm_topk_prob:
        topk_weight = topk_weight / (topk_weight.sum(dim=-1, keepdim=True) + 1e-20)
    topk_weight = topk_weight * routed_scaling_factor
    return topk_idx, topk_weight


def gate_margins_fp64(x, weight, bias, *, top_k, n_group=1, topk_group=1,
                      scoring_func="sigmoid") -> torch.Tensor:
    """Per-token smallest selection gap when the router is evaluated in fp64.  A
    token is admissible for bit-exact routing comparison only if its gap is well
    above f32 summation noise: two correct f32 routers may legitimately differ on
    a token whose k-th and (k+1)-th scores are closer than that."""
    scores = gate_scores(x, weight, scoring_func, dtype=torch.float64)
    b = None if bias is None else bias.double()
    _, margin = gate_select(scores, b, top_k, n_group, topk_group)
    return margin


def gate_margin_fp64(x, weight, bias, **kw) -> float:
    return float(gate_margins_fp64(x, weight, bias, **kw).min())


def canonical_rows(topk_idx: torch.Tensor, topk_weight: torch.Tensor):
    """Sort each row by expert id (weights permuted alongside) so two routers
    that emit the same set in a different order compare equal."""
    order = torch.sort(topk_idx, dim=-1, stable=True)[1]
    return topk_idx.gather(1, order), topk_weight.gather(1, order)


# --------------------------------------------------------------------------
# Histogram and permutation metadata
# --------------------------------------------------------------------------
def tokens_per_expert(topk_ids: torch.Tensor, num_experts: int) -> torch.Tensor:
    """moe/all2all_moe.py:188-192: one-hot scatter then column sum -> int64 [E]."""
    cnts = topk_ids.new_zeros((topk_ids.shape[0], num_experts))
    cnts.scatter_(1, topk_ids, 1)
    return cnts.sum(dim=0)


def run_moe_ep_preproess(topk_ids: torch.Tensor, num_experts: int):
    """moe/group_gemm_kernel.py:48-78.

    reorder_topk_ids int64 [T*k]: expert ids stably sorted (:52)
    src2dst          int32 [T*k]: flat slot -> row in expert order (:37-45)
    seg_indptr       int64 [E+1]: seg_indptr[e+1] = #ids <= e (:19-34), [0] = 0
    """
    flat = topk_ids.reshape(-1)
    reorder_topk_ids, reorder_ids = torch.sort(flat, stable=True)
    n = flat.numel()
    src2dst = torch.empty(n, dtype=torch.int32, device=flat.device)
    src2dst[reorder_ids] = torch.arange(n, dtype=torch.int32, device=flat.device)
    counts = torch.bincount(flat, minlength=num_experts)[:num_experts]
    seg_indptr = torch.zeros(num_experts + 1, dtype=torch.int64, device=flat.device)
    seg_indptr[1:] = torch.cumsum(counts, 0)
    return reorder_topk_ids, src2dst, seg_indptr


# --------------------------------------------------------------------------
# fp8 e4m3 quantizers and blockwise GEMM  (quantization/fp8_kernel.py)
# --------------------------------------------------------------------------
def act_quant_fp8(x: torch.Tensor, block_size: int = 128):
    """quantization/fp8_kernel.py:23-30: per 128 contiguous elements
    s = amax/448 (fp32), y = (x/s) cast to e4m3 with round-to-nearest-even.
    amax == 0 gives s == 0 and y == NaN exactly as the reference does."""
    assert x.is_contiguous() and x.shape[-1] % block_size == 0
    g = x.float().reshape(-1, block_size)
    s = _div_const(g.abs().amax(dim=-1), FP8_MAX)
    y = (g / s.unsqueeze(-1)).to(FP8)
    return (y.reshape(x.shape),
            s.reshape(*x.shape[:-1], x.shape[-1] // block_size))


def _blocks(x: torch.Tensor, bs: int):
    M, N = x.shape
    pm, pn = (-M) % bs, (-N) % bs
    xp = F.pad(x, (0, pn, 0, pm))
    return xp.reshape((M + pm) // bs, bs, (N + pn) // bs, bs).permute(0, 2, 1, 3), M, N


def weight_quant_fp8(w: torch.Tensor, block_size: int = 128):
    """128x128-block e4m3 weight quantizer: s = amax/448 (fp32), y = w/s.
    The fp8 analogue of quantization/int8_kernel.py:59-113 (same block grid and
    scale shape [ceil(M/bs), ceil(N/bs)]); the reference ships no fp8 weight
    quantizer."""
    blk, M, N = _blocks(w.float(), block_size)
    s = _div_const(blk.abs().amax(dim=(-1, -2)), FP8_MAX)
    y = blk / s[..., None, None]
    y = y.permute(0, 2, 1, 3).reshape(blk.shape[0] * block_size, blk.shape[1] * block_size)
    return y[:M, :N].contiguous().to(FP8), s


def weight_dequant_fp8(x: torch.Tensor, s: torch.Tensor, block_size: int = 128,
                       dtype=torch.float32):
    """quantization/fp8_kernel.py:55-105: y = x.float() * s[block_m, block_n]."""
    M, N = x.shape
    se = s.float().repeat_interleave(block_size, 0)[:M].repeat_interleave(block_size, 1)[:, :N]
    return (x.float() * se).to(dtype)


def fp8_gemm(a, a_s, b, b_s, out_dtype=torch.bfloat16, block: int = 128):
    """quantization/fp8_kernel.py:108-190: C = A.B^T with per-K-block promotion
    acc += dot(a_kb, b_kb) * a_s[m,kb] * b_s[n//128,kb] (fp32), cast at the end."""
    K = a.shape[-1]
    a2 = a.reshape(-1, K)
    as2 = a_s.reshape(-1, a_s.shape[-1]).float()
    N = b.shape[0]
    acc = torch.zeros(a2.shape[0], N, dtype=torch.float32, device=a.device)
    bs_e = b_s.float().repeat_interleave(block, 0)[:N]          # [N, K/128]
    for kb in range((K + block - 1) // block):
        ks = slice(kb * block, min(K, (kb + 1) * block))
        d = a2[:, ks].float() @ b[:, ks].float().t()
        acc += d * as2[:, kb:kb + 1] * bs_e[:, kb].unsqueeze(0)
    return acc.to(out_dtype).reshape(*a.shape[:-1], N)


def grouped_gemm_blockwise(a, a_s, b, b_s, seg_indptr, weight_indices,
                           out_dtype=torch.bfloat16, block: int = 128):
    """moe/group_gemm_kernel.py:291-428 with group_k>0 (and its torch twin
    moe/sglang_moe_all_gather_all_reduce.py:58-159): for each group g rows
    [seg[g], seg[g+1]) use weight b[weight_indices[g]] [N,K] and scales
    b_s[weight_indices[g]] [N/128, K/128]; rows outside every group are left 0."""
    M, K = a.shape
    N = b.shape[1]
    c = torch.zeros(M, N, dtype=out_dtype, device=a.device)
    seg = seg_indptr.tolist()
    widx = weight_indices.tolist()
    for g in range(len(widx)):
        m0, m1 = seg[g], seg[g + 1]
        if m1 <= m0:
            continue
        e = widx[g]
        c[m0:m1] = fp8_gemm(a[m0:m1], a_s[m0:m1], b[e], b_s[e], out_dtype, block)
    return c


def grouped_gemm_plain(a, b, seg_indptr, weight_indices, out_dtype=None):
    """moe/group_gemm_kernel.py:291-428 with group_k == 0: C[seg] = A[seg].B[e]^T
    with fp32 accumulation."""
    out_dtype = out_dtype or a.dtype
    c = torch.zeros(a.shape[0], b.shape[1], dtype=out_dtype, device=a.device)
    seg = seg_indptr.tolist()
    for g, e in enumerate(weight_indices.tolist()):
        m0, m1 = seg[g], seg[g + 1]
        if m1 > m0:
            c[m0:m1] = (a[m0:m1].float() @ b[e].float().t()).to(out_dtype)
    return c


# --------------------------------------------------------------------------
# int8 quantizers
# --------------------------------------------------------------------------
def act_quant_int8(x: torch.Tensor, block_size: int = 128, rounding: str = "half_away"):
    """quantization/int8_kernel.py:23-31 (rounding='half_away', libdevice.round)
    or quantization/w4a8_kernel.py:159-168 (rounding='floor_half',
    floor(x/s + 0.5)).  s = amax/127 (fp32), stored as fp16."""
    g = x.float().reshape(-1, block_size)
    s = _div_const(g.abs().amax(dim=-1), 127.0)
    q = g / s.unsqueeze(-1)
    if rounding == "half_away":
        q = torch.sign(q) * torch.floor(q.abs() + 0.5)
    elif rounding == "floor_half":
        q = torch.floor(q + 0.5)
    else:
        raise ValueError(rounding)
    return (q.to(torch.int8).reshape(x.shape),
            s.to(torch.float16).reshape(*x.shape[:-1], x.shape[-1] // block_size))


def weight_quant_int8(x: torch.Tensor, block_size: int = 128):
    """quantization/int8_kernel.py:59-113: per 128x128 block (edge blocks masked, :76-79)
    s = amax/127 in fp32, y = libdevice.round(x / s) (half away from zero) as int8, s stored as
    fp16 [ceil(M/128), ceil(N/128)].  The Triton kernel cannot run in the CPU interpreter
    (libdevice), so this function is pinned by its formula only."""
    M, N = x.shape
    blk, _, _ = _blocks(x.float(), block_size)
    s = _div_const(blk.abs().amax(dim=(-1, -2)), 127.0)
    q = blk / s[..., None, None]
    q = torch.sign(q) * torch.floor(q.abs() + 0.5)
    q = q.permute(0, 2, 1, 3).reshape(blk.shape[0] * block_size, -1)[:M, :N]
    return torch.nan_to_num(q, nan=0.0).to(torch.int8).contiguous(), s.to(torch.float16)


def weight_dequant_int8(x: torch.Tensor, s: torch.Tensor, block_size: int = 128, dtype=torch.float32):
    """quantization/int8_kernel.py:116-170: y = float(x) * s[i/128, j/128], cast to the default dtype."""
    M, N = x.shape
    se = s.float().repeat_interleave(block_size, 0)[:M].repeat_interleave(block_size, 1)[:, :N]
    return (x.float() * se).to(dtype)


# --------------------------------------------------------------------------
# Quantized all-reduce  (quant_communication/quant_all2all_allreduce.py:52-99)
# --------------------------------------------------------------------------
def comm_quant(x: torch.Tensor, kind: str):
    """Payload quantizer of the quantized all-reduce over 1x128 groups: kind "fp8" = act_quant_fp8
    (e4m3, f32 scales); kind "int8" = quant_communication/quant_utils.py:9-32 (s = amax/127 stored as f16,
    y = floor(x/s + 0.5)), which is act_quant_int8 with rounding='floor_half'."""
    return act_quant_fp8(x) if kind == "fp8" else act_quant_int8(x, rounding="floor_half")


def comm_dequant_sum(q: torch.Tensor, s: torch.Tensor, out_dtype):
    """quant_all2all_allreduce.py:73-80: q [n, R, H], s [n, R, H/128]; each source is dequantized as
    quant_utils.py:75-83 / 176-180 do (product in the scales' dtype, cast to the output dtype), the sources
    are summed in f32 and the sum is cast to the output dtype.  Groups with scale 0 decode to zero."""
    se = s.repeat_interleave(128, dim=-1)
    v = torch.where(se == 0, torch.zeros((), dtype=torch.float32), q.float())
    prod = (v * se.float()).to(s.dtype).to(out_dtype)
    return prod.float().sum(dim=0).to(out_dtype)


def quant_allreduce(xs, kind: str):
    """The whole scheme for a list of per-rank tensors [T, H] (ranks simulated in-process): returns the tensor
    every rank ends up with.  Rows are padded to a multiple of the rank count."""
    ep = len(xs)
    T, H = xs[0].shape
    R = -(-T // ep)
    dt = xs[0].dtype
    pad = [torch.cat([x, x.new_zeros(R * ep - T, H)]) for x in xs]
    qs = [comm_quant(p, kind) for p in pad]
    chunks = []
    for r in range(ep):                                   # rank r reduces rows [r*R, (r+1)*R)
        q = torch.stack([qs[s_][0][r * R:(r + 1) * R] for s_ in range(ep)])
        s = torch.stack([qs[s_][1][r * R:(r + 1) * R] for s_ in range(ep)])
        chunks.append(comm_dequant_sum(q, s, dt))
    out = []
    for c in chunks:
        q2, s2 = comm_quant(c, kind)
        out.append(comm_dequant_sum(q2.unsqueeze(0), s2.unsqueeze(0), dt))
    return torch.cat(out)[:T]


# --------------------------------------------------------------------------
# Reorder / activation / combine kernels  (moe/group_gemm_kernel.py)
# --------------------------------------------------------------------------
def pre_reorder(x, src2dst, topk_ids, a1_scales, start_expert_id, end_expert_id,
                out: torch.Tensor):
    """moe/group_gemm_kernel.py:81-117.  Rows of `out` for non-local slots are
    left untouched."""
    T, k = topk_ids.shape
    s2d = src2dst.view(T, k).long()
    for j in range(k):
        e = topk_ids[:, j]
        sel = (e >= start_expert_id) & (e <= end_expert_id)
        if not bool(sel.any()):
            continue
        rows = x[sel].float()
        if a1_scales is not None:
            rows = rows * (1.0 / a1_scales[(e[sel] - start_expert_id)].float()).unsqueeze(-1)
        out[s2d[sel, j]] = rows.to(out.dtype)
    return out


def _act_and_mul(gateup, reorder_topk_ids, scales, start_expert_id, end_expert_id, out, act):
    half = gateup.shape[1] // 2
    sel = (reorder_topk_ids >= start_expert_id) & (reorder_topk_ids <= end_expert_id)
    g = gateup[sel, :half].float()
    u = gateup[sel, half:]
    g = act(g).to(gateup.dtype)
    if scales is not None:
        sc = (1.0 / scales[(reorder_topk_ids[sel] - start_expert_id)].float()).to(gateup.dtype)
        r = g * u * sc.unsqueeze(-1)
    else:
        r = g * u
    out[sel] = r.to(out.dtype)
    return out


def silu_and_mul(gateup, reorder_topk_ids, scales, start_expert_id, end_expert_id, out):
    """moe/group_gemm_kernel.py:120-168: silu in fp32, cast to the input dtype,
    product gate*up*(1/scale) in the input dtype, cast to the output dtype."""
    return _act_and_mul(gateup, reorder_topk_ids, scales, start_expert_id, end_expert_id,
                        out, lambda g: g * torch.sigmoid(g))


def gelu_and_mul(gateup, reorder_topk_ids, scales, start_expert_id, end_expert_id, out):
    """moe/group_gemm_kernel.py:176-235: tanh-GELU with tanh(x)=2*sigmoid(2x)-1."""
    def gelu(g):
        inner = 0.7978845608028654 * (g + 0.044715 * g * g * g)
        return 0.5 * g * (1 + (2 * torch.sigmoid(2 * inner) - 1))
    return _act_and_mul(gateup, reorder_topk_ids, scales, start_expert_id, end_expert_id,
                        out, gelu)


def post_reorder(down_output, src2dst, topk_ids, topk_weights, start_expert_id,
                 end_expert_id, acc_dtype=None):
    """moe/group_gemm_kernel.py:238-288: out[t] = sum_k down[src2dst[t,k]]*w[t,k]
    over local slots, accumulated in `acc_dtype` (the reference accumulates in the
    input dtype; the B200 kernel and moe/all2all_moe.py:270-278 accumulate in
    fp32); tokens with no local expert are zero."""
    T, k = topk_ids.shape
    acc_dtype = acc_dtype or down_output.dtype
    acc = torch.zeros(T, down_output.shape[1], dtype=acc_dtype, device=down_output.device)
    s2d = src2dst.view(T, k).long()
    for j in range(k):
        e = topk_ids[:, j]
        sel = (e >= start_expert_id) & (e <= end_expert_id)
        rows = down_output[s2d[:, j].clamp(0, down_output.shape[0] - 1)].to(acc_dtype)
        w = topk_weights[:, j].to(acc_dtype).unsqueeze(-1)
        acc = acc + torch.where(sel.unsqueeze(-1), rows * w, torch.zeros_like(rows))
    return acc.to(down_output.dtype)


# --------------------------------------------------------------------------
# Whole layer
# --------------------------------------------------------------------------
def expert_mlp(x, gate_w, up_w, down_w):
    """DeepseekV3MLP.forward (moe/all2all_moe.py:27-29) with silu."""
    return F.linear(F.silu(F.linear(x, gate_w)) * F.linear(x, up_w), down_w)


def moe_infer_dense(x, topk_ids, topk_weight, gate_ws, up_ws, down_ws):
    """DeepseekV3MoE.moe_infer at ep_size == 1 (moe/all2all_moe.py:187-280):
    sort slots by expert, run each expert on its slice, un-sort, weight in the
    routing-weight dtype (fp32) and sum over k, cast back."""
    T, k = topk_ids.shape
    flat = topk_ids.reshape(-1)
    idxs = torch.sort(flat, stable=True)[1]
    sorted_tokens = x[idxs // k]
    counts = torch.bincount(flat, minlength=len(gate_ws)).tolist()
    outs = torch.empty_like(sorted_tokens)
    s = 0
    for e, n in enumerate(counts):
        if n:
            outs[s:s + n] = expert_mlp(sorted_tokens[s:s + n], gate_ws[e], up_ws[e], down_ws[e])
        s += n
    new_x = torch.empty_like(outs)
    new_x[idxs] = outs
    return (new_x.view(T, k, -1).type(topk_weight.dtype)
            .mul_(topk_weight.unsqueeze(-1)).sum(dim=1).type(new_x.dtype))


def moe_layer_fp8(x, topk_ids, topk_weight, w13, w13_s, w2, w2_s, *,
                  ep_size: int = 1, out_dtype=torch.bfloat16, hidden_act: str = "silu"):
    """The quantized expert-parallel layer the B200 path implements, restated
    from the reference's pieces:

      permutation   moe/group_gemm_kernel.py:48-78 (stable sort by expert)
      act quant     quantization/fp8_kernel.py:23-30 per token, 1x128
      sharding      moe/all2all_moe.py:130-147 (rank r owns experts
                    [r*E/ep, (r+1)*E/ep)); the all-to-all of :206-268 only moves
                    rows, so with every rank simulated in-process the result is
                    independent of ep_size -- the loop below still walks the
                    ranks so per-rank segment bookkeeping is exercised
      GEMM-1        grouped blockwise GEMM with w13 = [gate ; up]
                    (moe/moe_numerical_equivalence_validation.py:87-88)
      activation    moe/group_gemm_kernel.py:120-168 (silu) or :176-235 (gelu), chosen as
                    moe/sglang_moe_all_gather_all_reduce.py:374-397 does (intermediate
                    rounded to out_dtype as the reference's gateup_output is)
      act quant 2   1x128 fp8 of the SwiGLU output
      GEMM-2        grouped blockwise GEMM with w2
      combine       moe/all2all_moe.py:270-278 (fp32 weighting and sum)

    w13 [E,2I,H] e4m3, w13_s [E,2I/128,H/128] fp32, w2 [E,H,I], w2_s [E,H/128,I/128].
    """
    T, k = topk_ids.shape
    E = w13.shape[0]
    H = x.shape[1]
    reorder_ids, src2dst, seg = run_moe_ep_preproess(topk_ids, E)
    S = T * k
    xq, xs = act_quant_fp8(x.contiguous())
    dst_tok = torch.empty(S, dtype=torch.long, device=x.device)
    dst_tok[src2dst.long()] = torch.arange(S, device=x.device) // k
    a1, a1s = xq[dst_tok], xs[dst_tok]
    down_out = torch.zeros(S, H, dtype=out_dtype, device=x.device)
    E_l = E // ep_size
    for r in range(ep_size):
        e0 = r * E_l
        lo, hi = int(seg[e0]), int(seg[e0 + E_l])
        if hi <= lo:
            continue
        seg_r = seg[e0:e0 + E_l + 1] - lo
        widx = torch.arange(e0, e0 + E_l)
        gu = grouped_gemm_blockwise(a1[lo:hi], a1s[lo:hi], w13, w13_s, seg_r, widx, out_dtype)
        h = torch.empty(hi - lo, gu.shape[1] // 2, dtype=out_dtype, device=x.device)
        act_mul = {"silu": silu_and_mul, "gelu": gelu_and_mul}[hidden_act]
        act_mul(gu, torch.zeros(hi - lo, dtype=torch.long), None, 0, 0, h)
        hq, hs = act_quant_fp8(h)
        down_out[lo:hi] = grouped_gemm_blockwise(hq, hs, w2, w2_s, seg_r, widx, out_dtype)
    y = (down_out[src2dst.long()].view(T, k, H).float()
         * topk_weight.float().unsqueeze(-1)).sum(dim=1)
    return y.to(out_dtype)


def _permuted_rows(x, topk_ids, num_experts):
    T, k = topk_ids.shape
    _, src2dst, seg = run_moe_ep_preproess(topk_ids, num_experts)
    dst_tok = torch.empty(T * k, dtype=torch.long, device=x.device)
    dst_tok[src2dst.long()] = torch.arange(T * k, device=x.device) // k
    return src2dst, seg, dst_tok


def _combine(down_out, src2dst, topk_weight, T, k, out_dtype):
    """moe/all2all_moe.py:270-278: f32 weighting and sum over k."""
    H = down_out.shape[1]
    return (down_out[src2dst.long()].view(T, k, H).float()
            * topk_weight.float().unsqueeze(-1)).sum(dim=1).to(out_dtype)


def moe_layer_w4a16(x, topk_ids, topk_weight, w13_q, w13_scale, w13_zero, w2_q, w2_scale, w2_zero,
                    out_dtype=torch.bfloat16, hidden_act: str = "silu"):
    """w4a16 layer: bf16 rows are permuted unquantized (moe/group_gemm_kernel.py:81-117); each
    expert multiplies by its dequantized int4 weights ((q - zero) * scale rounded to bf16, the
    zero-point extension of fast_dequant/simple_marlin/utils.py:98-136) with f32 accumulation;
    SwiGLU with the roundings of moe/group_gemm_kernel.py:120-168; f32 combine.
    w13_q uint8 [E,2I,H] (unpacked nibbles), scales/zeros bf16 [E,2I,H/128]; w2_* likewise."""
    T, k = topk_ids.shape
    E = w13_q.shape[0]
    src2dst, seg, dst_tok = _permuted_rows(x, topk_ids, E)
    a = x[dst_tok]
    down = torch.zeros(T * k, x.shape[1], dtype=out_dtype, device=x.device)
    segl = seg.tolist()
    for e in range(E):
        m0, m1 = segl[e], segl[e + 1]
        if m1 <= m0:
            continue
        w13 = w4a16_dequant(w13_q[e], w13_scale[e], w13_zero[e]).float()
        gu = (a[m0:m1].float() @ w13.t()).to(out_dtype)
        h = torch.empty(m1 - m0, gu.shape[1] // 2, dtype=out_dtype, device=x.device)
        {"silu": silu_and_mul, "gelu": gelu_and_mul}[hidden_act](gu, torch.zeros(m1 - m0, dtype=torch.long), None, 0, 0, h)
        w2 = w4a16_dequant(w2_q[e], w2_scale[e], w2_zero[e]).float()
        down[m0:m1] = (h.float() @ w2.t()).to(out_dtype)
    return _combine(down, src2dst, topk_weight, T, k, out_dtype)


def moe_layer_w4a8(x, topk_ids, topk_weight, w13, w2, out_dtype=torch.bfloat16, hidden_act: str = "silu"):
    """w4a8 layer: tokens are quantized to int8 per 1x128 group (quantization/w4a8_kernel.py:145-193)
    before the permutation; each expert runs w4a8_gemm (:317-448) for gate/up, SwiGLU
    (moe/group_gemm_kernel.py:120-168), re-quantizes to int8, runs w4a8_gemm for down; f32
    combine.  w13, w2: per-expert lists of (packed, s, s4, z4) from w4a8_weight_quant."""
    T, k = topk_ids.shape
    E = len(w13)
    src2dst, seg, dst_tok = _permuted_rows(x, topk_ids, E)
    xq, xs = act_quant_int8(x.contiguous(), rounding="floor_half")
    a, a_s = xq[dst_tok], xs[dst_tok]
    down = torch.zeros(T * k, x.shape[1], dtype=out_dtype, device=x.device)
    segl = seg.tolist()
    for e in range(E):
        m0, m1 = segl[e], segl[e + 1]
        if m1 <= m0:
            continue
        gu = w4a8_gemm(a[m0:m1], a_s[m0:m1], *w13[e], out_dtype=out_dtype)
        h = torch.empty(m1 - m0, gu.shape[1] // 2, dtype=out_dtype, device=x.device)
        {"silu": silu_and_mul, "gelu": gelu_and_mul}[hidden_act](gu, torch.zeros(m1 - m0, dtype=torch.long), None, 0, 0, h)
        hq, hs = act_quant_int8(h, rounding="floor_half")
        down[m0:m1] = w4a8_gemm(hq, hs, *w2[e], out_dtype=out_dtype)
    return _combine(down, src2dst, topk_weight, T, k, out_dtype)


def rel_fro(a: torch.Tensor, b: torch.Tensor) -> float:
    """Relative Frobenius error ||a-b|| / ||b|| in fp64."""
    a, b = a.double(), b.double()
    return float((a - b).norm() / b.norm().clamp_min(1e-300))


# --------------------------------------------------------------------------
# Bit packing  (quantization/bitpack.py)
# --------------------------------------------------------------------------
_PACK_DTYPE = {8: torch.uint8, 16: torch.int16, 32: torch.int32, 64: torch.int64}


def pack_weights_over_rows(W_q, W_nbits: int, packing_bitwidth: int, transpose: bool = False):
    """quantization/bitpack.py:9-36: word r, field i holds W_q[e*r+i, c] << (nbits*i)."""
    e = packing_bitwidth // W_nbits
    Wi = W_q.to(torch.int64)
    out = torch.zeros(Wi.shape[0] // e, Wi.shape[1], dtype=torch.int64, device=W_q.device)
    for i in range(e):
        out |= Wi[i::e, :] << (i * W_nbits)
    out = _wrap(out, packing_bitwidth)
    return (out.t() if transpose else out), e


def pack_weights_over_cols(W_q, W_nbits: int, packing_bitwidth: int, transpose: bool = False):
    """quantization/bitpack.py:38-67: word c, field i holds W_q[r, e*c+i] << (nbits*i)."""
    e = packing_bitwidth // W_nbits
    Wi = W_q.to(torch.int64)
    out = torch.zeros(Wi.shape[0], Wi.shape[1] // e, dtype=torch.int64, device=W_q.device)
    for i in range(e):
        out |= Wi[:, i::e] << (i * W_nbits)
    out = _wrap(out, packing_bitwidth)
    return (out.t() if transpose else out), e


def _wrap(v64: torch.Tensor, bits: int) -> torch.Tensor:
    if bits == 64:
        return v64
    if bits == 8:
        return (v64 & 0xFF).to(torch.uint8)
    half = 1 << (bits - 1)
    v = v64 & ((1 << bits) - 1)
    v = torch.where(v >= half, v - (1 << bits), v)
    return v.to(_PACK_DTYPE[bits])


def unpack_over_rows(packed, W_nbits: int, num_output_rows: int, dtype=torch.uint8):
    """quantization/bitpack.py:296-305."""
    e = num_output_rows // packed.shape[0]
    p = packed.to(torch.int64)
    shifts = torch.arange(e, device=packed.device, dtype=torch.int64) * W_nbits
    u = ((p.unsqueeze(-1) >> shifts) & ((1 << W_nbits) - 1)).to(dtype)
    return u.permute(0, 2, 1).reshape(num_output_rows, packed.shape[1])


def unpack_over_cols(packed, W_nbits: int, num_output_cols: int, dtype=torch.uint8):
    """quantization/bitpack.py:152-161."""
    e = num_output_cols // packed.shape[1]
    p = packed.to(torch.int64)
    shifts = torch.arange(e, device=packed.device, dtype=torch.int64) * W_nbits
    u = ((p.unsqueeze(-1) >> shifts) & ((1 << W_nbits) - 1)).to(dtype)
    return u.reshape(packed.shape[0], num_output_cols)


# --------------------------------------------------------------------------
# Two-level int4 weights + int8 activations  (quantization/w4a8_kernel.py)
# --------------------------------------------------------------------------
def w4a8_weight_quant(x: torch.Tensor, block_size: int = 128, group: int = 128):
    """quantization/w4a8_kernel.py:196-309.

    level 1 (:196-225): per 128x128 block s = amax/119 (fp32 -> fp16 for
      storage), y8 = clamp(floor(x/s + 0.5), -119, 119)
    level 2 (:228-262): per (row, 128-col group) s4 = floor((max-min)/15+0.5),
      z4 = floor(-min/s4 + 0.5), q = clamp(floor(y8/s4 + 0.5) + z4, 0, 15)
    pack (:300-305): 8 consecutive ROWS (output channels) per int32 word.

    Returns (packed int32 [M/8,N], s fp16 [M/128,N/128], s4 int8 [M,N/128],
    z4 int8 [M,N/128])."""
    M, N = x.shape
    blk, _, _ = _blocks(x.float(), block_size)
    s = _div_const(blk.abs().amax(dim=(-1, -2)), 119.0)
    y8 = torch.clamp(torch.floor(blk / s[..., None, None] + 0.5), -119.0, 119.0)
    y8 = y8.permute(0, 2, 1, 3).reshape(blk.shape[0] * block_size, -1)[:M, :N]
    g = y8.reshape(M, N // group, group)
    mx, mn = g.amax(-1), g.amin(-1)
    s4 = torch.floor(_div_const(mx - mn, 15.0) + 0.5)
    z4 = torch.floor(-mn / s4 + 0.5)
    q = torch.clamp(torch.floor(g / s4.unsqueeze(-1) + 0.5) + z4.unsqueeze(-1), 0, 15)
    q = q.reshape(M, N).to(torch.uint8)
    packed, _ = pack_weights_over_rows(q, 4, 32)
    return packed, s.to(torch.float16), s4.to(torch.int8), z4.to(torch.int8)


def w4a8_weight_int8(packed, s4, z4, group: int = 128):
    """quantization/w4a8_kernel.py:44-101: (q - z4) * s4 in int8 arithmetic
    (the int32 -> int8 cast wraps exactly as the reference's int8 product does)."""
    q = unpack_over_rows(packed, 4, packed.shape[0] * 8, torch.int8)
    M, N = q.shape
    g = q.reshape(M, N // group, group).to(torch.int32)
    w8 = (g - z4.to(torch.int32).unsqueeze(-1)) * s4.to(torch.int32).unsqueeze(-1)
    return w8.reshape(M, N).to(torch.int8)


def w4a8_weight_dequant(packed, s, s4, z4, block_size: int = 128, group: int = 128):
    """quantization/w4a8_kernel.py:104-142: int4 -> int8 -> * s (fp16 result)."""
    w8 = w4a8_weight_int8(packed, s4, z4, group).float()
    M, N = w8.shape
    se = s.float().repeat_interleave(block_size, 0)[:M].repeat_interleave(block_size, 1)[:, :N]
    return (w8 * se).to(torch.float16)


def w4a8_gemm(a, a_s, packed, b_s, b_s4, b_z4, out_dtype=torch.bfloat16, block: int = 128):
    """quantization/w4a8_kernel.py:317-448: per K block, int8 x int8 dot (exact
    in int32) times a_s[m,kb] * b_s[n//128,kb] accumulated in fp32."""
    K = a.shape[-1]
    a2 = a.reshape(-1, K)
    w8 = w4a8_weight_int8(packed, b_s4, b_z4, block)
    N = w8.shape[0]
    acc = torch.zeros(a2.shape[0], N, dtype=torch.float32, device=a.device)
    as2 = a_s.reshape(-1, a_s.shape[-1]).float()
    bs_e = b_s.float().repeat_interleave(block, 0)[:N]
    for kb in range(K // block):
        ks = slice(kb * block, (kb + 1) * block)
        d = (a2[:, ks].double() @ w8[:, ks].double().t()).float()
        acc += d * as2[:, kb:kb + 1] * bs_e[:, kb].unsqueeze(0)
    return acc.to(out_dtype).reshape(*a.shape[:-1], N)


# --------------------------------------------------------------------------
# w4a16  (fast_dequant/simple_marlin/utils.py)
# --------------------------------------------------------------------------
def w4a16_fake_quantize_sym(weight: torch.Tensor, groupsize: int = -1):
    """fast_dequant/simple_marlin/utils.py:98-136: weight [K,N]; per (group
    along K, column) scale = 2*amax/15; q = clamp(round(w/scale)+8, 0, 15);
    ref = (q-8)*scale.  Returns (ref, q int32 [K,N], scale [K/g, N])."""
    K, N = weight.shape
    g = K if groupsize == -1 else groupsize
    w = weight.reshape(K // g, g, N)
    scale = w.abs().amax(dim=1, keepdim=True)
    scale = scale * (2 / 15)
    q = torch.round(w / scale).int() + 8
    q = torch.clamp(q, 0, 15)
    ref = (q - 8).to(weight.dtype) * scale
    return ref.reshape(K, N), q.reshape(K, N), scale.reshape(K // g, N)


def w4a16_quantize_asym(weight_nk: torch.Tensor, groupsize: int = 128,
                        dtype=torch.bfloat16):
    """Asymmetric extension of fast_dequant/simple_marlin/utils.py:98-136 for
    nn.Linear-layout weights [N,K] grouped along K: scale = (max-min)/15 and
    zero = round(-min/scale), both rounded to `dtype`;
    q = clamp(round(w/scale) + zero, 0, 15); dequant = (q - zero) * scale.
    Returns (q uint8 [N,K], scale [N,K/g], zero [N,K/g])."""
    N, K = weight_nk.shape
    w = weight_nk.float().reshape(N, K // groupsize, groupsize)
    mx, mn = w.amax(-1), w.amin(-1)
    scale = ((mx - mn) / 15.0).clamp_min(1e-8).to(dtype)
    zero = torch.round(-mn / scale.float()).clamp(0, 15).to(dtype)
    q = torch.clamp(torch.round(w / scale.float().unsqueeze(-1)) + zero.float().unsqueeze(-1), 0, 15)
    return q.reshape(N, K).to(torch.uint8), scale, zero


def w4a16_dequant(q, scale, zero, groupsize: int = 128, dtype=torch.bfloat16):
    N, K = q.shape
    g = q.float().reshape(N, K // groupsize, groupsize)
    w = (g - zero.float().unsqueeze(-1)) * scale.float().unsqueeze(-1)
    return w.reshape(N, K).to(dtype)


def marlin_perm():
    """The 1024-entry weight permutation and the two scale permutations of
    fast_dequant/simple_marlin/utils.py:20-46."""
    perm = []
    for i in range(32):
        col = i // 4
        perm1 = [16 * row + col + 8 * block
                 for block in (0, 1)
                 for row in (2 * (i % 4), 2 * (i % 4) + 1, 2 * (i % 4 + 4), 2 * (i % 4 + 4) + 1)]
        for j in range(4):
            perm.extend(p + 256 * j for p in perm1)
    perm = torch.tensor(perm).reshape(-1, 8)[:, [0, 2, 4, 6, 1, 3, 5, 7]].reshape(-1)
    scale_perm = [i + 8 * j for i in range(8) for j in range(8)]
    scale_perm_single = [2 * i + j for i in range(4) for j in (0, 1, 8, 9, 16, 17, 24, 25)]
    return perm, scale_perm, scale_perm_single


def marlin_pack(q_kn: torch.Tensor, scale: torch.Tensor, groupsize: int = -1):
    """fast_dequant/simple_marlin/utils.py:53-95: q int32 [K,N] -> int32
    [K/16, N*16/8]; scales permuted with the grouped or single permutation."""
    perm, sp, sps = marlin_perm()
    K, N = q_kn.shape
    sc = scale.reshape(1, -1)
    p = sp if groupsize != -1 else sps
    sc = sc.reshape(-1, len(p))[:, p].reshape(-1, N).contiguous()
    w = q_kn.reshape(K // 16, 16, N // 16, 16).permute(0, 2, 1, 3).reshape(K // 16, N * 16)
    w = w.reshape(-1, perm.numel())[:, perm].reshape(w.shape).to(torch.int64)
    out = torch.zeros(w.shape[0], w.shape[1] // 8, dtype=torch.int64)
    for i in range(8):
        out |= w[:, i::8] << (4 * i)
    return _wrap(out, 32), sc
