"""Generate tests/golden/reference_vectors.npz by RUNNING the reference.

Usage:  python tests/golden/make_golden.py --reference <path to the reference checkout>

The reference checkout is imported as-is (its moe/ and quantization/ folders
are put on sys.path exactly as its own scripts do).  Its Triton kernels are
executed on CPU through Triton's interpreter (TRITON_INTERPRET=1); its torch
code runs natively.  ResultCollector.save (which writes .pt files on every
forward) is replaced by a no-op.  Nothing here is needed at test time: the
tests read only the committed .npz.

Every array is stored with a key "<case>/<name>"; bf16/fp16 tensors are stored
as float32, fp8 tensors as their uint8 bit patterns.
"""
import argparse
import os
import sys

os.environ["TRITON_INTERPRET"] = "1"

import numpy as np
import torch


def _np(t: torch.Tensor):
    if t.dtype in (torch.float8_e4m3fn,):
        return t.view(torch.uint8).numpy()
    if t.dtype in (torch.bfloat16, torch.float16):
        return t.float().numpy()
    return t.detach().cpu().numpy()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", required=True)
    ap.add_argument("--out", default=os.path.join(os.path.dirname(os.path.abspath(__file__)),
                                                  "reference_vectors.npz"))
    args = ap.parse_args()
    ref = os.path.abspath(args.reference)
    for sub in ("", "quantization", "moe"):
        sys.path.insert(0, os.path.join(ref, sub))

    import utils as ref_moe_utils
    ref_moe_utils.ResultCollector.save = staticmethod(lambda *a, **k: None)
    import all2all_moe as ref_a2a
    import group_gemm_kernel as ref_ggk
    import sglang_moe_all_gather_all_reduce as ref_epmoe
    import fp8_kernel as ref_fp8
    import bitpack as ref_bitpack
    import w4a8_kernel as ref_w4a8
    from config import Config

    out = {}

    def put(case, **kw):
        for k, v in kw.items():
            out[f"{case}/{k}"] = _np(v) if isinstance(v, torch.Tensor) else np.asarray(v)

    # ---------------- MoEGate.forward (moe/all2all_moe.py:60-118) ----------------
    for case, (T, H, E, k, ng, tg, scale, seed) in {
        "gate_small": (48, 64, 16, 4, 4, 2, 2.5, 11),
        "gate_v3": (24, 128, 256, 8, 8, 4, 2.5, 12),
        "gate_flat": (40, 96, 8, 2, 1, 1, 1.0, 13),
    }.items():
        g = torch.Generator().manual_seed(seed)
        cfg = Config()
        cfg.hidden_size, cfg.n_routed_experts, cfg.num_experts_per_tok = H, E, k
        cfg.n_group, cfg.topk_group, cfg.routed_scaling_factor = ng, tg, scale
        gate = ref_a2a.MoEGate(cfg).eval()
        W = torch.randn(E, H, generator=g) * 0.3
        bias = torch.rand(E, generator=g) * 0.2
        x = torch.randn(1, T, H, generator=g).to(torch.bfloat16)
        with torch.no_grad():
            gate.weight.copy_(W)
            gate.e_score_correction_bias.copy_(bias)
            idx, w = gate(x)
        put(case, x=x[0], W=W, bias=bias, topk_idx=idx, topk_weight=w,
            params=np.array([k, ng, tg], dtype=np.int64), scale=np.float64(scale))

    # ---------------- DeepseekV3MoE.forward, ep_size=1 (moe/all2all_moe.py:167-280) ----
    g = torch.Generator().manual_seed(21)
    cfg = Config()
    cfg.hidden_size, cfg.moe_intermediate_size = 64, 32
    cfg.n_routed_experts, cfg.num_experts_per_tok = 8, 2
    cfg.n_group, cfg.topk_group, cfg.routed_scaling_factor = 1, 1, 1.0
    cfg.n_shared_experts = None
    cfg.ep_size = 1
    model = ref_a2a.DeepseekV3MoE(cfg).eval()
    with torch.no_grad():
        model.gate.weight.copy_(torch.randn(8, 64, generator=g) * 0.3)
        gw = torch.randn(8, 32, 64, generator=g) * 0.1
        uw = torch.randn(8, 32, 64, generator=g) * 0.1
        dw = torch.randn(8, 64, 32, generator=g) * 0.1
        for e in range(8):
            model.experts[e].gate_proj.weight.copy_(gw[e])
            model.experts[e].up_proj.weight.copy_(uw[e])
            model.experts[e].down_proj.weight.copy_(dw[e])
        x = torch.randn(2, 20, 64, generator=g)
        idx, w = model.gate(x)
        y = model(x)
    put("moe_dense", x=x.view(-1, 64), gate_W=model.gate.weight.detach(), gate_w=gw, up_w=uw,
        down_w=dw, topk_idx=idx, topk_weight=w, y=y.view(-1, 64))

    # ---------------- same with shared experts (moe/all2all_moe.py:161-165, 182-183) ----
    cfg.n_shared_experts = 2
    model_s = ref_a2a.DeepseekV3MoE(cfg).eval()
    g2 = torch.Generator().manual_seed(22)
    with torch.no_grad():
        model_s.gate.weight.copy_(model.gate.weight)
        for e in range(8):
            model_s.experts[e].gate_proj.weight.copy_(gw[e])
            model_s.experts[e].up_proj.weight.copy_(uw[e])
            model_s.experts[e].down_proj.weight.copy_(dw[e])
        sg = torch.randn(64, 64, generator=g2) * 0.1
        su = torch.randn(64, 64, generator=g2) * 0.1
        sd = torch.randn(64, 64, generator=g2) * 0.1
        model_s.shared_experts.gate_proj.weight.copy_(sg)
        model_s.shared_experts.up_proj.weight.copy_(su)
        model_s.shared_experts.down_proj.weight.copy_(sd)
        y_s = model_s(x)
    put("moe_dense_shared", shared_gate_w=sg, shared_up_w=su, shared_down_w=sd, y=y_s.view(-1, 64))

    # ---------------- EPMoE.forward, one rank, fp16, unquantized ---------------------------
    # (moe/sglang_moe_all_gather_all_reduce.py:267-446: gate -> run_moe_ep_preproess -> pre_reorder ->
    #  grouped GEMM -> silu_and_mul -> grouped GEMM -> post_reorder, its Triton kernels interpreted)
    import sglang_moe_all_gather_all_reduce as ref_ep
    cfg_e = Config()
    cfg_e.hidden_size, cfg_e.moe_intermediate_size = 64, 32
    cfg_e.n_routed_experts, cfg_e.num_experts_per_tok = 8, 2
    cfg_e.n_group, cfg_e.topk_group, cfg_e.routed_scaling_factor = 1, 1, 1.0
    cfg_e.n_shared_experts, cfg_e.ep_size = None, 1
    cfg_e.quantize_method, cfg_e.use_block_quant = None, False
    torch.set_default_dtype(torch.float16)
    epmoe = ref_ep.EPMoE(cfg_e).eval()
    torch.set_default_dtype(torch.float32)
    ge = torch.Generator().manual_seed(31)
    with torch.no_grad():
        epmoe.gate.weight.copy_(torch.randn(8, 64, generator=ge) * 0.3)
        epmoe.w13_weight.copy_((torch.randn(8, 64, 64, generator=ge) * 0.1).half())
        epmoe.w2_weight.copy_((torch.randn(8, 64, 32, generator=ge) * 0.1).half())
        xe = torch.randn(1, 24, 64, generator=ge).half()
        ie, we = epmoe.gate(xe)
        ye = epmoe(xe)
    put("epmoe_fp16", x=xe[0], gate_W=epmoe.gate.weight.detach(), w13=epmoe.w13_weight.detach(),
        w2=epmoe.w2_weight.detach(), topk_idx=ie, topk_weight=we, y=ye[0])

    # ---------------- run_moe_ep_preproess (moe/group_gemm_kernel.py:48-78) -----------
    for case, (T, k, E, seed) in {"prep_small": (6, 2, 4, 31), "prep_skew": (200, 8, 64, 32),
                                  "prep_empty_experts": (33, 2, 32, 33)}.items():
        g = torch.Generator().manual_seed(seed)
        logits = torch.randn(T, E, generator=g)
        if case == "prep_skew":
            logits[:, :4] += 3.0
        if case == "prep_empty_experts":
            logits[:, 5:20] -= 100.0
        ids = logits.topk(k, dim=-1)[1]
        r_ids, s2d, seg = ref_ggk.run_moe_ep_preproess(ids, E)
        put(case, topk_ids=ids, reorder_topk_ids=r_ids, src2dst=s2d, seg_indptr=seg,
            num_experts=np.int64(E))

    # ---------------- reorder / activation / combine kernels --------------------------
    g = torch.Generator().manual_seed(41)
    T, k, E, H, I = 10, 2, 8, 48, 40
    ids = torch.randn(T, E, generator=g).topk(k, dim=-1)[1]
    tw = torch.rand(T, k, generator=g)
    r_ids, s2d, seg = ref_ggk.run_moe_ep_preproess(ids, E)
    x = torch.randn(T, H, generator=g).to(torch.float16)
    for name, (lo, hi) in {"all": (0, 7), "part": (2, 5)}.items():
        buf = torch.zeros(T * k, H, dtype=torch.float16)
        ref_ggk.pre_reorder_triton_kernel[(T,)](x, buf, s2d, ids, None, lo, hi, k, H, BLOCK_SIZE=512)
        gu = (torch.randn(T * k, 2 * I, generator=g)).to(torch.float16)
        d_silu = torch.zeros(T * k, I, dtype=torch.float16)
        ref_ggk.silu_and_mul_triton_kernel[(T * k,)](gu, d_silu, 2 * I, r_ids, None, lo, hi, BLOCK_SIZE=512)
        d_gelu = torch.zeros(T * k, I, dtype=torch.float16)
        ref_ggk.gelu_and_mul_triton_kernel[(T * k,)](gu, d_gelu, 2 * I, r_ids, None, lo, hi, BLOCK_SIZE=512)
        down = torch.randn(T * k, H, generator=g).to(torch.float16)
        o = torch.full((T, H), 7.0, dtype=torch.float16)
        ref_ggk.post_reorder_triton_kernel[(T,)](down, o, s2d, ids, tw, lo, hi, k, H, BLOCK_SIZE=512)
        put(f"reorder_{name}", x=x, topk_ids=ids, topk_weights=tw, src2dst=s2d,
            reorder_topk_ids=r_ids, lohi=np.array([lo, hi]), pre=buf, gateup=gu, silu=d_silu,
            gelu=d_gelu, down=down, post=o)

    # ---------------- grouped GEMM: Triton fp16 branch and the torch twin -------------
    g = torch.Generator().manual_seed(51)
    Eg, N, K = 4, 96, 128
    seg = torch.tensor([0, 5, 5, 70, 97], dtype=torch.int64)
    a = (torch.randn(97, K, generator=g) * 0.5).to(torch.float16)
    b = (torch.randn(Eg, N, K, generator=g) * 0.1).to(torch.float16)
    widx = torch.tensor([2, 0, 3, 1], dtype=torch.int64)
    c = torch.zeros(97, N, dtype=torch.float16)
    ref_ggk.grouped_gemm_triton(a, b, c, Eg, True, seg, widx)
    c2 = torch.zeros(97, N, dtype=torch.float16)
    ref_epmoe.grouped_gemm_pytorch(a, b, c2, Eg, seg, widx)
    put("ggemm_fp16", a=a, b=b, seg_indptr=seg, weight_indices=widx, c_triton=c, c_torch=c2)

    # ---------------- fp8: act_quant scales, weight_dequant, blockwise GEMM ----------
    g = torch.Generator().manual_seed(61)
    x = torch.randn(6, 384, generator=g).to(torch.bfloat16)
    x[1, 128:256] = 0.0                                   # amax == 0 group
    _, s_ref = ref_fp8.act_quant(x)                       # interpreter: scales are exact,
    put("fp8_act", x=x, s=s_ref)                          # its e4m3 cast is not (see test)
    M, N, K = 40, 256, 256
    aq = (torch.randn(M, K, generator=g) * 100).clamp(-448, 448).to(torch.float8_e4m3fn)
    bq = (torch.randn(N, K, generator=g) * 100).clamp(-448, 448).to(torch.float8_e4m3fn)
    a_s = torch.rand(M, K // 128, generator=g) * 0.01 + 1e-3
    b_s = torch.rand(N // 128, K // 128, generator=g) * 0.01 + 1e-3
    cc = torch.empty(M, N, dtype=torch.float32)
    ref_fp8.fp8_gemm_kernel.fn[(M // 16 + 1, N // 64)](aq, bq, cc, a_s, b_s, M, N, K,
                                                       BLOCK_SIZE_M=16, BLOCK_SIZE_N=64, BLOCK_SIZE_K=128)
    wd = torch.empty(N, K, dtype=torch.float32)
    ref_fp8.weight_dequant_kernel[(N // 128, K // 128)](bq, b_s, wd, N, K, BLOCK_SIZE=128)
    put("fp8_gemm", a=aq, a_s=a_s, b=bq, b_s=b_s, c=cc, b_dequant=wd)

    # ---------------- bitpack (quantization/bitpack.py) -------------------------------
    g = torch.Generator().manual_seed(71)
    # 64-bit words are left out: the reference shifts in int32 there (bitpack.py:14, 25-28)
    for nbits, width in ((4, 32), (4, 8), (2, 16), (8, 32), (1, 8)):
        Wq = torch.randint(0, 2 ** nbits, (64, 128), generator=g, dtype=torch.int32).to(torch.uint8)
        pr_t, e = ref_bitpack.pack_weights_over_rows_torch(Wq, nbits, width, False)
        pc_t, _ = ref_bitpack.pack_weights_over_cols_torch(Wq, nbits, width, False)
        case = f"bitpack_{nbits}_{width}"
        put(case, W=Wq, rows=pr_t, cols=pc_t, e=np.int64(e))
        if width <= 32:
            pr, _ = ref_bitpack.pack_weights_over_rows(Wq, nbits, width, False)
            pc, _ = ref_bitpack.pack_weights_over_cols(Wq, nbits, width, False)
            assert torch.equal(pr, pr_t) and torch.equal(pc, pc_t)
            assert torch.equal(ref_bitpack.unpack_over_rows(pr, nbits, 64), Wq)
            assert torch.equal(ref_bitpack.unpack_over_cols(pc, nbits, 128), Wq)

    # ---------------- two-level int4 (quantization/w4a8_kernel.py) -------------------
    g = torch.Generator().manual_seed(81)
    w = torch.randn(256, 256, generator=g) * 0.02
    packed, s, s4, z4 = ref_w4a8.weight_quant(w)
    deq = ref_w4a8.weight_dequant(packed, s, s4, z4)
    xa = torch.randn(24, 256, generator=g)
    a8, a8s = ref_w4a8.act_quant(xa)
    M, N, K = 24, 256, 256
    c = torch.empty(M, N, dtype=torch.float32)
    ref_w4a8.w4a8_gemm_kernel.fn[(M // 16 + 1, N // 64)](
        a8, packed, c, a8s, s, s4, z4, M, N, K, 128,
        BLOCK_SIZE_M=16, BLOCK_SIZE_N=64, BLOCK_SIZE_K=128,
        elements_per_sample=8, w_bits=4, unpack_mask=15)
    put("w4a8", w=w, packed=packed, s=s, s4=s4, z4=z4, dequant=deq, x=xa, a8=a8, a8s=a8s, c=c)

    # ---------------- Marlin-order int4 (fast_dequant/simple_marlin/utils.py) --------
    import importlib.util
    spec = importlib.util.spec_from_file_location(
        "ref_marlin_utils", os.path.join(ref, "fast_dequant", "simple_marlin", "utils.py"))
    mu = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mu)
    g = torch.Generator().manual_seed(91)
    wkn = (torch.randn(256, 128, generator=g) * 0.05).half()
    for gs in (128, -1):
        refw, q, sc = mu.QuantUtils.fake_quantize(wkn, gs)
        pk, psc = mu.QuantUtils.pack(q, sc, gs)
        put(f"marlin_g{gs}", w=wkn, ref=refw, q=q, scale=sc, packed=pk, packed_scale=psc)

    np.savez_compressed(args.out, **out)
    print(f"wrote {args.out}: {len(out)} arrays, {os.path.getsize(args.out)} bytes")


if __name__ == "__main__":
    main()
