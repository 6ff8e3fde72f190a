"""CPU-only checks: the C-ABI library builds, loads and exports what include/b200moe.h
declares; host-side argument validation; the expert-parallel exchange plumbing under gloo."""
import os
import re
import subprocess
import sys

import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module")
def native():
    from llm_kernels_b200 import build, _native
    build.build()
    return _native


def test_library_exports_every_declared_symbol(native):
    header = open(os.path.join(ROOT, "include", "b200moe.h")).read()
    declared = set(re.findall(r"\b(b200moe_[a-z0-9_]+)\s*\(", header))
    assert declared, "no declarations found"
    lib = native.lib()
    for name in sorted(declared):
        assert hasattr(lib, name), f"{name} declared in b200moe.h but not exported"
    assert declared == set(native.SIGNATURES), "ctypes table and header disagree"
    assert lib.b200moe_abi_version() == 2
    assert lib.b200moe_status_string(0) == b"ok"


def test_argument_validation_without_a_gpu(native):
    lib = native.lib()
    # cols not a multiple of 128 -> BAD_SHAPE before any CUDA call
    assert lib.b200moe_act_quant_fp8(16, native.BF16, 4, 100, 16, 100, 16, 1, None) == 1
    assert b"divisible by block_size" in lib.b200moe_last_error()
    assert lib.b200moe_router_topk(16, native.BF16, 16, None, 4, 128, 8, 2, 8, 4, 0, 1, 1.0, 16, 16, None) == 1
    assert lib.b200moe_route_metadata_workspace_bytes(32768, 256) == 32 * 256 * 4
    assert lib.b200moe_pack_bits(16, 16, 8, 8, 3, 32, 1, None) == 4
    assert lib.b200moe_gemm_fp8_block(16, 16, 16, 16, 16, native.BF16, 128, 100, 128, None) == 1
    assert lib.b200moe_gemm_fp8_block(None, 16, 16, 16, 16, native.BF16, 128, 128, 128, None) == 4
    with pytest.raises(AssertionError):
        native.check(1)


def test_operators_refuse_cpu_tensors(native):
    from llm_kernels_b200.quantization import fp8_kernel, bitpack
    from llm_kernels_b200.moe import group_gemm_kernel as G
    with pytest.raises(RuntimeError):
        fp8_kernel.act_quant(torch.zeros(2, 128))
    with pytest.raises(RuntimeError):
        bitpack.pack_weights_over_rows(torch.zeros(8, 8, dtype=torch.uint8), 4, 32)
    with pytest.raises(RuntimeError):
        G.run_moe_ep_preproess(torch.zeros(4, 2, dtype=torch.int64), 8)


def test_config_attribute_surface():
    from llm_kernels_b200.moe.config import Config
    c = Config()
    for name in ["hidden_size", "moe_intermediate_size", "n_routed_experts", "num_experts_per_tok",
                 "routed_scaling_factor", "scoring_func", "topk_method", "n_group", "topk_group",
                 "norm_topk_prob", "n_shared_experts", "ep_size", "hidden_act", "use_triton_group_gemm",
                 "quantize_method", "use_block_quant", "w_quant_block_size", "a_quant_block_size",
                 "w_bit", "a_bit", "w_dtype", "a_dtype"]:
        assert hasattr(c, name), name


def test_compare_tensors_metric():
    from llm_kernels_b200.moe.utils import ResultAnalyzer
    a = torch.randn(8, 16)
    r = ResultAnalyzer.compare_tensors(a, a + 1e-5)
    assert r["is_equivalent"] and r["min_sim_val"] > 0.999


_WORKER = r'''
import os, sys, torch, torch.distributed as dist
sys.path.insert(0, sys.argv[1])
from llm_kernels_b200.moe import ep_comm
from oracle import restate as R
rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
dist.init_process_group("gloo", rank=rank, world_size=world)
E, k, H, T = 8, 2, 16, 20 + 7 * rank           # ragged: ranks hold different token counts
g = torch.Generator().manual_seed(100 + rank)
x = torch.randn(T, H, generator=g)
ids = torch.rand(T, E, generator=g).topk(k, dim=-1)[1]
w = torch.rand(T, k, generator=g)
_, s2d, seg = R.run_moe_ep_preproess(ids, E)
send = torch.empty(T * k, H)
send[s2d.long()] = x.repeat_interleave(k, 0)
plan = ep_comm.plan_exchange(seg, world)
recv = torch.empty(plan.recv_rows, H)
ep_comm.dispatch(plan, send, recv)
# "expert" e multiplies by (e + 1): every received run must reach the right local expert
El = E // world
out = torch.empty_like(recv)
sg = plan.seg_indptr.tolist()
for gi, le in enumerate(plan.weight_indices.tolist()):
    out[sg[gi]:sg[gi + 1]] = recv[sg[gi]:sg[gi + 1]] * (rank * El + le + 1)
back = torch.empty(T * k, H)
ep_comm.combine(plan, out, back)
y = (back[s2d.long()].view(T, k, H) * w.unsqueeze(-1)).sum(1)
want = (x.unsqueeze(1) * (ids + 1).unsqueeze(-1).float() * w.unsqueeze(-1)).sum(1)
assert plan.recv_counts.shape == (world, El)
assert int(plan.seg_indptr[-1]) == plan.recv_rows
torch.testing.assert_close(y, want, rtol=1e-5, atol=1e-5)
# total rows conserved across the job
tot = torch.tensor([plan.recv_rows, T * k]); dist.all_reduce(tot)
assert int(tot[0]) == int(tot[1])
# pipelined plan: experts visited in (pass, owner, expert-in-pass) order, 2 passes
P = 2
order = ep_comm.expert_order(E, world, P, "cpu")
ids_r = order[ids]
_, s2d, seg = R.run_moe_ep_preproess(ids_r, E)
send = torch.empty(T * k, H)
send[s2d.long()] = x.repeat_interleave(k, 0)
pp = ep_comm.plan_exchange_pipelined(seg, world, P)
recv = torch.empty(pp.recv_rows, H)
out = torch.empty_like(recv)
back = torch.empty(T * k, H)
Ep = El // P
sg = pp.seg_indptr.tolist()
for p in range(P):
    ep_comm.dispatch_pass(pp, p, send, recv)
    for gi in range(p * pp.groups_per_pass, (p + 1) * pp.groups_per_pass):
        le = int(pp.weight_indices[gi])
        assert p * Ep <= le < (p + 1) * Ep
        out[sg[gi]:sg[gi + 1]] = recv[sg[gi]:sg[gi + 1]] * (rank * El + le + 1)
    ep_comm.combine_pass(pp, p, out, back)
y = (back[s2d.long()].view(T, k, H) * w.unsqueeze(-1)).sum(1)
torch.testing.assert_close(y, want, rtol=1e-5, atol=1e-5)
assert sg[-1] == pp.recv_rows == pp.recv_off[-1]
# merged view: gather_map brings every expert's rows from all sources together
merged = recv[pp.gather_map.long()]
ms = pp.merged_seg.tolist()
out2 = torch.empty_like(recv)
for gi, le in enumerate(pp.merged_widx.tolist()):
    out2[pp.gather_map.long()[ms[gi]:ms[gi + 1]]] = merged[ms[gi]:ms[gi + 1]] * (rank * El + le + 1)
assert ms[-1] == pp.recv_rows and sorted(pp.gather_map.tolist()) == list(range(pp.recv_rows))
torch.testing.assert_close(out2, out)
# pushed-exchange plan: offsets must describe the same layout as the all-to-all plan
pl = ep_comm.plan_push(seg, world, P, rank)
assert pl.base.in_splits == pp.in_splits and pl.base.out_splits == pp.out_splits
assert torch.equal(pl.base.gather_map, pp.gather_map) and torch.equal(pl.base.merged_seg, pp.merged_seg)
# gather every rank's view of the offsets and cross-check: what I think I write at peer d must be
# where d expects rows from me, and the back offsets must mirror the peers' send offsets
mine = torch.tensor([pl.dst_off, pl.src_off, pl.back_off, pl.mine_off])          # [4, P, world]
allv = [torch.empty_like(mine) for _ in range(world)]
dist.all_gather(allv, mine)
for p in range(P):
    for d in range(world):
        assert pl.dst_off[p][d] == int(allv[d][3][p][rank]), "dispatch offset mismatch"
        assert pl.back_off[p][d] == int(allv[d][1][p][rank]), "combine offset mismatch"
dist.destroy_process_group()
print("OK", rank)
'''


def test_ep_exchange_world_size_2_gloo(tmp_path):
    script = tmp_path / "worker.py"
    script.write_text(_WORKER)
    port = 29500 + os.getpid() % 1000
    procs = []
    for r in range(2):
        env = dict(os.environ, RANK=str(r), WORLD_SIZE="2", MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
        procs.append(subprocess.Popen([sys.executable, str(script), ROOT], env=env, stdout=subprocess.PIPE,
                                      stderr=subprocess.STDOUT, text=True))
    for p in procs:
        out, _ = p.communicate(timeout=180)
        assert p.returncode == 0, out


def test_marlin_quantutils_match_reference_vectors(golden):
    """fast_dequant/simple_marlin/utils.py:53-136 on CPU tensors: bit-exact against the reference's output."""
    import numpy as np
    from llm_kernels_b200.fast_dequant.simple_marlin.utils import QuantUtils
    for tag, gs in (("marlin_g128", 128), ("marlin_g-1", -1)):
        c = golden.case(tag)
        f = lambda k, dt: torch.from_numpy(np.ascontiguousarray(c[k])).to(dt)
        ref, q, sc = QuantUtils.fake_quantize(f("w", torch.float16), gs)
        assert torch.equal(ref, f("ref", torch.float16)) and torch.equal(q, f("q", torch.int32))
        assert torch.equal(sc, f("scale", torch.float16))
        pk, ps = QuantUtils.pack(q, sc, gs)
        assert torch.equal(pk, f("packed", torch.int32)) and torch.equal(ps, f("packed_scale", torch.float16))


def test_marlin_mul_rejects_like_the_reference_binding():
    """Argument checks of fast_dequant/simple_marlin/marlin_w4a16_gemm.cpp:38-88 happen before any launch,
    so they can be exercised without a GPU."""
    import pytest
    from llm_kernels_b200.fast_dequant.simple_marlin import mul
    A = torch.zeros(16, 128, dtype=torch.half)
    B = torch.zeros(8, 128, dtype=torch.int32)
    C = torch.zeros(16, 64, dtype=torch.half)
    s = torch.ones(1, 64, dtype=torch.half)
    with pytest.raises(RuntimeError, match="divisible by 16"):
        mul(A[:15], B, C[:15], s, None)
    with pytest.raises(RuntimeError, match="same CUDA device"):
        mul(A, B, C, s, None)                   # CPU tensors: there is no CPU path


def test_operators_refuse_tensors_of_another_device(native, monkeypatch):
    """require_cuda: a tensor that lives on a GPU other than the current one must raise before any launch
    (the launchers use the current device's stream; a foreign pointer would be dereferenced on the wrong GPU)."""
    from types import SimpleNamespace
    monkeypatch.setattr(torch.cuda, "current_device", lambda: 0)
    here = SimpleNamespace(is_cuda=True, device=SimpleNamespace(index=0))
    there = SimpleNamespace(is_cuda=True, device=SimpleNamespace(index=1))
    native.require_cuda(here, None, here)
    with pytest.raises(RuntimeError, match="current device"):
        native.require_cuda(here, there)


def test_sglang_mirror_exports_grouped_gemm_runner():
    """The reference's EPMoE builds `GroupedGemmRunner(device)` and calls it with grouped_gemm_triton's argument
    order (moe/sglang_moe_all_gather_all_reduce.py:25-55); the mirror module exports the same class."""
    import inspect
    from llm_kernels_b200.moe import sglang_moe_all_gather_all_reduce as M
    r = M.GroupedGemmRunner("cuda")
    assert isinstance(r, torch.nn.Module) and r.use_flashinfer is False
    names = list(inspect.signature(r.forward).parameters)
    assert names == ["a", "b", "c", "batch_size", "weight_column_major", "seg_indptr", "weight_indices",
                     "use_fp8_w8a8", "scale_a", "scale_b", "block_shape"]
    with pytest.raises(RuntimeError):          # CPU tensors are refused like everywhere else
        z = torch.zeros(2, 128, dtype=torch.float16)
        r(z, torch.zeros(1, 128, 128, dtype=torch.float16), torch.zeros(2, 128, dtype=torch.float16), 1, True,
          torch.tensor([0, 2]))


_QAR_WORKER = r'''
import os, sys, torch, torch.distributed as dist
sys.path.insert(0, sys.argv[1])
from llm_kernels_b200.moe import ep_comm
from oracle import restate as R
rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
dist.init_process_group("gloo", rank=rank, world_size=world)
T, H = 37, 256                                   # 37 rows: not a multiple of the rank count -> padded chunk
xs = []
for r in range(world):                           # every rank can rebuild every rank's input (seeded)
    g = torch.Generator().manual_seed(500 + r)
    t = torch.randn(T, H, generator=g).to(torch.bfloat16)
    t[3 + r] = 0                                 # an all-zero row: zero scale, NaN payload, must decode to zero
    xs.append(t)
for kind in ("int8", "fp8"):
    x = xs[rank].clone()
    quant = lambda t: R.comm_quant(t, kind)
    def dsum(q, s, out):
        out.copy_(R.comm_dequant_sum(q, s, out.dtype))
    ep_comm.quant_allreduce(x, quant, dsum)
    want = R.quant_allreduce(xs, kind)           # the scheme with the ranks simulated in one process
    assert torch.equal(x, want), kind
    exact = sum(t.float() for t in xs)
    if kind == "int8":                           # the reference's own acceptance test (quant_all2all_allreduce.py:104)
        assert torch.allclose(x.float(), exact, rtol=1e-2, atol=1e-1)
    else:                                        # e4m3 keeps 3 mantissa bits, twice: a few per cent
        assert R.rel_fro(x.float(), exact) < 6e-2
    assert not bool(x.isnan().any())
dist.destroy_process_group()
print("OK", rank)
'''


@pytest.mark.parametrize("world", [2, 3])
def test_quantized_allreduce_plumbing_gloo(tmp_path, world):
    """ep_comm.quant_allreduce (all-to-all of quantized chunks, local sum, re-quantize, all-gather) on gloo ranks
    with the oracle's quantizers plugged in: identical to the oracle's in-process simulation of the scheme."""
    script = tmp_path / "qar_worker.py"
    script.write_text(_QAR_WORKER)
    port = 29500 + (os.getpid() + 17 * world) % 1000
    procs = []
    for r in range(world):
        env = dict(os.environ, RANK=str(r), WORLD_SIZE=str(world), MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
        procs.append(subprocess.Popen([sys.executable, str(script), ROOT], env=env, stdout=subprocess.PIPE,
                                      stderr=subprocess.STDOUT, text=True))
    for p in procs:
        out, _ = p.communicate(timeout=180)
        assert p.returncode == 0, out


def test_raw_nibble_range_check_of_the_fused_w4a8_path():
    """DeepseekV3MoE._raw_nibbles_ok decides whether the fused w4a8 GEMM (raw nibbles on the tensor core, (q - z4) * s4
    applied to the dot product) may serve a weight: it must accept the reference quantizer's output
    (quantization/w4a8_kernel.py:228-262) and reject a weight whose (q - z4) * s4 leaves int8 for a nibble it holds
    (the reference casts that product to int8, :362-380).  Pure tensor arithmetic: runs on the host."""
    from types import SimpleNamespace
    from oracle import restate as R
    from llm_kernels_b200.moe.all2all_moe import DeepseekV3MoE
    g = torch.Generator().manual_seed(5)
    packed, _, s4, z4 = R.w4a8_weight_quant(torch.randn(256, 512, generator=g) * 0.05)[:4]
    fake = SimpleNamespace(w13_qweight=packed[None].clone(), w13_s4=s4[None].clone(), w13_z4=z4[None].clone(),
                           _buffers_cache={})
    assert DeepseekV3MoE._raw_nibbles_ok(fake, "w13")
    fake.w13_s4[0, 0, 0] = 127
    fake.w13_z4[0, 0, 0] = 0
    fake.w13_qweight[0, 0, 0] |= 0xF                       # a nibble 15 in that scale group: 15 * 127 wraps in int8
    assert not DeepseekV3MoE._raw_nibbles_ok(fake, "w13")
    fake.w13_qweight[0, 0, :128] &= ~0xF                   # no nibble above 0 left in the group: (0 - 0) * 127 fits
    assert DeepseekV3MoE._raw_nibbles_ok(fake, "w13")
