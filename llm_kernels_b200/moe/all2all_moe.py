"""Expert-parallel quantized MoE layer with the call surface of the reference's
moe/all2all_moe.py: ``MoEGate(config).forward(h) -> (topk_idx, topk_weight)`` (:60-118)
and ``DeepseekV3MoE(config).forward(hidden_states[B,S,H]) -> [B,S,H]`` (:167-184).

Where the reference runs a per-expert Python loop (``moe_infer``, :186-280) and leaves
its fused path as a stub (``triton_group_gemm_moe_infer``, :282-286), this module runs
one fused pipeline of sm_100a kernels:

    router_topk -> route_metadata -> permute + 1x128 e4m3 quantize
      -> [dispatch of fp8 rows + scales, one packed record per row]
      -> grouped GEMM-1 (tcgen05) with SwiGLU + re-quantize in the epilogue
      -> grouped GEMM-2 (tcgen05)
      -> [return of bf16 rows to their source ranks]
      -> routing-weighted un-permute (f32 accumulate)

With expert parallelism the two bracketed steps are, by default, part of the kernels next to them
(config.ep_exchange = "fused": the permute kernel copies each record into its owner's peer-mapped
buffer and the second GEMM stores each output row into its source rank's buffer, both over NVLink);
"nccl" runs them as all_to_all_single calls like the reference, "push" as copy-engine peer copies.

Experts are sharded as in the reference (:130-147): rank r owns experts
[r*E/ep, (r+1)*E/ep).  Expert weights live in the fused layout of the reference's
grouped path (moe/sglang_moe_all_gather_all_reduce.py:208-264): w13 [E_l, 2I, H] =
[gate ; up], w2 [E_l, H, I], both e4m3 with f32 128x128 block scales.
"""
import math
from typing import Optional

import torch
import torch.distributed as dist
from torch import nn

from .. import _native as N
from ..quantization import fp8_kernel, w4a8_kernel, w4a16_kernel
from . import ep_comm
from . import group_gemm_kernel as G
from .config import Config  # noqa: F401  (re-exported like the reference does)
from .utils import ResultCollector  # noqa: F401


class DeepseekV3MLP(nn.Module):
    """reference :13-29: ``down_proj(act_fn(gate_proj(x)) * up_proj(x))`` with three bias-free
    nn.Linear layers (weights [out, in]).  Same constructor and parameter names; the forward pass
    of a bf16 module on the GPU is two tcgen05 GEMMs, the first with SiLU(gate)*up fused in its
    epilogue with the roundings a bf16 torch module produces."""

    def __init__(self, config, hidden_size=None, intermediate_size=None):
        super().__init__()
        self.config = config
        self.hidden_size = config.hidden_size if hidden_size is None else hidden_size
        self.intermediate_size = config.intermediate_size if intermediate_size is None else intermediate_size
        self.hidden_act = getattr(config, "hidden_act", "silu")
        if self.hidden_act not in ("silu", "gelu"):
            raise NotImplementedError(f"hidden_act {self.hidden_act!r}: the fused epilogues implement silu and gelu")
        self.gate_proj = nn.Linear(self.hidden_size, self.intermediate_size, bias=False)
        self.up_proj = nn.Linear(self.hidden_size, self.intermediate_size, bias=False)
        self.down_proj = nn.Linear(self.intermediate_size, self.hidden_size, bias=False)
        self._w13_key = None

    def _fused_gate_up(self):
        g, u = self.gate_proj.weight, self.up_proj.weight
        key = (g.data_ptr(), g._version, u.data_ptr(), u._version)
        if self._w13_key != key:
            self._w13 = torch.cat([g.detach(), u.detach()], dim=0).unsqueeze(0).contiguous()
            self._w13_key = key
        return self._w13

    @torch.no_grad()
    def forward(self, x):
        N.require_cuda(x, self.gate_proj.weight)
        assert x.dtype == torch.bfloat16 and self.gate_proj.weight.dtype == torch.bfloat16, \
            "DeepseekV3MLP runs as a bfloat16 module (module.to(torch.bfloat16))"
        H, I = self.hidden_size, self.intermediate_size
        assert H % 128 == 0 and I % 128 == 0, "hidden and intermediate sizes must be multiples of 128"
        x2 = x.reshape(-1, H)
        if not x2.is_contiguous():
            x2 = x2.contiguous()
        M = x2.shape[0]
        seg = torch.tensor([0, M], dtype=torch.int64, device=x.device)
        h = torch.empty(M, I, dtype=torch.bfloat16, device=x.device)
        G.grouped_gemm_bf16(x2, self._fused_gate_up(), seg, None, h, epilogue=2 if self.hidden_act == "silu" else 5)
        y = torch.empty(M, H, dtype=torch.bfloat16, device=x.device)
        G.grouped_gemm_bf16(h, self.down_proj.weight.detach().unsqueeze(0), seg, None, y, epilogue=0)
        return y.view(*x.shape[:-1], H)


class MoEGate(nn.Module):
    """Router (reference :31-118): f32 logits, sigmoid (or softmax) scores, optional
    e_score_correction_bias, group-limited top-k, renormalisation, scaling."""

    def __init__(self, config):
        super().__init__()
        self.config = config
        self.top_k = config.num_experts_per_tok
        self.n_routed_experts = config.n_routed_experts
        self.routed_scaling_factor = config.routed_scaling_factor
        self.scoring_func = config.scoring_func
        self.topk_method = config.topk_method
        self.n_group = config.n_group
        self.topk_group = config.topk_group
        self.norm_topk_prob = config.norm_topk_prob
        self.gating_dim = config.hidden_size
        self.weight = nn.Parameter(torch.empty((self.n_routed_experts, self.gating_dim), dtype=torch.float32))
        if self.topk_method == "noaux_tc":
            self.e_score_correction_bias = nn.Parameter(torch.zeros((self.n_routed_experts), dtype=torch.float32))
        self.reset_parameters()

    def reset_parameters(self) -> None:
        nn.init.kaiming_uniform_(self.weight, a=math.sqrt(5))

    @torch.no_grad()
    def forward(self, hidden_states):
        if self.scoring_func not in ("sigmoid", "softmax"):
            raise NotImplementedError(f"insupportable scoring function for MoE gating: {self.scoring_func}")
        if self.topk_method != "noaux_tc":
            raise NotImplementedError(f"insupportable TopK function for MoE gating: {self.topk_method}")
        assert not self.training
        h = hidden_states.shape[-1]
        x = hidden_states.reshape(-1, h)
        N.require_cuda(x, self.weight)
        if not x.is_contiguous():
            x = x.contiguous()
        T = x.shape[0]
        topk_idx = torch.empty((T, self.top_k), dtype=torch.int64, device=x.device)
        topk_weight = torch.empty((T, self.top_k), dtype=torch.float32, device=x.device)
        w = self.weight if self.weight.dtype == torch.float32 else self.weight.float()
        bias = self.e_score_correction_bias
        bias = bias if bias.dtype == torch.float32 else bias.float()
        E = self.n_routed_experts
        scoring = 0 if self.scoring_func == "sigmoid" else 1
        if x.dtype == torch.bfloat16 and h % 64 == 0 and T >= 1:
            # tensor-core path: logits from bf16 MMAs against the weight split into three bf16 parts (zero rows pad
            # the expert count to a multiple of 128); the K loop is split so that a small batch still spreads over
            # many SMs (a decode batch is one m-tile)
            w3 = self._split_weight(w)
            Ep = w3.shape[0]
            tiles = ((T + 127) // 128) * ((Ep + 255) // 256)
            kb = 3 * h // 64
            # Splits also bound the length of one tensor-core accumulation (about 16 K blocks of 64): the f32
            # accumulator of the MMA truncates, and the error of a long chain reaches the routing weights (measured
            # 5e-5 relative for 4096-term dot products in two splits, below 1e-5 with short chains); the partial sums
            # are added with IEEE roundings by the selection kernel.
            ks = max(1, min(16, max(148 // tiles, -(-kb // 16))))
            while ks > 1 and -(-kb // ks) * (ks - 1) >= kb:
                ks -= 1
            part = self._scratch(ks * T * Ep)
            N.check(N.lib().b200moe_router_logits_bf16x3(N.ptr(x), N.ptr(w3), N.ptr(part), T, h, Ep, ks, N.stream()))
            N.check(N.lib().b200moe_router_select(
                N.ptr(part), ks, Ep, N.ptr(bias), T, E, self.top_k, self.n_group, self.topk_group, scoring,
                1 if self.norm_topk_prob else 0, float(self.routed_scaling_factor),
                N.ptr(topk_idx), N.ptr(topk_weight), N.stream()))
        else:
            N.check(N.lib().b200moe_router_topk(
                N.ptr(x), N.dtype_code(x.dtype), N.ptr(w), N.ptr(bias), T, h, E,
                self.top_k, self.n_group, self.topk_group, scoring,
                1 if self.norm_topk_prob else 0, float(self.routed_scaling_factor),
                N.ptr(topk_idx), N.ptr(topk_weight), N.stream()))
        return topk_idx, topk_weight

    def _split_weight(self, w):
        """[hi | mid | lo] bf16 parts of the f32 router weight, [E rounded up to a multiple of 128, 3H] (zero rows
        after the last expert); rebuilt when the weight changes."""
        key = (w.data_ptr(), w._version, tuple(w.shape))
        if getattr(self, "_w3_key", None) != key:
            hi = w.to(torch.bfloat16)
            r1 = w - hi.float()
            mid = r1.to(torch.bfloat16)
            lo = (r1 - mid.float()).to(torch.bfloat16)
            w3 = torch.cat([hi, mid, lo], dim=1)
            pad = -w.shape[0] % 128
            if pad:
                w3 = torch.cat([w3, w3.new_zeros(pad, w3.shape[1])], dim=0)
            self._w3 = w3.contiguous()
            self._w3_key = key
        return self._w3

    def _scratch(self, n):
        t = getattr(self, "_partials", None)
        if t is None or t.numel() < n or t.device != self.weight.device:
            t = torch.empty(n, dtype=torch.float32, device=self.weight.device)
            self._partials = t
        return t


class DeepseekV3MoE(nn.Module):
    """A mixed expert module (reference :120-286) over quantized fused expert weights.

    config.quantize_method selects the expert path:
      "fp8_block"  e4m3 weights, 128x128 f32 scales; activations e4m3 1x128 (dispatch payload:
                   e4m3 row + f32 scales in one record); GEMM-1 fuses SwiGLU + re-quantization
      "w4a16"      asymmetric group-128 int4 weights (bf16 scale/zero); bf16 activations
                   (dispatch payload: bf16 rows); GEMM-1 fuses SwiGLU
      "w4a8"       two-level int4 weights of quantization/w4a8_kernel.py; int8 activations
                   1x128 with f16 scales (dispatch payload: int8 row + scales in one record)
    """

    METHODS = ("fp8_block", "w4a16", "w4a8")

    def __init__(self, config, device=None):
        super().__init__()
        self.config = config
        self.num_experts_per_tok = config.num_experts_per_tok
        self.method = getattr(config, "quantize_method", "fp8_block")
        if self.method not in self.METHODS:
            raise NotImplementedError(f"quantize_method {self.method!r}")
        # activation of the expert FFNs (reference moe/sglang_moe_all_gather_all_reduce.py:374-397): SiLU or tanh-GELU
        self.hidden_act = getattr(config, "hidden_act", "silu")
        if self.hidden_act not in ("silu", "gelu"):
            raise NotImplementedError(f"hidden_act {self.hidden_act!r}: the fused GEMM-1 epilogues implement silu and gelu")
        self._gelu = self.hidden_act == "gelu"
        if hasattr(config, "ep_size") and config.ep_size > 1:
            assert config.ep_size == dist.get_world_size()
            self.ep_size = config.ep_size
            self.ep_rank = dist.get_rank()
        else:
            self.ep_size, self.ep_rank = 1, 0
        E, H, I = config.n_routed_experts, config.hidden_size, config.moe_intermediate_size
        assert E % self.ep_size == 0
        assert H % 128 == 0 and I % 128 == 0, "hidden and intermediate sizes must be multiples of 128"
        self.experts_per_rank = E // self.ep_size
        El = self.experts_per_rank
        # pipeline passes of the expert-parallel exchange (config.ep_passes; 1 = no overlap)
        want = int(getattr(config, "ep_passes", 1)) if self.ep_size > 1 else 1
        self.passes = max(p for p in (1, 2, 4, 8) if p <= max(want, 1) and El % p == 0)
        # "nccl": all_to_all_single with split sizes; "push": peer copies on the copy engines;
        # "fused": records and results stored straight into the peers' buffers by the permute kernel
        # and the down projection (fp8_block only; no host read, no pipeline passes)
        # "all2all": tokens are data-parallel and rows travel to their experts (reference
        # moe/all2all_moe.py); "allreduce": every rank sees all tokens, runs its own experts on them and
        # the outputs are summed across ranks (reference moe/sglang_moe_all_gather_all_reduce.py:267-446)
        self.strategy = getattr(config, "ep_strategy", "all2all") if self.ep_size > 1 else "all2all"
        assert self.strategy in ("all2all", "allreduce")
        # default ("auto"): "fused" for fp8_block, "nccl" for the int4 methods
        self.exchange = getattr(config, "ep_exchange", "auto") if self.ep_size > 1 else "none"
        # payload of the all-reduce of the "allreduce" strategy: None = bf16 NCCL all-reduce; "fp8" / "int8" = the
        # reference's quantized all-reduce (quant_communication/quant_all2all_allreduce.py:52-99)
        self.allreduce_quant = getattr(config, "allreduce_quant", None)
        assert self.allreduce_quant in (None, "fp8", "int8")
        if self.strategy == "allreduce":
            self.exchange, self.passes = "none", 1
        if self.exchange == "auto":
            self.exchange = "fused" if self.method == "fp8_block" else "nccl"
        assert self.exchange in ("nccl", "push", "fused", "none")
        if self.exchange == "fused":
            assert self.method == "fp8_block", "ep_exchange='fused' is built for quantize_method='fp8_block'"
            self.passes = 1
        self._fx = None
        self.recv_capacity = float(getattr(config, "ep_recv_capacity", 2.0))   # receive rows / (T*k)
        self._xch = None
        # with pipeline passes the expert GEMMs leave SMs for the NCCL kernels that run beside them
        # (config.ep_gemm_ctas; passed with each of this layer's GEMM calls)
        self._gemm_ctas = int(getattr(config, "ep_gemm_ctas", 0)) if self.passes > 1 else 0
        dev = device if device is not None else torch.device("cuda", torch.cuda.current_device())
        self._dev = dev
        reg = lambda name, t: self.register_buffer(name, t, persistent=True)
        z = lambda *shape, dtype: torch.zeros(*shape, dtype=dtype, device=dev)
        if self.method == "fp8_block":
            f8 = torch.float8_e4m3fn
            reg("w13_weight", z(El, 2 * I, H, dtype=f8))
            reg("w13_weight_scale", torch.ones(El, 2 * I // 128, H // 128, dtype=torch.float32, device=dev))
            reg("w2_weight", z(El, H, I, dtype=f8))
            reg("w2_weight_scale", torch.ones(El, H // 128, I // 128, dtype=torch.float32, device=dev))
        elif self.method == "w4a16":
            reg("w13_qweight", z(El, 2 * I, H // 8, dtype=torch.int32))
            reg("w13_scale", z(El, 2 * I, H // 128, dtype=torch.bfloat16))
            reg("w13_zero", z(El, 2 * I, H // 128, dtype=torch.bfloat16))
            reg("w2_qweight", z(El, H, I // 8, dtype=torch.int32))
            reg("w2_scale", z(El, H, I // 128, dtype=torch.bfloat16))
            reg("w2_zero", z(El, H, I // 128, dtype=torch.bfloat16))
        else:
            reg("w13_qweight", z(El, 2 * I // 8, H, dtype=torch.int32))
            reg("w13_weight_scale", z(El, 2 * I // 128, H // 128, dtype=torch.float32))
            reg("w13_s4", z(El, 2 * I, H // 128, dtype=torch.int8))
            reg("w13_z4", z(El, 2 * I, H // 128, dtype=torch.int8))
            reg("w2_qweight", z(El, H // 8, I, dtype=torch.int32))
            reg("w2_weight_scale", z(El, H // 128, I // 128, dtype=torch.float32))
            reg("w2_s4", z(El, H, I // 128, dtype=torch.int8))
            reg("w2_z4", z(El, H, I // 128, dtype=torch.int8))
        self.gate = MoEGate(config).to(dev)
        # Shared experts (reference :161-165, 182-183): one DeepseekV3MLP of width
        # n_shared_experts * moe_intermediate_size applied to every token, unquantized as in the
        # reference (plain bf16 nn.Linear layers there), added to the routed output.
        self.n_shared = int(config.n_shared_experts or 0)
        if self.n_shared:
            Is = I * self.n_shared
            reg("shared_w13", z(1, 2 * Is, H, dtype=torch.bfloat16))     # [gate_proj ; up_proj]
            reg("shared_w2", z(1, H, Is, dtype=torch.bfloat16))          # down_proj
            self._shared_stream = None
        # int4 methods: up to this many rows per expert group on average the dequantization runs inside the GEMMs
        # (every tile converts its weights once); above it the weights are expanded once per forward instead
        # (measured break-even: 64 rows for w4a8, whose tiles hold 64 tokens; 256 for w4a16, whose tiles hold 128)
        self.w4_fused_rows_per_group = int(getattr(config, "w4_fused_rows_per_group",
                                                   256 if self.method == "w4a16" else 64))
        self._buffers_cache = {}
        self._status = torch.zeros(1, dtype=torch.int32, device=dev)
        self._last_recv_rows = None
        # Optional per-stage timing: set to a list and every forward appends
        # (stage name, CUDA event recorded when the stage's launches were queued).
        self.stage_events = None

    def _mark(self, name):
        if self.stage_events is not None:
            ev = torch.cuda.Event(enable_timing=True)
            ev.record()
            self.stage_events.append((name, ev))

    # ---- weights ---------------------------------------------------------------------
    @torch.no_grad()
    def load_expert(self, local_idx: int, gate_w: torch.Tensor, up_w: torch.Tensor, down_w: torch.Tensor):
        """Quantizes one expert's nn.Linear weights (gate/up [I,H], down [H,I], the layout of
        DeepseekV3MLP, reference :13-29) into the fused tensors of the configured method."""
        w13 = torch.cat([gate_w, up_w], dim=0).contiguous()
        w2 = down_w.contiguous()
        if self.method == "fp8_block":
            q, s = fp8_kernel.weight_quant(w13)
            self.w13_weight[local_idx].copy_(q)
            self.w13_weight_scale[local_idx].copy_(s)
            q, s = fp8_kernel.weight_quant(w2)
            self.w2_weight[local_idx].copy_(q)
            self.w2_weight_scale[local_idx].copy_(s)
        elif self.method == "w4a16":
            for name, w in (("w13", w13), ("w2", w2)):
                packed, sc, zp = w4a16_kernel.weight_quant(w)
                getattr(self, f"{name}_qweight")[local_idx].copy_(packed)
                getattr(self, f"{name}_scale")[local_idx].copy_(sc)
                getattr(self, f"{name}_zero")[local_idx].copy_(zp)
        else:
            for name, w in (("w13", w13), ("w2", w2)):
                packed, s, s4, z4 = w4a8_kernel.weight_quant(w.float().contiguous())
                getattr(self, f"{name}_qweight")[local_idx].copy_(packed)
                getattr(self, f"{name}_weight_scale")[local_idx].copy_(s.float())
                getattr(self, f"{name}_s4")[local_idx].copy_(s4)
                getattr(self, f"{name}_z4")[local_idx].copy_(z4)

    def load_shared_experts(self, gate_w: torch.Tensor, up_w: torch.Tensor, down_w: torch.Tensor):
        """Weights of the shared DeepseekV3MLP: gate_proj/up_proj [I*n_shared, H], down_proj [H, I*n_shared]."""
        assert self.n_shared, "config.n_shared_experts is 0"
        self.shared_w13[0].copy_(torch.cat([gate_w, up_w], dim=0))
        self.shared_w2[0].copy_(down_w)

    def _shared_begin(self, x):
        """gate/up projection + SwiGLU of the shared experts on a side stream: it needs only x, so it
        fills the SMs while the routed path waits on its exchange.  Returns (h, event)."""
        T, H = x.shape
        Is = self.shared_w2.shape[2]
        if self._shared_stream is None:
            self._shared_stream = torch.cuda.Stream(device=self._dev)
        side, main = self._shared_stream, torch.cuda.current_stream()
        seg = self._buffers_cache.get(("shared_seg", T))
        if seg is None:
            seg = self._buffers_cache[("shared_seg", T)] = torch.tensor([0, T], dtype=torch.int64, device=self._dev)
        h = self._buf("shared_h", (T, Is), torch.bfloat16)
        side.wait_stream(main)
        with torch.cuda.stream(side):
            G.grouped_gemm_bf16(x, self.shared_w13, seg, None, h, epilogue=5 if self._gelu else 2,
                                status_word=self._status)
            ev = torch.cuda.Event()
            ev.record(side)
        return h, seg, ev

    def _shared_finish(self, fork, y):
        """down projection of the shared experts, added into the routed output in the GEMM's stores:
        y = bf16(y + bf16(h @ w2^T)), the sum the reference forms at :183."""
        h, seg, ev = fork
        torch.cuda.current_stream().wait_event(ev)
        G.grouped_gemm_bf16(h, self.shared_w2, seg, None, y, epilogue=3, status_word=self._status)
        self._mark("shared_experts")

    def _buf(self, name, shape, dtype):
        t = self._buffers_cache.get(name)
        n = 1
        for d in shape:
            n *= d
        if t is None or t.dtype != dtype or t.numel() < n:
            t = torch.empty(max(n, 1), dtype=dtype, device=self._dev)
            self._buffers_cache[name] = t
        return t[:n].view(*shape)

    # ---- forward ---------------------------------------------------------------------
    @torch.no_grad()
    def forward(self, hidden_states):
        orig_shape = hidden_states.shape
        self._mark("start")
        topk_idx, topk_weight = self.gate(hidden_states)
        self._mark("router")
        x = hidden_states.reshape(-1, orig_shape[-1])
        if not x.is_contiguous():
            x = x.contiguous()
        fork = self._shared_begin(x) if self.n_shared else None
        y = self.triton_group_gemm_moe_infer(x, topk_idx, topk_weight)
        if self.n_shared:
            self._shared_finish(fork, y)
        return y.view(*orig_shape)

    def make_graphed(self, example: torch.Tensor, warmup: int = 2):
        """Captures one forward pass for inputs of `example`'s shape and dtype into a CUDA graph and
        returns `run(x) -> y` (single-rank layers).  The layer's launch sequence is fixed and reads nothing
        back to the host.  For small batches, where the step is a dozen launches of a few microseconds
        each, replaying the graph removes the per-launch host cost.  `y` is a static buffer that the next
        `run` overwrites; a device-side timeout still shows up in `check_status()`.  Restricted to
        ep_size == 1: an expert-parallel step interleaves NCCL collectives with kernels that store into
        peer-mapped buffers, and capturing that sequence is not supported here."""
        assert self.ep_size == 1, "make_graphed supports ep_size == 1"
        cur = torch.cuda.current_stream()
        side = torch.cuda.Stream(device=self._dev)
        static_in = example.detach().clone()
        side.wait_stream(cur)
        with torch.cuda.stream(side):              # warm-up: buffers, peer mappings, driver entry points
            for _ in range(max(warmup, 1)):
                self(static_in)
        cur.wait_stream(side)
        torch.cuda.synchronize(self._dev)
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            static_out = self(static_in)

        def run(x: torch.Tensor) -> torch.Tensor:
            static_in.copy_(x, non_blocking=True)
            graph.replay()
            return static_out
        run.graph, run.static_input, run.static_output = graph, static_in, static_out
        return run

    # the reference's unfused entry point routes to the same pipeline
    def moe_infer(self, x, topk_ids, topk_weight):
        return self.triton_group_gemm_moe_infer(x, topk_ids, topk_weight)

    def _record_bytes(self, H):
        """Bytes of one dispatched row: payload, then f32 scales, padded to 16 (TMA row alignment)."""
        if self.method == "w4a16":
            return 2 * H
        return (H + (H // 128) * 4 + 15) // 16 * 16

    @torch.no_grad()
    def triton_group_gemm_moe_infer(self, x, topk_ids, topk_weight):
        """The fused expert-parallel pipeline (finishes the stub at reference :282-286)."""
        cfg = self.config
        T, H = x.shape
        k = topk_ids.shape[1]
        E = cfg.n_routed_experts
        S = T * k
        assert x.dtype == torch.bfloat16, "activations must be bfloat16"
        ep = self.ep_size
        # With expert parallelism the experts are visited in (pass, owner rank, expert-in-pass)
        # order so that every pipeline pass is contiguous on both sides of the exchange.
        ids = topk_ids if ep == 1 or self.passes == 1 else self._expert_order()[topk_ids]   # one pass: identity
        reorder_ids, src2dst, seg_indptr = G.run_moe_ep_preproess(ids, E)
        self._mark("route_metadata")
        rec = self._record_bytes(H)
        send = self._buf("send", (S, rec), torch.uint8)
        # The exchange plan needs only the per-expert counts: its count all-to-all and its one host
        # read are issued before the permute kernel, which then runs while the host builds the plan.
        push = ep > 1 and self.exchange == "push"
        if ep > 1 and self.strategy == "allreduce":
            return self._run_allreduce(x, ids, topk_weight, src2dst, seg_indptr, T, H, k, E, rec)
        if ep > 1 and self.exchange == "fused":
            down = self._run_fused(x, ids, src2dst, seg_indptr, S, H, rec)
            out = torch.empty((T, H), dtype=x.dtype, device=x.device)
            G.post_reorder_triton_kernel[(T,)](down, out, src2dst, ids, topk_weight, 0, E - 1, k, H,
                                               BLOCK_SIZE=512)
            self._mark("post_reorder")
            return out
        if ep == 1:
            plan = None
        elif push:
            pplan = ep_comm.plan_push(seg_indptr, ep, self.passes, self.ep_rank)
            plan = pplan.base
        else:
            plan = ep_comm.plan_exchange_pipelined(seg_indptr, ep, self.passes)
        if self.method == "fp8_block":
            G.permute_quant_fp8(x, src2dst, ids, 0, E - 1, send[:, :H],
                                send[:, H:H + (H // 128) * 4].view(torch.float32))
        elif self.method == "w4a8":
            G.permute_quant_int8(x, src2dst, ids, 0, E - 1, send[:, :H],
                                 send[:, H:H + (H // 128) * 4].view(torch.float32), rounding="floor_half")
        else:
            G.pre_reorder_triton_kernel[(T,)](x, send.view(torch.bfloat16), src2dst, ids, None, 0, E - 1, k, H,
                                              BLOCK_SIZE=512)
        self._mark("permute_quant")
        ctx = {}
        run = self._experts

        if ep == 1:
            self.last_recv_rows = S
            down = self._buf("down", (S, H), torch.bfloat16)
            self._last = (send, S, seg_indptr, None)
            if S > 0:
                run(ctx, send, S, seg_indptr, None, down, (0, S))
        elif push:
            down = self._run_pushed(ctx, run, pplan, send, S, H, rec)
        else:
            P = self.passes
            rows = plan.recv_rows
            self.last_recv_rows = rows
            recv = self._buf("recv", (max(rows, 1), rec), torch.uint8)[:rows]
            down_r = self._buf("down", (max(rows, 1), H), torch.bfloat16)[:rows]
            back = self._buf("back", (S, H), torch.bfloat16)
            self._last = (recv, rows, plan.seg_indptr, plan.weight_indices)
            main, comm = torch.cuda.current_stream(), self._comm_stream()
            ready = torch.cuda.Event()
            ready.record(main)
            got = [torch.cuda.Event() for _ in range(P)]
            done = [torch.cuda.Event() for _ in range(P)]
            with torch.cuda.stream(comm):
                comm.wait_event(ready)
                for p in range(P):
                    ep_comm.dispatch_pass(plan, p, send, recv)
                    got[p].record(comm)
            gpp = plan.groups_per_pass
            merge = self.method == "fp8_block"      # rows of one expert from all sources -> one GEMM group
            if merge:
                merged = self._buf("merged", (max(rows, 1), rec), torch.uint8)[:rows]
                ctx["c_row_map"] = plan.gather_map
                self._last = (merged, rows, plan.merged_seg, plan.merged_widx)
            epp = plan.experts_per_pass
            for p in range(P):
                main.wait_event(got[p])
                r0, r1 = plan.recv_off[p], plan.recv_off[p + 1]
                if r1 > r0 and merge:
                    G.gather_rows(recv, merged[r0:r1], plan.gather_map[r0:r1])
                    run(ctx, merged, rows, plan.merged_seg[p * epp:(p + 1) * epp + 1],
                        plan.merged_widx[p * epp:(p + 1) * epp], down_r, (r0, r1))
                elif r1 > r0:
                    run(ctx, recv, rows, plan.seg_indptr[p * gpp:(p + 1) * gpp + 1],
                        plan.weight_indices[p * gpp:(p + 1) * gpp], down_r, (r0, r1))
                done[p].record(main)
                with torch.cuda.stream(comm):
                    comm.wait_event(done[p])
                    ep_comm.combine_pass(plan, p, down_r, back)
                    if p == P - 1:
                        ready.record(comm)
            main.wait_event(ready)
            self._mark("experts_and_exchange")
            down = back
        out = torch.empty((T, H), dtype=x.dtype, device=x.device)
        G.post_reorder_triton_kernel[(T,)](down, out, src2dst, ids, topk_weight, 0, E - 1, k, H,
                                           BLOCK_SIZE=512)
        self._mark("post_reorder")
        return out

    @property
    def last_recv_rows(self):
        """Rows this rank's experts processed in the last forward (synchronises in 'fused' mode)."""
        v = self._last_recv_rows
        return int(v.item()) if torch.is_tensor(v) else v

    @last_recv_rows.setter
    def last_recv_rows(self, v):
        self._last_recv_rows = v

    def _run_allreduce(self, x, ids, topk_weight, src2dst, seg_indptr, T, H, k, E, rec):
        """Every rank holds all T tokens: permute + quantize only the slots of this rank's experts
        (the start/end expert ids of reference sglang_moe_all_gather_all_reduce.py:312-324), run them,
        un-permute into a partial output and sum the partial outputs over the ranks (:441-442)."""
        El = self.experts_per_rank
        lo, hi = self.ep_rank * El, self.ep_rank * El + El - 1
        S = T * k
        send = self._buf("send", (S, rec), torch.uint8)
        if self.method == "fp8_block":
            G.permute_quant_fp8(x, src2dst, ids, lo, hi, send[:, :H], send[:, H:H + (H // 128) * 4].view(torch.float32))
        elif self.method == "w4a8":
            G.permute_quant_int8(x, src2dst, ids, lo, hi, send[:, :H],
                                 send[:, H:H + (H // 128) * 4].view(torch.float32), rounding="floor_half")
        else:
            G.pre_reorder_triton_kernel[(T,)](x, send.view(torch.bfloat16), src2dst, ids, None, lo, hi, k, H,
                                              BLOCK_SIZE=512)
        self._mark("permute_quant")
        seg_local = seg_indptr[lo:hi + 2]                    # absolute row offsets of my experts' groups
        down = self._buf("down", (S, H), torch.bfloat16)
        self._last = (send, S, seg_local, None)
        self._last_recv_rows = seg_local[-1] - seg_local[0]
        if S > 0:
            getattr(self, "_experts_" + self.method)({}, send, S, seg_local, None, down, (0, S))
        out = torch.empty((T, H), dtype=x.dtype, device=x.device)
        G.post_reorder_triton_kernel[(T,)](down, out, src2dst, ids, topk_weight, lo, hi, k, H, BLOCK_SIZE=512)
        self._mark("post_reorder")
        if self.allreduce_quant is None:
            dist.all_reduce(out, op=dist.ReduceOp.SUM)
        else:
            ep_comm.quant_allreduce(out, self._ar_quant, G.dequant_sum)
        self._mark("all_reduce")
        return out

    def _ar_quant(self, t):
        """Quantizer of the all-reduce payload: e4m3 with f32 1x128 scales, or int8 (floor(v + 0.5), the rounding
        of the reference's communication quantizer, quant_communication/quant_utils.py:27-28) with f16 scales."""
        if self.allreduce_quant == "fp8":
            return fp8_kernel.act_quant(t)
        return w4a8_kernel.act_quant(t)

    def share_exchange_buffers(self, other: "DeepseekV3MoE"):
        """Uses `other`'s peer-mapped receive/return buffers (ep_exchange="fused") instead of allocating
        this layer's own: layers that run one after the other on a stream can share one pair (≈ 1 GB per
        rank at 4096 tokens, hidden 7168), because the two barriers of a forward pass already order a
        layer's reads before the next layer's remote writes.  Call after `other`'s first forward."""
        assert self.exchange == "fused" and other.exchange == "fused" and other._fx is not None
        assert (self.config.hidden_size, self.config.n_routed_experts, self.ep_size) == \
               (other.config.hidden_size, other.config.n_routed_experts, other.ep_size)
        self._fx = other._fx

    def _run_fused(self, x, ids, src2dst, seg_indptr, S, H, rec):
        """Exchange folded into the permute kernel and the down projection (ep_comm.FusedExchange)."""
        ep, E = self.ep_size, self.config.n_routed_experts
        if self._fx is None:
            smax = torch.tensor([S], dtype=torch.int64, device=self._dev)
            dist.all_reduce(smax, op=dist.ReduceOp.MAX)      # symmetric allocations: one size on every rank
            smax = max(int(smax.item()), 1)
            self._fx = ep_comm.FusedExchange(ep, self.ep_rank, self._dev, int(self.recv_capacity * smax), rec,
                                             smax, H, E)
        fx = self._fx
        assert S <= fx.slots, f"{S} routed slots, peer buffers were sized for {fx.slots} at the first call"
        # the previous forward's overflow flag has long reached the host (copied there right after its plan
        # kernel): a batch whose rows did not fit a peer buffer raises here instead of passing for a result
        fx.raise_if_overflowed()
        fx.gather_counts(seg_indptr)
        G.ep_plan(fx.counts_all, self.ep_rank, ep, fx.cap_rows, fx.recv_base, rec, fx.back_base, H * 2,
                  out=(fx.dst_base, fx.local_seg, fx.back_addr, fx.info))
        fx.publish_info()
        self._mark("exchange_plan")
        G.permute_quant_fp8_push(x, src2dst, ids, seg_indptr, fx.dst_base, rec, back_local=fx.back)
        fx.barrier()                                         # every rank's records have landed
        self._mark("permute_quant")
        self._last_recv_rows = fx.info[0]
        self._last = (fx.recv, fx.cap_rows, fx.local_seg, None)
        ctx = {"c_row_addr": fx.back_addr}
        self._experts_fp8_block(ctx, fx.recv, fx.cap_rows, fx.local_seg, None, fx.back, (0, fx.cap_rows))
        fx.barrier()                                         # every rank's results have landed
        self._mark("experts_and_exchange")
        return fx.back[:S]

    def _run_pushed(self, ctx, run, pplan, send, S, H, rec):
        """Exchange by peer copies on the copy engines (ep_comm.SymmExchange): every pass's rows are
        pushed up front, the GEMMs of pass p start when its rows have arrived everywhere, and its
        results are pushed back while pass p+1 computes."""
        plan, P, ep = pplan.base, self.passes, self.ep_size
        rows = plan.recv_rows
        self.last_recv_rows = rows
        if self._xch is None:
            # symmetric allocations must have one size on every rank: size them for the largest batch
            smax = torch.tensor([S], dtype=torch.int64, device=self._dev)
            dist.all_reduce(smax, op=dist.ReduceOp.MAX)
            smax = int(smax.item())
            self._xch = ep_comm.SymmExchange(ep, self.ep_rank, self._dev, int(self.recv_capacity * smax), rec, smax, H)
        xch = self._xch
        assert S <= xch.slots, f"{S} routed slots, peer buffers were sized for {xch.slots} at the first call"
        assert rows <= xch.cap_rows, f"received {rows} rows, capacity {xch.cap_rows} (raise config.ep_recv_capacity)"
        recv = xch.recv[:rows]
        down_r = self._buf("down", (max(rows, 1), H), torch.bfloat16)[:rows]
        merged = self._buf("merged", (max(rows, 1), rec), torch.uint8)[:rows]
        merge = self.method == "fp8_block"
        if merge:
            ctx["c_row_map"] = plan.gather_map
            self._last = (merged, rows, plan.merged_seg, plan.merged_widx)
        else:
            self._last = (recv, rows, plan.seg_indptr, plan.weight_indices)
        main = torch.cuda.current_stream()
        ready = torch.cuda.Event()
        ready.record(main)
        got = []
        for p in range(P):
            pieces = [(d, xch.peer_recv[d][pplan.dst_off[p][d]:pplan.dst_off[p][d] + plan.in_splits[p][d]],
                       send[pplan.src_off[p][d]:pplan.src_off[p][d] + plan.in_splits[p][d]]) for d in range(ep)]
            got.append(xch.push(ready, pieces))
        gpp, epp = plan.groups_per_pass, plan.experts_per_pass
        fin = None
        for p in range(P):
            main.wait_event(got[p])
            r0, r1 = plan.recv_off[p], plan.recv_off[p + 1]
            if r1 > r0 and merge:
                G.gather_rows(recv, merged[r0:r1], plan.gather_map[r0:r1])
                run(ctx, merged, rows, plan.merged_seg[p * epp:(p + 1) * epp + 1],
                    plan.merged_widx[p * epp:(p + 1) * epp], down_r, (r0, r1))
            elif r1 > r0:
                run(ctx, recv, rows, plan.seg_indptr[p * gpp:(p + 1) * gpp + 1],
                    plan.weight_indices[p * gpp:(p + 1) * gpp], down_r, (r0, r1))
            done = torch.cuda.Event()
            done.record(main)
            pieces = [(s_, xch.peer_back[s_][pplan.back_off[p][s_]:pplan.back_off[p][s_] + plan.out_splits[p][s_]],
                       down_r[pplan.mine_off[p][s_]:pplan.mine_off[p][s_] + plan.out_splits[p][s_]]) for s_ in range(ep)]
            fin = xch.push(done, pieces)
        main.wait_event(fin)
        self._mark("experts_and_exchange")
        return xch.back[:S]

    def _expert_order(self):
        t = self._buffers_cache.get("expert_order")
        if t is None:
            t = ep_comm.expert_order(self.config.n_routed_experts, self.ep_size, self.passes, self._dev)
            self._buffers_cache["expert_order"] = t
        return t

    def _comm_stream(self):
        if getattr(self, "_cs", None) is None:
            self._cs = torch.cuda.Stream(device=self._dev)
        return self._cs

    # ---- expert FFNs over the permuted rows ---------------------------------------------
    def _experts(self, *args):
        fn = getattr(self, "_experts_" + self.method)
        if self._gemm_ctas:
            with G.gemm_options(max_ctas=self._gemm_ctas):
                return fn(*args)
        return fn(*args)

    def _experts_fp8_block(self, ctx, buf, rows, seg, widx, down, rng):
        H, I = self.config.hidden_size, self.config.moe_intermediate_size
        a_q, a_s = buf[:, :H], buf[:, H:H + (H // 128) * 4].view(torch.float32)
        h_q = self._buf("h_q", (rows, I), torch.uint8)
        h_s = self._buf("h_s", (rows, I // 128), torch.float32)
        G.grouped_gemm_fp8(a_q, a_s, self.w13_weight, self.w13_weight_scale, seg, widx,
                           h_q, h_s, epilogue=4 if self._gelu else 1, status_word=self._status)
        self._mark("gemm1_swiglu")
        G.grouped_gemm_fp8(h_q, h_s, self.w2_weight, self.w2_weight_scale, seg, widx,
                           down, None, epilogue=0, status_word=self._status, c_row_map=ctx.get("c_row_map"),
                           c_row_addr=ctx.get("c_row_addr"))
        self._mark("gemm2")

    def _experts_w4a16(self, ctx, buf, rows, seg, widx, down, rng):
        I = self.config.moe_intermediate_size
        a = buf.view(torch.bfloat16)
        r0, r1 = rng
        if (r1 - r0) <= self.w4_fused_rows_per_group * (seg.numel() - 1):
            # few rows per expert (decode): the packed weights are dequantized inside the GEMMs, once per tile
            h = self._buf("h_bf16", (rows, I), torch.bfloat16)
            G.grouped_gemm_w4a16(a, self.w13_qweight, self._pairs("w13", "_scale", "_zero"), seg, widx, h,
                                 epilogue=5 if self._gelu else 2, status_word=self._status)
            self._mark("gemm1_swiglu")
            G.grouped_gemm_w4a16(h, self.w2_qweight, self._pairs("w2", "_scale", "_zero"), seg, widx, down,
                                 epilogue=0, status_word=self._status)
            self._mark("gemm2")
            return
        if "w13" not in ctx:      # many rows per expert: int4 -> bf16 once per forward, shared by the pipeline passes
            ctx["w13"] = w4a16_kernel.expand_bf16(self.w13_qweight, self.w13_scale, self.w13_zero)
            ctx["w2"] = w4a16_kernel.expand_bf16(self.w2_qweight, self.w2_scale, self.w2_zero)
            self._mark("expand_weights")
        h = self._buf("h_bf16", (rows, I), torch.bfloat16)
        G.grouped_gemm_bf16(a, ctx["w13"], seg, widx, h, epilogue=5 if self._gelu else 2, status_word=self._status)
        self._mark("gemm1_swiglu")
        G.grouped_gemm_bf16(h, ctx["w2"], seg, widx, down, epilogue=0, status_word=self._status)
        self._mark("gemm2")

    def _pairs(self, name, first="_s4", second="_z4"):
        """(s4, z4) -- or (scale, zero) -- of a weight in the layout the fused-dequantization kernels read; rebuilt
        when the tensors change."""
        s4, z4 = getattr(self, name + first), getattr(self, name + second)
        key = (s4.data_ptr(), s4._version, z4.data_ptr(), z4._version)
        hit = self._buffers_cache.get(("pairs", name))
        if hit is None or hit[0] != key:
            hit = (key, G.pair_scales_t(s4, z4))
            self._buffers_cache[("pairs", name)] = hit
        return hit[1]

    def _raw_nibbles_ok(self, name):
        """The fused w4a8 GEMM multiplies the raw nibbles and applies (q - z4) * s4 to the dot product, which equals
        the reference's int8 product (quantization/w4a8_kernel.py:362-380, where the product is cast to int8) only
        while (q - z4) * s4 stays inside int8 for every nibble the weight holds.  The reference's quantizer keeps it
        there (:228-262); any weight is checked once here (smallest and largest nibble of every scale group), and one
        that fails is expanded to int8 instead."""
        packed, s4, z4 = getattr(self, name + "_qweight"), getattr(self, name + "_s4"), getattr(self, name + "_z4")
        key = (packed.data_ptr(), packed._version, s4.data_ptr(), s4._version, z4.data_ptr(), z4._version)
        hit = self._buffers_cache.get(("raw_ok", name))
        if hit is None or hit[0] != key:
            W, R8, K = packed.shape                      # nibble i of a word: output row 8 r + i
            ok = True
            for e in range(W):                           # one expert at a time keeps the scratch small
                lo = torch.empty(R8, 8, K // 128, dtype=torch.int32, device=packed.device)
                hi = torch.empty_like(lo)
                for i in range(8):
                    q = ((packed[e] >> (4 * i)) & 15).view(R8, K // 128, 128)
                    lo[:, i], hi[:, i] = q.amin(-1), q.amax(-1)
                s, zz = s4[e].to(torch.int32).view(R8, 8, -1), z4[e].to(torch.int32).view(R8, 8, -1)
                a, b = (lo - zz) * s, (hi - zz) * s
                ok = ok and bool((torch.minimum(a, b).min() >= -128) & (torch.maximum(a, b).max() <= 127))
                if not ok:
                    break
            hit = (key, ok)
            self._buffers_cache[("raw_ok", name)] = hit
        return hit[1]

    def _experts_w4a8(self, ctx, buf, rows, seg, widx, down, rng):
        H, I = self.config.hidden_size, self.config.moe_intermediate_size
        a_q, a_s = buf[:, :H].view(torch.int8), buf[:, H:H + (H // 128) * 4].view(torch.float32)
        r0, r1 = rng                                   # the rows this call's groups cover
        h_q = self._buf("h_i8", (rows, I), torch.int8)
        h_s = self._buf("h_i8_s", (rows, I // 128), torch.float32)
        groups = seg.numel() - 1
        if (r1 - r0) <= self.w4_fused_rows_per_group * groups and self._raw_nibbles_ok("w13") and self._raw_nibbles_ok("w2"):
            # few rows per expert (decode): the packed weights are converted inside the GEMMs, once per tile;
            # act(gate)*up and the int8 re-quantization are GEMM-1's epilogue
            G.grouped_gemm_w4a8(a_q, a_s, self.w13_qweight, self._pairs("w13"), self.w13_weight_scale, seg, widx,
                                h_q, h_s, epilogue=4 if self._gelu else 1, status_word=self._status)
            self._mark("gemm1_swiglu")
            G.grouped_gemm_w4a8(h_q, h_s, self.w2_qweight, self._pairs("w2"), self.w2_weight_scale, seg, widx,
                                down, None, epilogue=0, status_word=self._status)
            self._mark("gemm2")
            return
        if "w13" not in ctx:      # many rows per expert: int4 -> int8 once per forward, shared by the pipeline passes
            ctx["w13"] = w4a8_kernel.expand_int8(self.w13_qweight, self.w13_s4, self.w13_z4)
            ctx["w2"] = w4a8_kernel.expand_int8(self.w2_qweight, self.w2_s4, self.w2_z4)
            self._mark("expand_weights")
        gu = self._buf("gateup", (rows, 2 * I), torch.bfloat16)
        G.grouped_gemm_i8(a_q, a_s, ctx["w13"], self.w13_weight_scale, seg, widx, gu, status_word=self._status)
        self._mark("gemm1")
        h = self._buf("h_bf16", (rows, I), torch.bfloat16)
        act_mul = G.gelu_and_mul_triton_kernel if self._gelu else G.silu_and_mul_triton_kernel
        act_mul[(r1 - r0,)](gu[r0:r1], h[r0:r1], 2 * I, None, None, 0, 0, BLOCK_SIZE=512)
        q, sc = w4a8_kernel.act_quant(h[r0:r1])
        h_q[r0:r1].copy_(q)
        h_s[r0:r1].copy_(sc)
        self._mark("silu_quant")
        G.grouped_gemm_i8(h_q, h_s, ctx["w2"], self.w2_weight_scale, seg, widx, down, status_word=self._status)
        self._mark("gemm2")

    @torch.no_grad()
    def time_expert_gemms(self, iters: int = 10):
        """Re-launches the two grouped GEMMs of the last forward on its resident inputs (all
        groups, current stream) and returns their average durations in ms, timed with CUDA
        events: (gemm1_ms, gemm2_ms, rows).  fp8_block only."""
        assert self.method == "fp8_block" and getattr(self, "_last", None) is not None
        buf, rows, seg, widx = self._last
        H, I = self.config.hidden_size, self.config.moe_intermediate_size
        a_q, a_s = buf[:, :H], buf[:, H:H + (H // 128) * 4].view(torch.float32)
        h_q = self._buf("h_q", (rows, I), torch.uint8)
        h_s = self._buf("h_s", (rows, I // 128), torch.float32)
        down = self._buf("down", (max(rows, 1), H), torch.bfloat16)[:rows]
        ev = [torch.cuda.Event(enable_timing=True) for _ in range(3)]
        t1 = t2 = 0.0
        for _ in range(iters):
            ev[0].record()
            G.grouped_gemm_fp8(a_q, a_s, self.w13_weight, self.w13_weight_scale, seg, widx, h_q, h_s,
                               epilogue=4 if self._gelu else 1, status_word=self._status)
            ev[1].record()
            G.grouped_gemm_fp8(h_q, h_s, self.w2_weight, self.w2_weight_scale, seg, widx, down, None, epilogue=0,
                               status_word=self._status)
            ev[2].record()
            ev[2].synchronize()
            t1 += ev[0].elapsed_time(ev[1])
            t2 += ev[1].elapsed_time(ev[2])
        return t1 / iters, t2 / iters, rows

    def check_status(self):
        """Raises if a kernel of an earlier forward reported a device-side timeout, or if rows of an earlier
        forward did not fit a peer buffer of the fused exchange (synchronises).  With ep_exchange="fused" a
        forward whose rows overflow `config.ep_recv_capacity` still completes -- the surplus rows contribute
        zeros -- and the NEXT forward raises; call this after the last forward of a sequence so that its
        overflow cannot go unnoticed either."""
        if self._fx is not None:
            torch.cuda.current_stream().synchronize()
            self._fx.raise_if_overflowed()
        s = int(self._status.item())
        if s:
            self._status.zero_()
            raise N.B200MoeError(s, "a bounded device-side wait expired inside a grouped GEMM")
