"""Benchmark of the expert-parallel quantized MoE layer.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

A step is one forward pass of the layer over one batch of synthetic tokens per rank
(configs[3] of the benchmark spec: DeepSeek-V3 shape, 256 experts, top-8, hidden 7168,
SwiGLU 2048, e4m3 weights with 128x128 scales, 4096 tokens per rank, Zipf-skewed expert
popularity; EP = N).  For N > 1 launch with torch.distributed.run, one rank per GPU.
Rank 0 prints ONE JSON line.

`value` is whole-job tokens/s with the tokens already resident in HBM, timed with CUDA
events on the launching stream (max over ranks).  `e2e` is the same metric through the
public layer call with HOST buffers: the pinned host->device copy of the step's tokens and
the device->host read of its output are inside the timed region, on copy streams of their own
so that they overlap the neighbouring steps' compute as in a serving loop.  `roofline` describes the
dominant kernel (the gate/up grouped GEMM), `cpu_baseline` times the CPU restatement of the
reference's torch path on the host cores on a bounded sample.  `parity` is a reduced-shape forward
through the same expert-parallel exchange the timed run uses, every rank checked against the CPU
oracle before anything is timed (the run fails above the tolerance).  At N = 1 `configs` adds
device-timed records of the other benchmark configurations (dense fp8 GEMM shapes, the w4a16
and w4a8 layers).

--impl reference times the CPU path alone: the reference is a set of Python scripts that exists
only on the development machine, so what runs here is oracle/restate.py's restatement of its
torch code path (MoEGate + the per-expert loop of moe_infer), every step over the full 4096-token
batch.
"""
import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

import torch

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

METRIC = "ep_moe_layer_tokens_per_s"
UNIT = "tokens/s"
NOMINAL_FP8_TFLOPS = 4500.0
NOMINAL_HBM_GBS = 8000.0
# dram__bytes_read.sum + dram__bytes_write.sum of ONE gate/up launch in the ncu capture summarised in
# profiles/gemm_block_kernel_fp8_cfg3_small.md (32 experts, 4096 rows).  At EP = 1 the full workload has
# 8x the experts and 8x the rows, and the traffic (weights once + rows once) grows in proportion.
NCU_GEMM1_SMALL = {"dram_bytes": 1026.601e6 + 16.708864e6, "experts": 32, "rows": 4096}


def _peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        d = json.load(open(path))
        return {"hbm_gbs": float(d["hbm_gbs"]), "bf16_tflops": float(d["bf16_tflops"]),
                "bf16_tflops_sustained": float(d.get("bf16_tflops_sustained", d["bf16_tflops"])),
                "source": "measured"}
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0, "source": "fallback"}


class ClockSampler:
    """Samples nvidia-smi clocks and throttle reasons of one GPU while the timed region runs."""
    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
         "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_id):
        self.index, self.proc, self.lines = gpu_id, None, []

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--id={self.index}", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits", "-lms", "50"],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except Exception:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            self.proc.kill()
        sm, mx, reasons = [], None, set()
        for ln in self.lines:
            f = [s.strip() for s in ln.split(",")]
            if len(f) < 9:
                continue
            try:
                sm.append(float(f[1])); mx = float(f[2])
            except ValueError:
                continue
            for name, val in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), f[5:9]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": mx,
                "reasons": sorted(reasons), "samples": len(sm)}


def _dist_env():
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    return rank, world, local


# ------------------------------------------------------------------------------------------
# CPU baseline: the reference's torch path (MoEGate + moe_infer per-expert loop,
# moe/all2all_moe.py:60-118, 186-280) as restated in oracle/restate.py, on the host cores.
# ------------------------------------------------------------------------------------------
def cpu_reference_run(shape, layer_weights_fn, sample_tokens, steps, warmup, budget_s=None):
    """Times gate + per-expert loop on `sample_tokens` tokens; returns (tokens/s, cores, tokens used).
    With budget_s the sample is resized after a probe step so that all steps fit the budget."""
    from oracle import restate as R
    from llm_kernels_b200 import workloads as WL
    torch.set_num_threads(os.cpu_count() or 1)
    cores = torch.get_num_threads()
    W, bias = WL.router_params(shape)
    gw, uw, dw = layer_weights_fn()           # bf16 CPU tensors [E,I,H], [E,I,H], [E,H,I]

    def one(x):
        t0 = time.perf_counter()
        idx, w = R.gate_forward(x, W, bias, top_k=shape.top_k, n_group=shape.n_group,
                                topk_group=shape.topk_group, scoring_func=shape.scoring,
                                routed_scaling_factor=shape.scaling)
        R.moe_infer_dense(x, idx, w, gw, uw, dw)
        return time.perf_counter() - t0

    if budget_s is not None:
        probe = one(WL.tokens(shape, rank=0, n=64))
        per_step = budget_s / max(steps + warmup, 1)
        # cost is roughly affine in tokens (weights stream once per step); scale conservatively
        sample_tokens = int(max(64, min(shape.tokens, 64 * per_step / max(probe, 1e-3))))
        sample_tokens -= sample_tokens % 64
    x = WL.tokens(shape, rank=0, n=sample_tokens)
    times = [one(x) for _ in range(warmup + steps)][warmup:]
    return sample_tokens / statistics.median(times), cores, sample_tokens


def cpu_weights_from_layer(layer, shape):
    """Dequantized bf16 copies of the layer's own quantized experts, moved to the host."""
    from oracle import restate as R
    E, I, H = shape.experts, shape.inter, shape.hidden
    gw = torch.empty(E, I, H, dtype=torch.bfloat16)
    uw = torch.empty(E, I, H, dtype=torch.bfloat16)
    dw = torch.empty(E, H, I, dtype=torch.bfloat16)
    for e in range(E):
        w13 = R.weight_dequant_fp8(layer.w13_weight[e], layer.w13_weight_scale[e], dtype=torch.bfloat16)
        gw[e].copy_(w13[:I]); uw[e].copy_(w13[I:])
        dw[e].copy_(R.weight_dequant_fp8(layer.w2_weight[e], layer.w2_weight_scale[e], dtype=torch.bfloat16))
    return gw, uw, dw


def cpu_weights_random(shape):
    """Host bf16 expert weights ~N(0, 0.02): one drawn matrix per projection, rescaled per expert
    (drawing 11 G normal variates on the host would take longer than the measurement)."""
    E, I, H = shape.experts, shape.inter, shape.hidden
    g = torch.Generator().manual_seed(shape.seed)
    base_g = torch.randn(I, H, generator=g) * 0.02
    base_u = torch.randn(I, H, generator=g) * 0.02
    base_d = torch.randn(H, I, generator=g) * 0.02
    gw = torch.empty(E, I, H, dtype=torch.bfloat16); uw = torch.empty_like(gw)
    dw = torch.empty(E, H, I, dtype=torch.bfloat16)
    for e in range(E):
        f = 1.0 + 0.001 * e
        gw[e] = (base_g * f).to(torch.bfloat16); uw[e] = (base_u * f).to(torch.bfloat16)
        dw[e] = (base_d * f).to(torch.bfloat16)
    return gw, uw, dw


def run_reference(args):
    rank, world, _ = _dist_env()
    if rank != 0:
        return
    from llm_kernels_b200 import workloads as WL
    shape = WL.CONFIG3 if args.shape == "cfg3" else WL.CONFIG3_SMALL
    t0 = time.perf_counter()
    # every step is one pass over the full batch of the workload (a fixed sample: the whole 4096 tokens)
    v, cores, sample = cpu_reference_run(shape, lambda: cpu_weights_random(shape), shape.tokens, args.steps,
                                         args.warmup)
    line = {
        "impl": "reference", "metric": METRIC, "value": v, "unit": UNIT, "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": 1e3 * sample / v,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16",
        "data": "synthetic", "config": _config(shape, args.gpus),
        "cpu_baseline": {"value": v, "unit": UNIT, "cores": cores, "kind": "port",
                         "sample": f"{sample} of {shape.tokens} tokens per step (fixed), all {shape.experts} experts, bf16 "
                                   f"weights, torch CPU per-expert loop, median of {args.steps} steps after "
                                   f"{args.warmup} ({time.perf_counter() - t0:.0f} s incl. setup)"},
        "e2e": {"value": v, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    print(json.dumps(line), flush=True)


def _config(shape, n):
    return {"workload": f"{'configs[3]' if shape.experts == 256 else 'configs[3] cut to 1/8 (profiling case)'}: DeepSeek-V3-shape fp8 blockwise MoE layer, EP={n}, {shape.tokens} tokens/rank, "
                        f"{shape.experts} experts top-{shape.top_k} (groups {shape.n_group}/{shape.topk_group}), hidden "
                        f"{shape.hidden}, SwiGLU {shape.inter}, Zipf(1.1)-biased routing, seed {shape.seed}",
            "tokens_per_rank": shape.tokens, "ep_size": n,
            "l2": "inputs larger than L2: each step streams the rank's expert weights "
                  f"({shape.experts // n * 3 * shape.hidden * shape.inter / 1e9:.2f} GB) and 4 rotating token batches"}


# ------------------------------------------------------------------------------------------
def bind_to_gpu_numa_node(dev):
    """Pins this process to the CPUs of the NUMA node its GPU hangs off, so that the pinned host buffers
    allocated afterwards are node-local (first touch) and N ranks' host<->device copies do not all land
    on one socket's memory.  Returns a short description, or None when the topology cannot be read."""
    try:
        props = torch.cuda.get_device_properties(dev)
        bdf = f"{props.pci_domain_id:04x}:{props.pci_bus_id:02x}:{props.pci_device_id:02x}.0"
        node = int(open(f"/sys/bus/pci/devices/{bdf}/numa_node").read())
        if node < 0:
            return "single node (no NUMA affinity reported for the GPU)"
        cpus = set()
        for part in open(f"/sys/devices/system/node/node{node}/cpulist").read().strip().split(","):
            lo, _, hi = part.partition("-")
            cpus.update(range(int(lo), int(hi or lo) + 1))
        allowed = cpus & os.sched_getaffinity(0)
        if not allowed:
            return f"node{node}: none of its CPUs is in this process's affinity mask"
        os.sched_setaffinity(0, allowed)
        return f"node{node}:{len(allowed)}cpus"
    except Exception as e:
        return f"not bound ({type(e).__name__})"


def parity_check(world, rank, dev, exchange):
    """One reduced-shape forward (32 experts top-4 of 2 of 4 groups, hidden 512, SwiGLU 256, 96 + 32 r tokens on
    rank r) through the exchange the timed run uses; every rank compares with the CPU oracle, which does not
    depend on the EP degree.  Returns the dict for the JSON line (max / all over ranks)."""
    import torch.distributed as dist
    from dataclasses import replace
    from llm_kernels_b200 import workloads as WL
    from llm_kernels_b200.moe.all2all_moe import DeepseekV3MoE
    from oracle import restate as R
    shape = replace(WL.CONFIG3, tokens=96 + 32 * rank, hidden=512, inter=256, experts=32, n_group=4, topk_group=2,
                    top_k=4)
    cfg = WL.make_config(shape, ep_size=world)
    cfg.ep_exchange = exchange
    layer = DeepseekV3MoE(cfg, device=dev).eval()
    WL.fill_layer_cpu_seeded(layer, shape)
    x = WL.tokens(shape, rank=rank)
    xd = x.to(dev).view(1, shape.tokens, -1)
    layer(xd)
    y = layer(xd)                                   # second pass: buffers and peer mappings are re-used
    gi, gw = layer.gate(xd)
    layer.check_status()
    W, bias = WL.router_params(shape)
    kw = dict(top_k=shape.top_k, n_group=shape.n_group, topk_group=shape.topk_group, scoring_func=shape.scoring)
    ok = R.gate_margins_fp64(x, W, bias, **kw) > 1e-5
    idx, w = R.gate_forward(x, W, bias, routed_scaling_factor=shape.scaling, **kw)
    routing = bool(torch.equal(R.canonical_rows(gi.cpu(), gw.cpu())[0][ok], R.canonical_rows(idx, w)[0][ok]))
    q13, q2 = [], []
    for e in range(shape.experts):
        g, u, d = WL.expert_weights_cpu(shape, e)
        q13.append(R.weight_quant_fp8(torch.cat([g, u], 0)))
        q2.append(R.weight_quant_fp8(d))
    y_ref = R.moe_layer_fp8(x, idx, w, torch.stack([a for a, _ in q13]), torch.stack([s for _, s in q13]),
                            torch.stack([a for a, _ in q2]), torch.stack([s for _, s in q2]), ep_size=world)
    err = R.rel_fro(y.cpu().view(shape.tokens, -1).float(), y_ref.float())
    stat = torch.tensor([err, 0.0 if routing else 1.0], device=dev, dtype=torch.float64)
    rows = torch.tensor([layer.last_recv_rows, shape.tokens * shape.top_k], device=dev)
    if world > 1:
        dist.all_reduce(stat, op=dist.ReduceOp.MAX)
        dist.all_reduce(rows)
    del layer
    return {"rel_fro_max": float(stat[0]), "tolerance": 1e-2, "routing_exact": float(stat[1]) == 0.0,
            "rows_conserved": int(rows[0]) == int(rows[1]), "ep": world, "exchange": exchange,
            "case": "32 experts top-4 (groups 4/2), hidden 512, SwiGLU 256, 96 + 32*rank tokens per rank, "
                    "checked against the CPU oracle on every rank"}


def _time_launches(fn, n, dev):
    """Average device time (ms) of n back-to-back calls of fn(i), CUDA events on the current stream."""
    fn(0)
    torch.cuda.synchronize(dev)
    s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    s.record()
    for i in range(n):
        fn(i)
    e.record()
    e.synchronize()
    return s.elapsed_time(e) / n


def other_configs(dev, peaks, fp8_peak):
    """Device-timed records of the benchmark configurations that are not the headline (N = 1 only).
    cfg1: dense fp8 blockwise GEMM N = K = 7168, M in {16, 128, 1024, 4096}; the weight rotates over
    4 copies (205 MB > L2) so every launch streams it from HBM; 20 back-to-back launches.
    cfg2: w4a16 layer at full width (8 experts, H 4096, I 14336, 8192 tokens = the 16384 rows one rank's expert
    processes at EP = 8).  cfg4: w4a8 layer, 64 tokens, 256 experts."""
    from llm_kernels_b200 import workloads as WL
    from llm_kernels_b200.moe.all2all_moe import DeepseekV3MoE
    from llm_kernels_b200.quantization import fp8_kernel
    out = {}
    tensor_peak = fp8_peak or 2 * peaks["bf16_tflops"]
    N_, K = 7168, 7168
    g = torch.Generator(device=dev).manual_seed(1)
    bq, b_s = fp8_kernel.weight_quant(torch.randn(N_, K, generator=g, device=dev) * 0.02)
    bqs = [bq.clone() for _ in range(4)]
    cfg1 = {}
    for M in (16, 128, 1024, 4096):
        aq, a_s = fp8_kernel.act_quant(torch.randn(M, K, generator=g, device=dev).to(torch.bfloat16))
        ms = _time_launches(lambda i: fp8_kernel.fp8_gemm(aq, a_s, bqs[i & 3], b_s, out_dtype=torch.bfloat16), 20, dev)
        tf = 2.0 * M * N_ * K / (ms * 1e-3) / 1e12
        gbs = (N_ * K + M * K + 2 * M * N_ + 4 * (N_ // 128) * (K // 128) + 4 * M * (K // 128)) / (ms * 1e-3) / 1e9
        cfg1[str(M)] = {"us": ms * 1e3, "tflops": tf, "frac_of_fp8_burst_peak": tf / tensor_peak, "gbs": gbs,
                        "frac_of_hbm_peak": gbs / peaks["hbm_gbs"]}
    out["cfg1_dense_fp8_gemm_n7168_k7168"] = cfg1
    del bqs, bq
    for name, shape in (("cfg2_w4a16_mixtral_8192tok", WL.CONFIG2), ("cfg4_w4a8_decode_64tok", WL.CONFIG4)):
        layer = DeepseekV3MoE(WL.make_config(shape), device=dev).eval()
        WL.fill_layer_gpu(layer, shape)
        x = WL.tokens(shape, device=dev).view(1, shape.tokens, -1)
        for _ in range(2):
            layer(x)
        layer.check_status()
        ms = _time_launches(lambda i: layer(x), 10, dev)
        layer.stage_events = []
        for _ in range(5):
            layer(x)
        torch.cuda.synchronize(dev)
        ev, st = layer.stage_events, {}
        layer.stage_events = None
        for (n0, e0), (n1, e1) in zip(ev[:-1], ev[1:]):
            if n1 != "start":
                st[n1] = st.get(n1, 0.0) + e0.elapsed_time(e1) / 5
        rows = shape.tokens * shape.top_k
        rec = {"ms_per_step": ms, "tokens_per_s": shape.tokens / (ms * 1e-3), "stages_ms": st,
               "gemm_tflops_whole_step": 6.0 * shape.hidden * shape.inter * rows / (ms * 1e-3) / 1e12}
        wbytes = shape.experts * 3 * shape.hidden * shape.inter // 2          # packed int4
        rec["packed_weight_gbs_whole_step"] = wbytes / (ms * 1e-3) / 1e9
        if shape.method == "w4a16":
            rec["frac_of_bf16_peak_whole_step"] = rec["gemm_tflops_whole_step"] / peaks["bf16_tflops"]
        else:
            rec["frac_of_hbm_peak_whole_step"] = rec["packed_weight_gbs_whole_step"] / peaks["hbm_gbs"]
        out[name] = rec
        del layer
        torch.cuda.empty_cache()
    return out


def run_w4a8_small(args):
    """`--shape cfg4-small`: the decode-regime w4a8 layer of configs[4] cut to 64 experts (1.4 GB of packed weights,
    well above L2, small enough for a profiler capture), 64 tokens top-8 on one GPU.  Prints one JSON line with the
    device time of the step and of its stages; it is a profiling aid, not the benchmark."""
    from dataclasses import replace
    from llm_kernels_b200 import workloads as WL
    from llm_kernels_b200.moe.all2all_moe import DeepseekV3MoE
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    shape = replace(WL.CONFIG4, experts=64)
    layer = DeepseekV3MoE(WL.make_config(shape), device=dev).eval()
    WL.fill_layer_gpu(layer, shape)
    x = WL.tokens(shape, device=dev).view(1, shape.tokens, -1)
    for _ in range(args.warmup):
        layer(x)
    layer.check_status()
    ms = _time_launches(lambda i: layer(x), args.steps, dev)
    layer.stage_events = []
    for _ in range(args.steps):
        layer(x)
    torch.cuda.synchronize(dev)
    ev, st = layer.stage_events, {}
    for (n0, e0), (n1, e1) in zip(ev[:-1], ev[1:]):
        if n1 != "start":
            st[n1] = st.get(n1, 0.0) + e0.elapsed_time(e1) / args.steps
    wbytes = shape.experts * 3 * shape.hidden * shape.inter // 2
    print(json.dumps({"metric": "w4a8_decode_layer_ms_per_step", "value": ms, "unit": "ms", "n_gpus": 1,
                      "steps": args.steps, "warmup": args.warmup, "higher_is_better": False, "dtype": "int4 x int8",
                      "data": "synthetic", "config": {"workload": "configs[4] with 64 of its 256 experts, 64 tokens top-8"},
                      "stages_ms": st, "packed_weight_bytes": wbytes,
                      "packed_weight_gbs_whole_step": wbytes / (ms * 1e-3) / 1e9}), flush=True)


def measure_fp8_peak(dev):
    """Dense e4m3 GEMM 8192^3 through torch._scaled_mm (cuBLASLt), TFLOP/s: (burst, sustained).  burst = best of
    12 single launches (the figure for a kernel timed alone); sustained = back-to-back launches for about one
    second under the power cap (the figure for a kernel timed inside a long loop, as the expert GEMMs are)."""
    try:
        n = 8192
        a = torch.randn(n, n, device=dev).to(torch.float8_e4m3fn)
        b = torch.randn(n, n, device=dev).to(torch.float8_e4m3fn).t()
        one = torch.ones((), device=dev)
        run = lambda: torch._scaled_mm(a, b, scale_a=one, scale_b=one, out_dtype=torch.bfloat16)
        best = None
        for _ in range(12):
            s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            s.record()
            run()
            e.record(); e.synchronize()
            ms = s.elapsed_time(e)
            best = ms if best is None else min(best, ms)
        reps = max(20, int(1000.0 / best))
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s.record()
        for _ in range(reps):
            run()
        e.record(); e.synchronize()
        flops = 2.0 * n ** 3
        return flops / (best * 1e-3) / 1e12, flops * reps / (s.elapsed_time(e) * 1e-3) / 1e12
    except Exception:
        return None, None


def run_ours(args):
    import torch.distributed as dist
    from llm_kernels_b200 import workloads as WL
    from llm_kernels_b200.moe.all2all_moe import DeepseekV3MoE

    rank, world, local = _dist_env()
    assert world == args.gpus, f"--gpus {args.gpus} but WORLD_SIZE={world} (launch with torch.distributed.run)"
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    # stdout carries ONE JSON line.  Libraries that write to file descriptor 1 on their own (NCCL prints its
    # version banner there) are sent to stderr for the duration of the run; the line is printed on the saved
    # descriptor at the end.
    sys.stdout.flush()
    json_fd = os.dup(1)
    os.dup2(2, 1)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    numa = bind_to_gpu_numa_node(dev)          # before any pinned host allocation
    shape = WL.CONFIG3 if args.shape == "cfg3" else WL.CONFIG3_SMALL
    T, H, k = shape.tokens, shape.hidden, shape.top_k

    cfg = WL.make_config(shape, ep_size=world)
    cfg.ep_passes, cfg.ep_gemm_ctas, cfg.ep_exchange = args.ep_passes, args.ep_gemm_ctas, args.ep_exchange
    layer = DeepseekV3MoE(cfg, device=dev).eval()
    WL.fill_layer_gpu(layer, shape)
    nbatch = 4
    xs = [WL.tokens(shape, rank=rank * 16 + i, device=dev).view(1, T, H) for i in range(nbatch)]
    host_in = [x.cpu().pin_memory() for x in xs]

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def timed(fn, steps, drain=None):
        barrier()
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s.record()
        for i in range(steps):
            fn(i)
        if drain is not None:
            drain()                # work on other streams that belongs to the timed steps
        e.record()
        barrier()
        ms = torch.tensor([s.elapsed_time(e)], device=dev)
        if world > 1:
            dist.all_reduce(ms, op=dist.ReduceOp.MAX)
        return float(ms.item())

    step = lambda i: layer(xs[i % nbatch])

    # End to end: every step's tokens start in pinned host memory and its output ends in pinned host
    # memory, all inside the timed region.  The loop is the one a serving caller writes: the copy of step
    # i+1's tokens (copy-in stream) and the read-back of step i-1's output (copy-out stream) run on the
    # copy engines while step i computes.  Four device input buffers and four host output buffers: the copies may
    # run a few steps ahead, which absorbs the step-to-step jitter of the host's copy bandwidth when several ranks
    # share it (every step of the layer waits for the slowest rank's tokens).
    main_stream = torch.cuda.current_stream()
    s_in, s_out = torch.cuda.Stream(device=dev), torch.cuda.Stream(device=dev)
    NBUF = 4
    dev_ins = [torch.empty(1, T, H, dtype=torch.bfloat16, device=dev) for _ in range(NBUF)]
    host_outs = [torch.empty(T, H, dtype=torch.bfloat16).pin_memory() for _ in range(NBUF)]
    ev_in = [torch.cuda.Event() for _ in range(NBUF)]
    ev_read = [torch.cuda.Event() for _ in range(NBUF)]    # step finished reading dev_ins[b]
    ev_done = [torch.cuda.Event() for _ in range(NBUF)]    # host_outs[b] holds its step's output

    def step_e2e(i):
        b = i % NBUF
        with torch.cuda.stream(s_in):
            s_in.wait_event(ev_read[b])
            dev_ins[b].copy_(host_in[i % nbatch], non_blocking=True)
            ev_in[b].record(s_in)
        main_stream.wait_event(ev_in[b])
        y = layer(dev_ins[b])
        ev_read[b].record(main_stream)
        y.record_stream(s_out)
        with torch.cuda.stream(s_out):
            s_out.wait_event(ev_read[b])
            host_outs[b].copy_(y.view(T, H), non_blocking=True)
            ev_done[b].record(s_out)

    def e2e_drain():
        s_out.synchronize()                                 # the caller holds every result

    # parity first: a reduced-shape forward through the same exchange, every rank against the CPU oracle
    parity = parity_check(world, rank, dev, layer.exchange if world > 1 else "none") if args.parity else None

    for i in range(args.warmup):
        step(i)
    layer.check_status()
    sampler = ClockSampler("GPU-" + str(torch.cuda.get_device_properties(dev).uuid))
    sampler.start()
    time.sleep(1.0)
    # the timed region (exactly `steps` steps between barriers) is taken `repeats` times back to back so that
    # the clock sampler sees load for long enough; the median region is reported, all of them are listed
    regions = [timed(step, args.steps) for _ in range(args.repeats)]
    ms = statistics.median(regions)
    layer.check_status()
    for i in range(min(args.warmup, 3)):
        step_e2e(i)
    e2e_drain()
    regions_e2e = [timed(step_e2e, args.steps, drain=e2e_drain) for _ in range(args.repeats)]
    ms_e2e = statistics.median(regions_e2e)
    clocks = sampler.stop()

    # ceiling of the host<->device traffic alone: every rank copies one step's input in and one step's output
    # out at the same time, no compute
    dev_out = torch.empty(T, H, dtype=torch.bfloat16, device=dev)

    def copy_only(i):
        b = i % NBUF
        with torch.cuda.stream(s_in):
            dev_ins[b].copy_(host_in[i % nbatch], non_blocking=True)
        with torch.cuda.stream(s_out):
            host_outs[b].copy_(dev_out, non_blocking=True)

    def copy_drain():
        torch.cuda.current_stream().wait_stream(s_in)
        torch.cuda.current_stream().wait_stream(s_out)

    ms_copy = timed(copy_only, args.steps, drain=copy_drain)

    # per-stage device times (separate pass, events between the stages)
    layer.stage_events = []
    barrier()
    for i in range(args.steps):
        step(i)
    torch.cuda.synchronize()
    ev = layer.stage_events
    layer.stage_events = None
    stages = {}
    for (n0, e0), (n1, e1) in zip(ev[:-1], ev[1:]):
        if n1 != "start":
            stages[n1] = stages.get(n1, 0.0) + e0.elapsed_time(e1)
    stages = {n: v / args.steps for n, v in stages.items()}
    rows = layer.last_recv_rows
    seg_last = layer._last[2]                                   # group table of the last forward on this rank
    active = int(((seg_last[1:] - seg_last[:-1]) > 0).sum().item())   # experts that received rows
    barrier()
    g1_ms, g2_ms, _ = layer.time_expert_gemms(max(3, min(args.steps, 10)))   # kernels alone, all groups
    barrier()

    if rank == 0:
        peaks = _peaks()
        tokens_per_s = world * T * args.steps / (ms * 1e-3)
        e2e_tokens_per_s = world * T * args.steps / (ms_e2e * 1e-3)
        El, I = shape.experts // world, shape.inter
        # dominant kernel: gate/up grouped GEMM.  Algorithmic bytes per launch: the w13 (e4m3) + f32 block
        # scales of every local expert THAT RECEIVED ROWS once (experts without rows are skipped by the
        # kernel and must not be credited), the activation rows (packed e4m3 + f32 scales) once, the e4m3
        # SwiGLU output + scales once.
        g1_bytes = (active * (2 * I * H + (2 * I // 128) * (H // 128) * 4) + rows * (H + H // 32) + rows * (I + I // 32))
        g1_flops = 4.0 * H * I * rows
        g2_flops = 2.0 * H * I * rows
        stages["gemm1_alone"], stages["gemm2_alone"] = g1_ms, g2_ms
        if world == 1:      # inside the step the two launches run back to back on one stream: use those events
            g1_s, g2_s = stages["gemm1_swiglu"] * 1e-3, stages["gemm2"] * 1e-3
        else:               # with the exchange in between the in-step events include waits: use the re-launches
            g1_s, g2_s = g1_ms * 1e-3, g2_ms * 1e-3
        hbm_bound = world == 1
        fp8_peak, fp8_sustained = measure_fp8_peak(dev) if args.fp8_peak else (None, None)
        # the expert GEMMs are timed inside loops of tens of milliseconds: the sustained figure is their peak
        tensor_peak = fp8_sustained or 2 * peaks["bf16_tflops_sustained"]
        if hbm_bound:
            ach = g1_bytes / g1_s / 1e9
            roof = {"kernel": "gemm_block_kernel<fp8> (gate/up + SwiGLU epilogue)", "bound": "hbm", "achieved": ach,
                    "peak": peaks["hbm_gbs"], "unit": "GB/s", "frac": ach / peaks["hbm_gbs"],
                    # ncu DRAM bytes of the 32-expert capture (all 32 active), scaled by the experts that stream
                    # weights here: traffic is weight-dominated and grows in proportion
                    "traffic": NCU_GEMM1_SMALL["dram_bytes"] * active / NCU_GEMM1_SMALL["experts"]
                    if rows == NCU_GEMM1_SMALL["rows"] * El // NCU_GEMM1_SMALL["experts"] else None,
                    "peak_source": f"{peaks['source']} copy bandwidth", "algorithmic_bytes": g1_bytes,
                    "active_experts": active}
        else:
            ach = g1_flops / g1_s / 1e12
            roof = {"kernel": "gemm_block_kernel<fp8> (gate/up + SwiGLU epilogue)", "bound": "tensor", "achieved": ach,
                    "peak": tensor_peak, "unit": "TFLOP/s", "frac": ach / tensor_peak, "traffic": None,
                    "peak_source": "torch._scaled_mm e4m3 8192^3 back to back for 1 s in this run (sustained; the "
                                   "kernel is timed in a loop of the same kind)" if fp8_sustained else
                                   f"2 x {peaks['source']} sustained bf16 cuBLAS",
                    "frac_of_burst_peak": ach / fp8_peak if fp8_peak else None,
                    "frac_of_nominal_fp8_4500": ach / NOMINAL_FP8_TFLOPS, "algorithmic_flops": g1_flops}
        line = {
            "metric": METRIC, "value": tokens_per_s, "unit": UNIT, "n_gpus": world, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": ms / args.steps, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "fp8_e4m3", "data": "synthetic", "config": _config(shape, world),
            "clocks": clocks,
            "e2e": {"value": e2e_tokens_per_s, "unit": UNIT, "h2d_bytes_per_step": T * H * 2,
                    "d2h_bytes_per_step": T * H * 2, "ms_per_step": ms_e2e / args.steps,
                    "ms_per_step_all": [r / args.steps for r in regions_e2e],
                    "copy_only_ms_per_step": ms_copy / args.steps, "host_numa_binding": numa},
            "repeats": args.repeats, "ms_per_step_all": [r / args.steps for r in regions],
            # this library's kernels per step: router GEMM + selection, 3 of the counting sort, permute,
            # un-permute (7); then 2 grouped GEMMs per pass (+ 1 row gather per pass behind the NCCL and
            # copy-engine exchanges), or 2 plan kernels + 2 grouped GEMMs for the fused exchange
            "gpu_launches": (7 + (4 if layer.exchange == "fused" else (2 if world == 1 else 3) * layer.passes)) * args.steps,
            "roofline": roof,
            "tokens_per_s_per_gpu": tokens_per_s / world,
            "stages_ms": stages, "rows_rank0": rows,
            "grouped_gemm": {"gemm1_tflops": g1_flops / g1_s / 1e12, "gemm2_tflops": g2_flops / g2_s / 1e12,
                             "both_tflops": (g1_flops + g2_flops) / (g1_s + g2_s) / 1e12,
                             "frac_of_nominal_fp8_4500": (g1_flops + g2_flops) / (g1_s + g2_s) / 1e12 / NOMINAL_FP8_TFLOPS,
                             "fp8_peak_measured_tflops": fp8_peak, "fp8_peak_sustained_tflops": fp8_sustained},
        }
        if world > 1:
            # Expert-parallel exchange on rank 0: rows that arrive from / return to the other ranks (about
            # (N-1)/N of the rows it computes), bytes of their records and results, and what of the exchange is not
            # hidden: the plan, the permute + push + barrier stage beyond the time the same kernel needs for its HBM
            # traffic alone, and the down projection's remote stores (GEMM in the step minus the GEMM alone).
            rec = H + (H // 128) * 4
            remote_rows = rows * (world - 1) / world
            local_permute_ms = (T * H * 2 + T * k * rec) / (peaks["hbm_gbs"] * 1e9) * 1e3
            push_ms = max(stages.get("permute_quant", 0.0) - local_permute_ms, 1e-6)
            ret_ms = max(stages.get("gemm2", 0.0) - g2_ms, 0.0)
            line["nvlink"] = {
                "dispatch_bytes": remote_rows * rec, "dispatch_gbs": remote_rows * rec / (push_ms * 1e-3) / 1e9,
                "return_bytes": remote_rows * H * 2, "return_extra_ms": ret_ms,
                "exposed_ms": stages.get("exchange_plan", 0.0) + push_ms + ret_ms}
        if parity is not None:
            line["parity"] = parity
        if world == 1 and args.cpu_tokens > 0:
            t0 = time.perf_counter()
            v, cores, _ = cpu_reference_run(shape, lambda: cpu_weights_from_layer(layer, shape), args.cpu_tokens, 2, 1)
            line["cpu_baseline"] = {
                "value": v, "unit": UNIT, "cores": cores, "kind": "port",
                "sample": f"{args.cpu_tokens} of {T} tokens, all {shape.experts} experts (dequantized bf16 copies of the "
                          f"same weights), torch CPU per-expert loop, median of 2 after 1 warm-up "
                          f"({time.perf_counter() - t0:.0f} s incl. setup)"}
        if world == 1 and args.configs:
            xs.clear(); dev_ins.clear()
            layer._buffers_cache.clear()
            layer.to_empty(device="cpu")                   # frees the 11 GB of expert weights on the device
            torch.cuda.empty_cache()
            line["configs"] = other_configs(dev, peaks, fp8_peak)
        sys.stdout.flush()
        os.write(json_fd, (json.dumps(line) + "\n").encode())
    os.close(json_fd)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()
    if parity is not None and not (parity["rel_fro_max"] < parity["tolerance"] and parity["routing_exact"]
                                   and parity["rows_conserved"]):
        sys.stderr.write(f"parity check failed: {parity}\n")
        sys.exit(3)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--shape", default="cfg3", choices=["cfg3", "small", "cfg4-small"],
                    help="cfg3 = the benchmark configuration; small = 1/8 of its experts and tokens (profiler captures); "
                         "cfg4-small = only the w4a8 decode layer of configs[4] with 64 experts (profiler captures)")
    ap.add_argument("--ep-passes", type=int, default=1,
                    help="pipeline passes of the EP exchange (N > 1); 1 = exchange and GEMMs back to back")
    ap.add_argument("--ep-exchange", default="auto", choices=["auto", "nccl", "push", "fused"],
                    help="auto = fused; nccl = all_to_all_single; push = peer copies on the copy engines (symmetric memory); "
                         "fused = records and results stored into the peers' buffers by the permute kernel and "
                         "the down projection")
    ap.add_argument("--ep-gemm-ctas", type=int, default=0,
                    help="GEMM grid cap while NCCL kernels overlap (N > 1, passes > 1); 0 = all SMs")
    ap.add_argument("--cpu-tokens", type=int, default=512, help="tokens in the CPU baseline sample (0 = skip)")
    ap.add_argument("--no-fp8-peak", dest="fp8_peak", action="store_false")
    ap.add_argument("--no-parity", dest="parity", action="store_false", help="skip the reduced-shape parity pass")
    ap.add_argument("--no-configs", dest="configs", action="store_false",
                    help="skip the records of the other benchmark configurations (N = 1)")
    ap.add_argument("--repeats", type=int, default=5, help="timed regions of `steps` steps; the median is reported")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3)
    if args.impl == "reference":
        run_reference(args)
    elif args.shape == "cfg4-small":
        run_w4a8_small(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
