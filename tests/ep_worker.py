"""One rank of the expert-parallel parity check (launched by tests/test_gpu_ep.py).

Every rank routes its own tokens, the fused layer exchanges fp8 records over NCCL, and the
rank's output is compared with the CPU oracle, which does not depend on the EP degree."""
import os
import sys
from dataclasses import replace

import torch
import torch.distributed as dist

ROOT = sys.argv[1]
sys.path.insert(0, ROOT)

from llm_kernels_b200 import workloads as WL                      # noqa: E402
from llm_kernels_b200.moe.all2all_moe import DeepseekV3MoE        # noqa: E402
from oracle import restate as R                                   # noqa: E402


def main():
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", device_id=dev)
    strategy = os.environ.get("EP_STRATEGY", "all2all")
    # all-to-all: every rank routes its own (differently sized) batch; all-reduce: all ranks see one batch
    shape = replace(WL.CONFIG3, tokens=96 + (32 * rank if strategy == "all2all" else 0), hidden=512, inter=256,
                    experts=32, n_group=4, topk_group=2, top_k=4)
    cfg = WL.make_config(shape, ep_size=world)
    cfg.ep_strategy = strategy
    cfg.ep_passes = int(os.environ.get("EP_PASSES", "1"))
    cfg.ep_exchange = os.environ.get("EP_EXCHANGE", "nccl")
    cfg.allreduce_quant = os.environ.get("EP_AR_QUANT") or None
    layer = DeepseekV3MoE(cfg, device=dev).eval()
    WL.fill_layer_cpu_seeded(layer, shape)
    x = WL.tokens(shape, rank=rank if strategy == "all2all" else 0)
    y = layer(x.to(dev).view(1, shape.tokens, -1))
    y = layer(x.to(dev).view(1, shape.tokens, -1))      # twice: buffers and peer mappings are re-used
    layer.check_status()
    torch.cuda.synchronize()
    if layer.exchange == "fused":
        # a second layer on the first one's peer buffers (layers of a model run one after the other)
        layer2 = DeepseekV3MoE(cfg, device=dev).eval()
        WL.fill_layer_cpu_seeded(layer2, shape)
        layer2.share_exchange_buffers(layer)
        y2 = layer2(x.to(dev).view(1, shape.tokens, -1))
        y1 = layer(x.to(dev).view(1, shape.tokens, -1))
        layer2.check_status()
        assert torch.equal(y2, y) and torch.equal(y1, y), "shared peer buffers changed the result"

    W, bias = WL.router_params(shape)
    kw = dict(top_k=shape.top_k, n_group=shape.n_group, topk_group=shape.topk_group, scoring_func=shape.scoring)
    idx, w = R.gate_forward(x, W, bias, routed_scaling_factor=shape.scaling, **kw)
    q13, q2 = [], []
    for e in range(shape.experts):
        g, u, d = WL.expert_weights_cpu(shape, e)
        q13.append(R.weight_quant_fp8(torch.cat([g, u], 0)))
        q2.append(R.weight_quant_fp8(d))
    y_ref = R.moe_layer_fp8(x, idx, w, torch.stack([a for a, _ in q13]), torch.stack([s for _, s in q13]),
                            torch.stack([a for a, _ in q2]), torch.stack([s for _, s in q2]), ep_size=world)
    err = R.rel_fro(y.cpu().view(shape.tokens, -1).float(), y_ref.float())
    own = shape.tokens * shape.top_k if strategy == "all2all" or rank == 0 else 0
    rows = torch.tensor([layer.last_recv_rows, own], device=dev)
    dist.all_reduce(rows)
    assert int(rows[0]) == int(rows[1]), "rows are not conserved across the exchange"
    # an 8-bit all-reduce payload adds its own quantization error twice (int8: ~1e-2, e4m3: a few per cent)
    tol = {None: 1e-2, "int8": 2e-2, "fp8": 6e-2}[cfg.allreduce_quant]
    assert err < tol, f"rank {rank}: rel_fro {err}"
    print(f"rank {rank} ok rel_fro={err:.2e} recv_rows={layer.last_recv_rows}", flush=True)
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
