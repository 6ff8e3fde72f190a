"""Host-side plumbing of the expert-parallel exchange (device-agnostic torch.distributed
calls; NCCL over NVLink on GPUs, gloo in the CPU tests).

Replaces the count exchange, the four host synchronisations and the list-form
all_to_all of the reference's moe_infer (moe/all2all_moe.py:206-227, :260-268) with
one count all-to-all, ONE host read of 2*ep integers, and all_to_all_single calls
with split sizes.  Rows are already ordered by destination rank because experts are
range-partitioned (moe/all2all_moe.py:133-146) and rows are sorted by expert id.
"""
from dataclasses import dataclass
from typing import List

import torch
import torch.distributed as dist


@dataclass
class ExchangePlan:
    in_splits: List[int]       # rows this rank sends to each peer
    out_splits: List[int]      # rows this rank receives from each peer
    recv_rows: int
    recv_counts: torch.Tensor  # int64 [ep, E_local]: rows from (source rank, local expert)
    seg_indptr: torch.Tensor   # int64 [ep*E_local + 1]: row offsets of the received runs
    weight_indices: torch.Tensor  # int64 [ep*E_local]: local expert of each run


def plan_exchange(seg_indptr: torch.Tensor, ep_size: int, group=None) -> ExchangePlan:
    """seg_indptr int64 [E+1] over GLOBAL experts (exclusive prefix of per-expert row counts)."""
    E = seg_indptr.numel() - 1
    El = E // ep_size
    counts = (seg_indptr[1:] - seg_indptr[:-1]).view(ep_size, El).contiguous()
    recv_counts = torch.empty_like(counts)
    dist.all_to_all_single(recv_counts, counts, group=group)
    sizes = torch.stack([counts.sum(1), recv_counts.sum(1)]).cpu()     # the one host sync
    in_splits, out_splits = sizes[0].tolist(), sizes[1].tolist()
    seg = torch.zeros(ep_size * El + 1, dtype=torch.int64, device=seg_indptr.device)
    seg[1:] = torch.cumsum(recv_counts.reshape(-1), 0)
    widx = torch.arange(El, dtype=torch.int64, device=seg_indptr.device).repeat(ep_size)
    return ExchangePlan(in_splits, out_splits, int(sum(out_splits)), recv_counts, seg, widx)


def dispatch(plan: ExchangePlan, send_rows: torch.Tensor, recv_rows: torch.Tensor, group=None):
    """send_rows [S, R] (sorted by global expert) -> recv_rows [plan.recv_rows, R] ordered by
    (source rank, local expert)."""
    dist.all_to_all_single(recv_rows, send_rows, output_split_sizes=plan.out_splits,
                           input_split_sizes=plan.in_splits, group=group)
    return recv_rows


def combine(plan: ExchangePlan, expert_out: torch.Tensor, back_rows: torch.Tensor, group=None):
    """Inverse of dispatch: expert_out [plan.recv_rows, H] -> back_rows [S, H] in the sender's
    expert-sorted order (reference :264-267 with the split lists swapped)."""
    dist.all_to_all_single(back_rows, expert_out, output_split_sizes=plan.in_splits,
                           input_split_sizes=plan.out_splits, group=group)
    return back_rows
