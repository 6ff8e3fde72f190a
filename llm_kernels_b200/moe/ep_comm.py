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


# --------------------------------------------------------------------------------------------
# Pipelined exchange: the local experts of every rank are cut into `passes` ranges.  Rows are
# ordered (pass, destination rank, expert-in-pass) on the sender and (pass, source rank,
# expert-in-pass) on the receiver, so each pass is one contiguous all_to_all_single in each
# direction and one contiguous run of GEMM groups; pass p+1 is dispatched and pass p-1 is
# combined while the expert GEMMs of pass p run.
# --------------------------------------------------------------------------------------------
def expert_order(num_experts: int, ep_size: int, passes: int, device) -> torch.Tensor:
    """remap int64 [E]: position of global expert e in the (pass, owner rank, expert-in-pass) order."""
    El = num_experts // ep_size
    Ep = El // passes
    e = torch.arange(num_experts, device=device)
    dest, loc = e // El, e % El
    return (loc // Ep) * (ep_size * Ep) + dest * Ep + (loc % Ep)


@dataclass
class PipelinedPlan:
    passes: int
    in_splits: List[List[int]]     # [pass][dest]  rows sent
    out_splits: List[List[int]]    # [pass][src]   rows received
    send_off: List[int]            # [pass+1] row offsets of the passes in the send buffer
    recv_off: List[int]            # [pass+1] row offsets of the passes in the receive buffer
    seg_indptr: torch.Tensor       # int64 [passes*ep*Ep + 1] over received rows
    weight_indices: torch.Tensor   # int64 [passes*ep*Ep] local expert of each received run
    groups_per_pass: int
    # The same rows merged per expert (all sources of an expert contiguous), which is what keeps the
    # GEMM's 128-row tiles full: merged row i is received row gather_map[i].
    merged_seg: torch.Tensor       # int64 [passes*Ep + 1]
    merged_widx: torch.Tensor      # int64 [passes*Ep]
    gather_map: torch.Tensor       # int32 [recv_rows]
    experts_per_pass: int

    @property
    def recv_rows(self) -> int:
        return self.recv_off[-1]


def plan_exchange_pipelined(seg_indptr: torch.Tensor, ep_size: int, passes: int, group=None) -> PipelinedPlan:
    """seg_indptr int64 [E+1] over experts in expert_order() positions."""
    E = seg_indptr.numel() - 1
    El = E // ep_size
    Ep = El // passes
    dev = seg_indptr.device
    counts = (seg_indptr[1:] - seg_indptr[:-1]).view(passes, ep_size, Ep)        # [pass, dest, j]
    send_c = counts.permute(1, 0, 2).contiguous()                                # [dest, pass, j]
    recv_c = torch.empty_like(send_c)
    dist.all_to_all_single(recv_c, send_c, group=group)                          # [src, pass, j]
    recv_counts = recv_c.permute(1, 0, 2).contiguous()                           # [pass, src, j]
    sizes = torch.stack([counts.sum(2), recv_counts.sum(2)]).cpu()               # the one host sync
    in_splits, out_splits = sizes[0].tolist(), sizes[1].tolist()
    send_off, recv_off = [0], [0]
    for p in range(passes):
        send_off.append(send_off[-1] + int(sum(in_splits[p])))
        recv_off.append(recv_off[-1] + int(sum(out_splits[p])))
    seg = torch.zeros(passes * ep_size * Ep + 1, dtype=torch.int64, device=dev)
    seg[1:] = torch.cumsum(recv_counts.reshape(-1), 0)
    j = torch.arange(Ep, dtype=torch.int64, device=dev)
    widx = (torch.arange(passes, dtype=torch.int64, device=dev).view(passes, 1, 1) * Ep
            + j.view(1, 1, Ep)).expand(passes, ep_size, Ep).reshape(-1).contiguous()
    R = recv_off[-1]
    c2 = recv_counts.reshape(passes, -1)
    base = torch.tensor(recv_off[:-1], dtype=torch.int64, device=dev).view(passes, 1)
    src_start = (torch.cumsum(c2, 1) - c2 + base).view(passes, ep_size, Ep)
    ct = recv_counts.transpose(1, 2).contiguous()                                # [pass, j, src]
    ct2 = ct.reshape(passes, -1)
    dst_start = (torch.cumsum(ct2, 1) - ct2 + base).view(passes, Ep, ep_size)
    delta = (src_start.transpose(1, 2) - dst_start).reshape(-1)
    gather_map = (torch.arange(R, dtype=torch.int64, device=dev)
                  + torch.repeat_interleave(delta, ct.reshape(-1), output_size=R)).to(torch.int32)
    mseg = torch.zeros(passes * Ep + 1, dtype=torch.int64, device=dev)
    mseg[1:] = torch.cumsum(ct.sum(2).reshape(-1), 0)
    mwidx = torch.arange(passes * Ep, dtype=torch.int64, device=dev)
    return PipelinedPlan(passes, in_splits, out_splits, send_off, recv_off, seg, widx, ep_size * Ep,
                         mseg, mwidx, gather_map, Ep)


def dispatch_pass(plan: PipelinedPlan, p: int, send_rows: torch.Tensor, recv_rows: torch.Tensor, group=None):
    dist.all_to_all_single(recv_rows[plan.recv_off[p]:plan.recv_off[p + 1]],
                           send_rows[plan.send_off[p]:plan.send_off[p + 1]],
                           output_split_sizes=plan.out_splits[p], input_split_sizes=plan.in_splits[p], group=group)


def combine_pass(plan: PipelinedPlan, p: int, expert_out: torch.Tensor, back_rows: torch.Tensor, group=None):
    dist.all_to_all_single(back_rows[plan.send_off[p]:plan.send_off[p + 1]],
                           expert_out[plan.recv_off[p]:plan.recv_off[p + 1]],
                           output_split_sizes=plan.in_splits[p], input_split_sizes=plan.out_splits[p], group=group)
