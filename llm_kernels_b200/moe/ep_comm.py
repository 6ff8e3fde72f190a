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


# --------------------------------------------------------------------------------------------
# Copy-engine exchange over peer-mapped (symmetric) memory.  NCCL's all-to-all moves the rows
# with SM kernels that need a few dozen SMs for bandwidth, while a persistent GEMM CTA owns its
# SM: the two cannot overlap.  Here every rank PUSHES its rows into the peers' receive buffers
# with cudaMemcpyAsync peer copies (copy engines, no SMs; one stream per peer), so pass p+1
# travels while the GEMMs of pass p run.  Arrival is published with a small NCCL all-reduce on
# the exchange stream (it runs after this rank's copies and completes only when every rank got
# there), so no hand-written cross-GPU spin-wait is involved.
# --------------------------------------------------------------------------------------------
class SymmExchange:
    """Peer-mapped receive/back buffers and the per-peer copy streams of one layer."""

    def __init__(self, ep_size: int, rank: int, device, cap_rows: int, rec_bytes: int, slots: int, hidden: int,
                 group=None):
        import torch.distributed._symmetric_memory as symm_mem
        grp = group if group is not None else dist.group.WORLD
        self.ep, self.rank, self.cap_rows, self.rec, self.slots = ep_size, rank, cap_rows, rec_bytes, slots
        self.recv = symm_mem.empty((cap_rows, rec_bytes), dtype=torch.uint8, device=device)
        self.back = symm_mem.empty((slots, hidden), dtype=torch.bfloat16, device=device)
        self._hr = symm_mem.rendezvous(self.recv, grp.group_name)
        self._hb = symm_mem.rendezvous(self.back, grp.group_name)
        self.peer_recv = [self.recv if r == rank else self._hr.get_buffer(r, (cap_rows, rec_bytes), torch.uint8)
                          for r in range(ep_size)]
        self.peer_back = [self.back if r == rank else self._hb.get_buffer(r, (slots, hidden), torch.bfloat16)
                          for r in range(ep_size)]
        self.copy_streams = [torch.cuda.Stream(device=device) for _ in range(ep_size)]
        self.sync_stream = torch.cuda.Stream(device=device)
        self._flag = torch.zeros(1, dtype=torch.float32, device=device)
        self.group = group

    def _fence(self, after_events):
        """All ranks' copies recorded in `after_events` (on this rank) and their peers' are done once the
        all-reduce queued here completes."""
        st = self.sync_stream
        for ev in after_events:
            st.wait_event(ev)
        with torch.cuda.stream(st):
            dist.all_reduce(self._flag, group=self.group)
        ev = torch.cuda.Event()
        ev.record(st)
        return ev

    def push(self, ready_event, pieces):
        """pieces: list of (peer, dst_tensor_slice_on_peer, src_slice).  Queues one peer copy per piece on
        that peer's stream after `ready_event`; returns the event that marks global completion."""
        evs = []
        for peer, dst, src in pieces:
            if src.numel() == 0:
                continue
            st = self.copy_streams[peer]
            st.wait_event(ready_event)
            with torch.cuda.stream(st):
                dst.copy_(src, non_blocking=True)
            ev = torch.cuda.Event()
            ev.record(st)
            evs.append(ev)
        return self._fence(evs)


@dataclass
class PushPlan:
    """Host-side offsets of the pushed exchange, from the all-gathered per-expert counts."""
    base: PipelinedPlan
    dst_off: List[List[int]]      # [pass][dest]  row in dest's receive buffer where my rows start
    src_off: List[List[int]]      # [pass][dest]  row in my send buffer where the rows for dest start
    back_off: List[List[int]]     # [pass][src]   row in src's back buffer where its (pass, me) block starts
    mine_off: List[List[int]]     # [pass][src]   row in my receive buffer where src's rows start


def plan_push(seg_indptr: torch.Tensor, ep_size: int, passes: int, rank: int, group=None) -> PushPlan:
    """Same ordering and GEMM groups as plan_exchange_pipelined, but every rank learns ALL ranks' counts
    (one all_gather of E integers per rank, one host read) so that it can compute where its rows land in
    each peer's buffers."""
    E = seg_indptr.numel() - 1
    El = E // ep_size
    Ep = El // passes
    dev = seg_indptr.device
    counts = (seg_indptr[1:] - seg_indptr[:-1]).contiguous()                     # [E] in (pass, dest, j) order
    allc = torch.empty(ep_size * E, dtype=torch.int64, device=dev)
    dist.all_gather_into_tensor(allc, counts, group=group)
    allc5 = allc.view(ep_size, passes, ep_size, Ep)                              # [src, pass, dest, j]
    recv_counts = allc5[:, :, rank, :].permute(1, 0, 2).contiguous()             # [pass, src, j]
    tot = allc5.sum(3).cpu()                                                     # [src, pass, dest]  (the host read)
    tot_l = tot.tolist()
    in_splits = [[tot_l[rank][p][d] for d in range(ep_size)] for p in range(passes)]
    out_splits = [[tot_l[s][p][rank] for s in range(ep_size)] for p in range(passes)]
    send_off, recv_off = [0], [0]
    for p in range(passes):
        send_off.append(send_off[-1] + sum(in_splits[p]))
        recv_off.append(recv_off[-1] + sum(out_splits[p]))
    # where do things land on the peers
    def recv_off_of(d, p):      # start of pass p in rank d's receive buffer
        return sum(tot_l[s][pp][d] for pp in range(p) for s in range(ep_size))
    def send_off_of(s, p):      # start of pass p in rank s's send buffer
        return sum(tot_l[s][pp][d] for pp in range(p) for d in range(ep_size))
    dst_off = [[recv_off_of(d, p) + sum(tot_l[s][p][d] for s in range(rank)) for d in range(ep_size)]
               for p in range(passes)]
    src_off = [[send_off[p] + sum(in_splits[p][:d]) for d in range(ep_size)] for p in range(passes)]
    back_off = [[send_off_of(s, p) + sum(tot_l[s][p][d] for d in range(rank)) for s in range(ep_size)]
                for p in range(passes)]
    mine_off = [[recv_off[p] + sum(out_splits[p][:s]) for s in range(ep_size)] for p in range(passes)]
    # device-side group tables (identical to plan_exchange_pipelined)
    seg = torch.zeros(passes * ep_size * Ep + 1, dtype=torch.int64, device=dev)
    seg[1:] = torch.cumsum(recv_counts.reshape(-1), 0)
    j = torch.arange(Ep, dtype=torch.int64, device=dev)
    widx = (torch.arange(passes, dtype=torch.int64, device=dev).view(passes, 1, 1) * Ep
            + j.view(1, 1, Ep)).expand(passes, ep_size, Ep).reshape(-1).contiguous()
    R = recv_off[-1]
    c2 = recv_counts.reshape(passes, -1)
    base_t = torch.tensor(recv_off[:-1], dtype=torch.int64, device=dev).view(passes, 1)
    src_start = (torch.cumsum(c2, 1) - c2 + base_t).view(passes, ep_size, Ep)
    ct = recv_counts.transpose(1, 2).contiguous()
    ct2 = ct.reshape(passes, -1)
    dst_start = (torch.cumsum(ct2, 1) - ct2 + base_t).view(passes, Ep, ep_size)
    delta = (src_start.transpose(1, 2) - dst_start).reshape(-1)
    gather_map = (torch.arange(R, dtype=torch.int64, device=dev)
                  + torch.repeat_interleave(delta, ct.reshape(-1), output_size=R)).to(torch.int32)
    mseg = torch.zeros(passes * Ep + 1, dtype=torch.int64, device=dev)
    mseg[1:] = torch.cumsum(ct.sum(2).reshape(-1), 0)
    mwidx = torch.arange(passes * Ep, dtype=torch.int64, device=dev)
    base = PipelinedPlan(passes, in_splits, out_splits, send_off, recv_off, seg, widx, ep_size * Ep,
                         mseg, mwidx, gather_map, Ep)
    return PushPlan(base, dst_off, src_off, back_off, mine_off)


# --------------------------------------------------------------------------------------------
# Exchange folded into the kernels.  The permute/quantize kernel stores every record straight into
# its owner's receive buffer and the down projection stores every output row straight into its
# source rank's return buffer, both through NVLink peer mappings; the only collective left is the
# all-gather of the per-expert counts, and nothing is read by the host (see csrc/ep_fused.cu).
# --------------------------------------------------------------------------------------------
class FusedExchange:
    """Peer-mapped receive/return buffers of one layer, their address tables, and the device-side
    plan outputs.  Construction is collective (symmetric allocation + rendezvous)."""

    def __init__(self, ep_size: int, rank: int, device, cap_rows: int, rec_bytes: int, slots: int, hidden: int,
                 num_experts: int, group=None):
        import torch.distributed._symmetric_memory as symm_mem
        grp = group if group is not None else dist.group.WORLD
        self.ep, self.rank, self.cap_rows, self.rec, self.slots = ep_size, rank, cap_rows, rec_bytes, slots
        self.group = group
        self.recv = symm_mem.empty((cap_rows, rec_bytes), dtype=torch.uint8, device=device)
        self.back = symm_mem.empty((slots, hidden), dtype=torch.bfloat16, device=device)
        self._hr = symm_mem.rendezvous(self.recv, grp.group_name)
        self._hb = symm_mem.rendezvous(self.back, grp.group_name)
        self._peers = ([self.recv if r == rank else self._hr.get_buffer(r, (cap_rows, rec_bytes), torch.uint8)
                        for r in range(ep_size)],
                       [self.back if r == rank else self._hb.get_buffer(r, (slots, hidden), torch.bfloat16)
                        for r in range(ep_size)])
        self.recv_base = torch.tensor([t.data_ptr() for t in self._peers[0]], dtype=torch.int64, device=device)
        self.back_base = torch.tensor([t.data_ptr() for t in self._peers[1]], dtype=torch.int64, device=device)
        El = num_experts // ep_size
        self.counts_all = torch.zeros(ep_size * num_experts, dtype=torch.int64, device=device)
        self.dst_base = torch.zeros(num_experts, dtype=torch.int64, device=device)
        self.local_seg = torch.zeros(El + 1, dtype=torch.int64, device=device)
        self.back_addr = torch.zeros(cap_rows, dtype=torch.int64, device=device)
        self.info = torch.zeros(2, dtype=torch.int32, device=device)
        self._info_host = torch.zeros(2, dtype=torch.int32).pin_memory()
        self._info_event = None
        self._flag = torch.zeros(1, dtype=torch.float32, device=device)

    def publish_info(self):
        """Queues a copy of the plan's {rows received, overflow flag} to pinned host memory behind the plan
        kernel; raise_if_overflowed() reads it once the copy has completed."""
        self._info_host.copy_(self.info, non_blocking=True)
        self._info_event = torch.cuda.Event()
        self._info_event.record()

    def raise_if_overflowed(self):
        if self._info_event is None:
            return
        self._info_event.synchronize()
        self._info_event = None
        if int(self._info_host[1]):
            from .. import _native as N
            raise N.B200MoeError(1, "expert-parallel exchange: a rank was sent more rows than its receive buffer "
                                    "holds (those rows contributed zeros); raise config.ep_recv_capacity")

    def gather_counts(self, seg_indptr: torch.Tensor):
        counts = (seg_indptr[1:] - seg_indptr[:-1]).contiguous()
        dist.all_gather_into_tensor(self.counts_all, counts, group=self.group)
        return self.counts_all

    def barrier(self):
        """Stream-ordered barrier across the ranks: the all-reduce completes on a rank only after every
        rank has reached it on its stream, i.e. after the kernels that stored into this rank's buffers
        (which end with a system-scope fence) have finished."""
        dist.all_reduce(self._flag, group=self.group)


# --------------------------------------------------------------------------------------------
# Quantized all-reduce of the all-gather/all-reduce strategy's output (the scheme of the reference's
# quant_communication/quant_all2all_allreduce.py:52-99): reduce-scatter as an all-to-all of quantized
# chunks, local dequantize + f32 sum, re-quantize, all-gather, dequantize.  The payload travels as a
# uint8 view ("NCCL does not support FP8 directly", :38) and the scales as a second message (:69-70).
# --------------------------------------------------------------------------------------------
def quant_allreduce(x: torch.Tensor, quant, dequant_sum, group=None) -> torch.Tensor:
    """In-place sum of x [T, H] over the ranks of `group` through 8-bit payloads.

    quant(t [R, H]) -> (payload uint8-viewable [R, H], scales [R, H/128]);
    dequant_sum(payload [n, R, H], scales [n, R, H/128], out [R, H]) writes, in out's dtype, the sum over the
    n sources of the dequantized chunks (each rounded to out's dtype first, f32 accumulation).
    Rows are padded to a multiple of the group size; rank r reduces rows [r*R, (r+1)*R)."""
    ep = dist.get_world_size(group)
    rank = dist.get_rank(group)
    T, H = x.shape
    R = -(-T // ep)                                   # rows per rank chunk
    if R * ep != T:
        xp = x.new_zeros(R * ep, H)
        xp[:T].copy_(x)
    else:
        xp = x
    # ---- stage A: quantize all chunks, exchange, dequantize + sum my chunk
    q, s = quant(xp)
    q8 = q.view(torch.uint8).view(ep, R, H)
    s3 = s.view(ep, R, -1)
    rq, rs = torch.empty_like(q8), torch.empty_like(s3)
    dist.all_to_all_single(rq, q8.contiguous(), group=group)
    dist.all_to_all_single(rs, s3.contiguous(), group=group)
    mine = x.new_empty(R, H)
    dequant_sum(rq.view(q.dtype), rs, mine)
    # ---- stage B: quantize the reduced chunk, gather everyone's, dequantize
    q2, s2 = quant(mine)
    gq = torch.empty(ep * R, H, dtype=torch.uint8, device=x.device)
    gs = torch.empty(ep * R, s2.shape[-1], dtype=s2.dtype, device=x.device)
    dist.all_gather_into_tensor(gq, q2.view(torch.uint8).view(R, H).contiguous(), group=group)
    dist.all_gather_into_tensor(gs, s2.view(R, -1).contiguous(), group=group)
    full = x.new_empty(ep * R, H)
    dequant_sum(gq.view(q.dtype).view(1, ep * R, H), gs.view(1, ep * R, -1), full)
    x.copy_(full[:T])
    return x
