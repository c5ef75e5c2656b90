"""Expert-parallel token exchange over NCCL (NVLink 5 / NVSwitch), standing in for the DeepEP
`Buffer` wrappers of the reference (dlblas/layers/moe/token_dispatcher.py:245-602).

One process per GPU; rank r owns experts [r * E_local, (r + 1) * E_local).  Each direction is one
variable-size all-to-all (`all_to_all_single` with split sizes).  The split sizes come from ONE
all-gather of a small count matrix followed by ONE device->host copy (the reference synchronises at
the same point: DeepEP hands back `recv_tokens_per_expert` as a Python list).  Rows are packed and
unpacked by the permutation / gather kernels of the CUDA extension; the planning below is plain
torch on small integer tensors and runs on any backend, so it is unit-tested with gloo on CPU.
"""
import os
from typing import List, Optional, Tuple, Union

import torch
import torch.distributed as dist

from ... import _C, ops
from ...utils.utils import DisposibleTensor


class CommEvent:
    """Event handed out by the async API; `current_stream_wait()` as on DeepEP's EventOverlap."""

    def __init__(self, event: Optional[torch.cuda.Event] = None):
        self.event = event

    def current_stream_wait(self):
        if self.event is not None:
            torch.cuda.current_stream().wait_event(self.event)


def _record_event() -> CommEvent:
    if torch.cuda.is_available():
        ev = torch.cuda.Event()
        ev.record()
        return CommEvent(ev)
    return CommEvent(None)


# ----------------------------------------------------------------------------------------------
# planning (device agnostic)
# ----------------------------------------------------------------------------------------------
class NormalPlan:
    """Exchange plan of the contiguous ("normal") mode: every token goes once to each rank that owns
    at least one of its routed experts."""

    def __init__(self):
        self.dst_pos = None          # int32 [T, W]: row in the send buffer or -1
        self.send_splits = None      # python lists
        self.recv_splits = None
        self.recv_tokens_per_expert = None   # python list, aligned
        self.num_tokens = 0
        self.num_send = 0
        self.num_recv = 0


def make_normal_plan(topk_ids: torch.Tensor, world_size: int, rank: int, num_local_experts: int,
                     group, expert_alignment: int = 128) -> NormalPlan:
    """topk_ids: [T, k] global expert ids (any negative id = unrouted slot).

    dst_pos[t, r] is the row of token t in the part of the send buffer that goes to rank r (rows of
    one rank are contiguous and in token order) or negative if rank r owns none of its experts.  On
    CUDA this is the stable counting sort of the extension applied to the (token, rank) pairs; the
    torch formulation below it is the same computation for CPU tensors."""
    t, k = topk_ids.shape
    dev = topk_ids.device
    ids = topk_ids.to(torch.int64)
    valid = ids >= 0
    if topk_ids.is_cuda:
        dest = ops.ep_dest_ranks(topk_ids.contiguous(), num_local_experts, world_size)
        _, _, _, pos, cnt = ops.sort_by_expert(dest, world_size, want_pos=True, want_counts=True)
        dst_pos = pos.view(t, world_size)
        per_rank = cnt.to(torch.int64)
    else:
        owner = torch.where(valid, ids // num_local_experts, torch.full_like(ids, world_size))
        need = torch.zeros(t, world_size + 1, dtype=torch.int32, device=dev)
        need.scatter_(1, owner, 1)
        need = need[:, :world_size]                                   # [T, W] 0/1
        per_rank = need.sum(dim=0, dtype=torch.int64)                 # rows sent to each rank
        offs = torch.cumsum(per_rank, 0) - per_rank
        within = torch.cumsum(need, dim=0, dtype=torch.int64) - need  # rank of the token among the rank's rows
        dst_pos = torch.where(need > 0, offs[None, :] + within, torch.full_like(within, -1)).to(torch.int32)
    per_expert = torch.bincount(ids[valid], minlength=world_size * num_local_experts)[:world_size * num_local_experts]
    mine = torch.cat([per_rank[:, None], per_expert.view(world_size, num_local_experts)], dim=1).contiguous()
    gathered = torch.empty(world_size, world_size, num_local_experts + 1, dtype=torch.int64, device=dev)
    if world_size > 1:
        dist.all_gather_into_tensor(gathered.view(world_size, -1), mine.view(1, -1), group=group)
    else:
        gathered[0] = mine
    host = gathered.cpu()                                         # the one synchronisation of the dispatch
    plan = NormalPlan()
    plan.dst_pos = dst_pos.contiguous()
    plan.send_splits = host[rank, :, 0].tolist()
    plan.recv_splits = host[:, rank, 0].tolist()
    per_exp = host[:, rank, 1:].sum(dim=0)
    al = expert_alignment
    plan.recv_tokens_per_expert = [int((c + al - 1) // al * al) for c in per_exp.tolist()]
    plan.num_tokens = t
    plan.num_send = int(sum(plan.send_splits))
    plan.num_recv = int(sum(plan.recv_splits))
    return plan


def localize_ids(ids: torch.Tensor, dest_rank: torch.Tensor, num_local_experts: int) -> torch.Tensor:
    """ids [n, k] global, dest_rank [n]: ids local to the destination rank, -1 where another rank owns it."""
    lo = (dest_rank * num_local_experts)[:, None]
    mine = (ids >= lo) & (ids < lo + num_local_experts)
    return torch.where(mine, ids - lo, torch.full_like(ids, -1))


def _a2a(out: torch.Tensor, inp: torch.Tensor, out_splits, in_splits, group, world_size: int):
    if world_size == 1:
        out.copy_(inp)
    else:
        dist.all_to_all_single(out, inp, output_split_sizes=out_splits, input_split_sizes=in_splits, group=group)


# ----------------------------------------------------------------------------------------------
# normal (prefill) mode
# ----------------------------------------------------------------------------------------------
class TokenDispatcherNormal:
    """`DeepEPTokenDispatcherNormal` of the reference (token_dispatcher.py:245-452) over NCCL."""

    def __init__(self, group, num_experts: int = None, num_local_experts: int = None, hidden_size: int = None,
                 params_dtype: torch.dtype = None, expert_alignment: int = 128):
        self.group = group
        self.num_experts = num_experts
        self.num_local_experts = num_local_experts
        self.hidden_size = hidden_size
        self.params_dtype = params_dtype
        self.expert_alignment = expert_alignment
        self.world_size = dist.get_world_size(group) if (dist.is_available() and dist.is_initialized()) else 1
        self.rank = dist.get_rank(group) if (dist.is_available() and dist.is_initialized()) else 0
        assert num_experts == num_local_experts * self.world_size, "experts must split evenly over the ranks"
        self.handle = None
        self.topk_idx = None
        self.topk_weights = None
        self.hidden_shape = None

    # ---- synchronous pair -------------------------------------------------------------------
    def dispatch(self, x: Union[torch.Tensor, Tuple[torch.Tensor, torch.Tensor]], topk_idx: torch.Tensor,
                 topk_weights: torch.Tensor, expert_list: List[int] = None, previous_event=None):
        hidden_states = x[0] if isinstance(x, tuple) else x
        self.hidden_shape = hidden_states.shape
        recv_x, recv_idx, recv_w, per_expert, handle, _ = self.dispatch_normal_async(
            x, topk_idx.to(torch.int64), topk_weights, self.num_experts, previous_event, async_finish=False)
        self.handle = handle
        self.topk_idx = recv_idx
        self.topk_weights = recv_w
        return recv_x, recv_idx, recv_w, per_expert

    def combine(self, hidden_states: torch.Tensor) -> torch.Tensor:
        out, _ = self.combine_normal_async(hidden_states, self.handle, async_finish=False)
        self.handle = None
        return out.view(self.hidden_shape)

    # ---- async flavoured API (same stream; events mark completion) ----------------------------
    def dispatch_normal_async(self, x, topk_idx: torch.Tensor, topk_weights: torch.Tensor,
                              num_experts: Optional[int] = None, previous_event=None, async_finish=True):
        """x: (e4m3 rows, fp32 scales) or unquantised rows.  Returns (recv_x, recv_topk_idx (local ids, -1 for
        other ranks' experts), recv_topk_weights, recv_tokens_per_expert (list, aligned), handle, event)."""
        if previous_event is not None:
            previous_event.current_stream_wait()
        x_q, x_s = x if isinstance(x, tuple) else (x, None)
        w_sz = self.world_size
        plan = make_normal_plan(topk_idx, w_sz, self.rank, self.num_local_experts, self.group, self.expert_alignment)
        # pack: one pass over the tokens, each row copied to its (<= W) destinations
        send_x, send_s = ops.permute_rows(x_q.view(torch.uint8) if x_q.element_size() == 1 else x_q, x_s, plan.dst_pos,
                                          w_sz, plan.num_send)
        return self._exchange(plan, send_x, send_s, x_q.dtype, topk_idx, topk_weights)

    def dispatch_from_hidden(self, hidden_states: torch.Tensor, topk_idx: torch.Tensor, topk_weights: torch.Tensor,
                             block_size: int = 128):
        """Quantise (per_token_group_quant_fp8 arithmetic) straight into the send buffer: one kernel reads each
        token once and writes its FP8 row and scales to every destination rank's part of the buffer."""
        self.hidden_shape = hidden_states.shape
        topk_idx = topk_idx.to(torch.int64)
        plan = make_normal_plan(topk_idx, self.world_size, self.rank, self.num_local_experts, self.group,
                                self.expert_alignment)
        send_x, send_s = ops.quant_fp8(hidden_states, block_size, _C.QUANT_DIV_EPS, 1e-10, False, plan.dst_pos,
                                       self.world_size, plan.num_send)
        recv_x, recv_idx, recv_w, per_expert, handle, _ = self._exchange(plan, send_x.view(torch.uint8), send_s,
                                                                         ops.FP8, topk_idx, topk_weights)
        self.handle, self.topk_idx, self.topk_weights = handle, recv_idx, recv_w
        return recv_x, recv_idx, recv_w, per_expert

    def _exchange(self, plan, send_x, send_s, x_dtype, topk_idx, topk_weights):
        w_sz, nle = self.world_size, self.num_local_experts
        t, k = topk_idx.shape
        dev = send_x.device
        n_send, n_recv = plan.num_send, plan.num_recv
        # per-row metadata travels as one [*, 2 kp] int32 row: global ids and the weights' bit patterns
        kp = (k + 1) // 2 * 2
        meta = torch.zeros(t, 2 * kp, dtype=torch.int32, device=dev)
        meta[:, :k] = topk_idx
        meta[:, kp:kp + k] = topk_weights.to(torch.float32).view(torch.int32)
        send_meta, _ = ops.permute_rows(meta.view(torch.uint8), None, plan.dst_pos, w_sz, n_send)
        recv_x = torch.empty(n_recv, send_x.shape[1], dtype=send_x.dtype, device=dev)
        recv_meta = torch.empty(n_recv, 8 * kp, dtype=torch.uint8, device=dev)
        _a2a(recv_x, send_x, plan.recv_splits, plan.send_splits, self.group, w_sz)
        recv_s = None
        if send_s is not None:
            recv_s = torch.empty(n_recv, send_s.shape[1], dtype=torch.float32, device=dev)
            _a2a(recv_s, send_s, plan.recv_splits, plan.send_splits, self.group, w_sz)
        _a2a(recv_meta, send_meta, plan.recv_splits, plan.send_splits, self.group, w_sz)
        rm = recv_meta.view(torch.int32)
        lo = self.rank * nle
        gid = rm[:, :k].to(torch.int64)
        recv_ids = torch.where((gid >= lo) & (gid < lo + nle), gid - lo, torch.full_like(gid, -1))
        recv_w = rm[:, kp:kp + k].view(torch.float32).contiguous()
        if recv_x.dtype != x_dtype:
            recv_x = recv_x.view(x_dtype)
        out_x = (recv_x, recv_s) if send_s is not None else recv_x
        return out_x, recv_ids, recv_w, plan.recv_tokens_per_expert, (plan,), _record_event()

    def combine_normal_async(self, x: torch.Tensor, handle: Tuple, previous_event=None, async_finish=True):
        if previous_event is not None:
            previous_event.current_stream_wait()
        (plan,) = handle
        w_sz = self.world_size
        back = torch.empty(plan.num_send, x.shape[1], dtype=x.dtype, device=x.device)
        _a2a(back, x.contiguous(), plan.send_splits, plan.recv_splits, self.group, w_sz)
        out = torch.empty(plan.num_tokens, x.shape[1], dtype=x.dtype, device=x.device)
        ones = torch.ones(plan.num_tokens, w_sz, dtype=torch.float32, device=x.device)
        # out[t] = sum over the ranks the token was sent to, in rank order (fp32 accumulation)
        ops.ep_gather(back, plan.dst_pos, ones, plan.dst_pos, out)
        return out, _record_event()

    def capture(self):
        return _record_event()

    def release(self):
        self.handle = None
        self.topk_idx = None
        self.topk_weights = None
        return True


# ----------------------------------------------------------------------------------------------
# low-latency (decode) mode: masked layout [E_local, max_tokens_per_rank * W, H]
# ----------------------------------------------------------------------------------------------
class LowLatencyPlan:
    def __init__(self):
        self.slot_pos = None       # int32 [T*k]: row of each (token, slot) pair in the send buffer
        self.send_splits = None
        self.recv_splits = None
        self.recv_dst = None       # int32 [n_recv]: row of each received pair in the masked layout
        self.masked_m = None       # int32 [E_local]
        self.num_send = 0
        self.num_recv = 0
        self.num_tokens = 0


def make_single_rank_plan(counts: torch.Tensor, num_pairs: int, rows_per_expert: int) -> LowLatencyPlan:
    """World of one: the plan stays on the device (no host round trip, so the layer can be captured in a CUDA
    graph).  Buffers are sized for all `num_pairs` (token, slot) pairs; pairs without an expert sort to the
    end of the send order and get destination -1."""
    dev = counts.device
    c = counts.to(torch.int64)
    plan = LowLatencyPlan()
    plan.num_send = plan.num_recv = num_pairs
    plan.send_splits = plan.recv_splits = [num_pairs]
    ends = torch.cumsum(c, 0)
    rows = torch.arange(num_pairs, dtype=torch.int64, device=dev)
    expert = torch.searchsorted(ends, rows, right=True)                  # expert of every sent row, E for the rest
    valid = expert < c.numel()
    e_safe = expert.clamp(max=c.numel() - 1)
    within = rows - (ends - c)[e_safe]
    plan.recv_dst = torch.where(valid, e_safe * rows_per_expert + within, torch.full_like(rows, -1)).to(torch.int32)
    plan.masked_m = counts.to(torch.int32)
    return plan


def make_low_latency_plan(counts: torch.Tensor, world_size: int, rank: int, num_local_experts: int, group,
                          rows_per_expert: int) -> LowLatencyPlan:
    """counts: int32/int64 [E] number of (token, slot) pairs this rank routes to every global expert."""
    dev = counts.device
    mine = counts.to(torch.int64).view(1, -1)
    e = mine.shape[1]
    gathered = torch.empty(world_size, e, dtype=torch.int64, device=dev)
    if world_size > 1:
        dist.all_gather_into_tensor(gathered, mine, group=group)
    else:
        gathered.copy_(mine)
    host = gathered.cpu()
    plan = LowLatencyPlan()
    per_rank = host[rank].view(world_size, num_local_experts).sum(dim=1)
    plan.send_splits = per_rank.tolist()
    local = host[:, rank * num_local_experts:(rank + 1) * num_local_experts]      # [W(src), E_local]
    plan.recv_splits = local.sum(dim=1).tolist()
    plan.num_send = int(sum(plan.send_splits))
    plan.num_recv = int(sum(plan.recv_splits))
    # received rows arrive grouped by source rank, inside a source sorted by local expert;
    # the masked layout wants, per expert, the rows of source 0 first, then source 1, ...
    before = torch.cumsum(local, dim=0) - local                                   # rows of earlier sources, per expert
    seg_rows = local.reshape(-1)                                                  # arrival order: source-major, expert-minor
    seg_base = (torch.arange(num_local_experts, dtype=torch.int64)[None, :] * rows_per_expert + before).reshape(-1)
    seg_first = torch.cumsum(seg_rows, 0) - seg_rows
    within = torch.arange(plan.num_recv, dtype=torch.int64) - torch.repeat_interleave(seg_first, seg_rows)
    plan.recv_dst = (torch.repeat_interleave(seg_base, seg_rows) + within).to(torch.int32).to(dev)
    plan.masked_m = local.sum(dim=0).to(torch.int32).to(dev)
    assert int(plan.masked_m.max()) <= rows_per_expert if plan.masked_m.numel() else True, \
        "an expert received more rows than max_tokens_per_rank * world_size"
    return plan


class TokenDispatcherLowLatency:
    """`DeepEPTokenDispatcherLowLatency` of the reference (token_dispatcher.py:455-602) over NCCL."""

    def __init__(self, group, num_experts: int = None, num_local_experts: int = None, hidden_size: int = None,
                 params_dtype: torch.dtype = None, return_recv_hook: bool = False,
                 num_max_dispatch_tokens_per_rank: int = 128):
        import os
        self.group = group
        self.num_experts = num_experts
        self.num_local_experts = num_local_experts
        self.hidden_size = hidden_size
        self.params_dtype = params_dtype
        self.world_size = dist.get_world_size(group) if (dist.is_available() and dist.is_initialized()) else 1
        self.rank = dist.get_rank(group) if (dist.is_available() and dist.is_initialized()) else 0
        self.num_max_dispatch_tokens_per_rank = int(os.getenv("DEEPEP_MAX_TOKENS_PER_RANK",
                                                              str(num_max_dispatch_tokens_per_rank)))
        self.return_recv_hook = return_recv_hook
        self.handle = None

    @property
    def rows_per_expert(self):
        return self.num_max_dispatch_tokens_per_rank * self.world_size

    def dispatch(self, hidden_states: torch.Tensor, topk_idx: torch.Tensor, topk_weights: torch.Tensor,
                 num_experts: int, use_fp8: bool = True):
        if num_experts is not None and self.num_experts is not None:
            assert self.num_experts == num_experts
        topk_idx = topk_idx.to(torch.int64)
        expected_m = (hidden_states.shape[0] * self.world_size * topk_idx.shape[1] + num_experts) // num_experts
        packed, masked_m, self.handle, event, _ = self.dispatch_async(hidden_states, topk_idx, num_experts, use_fp8,
                                                                      async_finish=False)
        return packed, topk_idx, topk_weights, masked_m, expected_m

    def dispatch_async(self, hidden_states: torch.Tensor, topk_idx: torch.Tensor, num_experts: Optional[int] = None,
                       use_fp8: bool = True, async_finish: bool = True):
        assert topk_idx.dtype == torch.int64
        assert use_fp8, "the masked layout of this package is FP8"
        assert hidden_states.shape[0] <= self.num_max_dispatch_tokens_per_rank
        t, k = topk_idx.shape
        h = hidden_states.shape[1]
        dev = hidden_states.device
        w_sz, nle, rpe = self.world_size, self.num_local_experts, self.rows_per_expert
        # pairs sorted by global expert = send order; the quantiser writes each token's row to its k slots
        _, _, _, pos, counts = ops.sort_by_expert(topk_idx, self.num_experts, want_pos=True, want_counts=True)
        # slots without an expert (id -1) sort first and are not sent: shift the others down, drop those
        unrouted = (pos < 0).sum().to(pos.dtype)
        pos = torch.where(pos >= 0, pos - unrouted, torch.full_like(pos, -1))
        if w_sz == 1:
            plan = make_single_rank_plan(counts, t * k, rpe)
        else:
            plan = make_low_latency_plan(counts, w_sz, self.rank, nle, self.group, rpe)
        plan.slot_pos, plan.num_tokens = pos, t
        send_x, send_s = ops.quant_fp8(hidden_states, 128, _C.QUANT_DIV_EPS, 1e-10, False, pos, k, plan.num_send)
        recv_x = torch.empty(plan.num_recv, h, dtype=torch.uint8, device=dev)
        recv_s = torch.empty(plan.num_recv, h // 128, dtype=torch.float32, device=dev)
        _a2a(recv_x, send_x.view(torch.uint8), plan.recv_splits, plan.send_splits, self.group, w_sz)
        _a2a(recv_s, send_s, plan.recv_splits, plan.send_splits, self.group, w_sz)
        packed_x, packed_s = ops.permute_rows(recv_x, recv_s, plan.recv_dst, 1, nle * rpe)
        packed = [DisposibleTensor(packed_x.view(ops.FP8).view(nle, rpe, h)),
                  DisposibleTensor(packed_s.view(nle, rpe, h // 128))]
        return packed, plan.masked_m, (plan,), _record_event(), (lambda: None)

    def combine(self, hidden_states: torch.Tensor, topk_idx: torch.Tensor, topk_weights: torch.Tensor):
        out, _, _ = self.combine_async(hidden_states, topk_idx.to(torch.int64), topk_weights.to(torch.float32),
                                       self.handle, async_finish=False)
        return out

    def combine_async(self, hidden_states: torch.Tensor, topk_idx: torch.Tensor, topk_weights: torch.Tensor,
                      handle: Tuple, async_finish: bool):
        assert topk_idx.dtype == torch.int64
        assert topk_weights.dtype == torch.float32
        (plan,) = handle
        nle, rpe, h = hidden_states.shape
        flat = hidden_states.reshape(nle * rpe, h)
        # back to arrival order: row i of the exchange buffer is masked-layout row recv_dst[i]
        ones = torch.ones(plan.num_recv, 1, dtype=torch.float32, device=flat.device)
        send_back = torch.empty(plan.num_recv, h, dtype=flat.dtype, device=flat.device)
        idx = plan.recv_dst.view(-1, 1)
        ops.ep_gather(flat, idx, ones, idx, send_back)
        back = torch.empty(plan.num_send, h, dtype=flat.dtype, device=flat.device)
        _a2a(back, send_back, plan.send_splits, plan.recv_splits, self.group, self.world_size)
        out = torch.empty(plan.num_tokens, h, dtype=flat.dtype, device=flat.device)
        # out[t] = sum_k w[t, k] * back[slot_pos[t, k]]
        ops.ep_gather(back, topk_idx.to(torch.int32).contiguous(), topk_weights.contiguous(),
                      plan.slot_pos.view(plan.num_tokens, -1), out)
        return out, _record_event(), (lambda: None)


# ----------------------------------------------------------------------------------------------
# low-latency (decode) mode over peer-to-peer stores: no host synchronisation at any number of ranks
# ----------------------------------------------------------------------------------------------
def make_low_latency_p2p_plan(c: torch.Tensor, me: int, num_local_experts: int, rows_per_expert: int,
                              topk_idx: torch.Tensor, rank_in: torch.Tensor):
    """Index arithmetic of the host-free low-latency exchange (plain torch on small integer tensors, any device).

    c int64 [W, E]: pair count of every source rank for every global expert (the all-gathered counts);
    topk_idx int64 [T, k] (negative: no expert); rank_in int32 [T * k]: rank of a pair among this rank's pairs of
    the same expert.  The rows of an expert's block on its owner are ordered by source rank, and inside a source by
    that rank; a rank's send order is by expert, then by that rank.  Returns, for this rank as a SOURCE,
    pair_rank / pair_row int32 [T * k] (owner rank and row of its [E_local * rows_per_expert] buffer, -1 = not
    sent: no expert, or the expert's block is full), pair_pos int32 [T * k] (row of this rank's own return buffer)
    and the mask `sent`; and, for this rank as an OWNER, masked_m int32 [E_local] and row_rank / row_pos int32
    [E_local * rows_per_expert]: source rank and return-buffer row of every row of its masked layout (-1 = unused)."""
    w, e = c.shape
    nle, rpe = num_local_experts, rows_per_expert
    dev = c.device
    ids = topk_idx.reshape(-1)
    valid = ids >= 0
    e_safe = ids.clamp(min=0)
    rows_before_me = c[:me].sum(dim=0)                           # rows of earlier sources, per expert
    row_in_expert = rows_before_me[e_safe] + rank_in.to(torch.int64)
    sent = valid & (row_in_expert < rpe)                         # an overfull expert drops its last arrivals
    neg = torch.full_like(ids, -1)
    pair_rank = torch.where(sent, e_safe // nle, neg).to(torch.int32)
    pair_row = torch.where(sent, (e_safe % nle) * rpe + row_in_expert, neg).to(torch.int32)
    sent_before = torch.cumsum(c[me], 0) - c[me]                 # this rank's pairs of lower experts
    pair_pos = torch.where(sent, sent_before[e_safe] + rank_in.to(torch.int64), neg).to(torch.int32)
    lo = me * nle
    loc = c[:, lo:lo + nle]                                      # [W, E_local]
    ends = torch.cumsum(loc, dim=0)                              # rows of sources 0..r, per local expert
    masked_m = ends[-1].clamp(max=rpe).to(torch.int32)
    row = torch.arange(rpe, device=dev, dtype=torch.int64)
    src = torch.searchsorted(ends.t().contiguous(), row[None, :].expand(nle, rpe).contiguous(), right=True)
    live = src < w
    src_c = src.clamp(max=w - 1)
    le_idx = torch.arange(nle, device=dev)[:, None].expand(nle, rpe)
    first_row = (ends - loc)[src_c, le_idx]                      # first row of that source inside the expert
    pairs_before = (torch.cumsum(c, dim=1) - c)[:, lo:lo + nle]  # [W, E_local]: the source's pairs of lower experts
    src_pos = pairs_before[src_c, le_idx] + (row[None, :] - first_row)
    row_rank = torch.where(live, src_c, torch.full_like(src_c, -1)).to(torch.int32).reshape(-1)
    row_pos = torch.where(live, src_pos, torch.full_like(src_pos, -1)).to(torch.int32).reshape(-1)
    return pair_rank, pair_row, pair_pos, sent, masked_m, row_rank, row_pos


class TokenDispatcherLowLatencyP2P:
    """`DeepEPTokenDispatcherLowLatency` of the reference (token_dispatcher.py:455-602) on symmetric memory.

    dispatch: the (token, slot) pairs are ranked inside their expert by the sort kernel; every rank stores its
    per-expert pair counts into all peers (an all-gather by stores) and, after a barrier, knows where its rows
    start inside every expert's block on the owning rank (rows of source 0 first, then source 1, ...).  One kernel
    then quantises each token once and stores it for each routed slot straight into the masked layout
    [E_local, max_tokens_per_rank * world, H] of the owner.  combine: the experts' rows go back to the rank they
    came from by indexed stores, and a weighted gather sums a token's slots.  Split sizes never reach the host,
    so the step can be captured in a CUDA graph on every rank.  All ranks must construct the dispatcher
    collectively and call dispatch / combine in the same order."""

    def __init__(self, group, num_experts: int = None, num_local_experts: int = None, hidden_size: int = None,
                 params_dtype: torch.dtype = None, return_recv_hook: bool = False,
                 num_max_dispatch_tokens_per_rank: int = 128, max_top_k: int = 8):
        self.group = group
        self.num_experts = num_experts
        self.num_local_experts = num_local_experts
        self.hidden_size = hidden_size
        self.params_dtype = params_dtype or torch.bfloat16
        single = group is None or not (dist.is_available() and dist.is_initialized())
        self.world_size = 1 if single else dist.get_world_size(group)
        self.rank = 0 if single else dist.get_rank(group)
        assert num_experts == num_local_experts * self.world_size, "experts must split evenly over the ranks"
        assert hidden_size % 128 == 0 and self.params_dtype in (torch.bfloat16, torch.float16)
        self.num_max_dispatch_tokens_per_rank = int(os.getenv("DEEPEP_MAX_TOKENS_PER_RANK",
                                                              str(num_max_dispatch_tokens_per_rank)))
        self.max_top_k = int(max_top_k)
        self.return_recv_hook = return_recv_hook
        w, h, nle, rpe = self.world_size, hidden_size, num_local_experts, self.rows_per_expert
        self.cnt_ints = (num_experts + 3) // 4 * 4                 # counts travel as whole 16-byte words
        self.send_rows = self.num_max_dispatch_tokens_per_rank * self.max_top_k
        sizes = [("allcnt", w * self.cnt_ints * 4), ("q", nle * rpe * h), ("s", nle * rpe * (h // 128) * 4),
                 ("comb", self.send_rows * h * 2)]
        # one rank: the same kernels on ordinary device memory ("peer 0" is this GPU), no barrier
        self._sym = _LocalBuffers(sizes) if self.world_size == 1 else _SymmetricBuffers(group, sizes)
        self.allcnt = self._sym.region("allcnt", w * self.cnt_ints * 4).view(torch.int32).view(w, self.cnt_ints)
        self.recv_q = self._sym.region("q", nle * rpe * h).view(ops.FP8).view(nle, rpe, h)
        self.recv_s = self._sym.region("s", nle * rpe * (h // 128) * 4).view(torch.float32).view(nle, rpe, h // 128)
        self.comb = self._sym.region("comb", self.send_rows * h * 2).view(self.params_dtype).view(self.send_rows, h)
        self.allcnt.zero_()
        torch.cuda.synchronize()
        if self.world_size > 1:
            dist.barrier(group=group)
        self.handle = None

    @property
    def rows_per_expert(self):
        return self.num_max_dispatch_tokens_per_rank * self.world_size

    def barrier(self, channel: int):
        self._sym.barrier(channel)

    def resync(self):
        self._sym.resync()

    def dispatch(self, hidden_states: torch.Tensor, topk_idx: torch.Tensor, topk_weights: torch.Tensor,
                 num_experts: int, use_fp8: bool = True):
        if num_experts is not None and self.num_experts is not None:
            assert self.num_experts == num_experts
        topk_idx = topk_idx.to(torch.int64)
        expected_m = (hidden_states.shape[0] * self.world_size * topk_idx.shape[1] + num_experts) // num_experts
        packed, masked_m, self.handle, event, _ = self.dispatch_async(hidden_states, topk_idx, num_experts, use_fp8,
                                                                      async_finish=False)
        return packed, topk_idx, topk_weights, masked_m, expected_m

    def dispatch_async(self, hidden_states: torch.Tensor, topk_idx: torch.Tensor, num_experts: Optional[int] = None,
                       use_fp8: bool = True, async_finish: bool = True):
        assert topk_idx.dtype == torch.int64
        assert use_fp8, "the masked layout of this package is FP8"
        t, k = topk_idx.shape
        # limits are checked before anything is stored or signalled (a rank that raises here has sent nothing)
        assert t <= self.num_max_dispatch_tokens_per_rank, "more tokens than num_max_dispatch_tokens_per_rank"
        assert k <= self.max_top_k, "more slots per token than the buffers were built for"
        e, nle, w, me, rpe = self.num_experts, self.num_local_experts, self.world_size, self.rank, self.rows_per_expert
        dev = hidden_states.device
        sym = self._sym
        # rank of every pair inside its expert (among this rank's pairs) and this rank's pair count per expert
        _, _, _, rank_in, counts = ops.sort_by_expert(topk_idx, e, want_rank=True, want_counts=True)
        if self.cnt_ints != e:
            counts = torch.cat([counts, counts.new_zeros(self.cnt_ints - e)])
        cnt_matrix = counts                                          # one rank: its own counts are the whole matrix
        if w > 1:
            _C.check(_C.lib().dlb_p2p_all_gather_small(_C.ptr(counts), self.cnt_ints * 4, w, me, sym.peers["allcnt"],
                                                      _C.stream(dev)))
            sym.barrier(0)
            cnt_matrix = self.allcnt
        # where every pair goes and where every row of the own layout came from: one kernel on the gathered counts
        # (the peers overwrite them only after this rank has passed the combine's barrier); the same arithmetic in
        # plain tensor operations is `make_low_latency_p2p_plan`
        pairs = t * k
        plan_ints = torch.empty(4 * pairs + nle + 2 * nle * rpe, dtype=torch.int32, device=dev)
        pair_rank, pair_row, pair_pos, ids_sent = (plan_ints[i * pairs:(i + 1) * pairs] for i in range(4))
        masked_m = plan_ints[4 * pairs:4 * pairs + nle]
        row_rank = plan_ints[4 * pairs + nle:4 * pairs + nle + nle * rpe]
        row_pos = plan_ints[4 * pairs + nle + nle * rpe:]
        ids_flat = topk_idx.contiguous().view(-1)
        _C.check(_C.lib().dlb_p2p_ll_plan(_C.ptr(cnt_matrix), self.cnt_ints, w, e, me, nle, rpe, _C.ptr(ids_flat),
                                          _C.ptr(rank_in), pairs, _C.ptr(pair_rank), _C.ptr(pair_row), _C.ptr(pair_pos),
                                          _C.ptr(ids_sent), _C.ptr(masked_m), _C.ptr(row_rank), _C.ptr(row_pos),
                                          _C.stream(dev)))
        _C.check(_C.lib().dlb_p2p_ll_quant_push(
            _C.ptr(hidden_states), _C.dtype_code(hidden_states.dtype), t, hidden_states.shape[1],
            hidden_states.stride(0), _C.QUANT_DIV_EPS, 1e-10, _C.ptr(pair_rank), _C.ptr(pair_row), k, w,
            sym.peers["q"], sym.peers["s"], _C.stream(dev)))
        sym.barrier(0)
        plan = (pair_pos.view(t, k), ids_sent.view(t, k), row_rank, row_pos, t, pair_row.view(t, k), masked_m)
        return [self.recv_q, self.recv_s], masked_m, plan, _record_event(), (lambda: None)

    def combine(self, hidden_states: torch.Tensor, topk_idx: torch.Tensor, topk_weights: torch.Tensor):
        out, _, _ = self.combine_async(hidden_states, topk_idx.to(torch.int64), topk_weights.to(torch.float32),
                                       self.handle, async_finish=False)
        return out

    def combine_async(self, hidden_states: torch.Tensor, topk_idx: torch.Tensor, topk_weights: torch.Tensor,
                      handle: Tuple, async_finish: bool):
        assert topk_idx.dtype == torch.int64
        assert topk_weights.dtype == torch.float32
        pair_pos, ids_sent, row_rank, row_pos, t, pair_row, masked_m = handle
        nle, rpe, h = hidden_states.shape
        assert hidden_states.dtype == self.comb.dtype and hidden_states.is_contiguous()
        dev = hidden_states.device
        sym = self._sym
        out = torch.empty(t, h, dtype=hidden_states.dtype, device=dev)
        if self.world_size == 1:
            # one rank: a token's rows are in this GPU's own layout; out[t] = sum_k w[t, k] * layout[pair_row[t, k]]
            ops.ep_gather(hidden_states.view(nle * rpe, h), ids_sent, topk_weights.contiguous(), pair_row, out)
            return out, _record_event(), (lambda: None)
        _C.check(_C.lib().dlb_p2p_push_rows_masked(_C.ptr(hidden_states), h * hidden_states.element_size(),
                                                  _C.ptr(masked_m), nle, rpe, _C.ptr(row_rank), _C.ptr(row_pos),
                                                  self.world_size, sym.peers["comb"], _C.stream(dev)))
        sym.barrier(1)
        # out[t] = sum_k w[t, k] * comb[pair_pos[t, k]]
        ops.ep_gather(self.comb, ids_sent, topk_weights.contiguous(), pair_pos, out)
        return out, _record_event(), (lambda: None)


# ----------------------------------------------------------------------------------------------
# normal (prefill) mode over peer-to-peer stores: no host synchronisation, no staging copies
# ----------------------------------------------------------------------------------------------
class _LocalBuffers:
    """Stand-in for `_SymmetricBuffers` on a single rank: one ordinary device allocation cut into the same named
    regions, this GPU as its only "peer", and no barrier (stream order is the order)."""

    def __init__(self, regions):
        import ctypes
        dev = torch.device("cuda", torch.cuda.current_device())
        self.device, self.world_size, self.rank = dev, 1, 0
        offs, total = {}, 0
        for name, n in regions:
            offs[name] = total
            total += (n + 255) // 256 * 256
        self._buf = torch.zeros(max(total, 256), dtype=torch.uint8, device=dev)
        self.offs = offs
        self.peers = {name: (ctypes.c_void_p * 1)(self._buf.data_ptr() + offs[name]) for name in offs}

    def region(self, name, nbytes):
        o = self.offs[name]
        return self._buf[o: o + nbytes]

    def barrier(self, channel: int):
        pass

    def resync(self):
        pass


class _SymmetricBuffers:
    """One symmetric-memory allocation per rank cut into named regions, the peers' addresses of every region, and
    the extension's bounded barrier on per-peer signal words (two independent sets, "channels")."""

    def __init__(self, group, regions):
        """regions: list of (name, bytes); all ranks must construct this collectively with equal sizes."""
        import ctypes

        import torch.distributed._symmetric_memory as symm_mem
        self.group = group
        self.world_size = dist.get_world_size(group)
        self.rank = dist.get_rank(group)
        w = self.world_size
        dev = torch.device("cuda", torch.cuda.current_device())
        self.device = dev

        def al(n):
            return (n + 255) // 256 * 256

        offs, total = {}, 0
        for name, n in list(regions) + [("sig", 256)]:
            offs[name] = total
            total += al(n)
        gname = group.group_name if hasattr(group, "group_name") else group
        self._buf = symm_mem.empty(total, dtype=torch.uint8, device=dev)
        self._hdl = symm_mem.rendezvous(self._buf, gname)
        bases = [int(p) for p in self._hdl.buffer_ptrs]
        self.offs = offs
        self.peers = {name: (ctypes.c_void_p * w)(*[b + offs[name] for b in bases]) for name in offs}
        self._buf[offs["sig"]: offs["sig"] + 256].zero_()
        self._sig_peers = [(ctypes.c_void_p * w)(*[bb + offs["sig"] + 64 * ch for bb in bases]) for ch in range(2)]
        # this rank's count of barriers per channel, on the device (the barrier kernel advances it)
        self._barrier_no = torch.zeros(2, dtype=torch.int32, device=dev)
        self.barrier_timeout_ns = int(float(os.environ.get("DLBLAS_EP_BARRIER_TIMEOUT_MS", "10000")) * 1e6)
        torch.cuda.synchronize(dev)
        dist.barrier(group=group)          # every rank's words are zero before anyone signals

    def region(self, name, nbytes):
        o = self.offs[name]
        return self._buf[o: o + nbytes]

    def barrier(self, channel: int):
        """Enqueues the next barrier of `channel` on the current stream (every rank must make the same calls in
        the same order).  If a peer does not arrive within DLBLAS_EP_BARRIER_TIMEOUT_MS (default 10 s), the kernel
        returns and `_C.check_status()` raises on this rank."""
        _C.check(_C.lib().dlb_p2p_barrier(self._sig_peers[channel], self.world_size, self.rank,
                                         _C.ptr(self._barrier_no[channel]), self.barrier_timeout_ns,
                                         _C.ptr(_C.status_word(self.device)), _C.stream(self.device)))

    def resync(self):
        """After a time-out (a rank skipped or missed a barrier): a host-side collective that brings the barrier
        counts of all ranks back in step.  Call it on every rank with no exchange in flight."""
        torch.cuda.synchronize(self.device)
        dist.all_reduce(self._barrier_no, op=dist.ReduceOp.MAX, group=self.group)
        torch.cuda.synchronize(self.device)
        dist.barrier(group=self.group)


class TokenDispatcherP2P:
    """Dispatch / combine through symmetric memory (`torch.distributed._symmetric_memory`): the
    quantiser of the extension stores every token's FP8 row, scales and routing metadata directly
    into the destination ranks' receive regions over NVLink, and the combine pushes result rows back
    the same way (csrc/p2p.cu).  Two device-side barriers per layer order the pushes; split sizes
    never travel to the host, so the layer runs without a CPU round trip.

    Receive buffers hold `world` regions of `max_tokens_per_rank` rows; unused rows carry id -1 and
    are skipped by the expert kernels.  All ranks must construct the dispatcher collectively."""

    def __init__(self, group, num_experts: int, num_local_experts: int, hidden_size: int,
                 params_dtype: torch.dtype = torch.bfloat16, max_tokens_per_rank: int = 8192, max_top_k: int = 8):
        self.group = group
        self.num_experts = num_experts
        self.num_local_experts = num_local_experts
        self.hidden_size = hidden_size
        self.params_dtype = params_dtype
        self.world_size = dist.get_world_size(group)
        self.rank = dist.get_rank(group)
        assert num_experts == num_local_experts * self.world_size, "experts must split evenly over the ranks"
        assert hidden_size % 128 == 0 and params_dtype in (torch.bfloat16, torch.float16)
        self.region_rows = int(max_tokens_per_rank)
        self.kp = (max_top_k + 1) // 2 * 2
        self.meta_ints = 2 * self.kp
        w, h = self.world_size, hidden_size
        rows = w * self.region_rows
        self.rows = rows
        sizes = [("q", rows * h), ("s", rows * (h // 128) * 4), ("meta", rows * self.meta_ints * 4), ("counts", 256),
                 ("comb", rows * h * 2)]
        self._sym = _SymmetricBuffers(group, sizes)
        self._peers = self._sym.peers
        self.recv_q = self._sym.region("q", rows * h).view(ops.FP8).view(rows, h)
        self.recv_s = self._sym.region("s", rows * (h // 128) * 4).view(torch.float32).view(rows, h // 128)
        self.recv_meta = self._sym.region("meta", rows * self.meta_ints * 4).view(torch.int32).view(rows, -1)
        self.recv_counts = self._sym.region("counts", 256).view(torch.int32)
        self.comb = self._sym.region("comb", rows * h * 2).view(params_dtype).view(rows, h)
        self.recv_counts.zero_()
        # constants of the combine, built once
        dev = self._sym.device
        self._region_base = (torch.arange(w, device=dev, dtype=torch.int32) * self.region_rows)[None, :]
        self._minus_one = torch.full((1, 1), -1, dtype=torch.int32, device=dev)
        self._ones = torch.ones(self.region_rows, w, dtype=torch.float32, device=dev)
        self._push_stream = None   # made on first use by push_slot_columns
        torch.cuda.synchronize()
        dist.barrier(group=group)
        self.handle = None
        self.hidden_shape = None

    def barrier(self, channel: int):
        """Enqueues the next barrier of `channel` on the current stream; see `_SymmetricBuffers.barrier`."""
        self._sym.barrier(channel)

    def resync(self):
        """Brings the barrier counts of all ranks back in step after a time-out; see `_SymmetricBuffers.resync`."""
        self._sym.resync()

    def dispatch_from_hidden(self, hidden_states: torch.Tensor, topk_idx: torch.Tensor, topk_weights: torch.Tensor,
                             block_size: int = 128, while_in_flight=None):
        """Returns ((recv_q, recv_s), recv_ids, recv_weights): `world * max_tokens_per_rank` rows, local
        expert ids with -1 for unused rows and for slots owned by other ranks.  `while_in_flight`, if given, is
        called between this rank's pushes and the barrier that waits for the peers': kernels it enqueues (work on
        local data only) run while the other ranks' rows are still crossing NVLink."""
        assert block_size == 128
        t, k = topk_idx.shape
        # checked before anything is pushed or signalled: a rank that raises here has sent nothing; its peers'
        # next barrier runs into its time limit and reports through the status word
        assert t <= self.region_rows, f"{t} tokens exceed max_tokens_per_rank={self.region_rows}"
        assert k <= self.kp, f"top_k {k} exceeds the {self.kp} slots the buffers were built for"
        w, dev = self.world_size, hidden_states.device
        self.hidden_shape = hidden_states.shape
        dest = ops.ep_dest_ranks(topk_idx.contiguous(), self.num_local_experts, w)
        _, _, _, within, counts = ops.sort_by_expert(dest, w, want_rank=True, want_counts=True)
        meta = torch.zeros(t, self.meta_ints, dtype=torch.int32, device=dev)
        meta[:, :k] = topk_idx
        meta[:, self.kp:self.kp + k] = topk_weights.to(torch.float32).view(torch.int32)
        p = self._peers
        _C.check(_C.lib().dlb_p2p_quant_push(
            _C.ptr(hidden_states), _C.dtype_code(hidden_states.dtype), t, hidden_states.shape[1],
            hidden_states.stride(0), _C.QUANT_DIV_EPS, 1e-10, _C.ptr(within), w, self.rank, self.region_rows,
            p["q"], p["s"], p["meta"], _C.ptr(meta), self.meta_ints, p["counts"], _C.ptr(counts), _C.stream(dev)))
        if while_in_flight is not None:
            while_in_flight()
        self.barrier(0)
        recv_ids = torch.empty(self.rows, k, dtype=torch.int64, device=dev)
        recv_w = torch.empty(self.rows, k, dtype=torch.float32, device=dev)
        _C.check(_C.lib().dlb_p2p_unpack_meta(_C.ptr(self.recv_meta), self.meta_ints, k, _C.ptr(self.recv_counts), w,
                                             self.region_rows, self.rank * self.num_local_experts,
                                             self.num_local_experts, _C.ptr(recv_ids), _C.ptr(recv_w), _C.stream(dev)))
        self.handle = (within.view(t, w), t)
        return (self.recv_q, self.recv_s), recv_ids, recv_w

    def combine(self, out_rows: torch.Tensor) -> torch.Tensor:
        """out_rows: [world * max_tokens_per_rank, H] results for the received rows (unused rows ignored)."""
        within, t = self.handle
        w, dev = self.world_size, out_rows.device
        assert out_rows.is_contiguous() and out_rows.shape == (self.rows, self.hidden_size)
        assert out_rows.dtype == self.comb.dtype
        _C.check(_C.lib().dlb_p2p_push_rows(_C.ptr(out_rows), self.hidden_size * out_rows.element_size(),
                                           _C.ptr(self.recv_counts), w, self.rank, self.region_rows,
                                           self._peers["comb"], _C.stream(dev)))
        return self._finish_combine(within, t, out_rows.dtype, dev)

    def combine_slots(self, slot_rows: torch.Tensor, recv_ids: torch.Tensor, while_in_flight=None) -> torch.Tensor:
        """slot_rows: [world * max_tokens_per_rank * k, H] weighted results of the individual (row, slot) pairs,
        recv_ids int64 [rows, k] the local expert ids from `dispatch_from_hidden`.  Sums a row's slots and
        stores the sum into the source rank's buffer in one kernel (no intermediate [rows, H] tensor)."""
        within, t = self.handle
        w, dev = self.world_size, slot_rows.device
        k = recv_ids.shape[1]
        assert slot_rows.is_contiguous() and slot_rows.shape == (self.rows * k, self.hidden_size)
        assert slot_rows.dtype == self.comb.dtype and recv_ids.dtype == torch.int64 and recv_ids.is_contiguous()
        _C.check(_C.lib().dlb_p2p_sum_push(_C.ptr(slot_rows), _C.dtype_code(slot_rows.dtype), _C.ptr(recv_ids), k,
                                          self.hidden_size, _C.ptr(self.recv_counts), w, self.rank, self.region_rows,
                                          self._peers["comb"], _C.stream(dev)))
        return self._finish_combine(within, t, slot_rows.dtype, dev, while_in_flight)

    def push_slot_columns(self, slot_rows: torch.Tensor, recv_ids: torch.Tensor, col_begin: int, col_count: int,
                          max_blocks: int = 0):
        """`combine_slots` for columns [col_begin, col_begin + col_count) only, queued on the dispatcher's push stream
        behind what the current stream has queued so far: the caller goes on computing the remaining columns while
        these travel.  `max_blocks` caps the push kernel's grid (it shares the GPU with the caller's next kernel).
        `finish_pushed_columns` must follow the last part."""
        k = recv_ids.shape[1]
        assert slot_rows.is_contiguous() and slot_rows.shape == (self.rows * k, self.hidden_size)
        assert slot_rows.dtype == self.comb.dtype and recv_ids.dtype == torch.int64 and recv_ids.is_contiguous()
        if self._push_stream is None:
            self._push_stream = torch.cuda.Stream(device=slot_rows.device)
        cur = torch.cuda.current_stream(slot_rows.device)
        self._push_stream.wait_stream(cur)
        slot_rows.record_stream(self._push_stream)
        recv_ids.record_stream(self._push_stream)
        _C.check(_C.lib().dlb_p2p_sum_push_cols(_C.ptr(slot_rows), _C.dtype_code(slot_rows.dtype), _C.ptr(recv_ids), k,
                                               self.hidden_size, _C.ptr(self.recv_counts), self.world_size, self.rank,
                                               self.region_rows, self._peers["comb"], self._push_stream.cuda_stream,
                                               int(col_begin), int(col_count), int(max_blocks)))

    def finish_pushed_columns(self, dtype, while_in_flight=None) -> torch.Tensor:
        """Joins the push stream, then barrier and gather as in `combine_slots`."""
        within, t = self.handle
        dev = self.comb.device
        torch.cuda.current_stream(dev).wait_stream(self._push_stream)
        return self._finish_combine(within, t, dtype, dev, while_in_flight)

    def _finish_combine(self, within, t, dtype, dev, while_in_flight=None):
        w = self.world_size
        if while_in_flight is not None:
            while_in_flight()
        self.barrier(1)
        idx = torch.where(within >= 0, within + self._region_base, self._minus_one).contiguous()
        ones = self._ones[:t]
        out = torch.empty(t, self.hidden_size, dtype=dtype, device=dev)
        # out[t] = sum over the ranks the token visited, in rank order (fp32 accumulation)
        ops.ep_gather(self.comb, idx, ones, idx, out)
        self.handle = None
        return out.view(self.hidden_shape)

    def release(self):
        self.handle = None
        return True
