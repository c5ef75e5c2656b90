"""`dlblas.layers.moe.ep_moe` (dlblas/layers/moe/ep_moe.py of the reference): the fused MoE layer classes.

DlblasTritonFusedMoEBlockedF8Impl (:413-484) runs on one GPU or expert-parallel by masking;
FusedMoENormal (:34-152) and FusedMoELowLatency (:155-347) exchange tokens between ranks through the
token dispatchers of this package (NCCL over NVLink instead of DeepEP)."""
import os
from typing import List, Optional, Tuple, Union

import torch
import torch.distributed as dist

from ... import _C, ops
from ...kernels.fp8 import per_token_group_quant_fp8
from ...kernels.fused_moe_v3 import fused_moe_v3
from ...kernels.moe import silu_and_mul_masked_post_quant_fwd
from ...utils.logger import get_logger
from ...utils.utils import DisposibleTensor
from .experts_distribution_recorder import ExpertsDistributionRecorder
from .kernels.blocked_fp8_fused_moe import _renormalize, moe_expert_forward
from .token_dispatcher import (TokenDispatcherLowLatency, TokenDispatcherLowLatencyP2P, TokenDispatcherNormal,
                               TokenDispatcherP2P)

logger = get_logger(__name__)

enable_moe_load_stats = os.environ.get("DLBLAS_MOE_LOAD_STATS", "false").lower() == "true"


class DlblasTritonFusedMoEBlockedF8Impl:
    """Block-scaled FP8 fused MoE layer (ep_moe.py:413-484).  The name is the reference's; the kernels
    underneath are the sm_100a CUDA extension."""

    def __init__(self, top_k: int, num_experts: int, renormalize: bool = False, block_size: int = 128,
                 out_dtype: torch.dtype = torch.float16, ep_size: int = 1):
        self.num_experts = num_experts
        self.top_k = top_k
        self.renormalize = renormalize
        self.block_size = block_size
        self.out_dtype = out_dtype
        self.ep_size = ep_size

    def support_ep(self):
        return True

    def ep_expert_list(self, world_size: int, rank: int):
        per_rank = (self.num_experts + world_size - 1) // world_size
        first = rank * per_rank
        return list(range(first, min(first + per_rank, self.num_experts)))

    def forward(self, hidden_states: torch.Tensor, topk_weights: torch.Tensor, topk_ids: torch.LongTensor,
                gate_up_weights: torch.Tensor, gate_up_scale: torch.Tensor, down_weights: torch.Tensor,
                down_scale: torch.Tensor, expert_list: List[int] = None):
        """hidden_states [..., H] bf16/fp16; topk_ids local to this rank's experts (-1 elsewhere) when
        `expert_list` is a strict subset, and then shifted by expert_list[0] in place as the reference does."""
        input_size = hidden_states.shape
        hidden_states = hidden_states.flatten(0, -2)
        expert_offset = 0
        num_experts = None
        if expert_list is not None and len(expert_list) != self.num_experts:
            expert_offset = expert_list[0]
            num_experts = self.num_experts
        e_local = gate_up_weights.shape[0]
        if num_experts is None:
            num_experts = e_local * self.ep_size if self.ep_size > 1 else e_local
        topk_weights = _renormalize(topk_weights, self.renormalize)
        if expert_offset != 0:
            topk_ids[topk_ids != -1] += expert_offset
        output = moe_expert_forward(hidden_states, None, None, gate_up_weights, gate_up_scale, down_weights,
                                    down_scale, topk_weights, topk_ids, self.top_k, hidden_states.dtype,
                                    expert_offset, num_experts, _C.QUANT_RECIP_MUL, group_size=self.block_size)
        _C.maybe_check_status(output.device)
        return output.unflatten(0, input_size[:-1])


class FusedMoELowLatency:
    """Expert-parallel decode layer on the masked layout [E_local, max_tokens * world, H]
    (ep_moe.py:155-347): dispatch casts to FP8, the experts run two masked grouped GEMMs with the fused
    silu*up + quantisation between them, combine applies the routing weights."""
    recorder = ExpertsDistributionRecorder(output_dir="/tmp/dlblas/decode_moe_stats")

    def __init__(self, ep_size: int, ep_group: dist.ProcessGroup, num_experts: int, hidden_dim: int,
                 layer_index: int, block_size: int = 128, out_dtype: torch.dtype = torch.bfloat16):
        self.num_experts = num_experts
        self.layer_index = layer_index
        self.block_size = block_size
        self.out_dtype = out_dtype
        # Exchange backend: the default is the peer-to-peer dispatcher (in-kernel stores into the owners' masked
        # layouts, no host round trip, CUDA-graph capturable; on one rank the same kernels on this GPU's own
        # memory); DLBLAS_EP_BACKEND=nccl selects the all-to-all with host-side split sizes.
        backend = os.environ.get("DLBLAS_EP_BACKEND", "p2p").lower()
        cls = TokenDispatcherLowLatencyP2P if backend == "p2p" else TokenDispatcherLowLatency
        self.token_dispatcher = cls(group=ep_group, num_experts=num_experts, num_local_experts=num_experts // ep_size,
                                    hidden_size=hidden_dim, params_dtype=out_dtype)

    def experts(self, hidden_states_fp8, gate_up_weight: torch.Tensor, gate_up_scale: torch.Tensor,
                gate_down_weight: torch.Tensor, gate_down_scale: torch.Tensor, masked_m: torch.Tensor,
                expected_m: int):
        """Masked-layout expert MLP: x [E_local, rows, H] e4m3 + scales, only the first masked_m[e] rows of every
        expert are valid.  `expected_m` (a scheduling hint of the reference's GEMM library) is not needed: the
        tile list is built on the device from masked_m."""
        x_q, x_s = hidden_states_fp8
        e_local, rows, hidden = x_q.shape
        width = gate_up_weight.size(1)                       # 2 * intermediate
        inter = width // 2
        dev = x_q.device
        valid_rows = masked_m if masked_m.dtype == torch.int32 else masked_m.to(torch.int32)
        tiles, max_tiles = ops.build_tiles_masked(valid_rows, rows)
        flat = e_local * rows

        # The masked GEMMs of a decode step stream weights at the HBM rate from far fewer SMs than the GPU has;
        # DLBLAS_DECODE_SM_MARGIN leaves that many SMs to kernels of other streams (a shared expert's small GEMMs,
        # which otherwise wait for the persistent CTAs to leave).
        margin = int(os.environ.get("DLBLAS_DECODE_SM_MARGIN", "0"))

        def gemm(a_q, a_s, w, w_s, out):
            ops.grouped_gemm(a_q, a_s, w, w_s, tiles, max_tiles, _C.EPI_STORE, out, sm_margin=margin)

        gate_up = torch.empty((e_local, rows, width), device=dev, dtype=self.out_dtype)
        gemm(DisposibleTensor.maybe_unwrap(x_q).view(flat, hidden), DisposibleTensor.maybe_unwrap(x_s).view(flat, -1),
             gate_up_weight, gate_up_scale, gate_up.view(flat, width))
        # the dispatch buffers are the largest tensors of the decode step: give them back as early as the
        # reference does (kernels already enqueued keep the memory alive through the caching allocator)
        for t in hidden_states_fp8:
            DisposibleTensor.maybe_dispose(t)
        act_q = torch.empty((e_local, rows, inter), device=dev, dtype=gate_down_weight.dtype)
        act_s = torch.empty((e_local, rows, inter // self.block_size), device=dev, dtype=torch.float32)
        silu_and_mul_masked_post_quant_fwd(gate_up, act_q, act_s, self.block_size, valid_rows)
        del gate_up
        out = torch.empty((e_local, rows, gate_down_weight.size(1)), device=dev, dtype=self.out_dtype)
        gemm(act_q.view(flat, inter), act_s.view(flat, -1), gate_down_weight, gate_down_scale, out.view(flat, -1))
        return out

    def forward(self, hidden_states: torch.Tensor, topk_weights: torch.Tensor, topk_ids: torch.LongTensor,
                up_weights: torch.Tensor, up_scale: torch.Tensor, down_weights: torch.Tensor,
                down_scale: torch.Tensor, expert_list: List[int] = None):
        if enable_moe_load_stats:
            FusedMoELowLatency.recorder.record(topk_ids, self.layer_index, self.num_experts)
        recv_hidden_states, topk_idx, topk_weights, masked_m, expected_m = self.token_dispatcher.dispatch(
            hidden_states, topk_ids, topk_weights, self.num_experts)
        out_states = self.experts(recv_hidden_states, up_weights, up_scale, down_weights, down_scale, masked_m,
                                  expected_m)
        out = self.token_dispatcher.combine(out_states, topk_idx, topk_weights)
        _C.maybe_check_status(out.device)
        return out

    def wait(self, event):
        event.current_stream_wait()

    def dispatch_async(self, hidden_states: torch.Tensor, topk_idx: torch.Tensor, num_experts: Optional[int] = None,
                       use_fp8: bool = True, async_finish: bool = True):
        return self.token_dispatcher.dispatch_async(hidden_states, topk_idx, num_experts, use_fp8, async_finish)

    def combine_async(self, hidden_states: torch.Tensor, topk_idx: torch.Tensor, topk_weights: torch.Tensor,
                      handle: tuple, async_finish: bool):
        return self.token_dispatcher.combine_async(hidden_states, topk_idx, topk_weights, handle, async_finish)

    def fusedmoe_forward(self, state, up_weight, up_scale, down_weight, down_scale):
        hidden_shape = state["raw_hidden_shape"]
        topk_idx = state["topk_idx"]
        d = self.token_dispatcher
        expected_m = (hidden_shape[0] * d.world_size * topk_idx.shape[1] + d.num_experts) // d.num_experts
        return self.experts(state["recv_hidden_states"], up_weight, up_scale, down_weight, down_scale,
                            state["recv_expert_count"], expected_m)


class FusedMoENormal:
    """Expert-parallel prefill layer: quantise, dispatch to the ranks that own the routed experts,
    run the experts on the received tokens, combine back (ep_moe.py:34-152)."""
    recorder = ExpertsDistributionRecorder(output_dir="/tmp/dlblas/prefill_moe_stats")

    def __init__(self, ep_size: int, ep_group: dist.ProcessGroup, num_experts: int, hidden_dim: int,
                 layer_index: int = 0, block_size: int = 128, top_k: int = 8,
                 out_dtype: torch.dtype = torch.bfloat16, chunk_size: Optional[int] = 32 * 1024,
                 expert_alignment: int = 128):
        self.layer_index = layer_index
        self.top_k = top_k
        self.num_experts = num_experts
        self.block_size = block_size
        self.num_local_experts = num_experts // ep_size
        self.token_dispatcher = TokenDispatcherNormal(group=ep_group, num_experts=num_experts,
                                                      num_local_experts=self.num_local_experts,
                                                      hidden_size=hidden_dim, params_dtype=out_dtype,
                                                      expert_alignment=expert_alignment)
        # Exchange backend: "p2p" = in-kernel stores into the peers' memory (default with more than one
        # rank), "nccl" = variable-size all-to-all.  DLBLAS_EP_MAX_TOKENS bounds the tokens per rank and call.
        # With p2p a call can be cut into DLBLAS_EP_CHUNKS token chunks (default 1 = off) that run on their own
        # streams with their own buffers, so that one chunk's pushes and barriers overlap the other chunk's GEMMs.
        backend = os.environ.get("DLBLAS_EP_BACKEND", "p2p" if ep_size > 1 else "nccl").lower()
        self.p2p_dispatcher = None
        self.p2p_chunks = []
        # Optional callables for work that needs local data only (e.g. a shared expert's GEMMs): `during_dispatch`
        # is called after this rank's tokens have been pushed and before the wait for the peers' tokens,
        # `during_combine` after the results have been pushed back and before the wait for the peers' results, so
        # the kernels they enqueue run while the other ranks' rows are in flight (peer-to-peer backend only).
        self.during_dispatch = None
        self.during_combine = None
        if backend == "p2p" and ep_size > 1:
            max_tokens = int(os.environ.get("DLBLAS_EP_MAX_TOKENS", "8192"))
            chunks = max(1, int(os.environ.get("DLBLAS_EP_CHUNKS", "1")))
            # fixed at construction from values every rank shares: all ranks must run the same sequence of
            # pushes and barriers whatever their own token counts are
            # ... and only where a chunk still brings about DLBLAS_EP_MIN_CHUNK_ROWS rows (default 1024) to every
            # local expert: with fewer, badly filled GEMM tiles cost more than the overlap wins (measured at EP 2)
            rows_per_expert = max_tokens * top_k // max(self.num_local_experts, 1) // chunks
            if rows_per_expert < int(os.environ.get("DLBLAS_EP_MIN_CHUNK_ROWS", "1024")):
                chunks = 1
            per_chunk = (max_tokens + chunks - 1) // chunks
            self.p2p_chunks = [TokenDispatcherP2P(ep_group, num_experts, self.num_local_experts, hidden_dim, out_dtype,
                                                  max_tokens_per_rank=per_chunk, max_top_k=top_k)
                               for _ in range(chunks)]
            self.p2p_dispatcher = self.p2p_chunks[0]
            self._chunk_streams = [torch.cuda.Stream() for _ in range(chunks - 1)]

    def _p2p_experts(self, d, hs, topk_ids, topk_weights, up_weights, up_scale, down_weights, down_scale):
        (rq, rs), rids, rw = d.dispatch_from_hidden(hs, topk_ids, topk_weights, self.block_size,
                                                    while_in_flight=self.during_dispatch)
        fused = os.environ.get("DLBLAS_EP_FUSED_COMBINE", "1") == "1"
        # DLBLAS_EP_W2_PARTS = p > 1: the second GEMM runs in p launches over windows of the hidden dimension, and the
        # rows' finished columns are summed and pushed back from a second stream while the next window is computed on
        # the other SMs (DLBLAS_EP_PUSH_SMS of them, default 16, are left to the push).
        parts = int(os.environ.get("DLBLAS_EP_W2_PARTS", "1"))
        if fused and parts > 1 and hs.shape[-1] % (256 * parts) == 0:
            push_sms = int(os.environ.get("DLBLAS_EP_PUSH_SMS", "16"))

            def push(y, col_begin, col_count):
                last = col_begin + col_count == hs.shape[-1]
                d.push_slot_columns(y, rids, col_begin, col_count, 0 if last else push_sms * 8)

            moe_expert_forward(None, rq, rs, up_weights, up_scale, down_weights, down_scale, rw, rids,
                               topk_ids.shape[1], hs.dtype, 0, self.num_local_experts, _C.QUANT_DIV_EPS,
                               skip_unrouted_rows=True, return_slot_rows=True, w2_column_parts=parts,
                               on_columns_done=push, sm_margin=push_sms)
            return d.finish_pushed_columns(hs.dtype, while_in_flight=self.during_combine)
        out_rows = moe_expert_forward(None, rq, rs, up_weights, up_scale, down_weights, down_scale, rw, rids,
                                      topk_ids.shape[1], hs.dtype, 0, self.num_local_experts,
                                      _C.QUANT_DIV_EPS, skip_unrouted_rows=True, return_slot_rows=fused)
        if fused:
            # sum over a row's local slots while pushing it back
            return d.combine_slots(out_rows, rids, while_in_flight=self.during_combine)
        return d.combine(out_rows)

    def forward(self, hidden_states: torch.Tensor, topk_weights: torch.Tensor, topk_ids: torch.LongTensor,
                up_weights: torch.Tensor, up_scale: torch.Tensor, down_weights: torch.Tensor,
                down_scale: torch.Tensor, expert_list: List[int] = None):
        if enable_moe_load_stats:
            FusedMoENormal.recorder.record(topk_ids, self.layer_index, self.num_experts)
        if self.p2p_dispatcher is not None:
            hs = hidden_states.flatten(0, -2) if hidden_states.dim() > 2 else hidden_states
            t = hs.shape[0]
            n = len(self.p2p_chunks)
            assert t <= n * self.p2p_chunks[0].region_rows, "more tokens than DLBLAS_EP_MAX_TOKENS"
            if n == 1:
                out = self._p2p_experts(self.p2p_chunks[0], hs, topk_ids, topk_weights, up_weights, up_scale,
                                        down_weights, down_scale)
                _C.maybe_check_status(out.device)
                return out.view(hidden_states.shape)
            main = torch.cuda.current_stream()
            step = min((t + n - 1) // n, self.p2p_chunks[0].region_rows) if t else 0
            outs = []
            for c in range(n):
                sl = slice(c * step, min((c + 1) * step, t))
                stream = main if c == 0 else self._chunk_streams[c - 1]
                if c > 0:
                    stream.wait_stream(main)
                with torch.cuda.stream(stream):
                    o = self._p2p_experts(self.p2p_chunks[c], hs[sl], topk_ids[sl].contiguous(),
                                          topk_weights[sl].contiguous(), up_weights, up_scale, down_weights, down_scale)
                    if c > 0:
                        o.record_stream(main)
                outs.append(o)
            for st in self._chunk_streams:
                main.wait_stream(st)
            _C.maybe_check_status(hs.device)
            return torch.cat(outs, dim=0).view(hidden_states.shape)
        # per_token_group_quant_fp8 fused with the packing of the send buffer (one pass over the tokens)
        x, recv_topk_ids, recv_topk_weights, recv_tokens_per_expert = self.token_dispatcher.dispatch_from_hidden(
            hidden_states.flatten(0, -2) if hidden_states.dim() > 2 else hidden_states, topk_ids, topk_weights,
            self.block_size)
        self.token_dispatcher.hidden_shape = hidden_states.shape
        out_states = fused_moe_v3(x, recv_topk_ids, recv_topk_weights, (up_weights, up_scale),
                                  (down_weights, down_scale), recv_tokens_per_expert)
        out = self.token_dispatcher.combine(out_states)
        _C.maybe_check_status(out.device)
        return out

    # --- split API used for two-batch overlap (ep_moe.py:100-152) ---
    def capture(self):
        return self.token_dispatcher.capture()

    def wait(self, event):
        self.token_dispatcher.release()
        event.current_stream_wait()

    def dispatch_async(self, x: Union[Tuple[torch.Tensor, torch.Tensor], torch.Tensor], topk_idx: torch.Tensor,
                       topk_weights: torch.Tensor, num_experts: Optional[int] = None, previous_event=None,
                       async_finish=True):
        if isinstance(x, torch.Tensor):
            x = per_token_group_quant_fp8(x, self.block_size)
        return self.token_dispatcher.dispatch_normal_async(x, topk_idx, topk_weights, num_experts, previous_event,
                                                           async_finish)

    def combine_async(self, x: torch.Tensor, handle: tuple, previous_event=None, async_finish=True):
        return self.token_dispatcher.combine_normal_async(x, handle, previous_event, async_finish)

    def release(self):
        return self.token_dispatcher.release()

    def fusedmoe_forward(self, state, up_weight, up_scale, down_weight, down_scale):
        return fused_moe_v3(state["recv_hidden_states"], state["recv_topk_idx"], state["recv_topk_weights"],
                            (up_weight, up_scale), (down_weight, down_scale), state["recv_tokens_per_expert"])

    def per_token_group_quant_fp8(self, x: torch.Tensor):
        return per_token_group_quant_fp8(x, self.block_size)


def build_deepep_moe(low_latency_mode: bool, ep_size: int, ep_group: dist.ProcessGroup, num_experts: int,
                     hidden_dim: int, block_size: int, top_k: int, out_dtype: torch.dtype, layer_idx: int = 0,
                     chunk_size: Optional[int] = 32 * 1024, expert_alignment: int = 128):
    """Factory with the reference's signature (ep_moe.py:375-410)."""
    if low_latency_mode:
        return FusedMoELowLatency(ep_size=ep_size, ep_group=ep_group, num_experts=num_experts, hidden_dim=hidden_dim,
                                  layer_index=layer_idx, block_size=block_size, out_dtype=out_dtype)
    return FusedMoENormal(ep_size=ep_size, ep_group=ep_group, num_experts=num_experts, hidden_dim=hidden_dim,
                          layer_index=layer_idx, block_size=block_size, top_k=top_k, out_dtype=out_dtype,
                          chunk_size=chunk_size, expert_alignment=expert_alignment)
