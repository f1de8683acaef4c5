"""`ElasticBuffer` / `EPHandle`: the elastic-style EP interface of Mooncake for one
NVLink domain, on the B200 exchange of this package.

Mirrors mooncake-wheel/mooncake/mooncake_elastic_buffer.py (class `EPHandle`
:35-81, `ElasticBuffer` :84-774): same constructor and method names, same
argument meaning, same shapes of what `dispatch` / `combine` return. Differences
a caller can see:

* the order of received rows is deterministic (source rank, then token index),
  with or without `deterministic=True`; with `do_expand` the rows of one expert
  are in receive order as well (the reference hands positions out atomically);
* `do_expand=True` does produce the expanded expert-major layout (the
  reference's wrapper warns that it returns the packed layout for now);
* one NVLink domain only: `num_scaleout_ranks` is always 1 (no hybrid mode);
* bf16 payloads only; an `(x_fp8, scale_packs)` tuple raises NotImplementedError;
* a cached handle recomputes the same layout from the handle's `topk_idx`
  instead of reusing slot indices, so it carries no restriction on `do_expand`;
* in a group, without `do_expand`, `recv_x` is by default a view of the buffer's
  symmetric memory (peers store the rows there; nothing is copied on the
  receiving side) and stays valid until the dispatch call after the next one on
  the same buffer; `ElasticBuffer(..., recv_in_place=False)` returns a tensor of
  its own instead (one more pass over the rows).
"""
from __future__ import annotations

import os
from typing import Any, List, Optional, Tuple, Union

import torch
import torch.distributed as dist

from . import ep
from .mooncake_ep_buffer import EventOverlap, _DeviceBytes, _stream_ptr


def _ceil_div(x: int, y: int) -> int:
    return (x + y - 1) // y


class EPHandle:
    """What `combine` (and a cached `dispatch`) needs from a `dispatch` call.
    Field names as in the reference (:46-81)."""

    def __init__(self, do_expand: bool, num_experts: int, expert_alignment: int,
                 num_max_tokens_per_rank: int, num_sms: int, topk_idx: torch.Tensor,
                 num_recv_tokens_per_expert_list: List[int],
                 psum_num_recv_tokens_per_scaleup_rank: torch.Tensor,
                 psum_num_recv_tokens_per_expert: torch.Tensor, recv_src_metadata: torch.Tensor,
                 dst_buffer_slot_idx: torch.Tensor,
                 token_metadata_at_forward: Optional[torch.Tensor] = None,
                 channel_linked_list: Optional[torch.Tensor] = None,
                 native_handle: Optional[Any] = None) -> None:
        assert topk_idx is not None
        self.do_expand = do_expand
        self.num_experts = num_experts
        self.expert_alignment = expert_alignment
        self.num_max_tokens_per_rank = num_max_tokens_per_rank
        self.num_sms = num_sms
        self.topk_idx = topk_idx
        self.psum_num_recv_tokens_per_scaleup_rank = psum_num_recv_tokens_per_scaleup_rank
        self.psum_num_recv_tokens_per_expert = psum_num_recv_tokens_per_expert
        self.num_recv_tokens_per_expert_list = num_recv_tokens_per_expert_list
        self.recv_src_metadata = recv_src_metadata
        self.dst_buffer_slot_idx = dst_buffer_slot_idx
        self.token_metadata_at_forward = token_metadata_at_forward
        self.channel_linked_list = channel_linked_list
        self.native_handle = native_handle
        # without a CPU sync an upper bound, after one the number of rows received (:79-81)
        self.num_recv_tokens = int(recv_src_metadata.shape[0])


class ElasticBuffer:
    def __init__(self, group: dist.ProcessGroup, num_bytes: Optional[int] = None,
                 num_max_tokens_per_rank: int = 0, hidden: int = 0, num_topk: int = 0,
                 use_fp8_dispatch: bool = False, deterministic: bool = False,
                 allow_hybrid_mode: bool = True, allow_multiple_reduction: bool = True,
                 prefer_overlap_with_compute: bool = True, sl_idx: int = 3,
                 num_allocated_qps: int = 0, num_cpu_timeout_secs: int = 300,
                 num_gpu_timeout_secs: int = 100, explicitly_destroy: bool = False,
                 recv_in_place: bool = True) -> None:
        if not allow_multiple_reduction:
            raise NotImplementedError("ElasticBuffer supports only allow_multiple_reduction=True")
        if use_fp8_dispatch:
            raise NotImplementedError("ElasticBuffer (B200): pre-quantised dispatch is not built; "
                                      "dispatch bf16")
        self.recv_in_place = recv_in_place
        self._views: dict = {}
        self.group = group
        self.backend = group
        self.rank_idx = group.rank()
        self.num_ranks = group.size()
        self.allow_hybrid_mode = allow_hybrid_mode
        self.allow_multiple_reduction = allow_multiple_reduction
        self.prefer_overlap_with_compute = prefer_overlap_with_compute
        self.deterministic = deterministic
        self.sl_idx = int(os.getenv("EP_OVERRIDE_RDMA_SL", sl_idx))
        self.num_allocated_qps = num_allocated_qps
        self.num_cpu_timeout_secs = num_cpu_timeout_secs
        self.num_gpu_timeout_secs = num_gpu_timeout_secs
        self.explicitly_destroy = explicitly_destroy
        self.num_max_tokens_per_rank = num_max_tokens_per_rank
        self.hidden = hidden
        self.num_topk = num_topk
        self.use_fp8_dispatch = use_fp8_dispatch
        if num_bytes is None:
            num_bytes = self.get_buffer_size_hint(group, num_max_tokens_per_rank, hidden,
                                                  num_topk=num_topk)
        self.num_bytes = num_bytes
        # one NVLink domain: every rank is a scale-up peer
        self.num_scaleout_ranks, self.num_scaleup_ranks = 1, self.num_ranks
        self.scaleout_rank_idx, self.scaleup_rank_idx = 0, self.rank_idx
        self.num_rdma_ranks, self.num_nvlink_ranks = 1, self.num_ranks
        self.runtime: Optional[ep.Buffer] = ep.Buffer(self.rank_idx, self.num_ranks, num_bytes, False)
        self._connect_native()
        torch.cuda.synchronize()
        if self.num_ranks > 1:
            dist.barrier(group)

    # ---------------------------------------------------------------- bootstrap
    def _active_ranks_mask(self) -> list:
        return [1] * self.num_ranks

    def _connect_native(self, is_update: bool = False) -> None:
        """Exchange memory handles and map every peer (reference :204-280)."""
        if self.num_ranks == 1:
            return
        mine = self.runtime.get_ipc_handle()
        device = (torch.device("cpu") if dist.get_backend(self.group) == "gloo"
                  else torch.device("cuda", torch.cuda.current_device()))
        local = torch.tensor(mine, dtype=torch.int32, device=device)
        gathered = [torch.empty_like(local) for _ in range(self.num_ranks)]
        dist.all_gather(gathered, local, self.group)
        self.runtime.sync_nvlink_ipc_handles([h.tolist() for h in gathered], self._active_ranks_mask())
        if not self.runtime.use_fast_path():
            raise RuntimeError(f"[Rank {self.rank_idx}] ElasticBuffer (B200): not every rank's buffer "
                               "could be mapped over NVLink; there is no fallback path")

    def update_ep_member(self) -> None:
        self._connect_native(True)

    def destroy(self) -> None:
        self.runtime = None

    # ------------------------------------------------------------------- sizing
    @staticmethod
    def get_buffer_size_hint(group: dist.ProcessGroup, num_max_tokens_per_rank: int, hidden: int,
                             num_topk: int = 0, use_fp8_dispatch: bool = False,
                             allow_hybrid_mode: bool = True,
                             allow_multiple_reduction: bool = True) -> int:
        """Bytes the buffer needs (reference :315-358)."""
        if group.size() == 1:
            return 0
        return ep.elastic_buffer_size_hint(num_max_tokens_per_rank, hidden, group.size(),
                                           max(num_topk, 1))

    def get_physical_domain_size(self) -> Tuple[int, int]:
        return self.num_rdma_ranks, self.num_nvlink_ranks

    def get_logical_domain_size(self) -> Tuple[int, int]:
        return self.num_scaleout_ranks, self.num_scaleup_ranks

    def get_theoretical_num_sms(self, num_experts: int, num_topk: int) -> int:
        """Accepted for interface parity; the kernels size their own grids."""
        return torch.cuda.get_device_properties(torch.cuda.current_device()).multi_processor_count

    def barrier(self, use_comm_stream: bool = True, with_cpu_sync: bool = False) -> None:
        """A barrier of the group on the device (reference :417-423)."""
        self.runtime.barrier(_stream_ptr(), 0)
        if with_cpu_sync:
            torch.cuda.synchronize()

    def _symmetric_tensor(self, ptr: int, nbytes: int, shape: tuple, device: torch.device) -> torch.Tensor:
        """A bf16 tensor over `nbytes` of symmetric memory at `ptr` (made once per span)."""
        key = (ptr, nbytes, shape)
        t = self._views.get(key)
        if t is None:
            raw = torch.as_tensor(_DeviceBytes(self.runtime, ptr, nbytes), device=device)
            t = self._views[key] = raw.view(torch.bfloat16).view(shape)
        return t

    def _timeout_us(self) -> int:
        return -1 if self.num_gpu_timeout_secs < 0 else int(self.num_gpu_timeout_secs) * 1_000_000

    # ----------------------------------------------------------------- dispatch
    def dispatch(self, x: Union[torch.Tensor, Tuple[torch.Tensor, torch.Tensor]],
                 topk_idx: Optional[torch.Tensor] = None,
                 topk_weights: Optional[torch.Tensor] = None, num_experts: Optional[int] = None,
                 num_max_tokens_per_rank: Optional[int] = None,
                 expert_alignment: Optional[int] = None, handle: Optional[EPHandle] = None,
                 do_expand: bool = False, do_cpu_sync: Optional[bool] = None,
                 num_sms: Optional[int] = None, async_with_compute_stream: bool = False):
        """Reference :437-714. Returns (recv_x, recv_topk_idx, recv_topk_weights, handle, event)."""
        if self.runtime is None:
            raise RuntimeError("ElasticBuffer has been destroyed")
        if isinstance(x, tuple):
            raise NotImplementedError("ElasticBuffer (B200): (x, scale_packs) input is not built")
        if handle is not None:
            if topk_idx is not None or topk_weights is not None:
                raise AssertionError("topk_idx and topk_weights must be None when cached handle is provided")
            if do_cpu_sync:
                raise AssertionError("Cannot do CPU sync with cached handle")
            if handle.native_handle is None:
                raise RuntimeError("Cached EPHandle is missing its native handle")
            topk_idx = handle.topk_idx
            num_max_tokens_per_rank = num_max_tokens_per_rank or handle.num_max_tokens_per_rank
            num_experts = num_experts or handle.num_experts
            expert_alignment = handle.expert_alignment if expert_alignment is None else expert_alignment
            num_sms = handle.num_sms if num_sms is None else num_sms
            do_expand = do_expand or handle.do_expand
            do_cpu_sync = False
        else:
            if topk_idx is None:
                raise AssertionError("topk_idx must be provided when cached handle is not provided")
            expert_alignment = 1 if expert_alignment is None else expert_alignment
            do_cpu_sync = True if do_cpu_sync is None else do_cpu_sync
        assert x.dim() == 2 and x.is_contiguous() and x.dtype == torch.bfloat16
        assert topk_idx.dtype == torch.int64 and topk_idx.is_contiguous()
        if num_experts is None:
            num_experts = int(torch.max(topk_idx).item()) + 1
        if num_max_tokens_per_rank is None:
            num_max_tokens_per_rank = self.num_max_tokens_per_rank or x.shape[0]
        if num_sms is None:
            num_sms = self.get_theoretical_num_sms(num_experts, topk_idx.shape[1])
        dev = x.device
        T, H, K = int(x.shape[0]), int(x.shape[1]), int(topk_idx.shape[1])
        L = num_experts // self.num_ranks
        n_cap = num_max_tokens_per_rank * self.num_ranks
        out_cap = n_cap * K if do_expand else n_cap

        active_ranks = torch.ones(self.num_ranks, dtype=torch.int32, device=dev)
        psum_expert = torch.empty(L + 1, dtype=torch.int32, device=dev)
        psum_rank = torch.empty(self.num_scaleup_ranks, dtype=torch.int32, device=dev)
        dst_buffer_slot_idx = torch.empty((T, K), dtype=torch.int32, device=dev)
        recv_x = None
        if self.recv_in_place and not do_expand:
            # where the exchange lands the rows: the flat tensor itself
            ptr, nbytes = self.runtime.next_recv_x(num_max_tokens_per_rank, H, self.num_ranks, False)
            if ptr:
                recv_x = self._symmetric_tensor(ptr, nbytes, (n_cap, H), dev)
        if recv_x is None:
            recv_x = torch.empty((out_cap, H), dtype=x.dtype, device=dev)
        recv_topk_idx = torch.empty((n_cap, K), dtype=topk_idx.dtype, device=dev)
        recv_topk_weights = (torch.empty((out_cap,) if do_expand else (n_cap, K), dtype=torch.float32,
                                         device=dev) if topk_weights is not None else None)
        recv_src_metadata = torch.empty((n_cap, K + 2), dtype=torch.int32, device=dev)
        if topk_weights is not None:
            assert topk_weights.dtype == torch.float32 and topk_weights.is_contiguous()
        # the handle keeps its own copy of the routing, as the reference's does (:679); the
        # copy is written by the call's first kernel
        kept_idx = handle.topk_idx if handle is not None else torch.empty_like(topk_idx)
        event = self.runtime.elastic_dispatch(
            x.data_ptr(), x.element_size(), 0, T, H, 0, 0, 0, topk_idx.data_ptr(), K,
            0 if topk_weights is None else topk_weights.data_ptr(), active_ranks.data_ptr(),
            num_experts, num_max_tokens_per_rank, expert_alignment, do_expand,
            async_with_compute_stream, _stream_ptr(), handle is not None, psum_rank.data_ptr(),
            psum_expert.data_ptr(), dst_buffer_slot_idx.data_ptr(), recv_x.data_ptr(), 0,
            recv_topk_idx.data_ptr(), 0 if recv_topk_weights is None else recv_topk_weights.data_ptr(),
            recv_src_metadata.data_ptr(), self._timeout_us(),
            0 if handle is not None else kept_idx.data_ptr())
        handle_psum_expert = psum_expert if do_expand else psum_expert[1:]

        counts: List[int] = []
        if do_cpu_sync:
            if event is not None:
                event.synchronize()
            rank_cpu, expert_cpu = psum_rank.cpu(), psum_expert.cpu()
            n_recv = int(rank_cpu[self.num_scaleup_ranks - 1])
            n_out = n_recv
            if do_expand:
                prev = 0
                for i in range(L):
                    cur = int(expert_cpu[i])
                    counts.append(cur - _ceil_div(prev, expert_alignment) * expert_alignment)
                    prev = cur
                n_out = 0 if L == 0 else int(expert_cpu[L - 1])
            else:
                counts = [int(expert_cpu[i + 1] - expert_cpu[i]) for i in range(L)]
            recv_x = recv_x[:n_out]
            recv_topk_idx = recv_topk_idx[:n_recv]
            if recv_topk_weights is not None:
                recv_topk_weights = recv_topk_weights[:n_out]
            recv_src_metadata = recv_src_metadata[:n_recv]

        out_handle = EPHandle(do_expand, num_experts, expert_alignment, num_max_tokens_per_rank,
                              num_sms, kept_idx, counts, psum_rank, handle_psum_expert,
                              recv_src_metadata, dst_buffer_slot_idx, None, None, native_handle=True)
        keep = (x, topk_idx, kept_idx, active_ranks, recv_x, recv_topk_idx, psum_rank, psum_expert,
                recv_src_metadata, dst_buffer_slot_idx) + \
            (() if topk_weights is None else (topk_weights, recv_topk_weights))
        return (recv_x, recv_topk_idx, recv_topk_weights, out_handle,
                EventOverlap(event, keep if async_with_compute_stream else None))

    # ------------------------------------------------------------------ combine
    def combine(self, x: torch.Tensor, handle: EPHandle, topk_weights: Optional[torch.Tensor] = None,
                num_sms: Optional[int] = None, async_with_compute_stream: bool = False):
        """Reference :716-774. Returns (combined_x, None, event)."""
        if self.runtime is None:
            raise RuntimeError("ElasticBuffer has been destroyed")
        if handle.native_handle is None:
            raise RuntimeError("EPHandle does not contain a native handle")
        assert x.dim() == 2 and x.is_contiguous() and x.dtype == torch.bfloat16
        if handle.do_expand and topk_weights is not None:
            # the reference asserts the same on the device (combine_official.cuh:70)
            raise AssertionError("topk_weights must be None with an expanded layout")
        dev = x.device
        active_ranks = torch.ones(self.num_ranks, dtype=torch.int32, device=dev)
        T, K = int(handle.topk_idx.shape[0]), int(handle.topk_idx.shape[1])
        combined_x = torch.empty((T, x.shape[1]), dtype=x.dtype, device=dev)
        event = self.runtime.elastic_combine(
            x.data_ptr(), int(x.shape[0]), int(x.shape[1]), handle.topk_idx.data_ptr(), T, K,
            0 if topk_weights is None else topk_weights.data_ptr(),
            handle.psum_num_recv_tokens_per_scaleup_rank.data_ptr(),
            handle.recv_src_metadata.data_ptr(), active_ranks.data_ptr(), handle.num_experts,
            handle.num_max_tokens_per_rank, handle.do_expand, async_with_compute_stream,
            _stream_ptr(), combined_x.data_ptr(), self._timeout_us())
        keep = (x, active_ranks, combined_x, handle.topk_idx, handle.recv_src_metadata) + \
            (() if topk_weights is None else (topk_weights,))
        return combined_x, None, EventOverlap(event, keep if async_with_compute_stream else None)
