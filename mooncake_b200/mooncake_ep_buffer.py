"""`Buffer` / `EventOverlap`: the torch-facing API of the EP path.

Drop-in for the reference's wrapper (mooncake-wheel/mooncake/
mooncake_ep_buffer.py:34-90 `EventOverlap`, :92-681 `Buffer`): same
constructor, `dispatch` / `combine` signatures, returned tensors, handle tuple
and error behaviour. What is different underneath:

* there is no torch fallback - without peer-mapped NVLink memory for every
  active rank the constructor raises instead of degrading;
* rows of an expert arrive in a fixed order (source rank, then token index),
  which is the order the reference's torch path produces;
* in a group the returned `recv_x` is a view of the buffer's symmetric memory:
  peers store the rows there directly, so dispatch moves no payload on the
  receiving side. It stays valid until the dispatch call after the next one
  on this buffer (two calls may be in flight, as with the reference's double
  buffering); `Buffer(..., recv_in_place=False)` returns a fresh tensor instead,
  at the price of one copy;
* zero-copy combine is built: `get_next_combine_buffer(handle)` returns the
  symmetric tensor the next `combine(..., zero_copy=True)` reads (the reference
  documents it, docs/source/design/mooncake-ep.md:165-167, and rejects it,
  :551,680);
* calls can be captured in CUDA graphs after `buffer.runtime.set_option("graph_mode", 1)`
  (include/mcep.h);
* the bootstrap only all-gathers the 64-byte memory handles
  (reference :271-285); the RDMA metadata exchange (:188-264) does not exist.
"""
from __future__ import annotations

import warnings
from typing import Any, Callable, Optional, Tuple, Union

import torch
import torch.distributed as dist

from . import ep


def _stream_ptr() -> int:
    return int(torch.cuda.current_stream().cuda_stream)


class _DeviceBytes:
    """A span of the buffer's symmetric memory, exposed through the CUDA array
    interface so torch can wrap it without copying. Holds the runtime object:
    tensors made from it keep the allocation alive."""

    def __init__(self, owner: object, ptr: int, nbytes: int):
        self._owner = owner
        self.__cuda_array_interface__ = {"shape": (nbytes,), "typestr": "|u1",
                                         "data": (ptr, False), "version": 3}


class EventOverlap:
    """An event plus the tensors that must outlive it (reference :34-90)."""

    def __init__(self, event: Optional["ep.EventHandle"] = None,
                 extra_tensors: Optional[Tuple[torch.Tensor, ...]] = None) -> None:
        self.event = event
        # kept alive here rather than via record_stream, which CUDA graphs reject
        self.extra_tensors = extra_tensors

    def current_stream_wait(self) -> None:
        assert self.event is not None
        self.event.current_stream_wait(_stream_ptr())

    def __enter__(self) -> Any:
        return self

    def __exit__(self, exc_type: Any, exc_val: Any, exc_tb: Any) -> None:
        if self.event is not None:
            self.event.current_stream_wait(_stream_ptr())


class Buffer:
    def __init__(self, group: dist.ProcessGroup, num_ep_buffer_bytes: int = 0,
                 disable_p2p: bool = False, recv_in_place: bool = True):
        self.recv_in_place = recv_in_place
        self._views = {}
        self.rank = group.rank()
        self.group_size = group.size()
        self.group = group
        self.backend = group
        self.num_ep_buffer_bytes = num_ep_buffer_bytes
        self.runtime = ep.Buffer(self.rank, self.group_size, num_ep_buffer_bytes, disable_p2p)
        self._use_fallback = False  # there is none; kept because callers read it
        self._warned_active_ranks = False
        self.connect()

    # ---------------------------------------------------------------- bootstrap
    def connect(self, is_update: bool = False) -> None:
        """Exchange memory handles and map every active peer (reference :185-304)."""
        if self.group_size == 1:
            return
        if not self.runtime.p2p_enabled():
            raise RuntimeError("Mooncake EP (B200): P2P disabled and no RDMA route exists; "
                               "there is no fallback path")
        mine = self.runtime.get_ipc_handle()
        if dist.get_backend(self.group) == "gloo":
            device = torch.device("cpu")
        else:
            device = torch.device("cuda", torch.cuda.current_device())
        local = torch.tensor(mine, dtype=torch.int32, device=device)
        gathered = [torch.empty_like(local) for _ in range(self.group_size)]
        dist.all_gather(gathered, local, self.group)
        handles = [h.tolist() for h in gathered]
        mask = self._active_ranks_tensor(torch.device("cpu")).tolist()
        self.runtime.sync_nvlink_ipc_handles(handles, mask)
        if not self.runtime.use_fast_path():
            raise RuntimeError(f"[Rank {self.rank}] Mooncake EP (B200): not every active rank's "
                               "buffer could be mapped over NVLink; there is no fallback path")

    def update_ep_member(self) -> None:
        """Re-import the peers' handles after a membership change (reference :306-307)."""
        self.connect(True)

    def _active_ranks_tensor(self, device: torch.device,
                             dtype: torch.dtype = torch.int32) -> torch.Tensor:
        """All ones unless the group's backend can report liveness (reference :315-341)."""
        try:
            is_mooncake = dist.get_backend(self.group) == "mooncake"
        except Exception:
            is_mooncake = False
        if is_mooncake:
            try:
                from mooncake.pg import get_active_ranks  # type: ignore
                return get_active_ranks(self.backend).to(device=device, dtype=dtype)
            except Exception:
                pass
        elif not self._warned_active_ranks:
            warnings.warn("Mooncake EP active_ranks is only available with the mooncake process "
                          "group. Treating all ranks as active.", RuntimeWarning, stacklevel=3)
            self._warned_active_ranks = True
        return torch.ones((self.group_size,), dtype=dtype, device=device)

    @staticmethod
    def get_ep_buffer_size_hint(num_max_dispatch_tokens_per_rank: int, hidden: int,
                                num_ranks: int, num_experts: int) -> int:
        return ep.get_ep_buffer_size_hint(num_max_dispatch_tokens_per_rank, hidden, num_ranks,
                                          num_experts)

    def _resolve_active_ranks(self, active_ranks: Optional[torch.Tensor],
                              device: torch.device) -> torch.Tensor:
        if active_ranks is None:
            return self._active_ranks_tensor(device=device)
        assert active_ranks.dim() == 1 and active_ranks.is_contiguous()
        assert active_ranks.dtype == torch.int32
        if active_ranks.numel() != self.group_size:  # reference :394-397
            return torch.ones((self.group_size,), dtype=torch.int32, device=device)
        return active_ranks

    def _symmetric_tensor(self, ptr: int, nbytes: int, shape: tuple, dtype: torch.dtype,
                          device: torch.device) -> torch.Tensor:
        """A tensor over `nbytes` of symmetric memory at `ptr` (made once per span)."""
        views = self.__dict__.setdefault("_views", {})
        key = (ptr, nbytes, shape, dtype)
        t = views.get(key)
        if t is None:
            raw = torch.as_tensor(_DeviceBytes(self.runtime, ptr, nbytes), device=device)
            t = views[key] = raw.view(dtype).view(shape)
        return t

    # ----------------------------------------------------------------- dispatch
    def dispatch(self, x: torch.Tensor, topk_idx: torch.Tensor, active_ranks: torch.Tensor,
                 num_max_dispatch_tokens_per_rank: int, num_experts: int, timeout_us: int,
                 use_fp8: Optional[bool] = None, async_finish: bool = False,
                 return_recv_hook: bool = False
                 ) -> Tuple[Union[Tuple[torch.Tensor, torch.Tensor], torch.Tensor], torch.Tensor,
                            Tuple, EventOverlap, Optional[Callable]]:
        """Send every token to the ranks owning its top-k experts (reference :360-535).

        Returns `(recv_x | (recv_x, scales), recv_count, handle, event, hook)` with
        `recv_x[E/R, R*M, H]`, `scales[E/R, R*M, H/128]` (a transposed view of
        `[E/R, H/128, R*M]` storage), `recv_count[E/R]` and
        `handle = (src_info, layout_range, M, H, E)`.
        """
        assert x.dim() == 2 and x.is_contiguous()
        assert x.dtype == torch.bfloat16
        assert topk_idx.dim() == 2 and topk_idx.is_contiguous()
        assert topk_idx.dtype == torch.int64
        assert x.size(0) == topk_idx.size(0)
        assert x.size(0) <= num_max_dispatch_tokens_per_rank
        assert x.size(1) % 16 == 0 and x.size(1) % 128 == 0
        assert num_experts % self.group_size == 0
        active_ranks = self._resolve_active_ranks(active_ranks, x.device)
        if use_fp8 is None:
            use_fp8 = True
        R, M, H = self.group_size, num_max_dispatch_tokens_per_rank, x.size(1)
        L = num_experts // R
        dev = x.device
        rx_dtype = torch.float8_e4m3fn if use_fp8 else torch.bfloat16
        recv_x = None
        if getattr(self, "recv_in_place", True):
            ptr, nbytes = self.runtime.next_recv_x(M, H, num_experts, use_fp8)
            if ptr:
                recv_x = self._symmetric_tensor(ptr, nbytes, (L, R * M, H), rx_dtype, dev)
        if recv_x is None:
            recv_x = torch.empty((L, R * M, H), device=dev, dtype=rx_dtype)
        recv_count = torch.empty((L,), dtype=torch.int32, device=dev)
        src_info = torch.empty((L, R * M), dtype=torch.int32, device=dev)
        layout_range = torch.empty((L, R), dtype=torch.int64, device=dev)
        scales = None
        if use_fp8:
            assert (R * M) % 4 == 0
            scales = torch.empty((L, H // 128, R * M), dtype=torch.float32,
                                 device=dev).transpose(1, 2)
        event, hook = self.runtime.dispatch(
            x.data_ptr(), topk_idx.data_ptr(), active_ranks.data_ptr(), x.size(0), H,
            topk_idx.size(1), M, num_experts, timeout_us, use_fp8, recv_x.data_ptr(),
            0 if scales is None else scales.data_ptr(), recv_count.data_ptr(),
            src_info.data_ptr(), layout_range.data_ptr(), async_finish, return_recv_hook,
            _stream_ptr())
        handle = (src_info, layout_range, M, H, num_experts)
        keep = (x, topk_idx, recv_x, scales, recv_count, src_info, layout_range)
        return ((recv_x, scales) if use_fp8 else recv_x, recv_count, handle,
                EventOverlap(event, keep if async_finish else None), hook)

    # ------------------------------------------------------------------ combine
    def combine(self, x: torch.Tensor, topk_idx: torch.Tensor, topk_weights: torch.Tensor,
                active_ranks: torch.Tensor, timeout_us: int, handle: tuple,
                zero_copy: bool = False, async_finish: bool = False,
                return_recv_hook: bool = False, out: Optional[torch.Tensor] = None
                ) -> Tuple[torch.Tensor, EventOverlap, Optional[Callable]]:
        """Bring the expert outputs back and reduce them with the top-k weights
        (reference :538-678). With `zero_copy` the expert outputs are read from the
        tensor `get_next_combine_buffer(handle)` returned and `x` only gives the
        shape."""
        assert x.dim() == 3 and x.is_contiguous()
        assert x.dtype == torch.bfloat16
        assert topk_idx.dim() == 2 and topk_idx.is_contiguous()
        assert topk_idx.dtype == torch.int64
        assert topk_weights.dim() == 2 and topk_weights.is_contiguous()
        assert topk_weights.dtype == torch.float32
        active_ranks = self._resolve_active_ranks(active_ranks, x.device)
        src_info, layout_range, M, hidden, num_experts = handle
        R = self.group_size
        assert x.size(0) == num_experts // R
        assert x.size(1) == R * M
        assert x.size(2) == hidden
        assert hidden % 16 == 0 and hidden % 128 == 0
        assert topk_idx.size() == topk_weights.size()
        assert topk_weights.size(0) <= M
        assert src_info.dim() == 2 and src_info.is_contiguous()
        assert src_info.dtype == torch.int32 and src_info.size(0) == x.size(0)
        assert layout_range.dim() == 2 and layout_range.is_contiguous()
        assert layout_range.dtype == torch.int64
        assert layout_range.size(0) == num_experts // R and layout_range.size(1) == R
        if out is not None:
            assert out.dim() == 2 and out.is_contiguous()
            assert out.size(0) == topk_weights.size(0) and out.size(1) == hidden
            assert out.dtype == x.dtype
            combined_x = out
        else:
            combined_x = torch.empty((topk_weights.size(0), hidden), dtype=x.dtype,
                                     device=x.device)
        event, hook = self.runtime.combine(
            x.data_ptr(), topk_idx.data_ptr(), topk_weights.data_ptr(), src_info.data_ptr(),
            layout_range.data_ptr(), active_ranks.data_ptr(), x.size(0), topk_weights.size(0),
            hidden, topk_weights.size(1), M, num_experts, timeout_us, zero_copy,
            combined_x.data_ptr(), async_finish, return_recv_hook, _stream_ptr())
        keep = (x, topk_idx, topk_weights, src_info, layout_range, combined_x)
        return combined_x, EventOverlap(event, keep if async_finish else None), hook

    def get_next_combine_buffer(self, handle: tuple) -> torch.Tensor:
        """The tensor `[E/R, R*M, H]` bf16 the next `combine(..., zero_copy=True)`
        reads: write the expert outputs into it instead of a tensor of your own.
        A single rank has no symmetric memory to write into; it gets an ordinary
        tensor and passes it to combine as `x`."""
        src_info, _, M, hidden, num_experts = handle
        R = self.group_size
        shape = (num_experts // R, R * M, hidden)
        ptr, nbytes = self.runtime.next_combine_buffer(M, hidden, num_experts)
        if not ptr:
            return torch.empty(shape, dtype=torch.bfloat16, device=src_info.device)
        return self._symmetric_tensor(ptr, nbytes, shape, torch.bfloat16, src_info.device)
