"""Native module of the package: the objects the reference exposes as
`mooncake._ep` / `mooncake.ep` (mooncake-ep/src/ep_py.cpp:14-46,
mooncake-wheel/mooncake/ep.py:1-26), bound with ctypes to the C ABI of
`libmcep.so` (include/mcep.h).

`Buffer`, `EventHandle`, `get_ep_buffer_size_hint` and `MAX_QP_COUNT` keep the
reference's names, argument order and return shapes. There is no CPU path:
if the shared library is missing it is built with nvcc, and if that fails the
import fails.
"""
from __future__ import annotations

import ctypes
import os
from typing import Callable, List, Optional, Tuple

from . import build as _build

_c = ctypes


class _DispatchArgs(_c.Structure):
    _fields_ = [
        ("x", _c.c_void_p), ("topk_idx", _c.c_void_p), ("active_ranks", _c.c_void_p),
        ("num_tokens", _c.c_int32), ("hidden", _c.c_int32), ("num_topk", _c.c_int32),
        ("num_max_dispatch_tokens_per_rank", _c.c_int32), ("num_experts", _c.c_int32),
        ("use_fp8", _c.c_int32), ("timeout_us", _c.c_int64),
        ("packed_recv_x", _c.c_void_p), ("packed_recv_x_scales", _c.c_void_p),
        ("packed_recv_count", _c.c_void_p), ("packed_recv_src_info", _c.c_void_p),
        ("packed_recv_layout_range", _c.c_void_p),
        ("async_finish", _c.c_int32), ("return_recv_hook", _c.c_int32),
        ("compute_stream", _c.c_uint64),
    ]


class _CombineArgs(_c.Structure):
    _fields_ = [
        ("x", _c.c_void_p), ("topk_idx", _c.c_void_p), ("topk_weights", _c.c_void_p),
        ("src_info", _c.c_void_p), ("layout_range", _c.c_void_p), ("active_ranks", _c.c_void_p),
        ("num_local_experts", _c.c_int32), ("num_combined_tokens", _c.c_int32),
        ("hidden", _c.c_int32), ("num_topk", _c.c_int32),
        ("num_max_dispatch_tokens_per_rank", _c.c_int32), ("num_experts", _c.c_int32),
        ("timeout_us", _c.c_int64), ("zero_copy", _c.c_int32),
        ("combined_x", _c.c_void_p),
        ("async_finish", _c.c_int32), ("return_recv_hook", _c.c_int32),
        ("compute_stream", _c.c_uint64),
    ]


class _ElasticDispatchArgs(_c.Structure):
    _fields_ = [
        ("x", _c.c_void_p), ("x_element_size", _c.c_int32), ("sf", _c.c_void_p),
        ("num_tokens", _c.c_int32), ("hidden", _c.c_int32), ("num_sf_packs", _c.c_int32),
        ("sf_token_stride", _c.c_int32), ("sf_hidden_stride", _c.c_int32),
        ("topk_idx", _c.c_void_p), ("num_topk", _c.c_int32), ("topk_weights", _c.c_void_p),
        ("active_ranks", _c.c_void_p),
        ("num_experts", _c.c_int32), ("num_max_tokens_per_rank", _c.c_int32),
        ("expert_alignment", _c.c_int32), ("do_expand", _c.c_int32), ("cached_mode", _c.c_int32),
        ("timeout_us", _c.c_int64), ("async_with_compute_stream", _c.c_int32),
        ("compute_stream", _c.c_uint64),
        ("psum_num_recv_tokens_per_scaleup_rank", _c.c_void_p),
        ("psum_num_recv_tokens_per_expert", _c.c_void_p), ("dst_buffer_slot_idx", _c.c_void_p),
        ("recv_x", _c.c_void_p), ("recv_x_scales", _c.c_void_p), ("recv_topk_idx", _c.c_void_p),
        ("recv_topk_weights", _c.c_void_p), ("recv_src_metadata", _c.c_void_p),
        ("copied_topk_idx", _c.c_void_p),
    ]


class _ElasticCombineArgs(_c.Structure):
    _fields_ = [
        ("x", _c.c_void_p), ("num_input_tokens", _c.c_int32), ("hidden", _c.c_int32),
        ("topk_idx", _c.c_void_p), ("num_combined_tokens", _c.c_int32), ("num_topk", _c.c_int32),
        ("topk_weights", _c.c_void_p), ("psum_num_recv_tokens_per_scaleup_rank", _c.c_void_p),
        ("recv_src_metadata", _c.c_void_p), ("active_ranks", _c.c_void_p),
        ("num_experts", _c.c_int32), ("num_max_tokens_per_rank", _c.c_int32),
        ("do_expand", _c.c_int32), ("timeout_us", _c.c_int64),
        ("async_with_compute_stream", _c.c_int32), ("compute_stream", _c.c_uint64),
        ("combined_x", _c.c_void_p),
    ]


def _load() -> ctypes.CDLL:
    # builds the library when it is missing or older than its sources (where the
    # sources and a compiler are present; a prebuilt library alone is taken as is)
    path = _build.build()
    L = ctypes.CDLL(path)
    vp, i32, i64, u64 = _c.c_void_p, _c.c_int, _c.c_int64, _c.c_uint64
    sig = {
        "mcep_last_error": (_c.c_char_p, []),
        "mcep_kernel_launch_count": (u64, []),
        "mcep_set_kernel_timing": (i32, [i32]),
        "mcep_drain_kernel_times": (i32, [_c.c_char_p, _c.c_size_t]),
        "mcep_get_ep_buffer_size_hint": (u64, [i32, i32, i32, i32]),
        "mcep_buffer_create": (i32, [i32, i32, i64, i32, _c.POINTER(vp)]),
        "mcep_buffer_destroy": (i32, [vp]),
        "mcep_buffer_ibgda_disabled": (i32, [vp]),
        "mcep_buffer_p2p_enabled": (i32, [vp]),
        "mcep_buffer_is_roce": (i32, [vp]),
        "mcep_buffer_use_fast_path": (i32, [vp]),
        "mcep_buffer_uses_fabric_handles": (i32, [vp]),
        "mcep_buffer_get_ipc_handle": (i32, [vp, _c.POINTER(_c.c_int32), i32, _c.POINTER(i32)]),
        "mcep_buffer_sync_nvlink_ipc_handles": (i32, [vp, _c.POINTER(_c.c_int32), i32,
                                                      _c.POINTER(_c.c_int32)]),
        "mcep_buffer_local_base": (i32, [vp, _c.POINTER(vp)]),
        "mcep_buffer_set_peer_bases": (i32, [vp, _c.POINTER(vp), _c.POINTER(_c.c_int32)]),
        "mcep_buffer_set_option": (i32, [vp, _c.c_char_p, i64]),
        "mcep_buffer_status": (i32, [vp, _c.POINTER(_c.c_int32), i32]),
        "mcep_buffer_barrier": (i32, [vp, vp, u64]),
        "mcep_buffer_call_counts": (i32, [vp, _c.POINTER(_c.c_uint32), _c.POINTER(_c.c_uint32)]),
        "mcep_buffer_next_recv_x": (i32, [vp, i32, i32, i32, i32, _c.POINTER(vp),
                                          _c.POINTER(_c.c_size_t)]),
        "mcep_buffer_next_combine_buffer": (i32, [vp, i32, i32, i32, _c.POINTER(vp),
                                                  _c.POINTER(_c.c_size_t)]),
        "mcep_launch_deferred": (i32, [_c.POINTER(vp), i32]),
        "mcep_dispatch": (i32, [vp, _c.POINTER(_DispatchArgs), _c.POINTER(vp), _c.POINTER(vp)]),
        "mcep_combine": (i32, [vp, _c.POINTER(_CombineArgs), _c.POINTER(vp), _c.POINTER(vp)]),
        "mcep_elastic_dispatch": (i32, [vp, _c.POINTER(_ElasticDispatchArgs), _c.POINTER(vp)]),
        "mcep_elastic_combine": (i32, [vp, _c.POINTER(_ElasticCombineArgs), _c.POINTER(vp)]),
        "mcep_elastic_buffer_size_hint": (u64, [i32, i32, i32, i32]),
        "mcep_event_create": (i32, [u64, _c.POINTER(vp)]),
        "mcep_event_current_stream_wait": (i32, [vp, u64]),
        "mcep_event_synchronize": (i32, [vp]),
        "mcep_event_free": (i32, [vp]),
        "mcep_hook_run": (i32, [vp]),
        "mcep_hook_free": (i32, [vp]),
        "mcep_routing_layout_scratch_bytes": (_c.c_size_t, []),
        "mcep_routing_layout": (i32, [vp, i32, i32, i32, i32, vp, vp, vp, vp, vp, u64]),
        "mcep_combine_single_rank_static": (i32, [vp, vp, vp, vp, vp, i32, i32, i32, i32, i32, vp,
                                                  u64]),
        "mcep_static_last_error": (_c.c_char_p, []),
        "mcep_static_status": (i32, [_c.POINTER(_c.c_int32)]),
    }
    for name, (res, args) in sig.items():
        fn = getattr(L, name)
        fn.restype, fn.argtypes = res, args
    return L


_lib = _load()

MAX_QP_COUNT = 256  # mooncake-ep/include/mooncake_ep_configs.cuh:5


def _check(rc: int) -> None:
    """Failures surface as RuntimeError, as the reference's EPException does
    through pybind (mooncake-ep/include/mooncake_ep_exception.cuh:12-24)."""
    if rc != 0:
        raise RuntimeError(_lib.mcep_last_error().decode())


def kernel_launch_count() -> int:
    return int(_lib.mcep_kernel_launch_count())


def set_kernel_timing(on: bool) -> None:
    _check(_lib.mcep_set_kernel_timing(1 if on else 0))


def drain_kernel_times() -> dict:
    """{kernel name: (launches, total milliseconds)} since timing was switched on."""
    buf = _c.create_string_buffer(1 << 16)
    _check(_lib.mcep_drain_kernel_times(buf, len(buf)))
    out = {}
    for line in buf.value.decode().splitlines():
        name, n, ms = line.split()
        out[name] = (int(n), float(ms))
    return out


def get_ep_buffer_size_hint(num_max_dispatch_tokens_per_rank: int, hidden: int,
                            num_ranks: int, num_experts: int) -> int:
    """mooncake-ep/include/mooncake_ep_buffer.h:197-203."""
    return int(_lib.mcep_get_ep_buffer_size_hint(num_max_dispatch_tokens_per_rank, hidden,
                                                 num_ranks, num_experts))


class EventHandle:
    """mooncake-ep/include/mooncake_ep_event.h:9-44: a CUDA event recorded on
    `stream_ptr` at construction."""

    def __init__(self, stream_ptr: int = 0, _adopt: Optional[int] = None):
        if _adopt is not None:
            self._h = _c.c_void_p(_adopt)
        else:
            h = _c.c_void_p()
            _check(_lib.mcep_event_create(stream_ptr, _c.byref(h)))
            self._h = h

    def current_stream_wait(self, stream_ptr: int) -> None:
        _check(_lib.mcep_event_current_stream_wait(self._h, stream_ptr))

    def synchronize(self) -> None:
        _check(_lib.mcep_event_synchronize(self._h))

    def __del__(self):
        h, self._h = getattr(self, "_h", None), None
        if h:
            _lib.mcep_event_free(h)


class _Hook:
    """The receive-phase callback (the `std::function<void()>` of the reference)."""

    def __init__(self, handle: int):
        self._h = _c.c_void_p(handle)

    def __call__(self) -> None:
        _check(_lib.mcep_hook_run(self._h))

    def __del__(self):
        h, self._h = getattr(self, "_h", None), None
        if h:
            _lib.mcep_hook_free(h)


class Buffer:
    """mooncake-ep/src/ep_py.cpp:28-46 / mooncake-ep/include/mooncake_ep_buffer.h:65-195."""

    def __init__(self, rank: int, num_ranks: int, num_ep_buffer_bytes: int,
                 disable_p2p: bool = False):
        self._h = _c.c_void_p()
        self.rank, self.num_ranks = rank, num_ranks
        _check(_lib.mcep_buffer_create(rank, num_ranks, num_ep_buffer_bytes,
                                       1 if disable_p2p else 0, _c.byref(self._h)))
        self._dargs = _DispatchArgs()
        self._cargs = _CombineArgs()

    def __del__(self):
        h, self._h = getattr(self, "_h", None), None
        if h:
            _lib.mcep_buffer_destroy(h)

    # -- RDMA surface of the reference: there is no RDMA route here ------------
    def ibgda_disabled(self) -> bool:
        return True

    def is_roce(self) -> bool:
        return False

    def update_local_qpns(self) -> None:
        return None

    def sync_ibgda_peers(self, *args) -> None:
        return None

    def get_mr_info(self) -> Tuple[int, int]:
        return (0, 0)

    def get_gid(self) -> Tuple[int, int]:
        return (0, 0)

    def get_local_qpns(self) -> List[int]:
        return []

    def get_local_lids(self) -> List[int]:
        return []

    # -- NVLink peer mapping ---------------------------------------------------
    def p2p_enabled(self) -> bool:
        return bool(_lib.mcep_buffer_p2p_enabled(self._h))

    def use_fast_path(self) -> bool:
        return bool(_lib.mcep_buffer_use_fast_path(self._h))

    def uses_fabric_handles(self) -> bool:
        """True when the buffer is shared through fabric handles (MC_USE_NVLINK_IPC=0
        and driver support) rather than CUDA IPC handles."""
        return bool(_lib.mcep_buffer_uses_fabric_handles(self._h))

    def get_ipc_handle(self) -> List[int]:
        out = (_c.c_int32 * 18)()  # 16 for a CUDA IPC handle, 18 for a fabric handle + size
        n = _c.c_int(0)
        _check(_lib.mcep_buffer_get_ipc_handle(self._h, out, 18, _c.byref(n)))
        return list(out[: n.value])

    def sync_nvlink_ipc_handles(self, remote_handles: List[List[int]],
                                active_ranks_mask: List[int]) -> None:
        n_per = max((len(h) for h in remote_handles), default=0)
        if n_per == 0:
            return
        flat = (_c.c_int32 * (n_per * self.num_ranks))()
        for r, h in enumerate(remote_handles[: self.num_ranks]):
            for i, v in enumerate(h):
                flat[r * n_per + i] = v
        mask = (_c.c_int32 * self.num_ranks)(*[int(v) for v in active_ranks_mask])
        _check(_lib.mcep_buffer_sync_nvlink_ipc_handles(self._h, flat, n_per, mask))

    # -- in-process groups / options / diagnostics (no reference counterpart) ---
    def local_base(self) -> int:
        p = _c.c_void_p()
        _check(_lib.mcep_buffer_local_base(self._h, _c.byref(p)))
        return int(p.value)

    def set_peer_bases(self, bases: List[int], available: Optional[List[int]] = None) -> None:
        arr = (_c.c_void_p * self.num_ranks)(*bases)
        av = (_c.c_int32 * self.num_ranks)(*(available or [1] * self.num_ranks))
        _check(_lib.mcep_buffer_set_peer_bases(self._h, arr, av))

    def set_option(self, name: str, value: int) -> None:
        _check(_lib.mcep_buffer_set_option(self._h, name.encode(), int(value)))

    def status(self) -> int:
        out = (_c.c_int32 * 1)()
        _check(_lib.mcep_buffer_status(self._h, out, 1))
        return int(out[0])

    def barrier(self, stream_ptr: int = 0, active_ranks_ptr: int = 0) -> None:
        """Device-side barrier of the group on `stream_ptr` (include/mcep.h:
        mcep_buffer_barrier): the ranks leave it within about a microsecond of
        each other."""
        _check(_lib.mcep_buffer_barrier(self._h, active_ranks_ptr or None, stream_ptr))

    def call_counts(self) -> Tuple[int, int]:
        """(dispatch calls, combine calls) made or adopted so far."""
        d, c = _c.c_uint32(), _c.c_uint32()
        _check(_lib.mcep_buffer_call_counts(self._h, _c.byref(d), _c.byref(c)))
        return int(d.value), int(c.value)

    def next_recv_x(self, num_max_dispatch_tokens_per_rank: int, hidden: int, num_experts: int,
                    use_fp8: bool) -> Tuple[int, int]:
        """(device pointer, bytes) of the in-place receive tensor of the next
        dispatch call, (0, 0) when there is none (include/mcep.h)."""
        p, n = _c.c_void_p(), _c.c_size_t()
        _check(_lib.mcep_buffer_next_recv_x(self._h, num_max_dispatch_tokens_per_rank, hidden,
                                            num_experts, int(use_fp8), _c.byref(p), _c.byref(n)))
        return int(p.value or 0), int(n.value)

    def next_combine_buffer(self, num_max_dispatch_tokens_per_rank: int, hidden: int,
                            num_experts: int) -> Tuple[int, int]:
        """(device pointer, bytes) of the tensor the next zero-copy combine reads."""
        p, n = _c.c_void_p(), _c.c_size_t()
        _check(_lib.mcep_buffer_next_combine_buffer(self._h, num_max_dispatch_tokens_per_rank,
                                                    hidden, num_experts, _c.byref(p),
                                                    _c.byref(n)))
        return int(p.value or 0), int(n.value)

    # -- the hot path ----------------------------------------------------------
    def dispatch(self, x_ptr: int, topk_idx_ptr: int, active_ranks_ptr: int, num_tokens: int,
                 hidden: int, num_topk: int, num_max_dispatch_tokens_per_rank: int,
                 num_experts: int, timeout_us: int, use_fp8: bool, packed_recv_x_ptr: int,
                 packed_recv_x_scales_ptr: int, packed_recv_count_ptr: int,
                 packed_recv_src_info_ptr: int, packed_recv_layout_range_ptr: int,
                 async_finish: bool, return_recv_hook: bool, compute_stream_ptr: int
                 ) -> Tuple[Optional[EventHandle], Optional[Callable[[], None]]]:
        a = self._dargs
        a.x, a.topk_idx, a.active_ranks = x_ptr, topk_idx_ptr, active_ranks_ptr
        a.num_tokens, a.hidden, a.num_topk = num_tokens, hidden, num_topk
        a.num_max_dispatch_tokens_per_rank = num_max_dispatch_tokens_per_rank
        a.num_experts, a.use_fp8, a.timeout_us = num_experts, int(use_fp8), timeout_us
        a.packed_recv_x, a.packed_recv_x_scales = packed_recv_x_ptr, packed_recv_x_scales_ptr
        a.packed_recv_count = packed_recv_count_ptr
        a.packed_recv_src_info = packed_recv_src_info_ptr
        a.packed_recv_layout_range = packed_recv_layout_range_ptr
        a.async_finish, a.return_recv_hook = int(async_finish), int(return_recv_hook)
        a.compute_stream = compute_stream_ptr
        ev, hk = _c.c_void_p(), _c.c_void_p()
        _check(_lib.mcep_dispatch(self._h, _c.byref(a), _c.byref(ev), _c.byref(hk)))
        return (EventHandle(_adopt=ev.value) if ev.value else None,
                _Hook(hk.value) if hk.value else None)

    def combine(self, x_ptr: int, topk_idx_ptr: int, topk_weights_ptr: int, src_info_ptr: int,
                layout_range_ptr: int, active_ranks_ptr: int, num_local_experts: int,
                num_combined_tokens: int, hidden: int, num_topk: int,
                num_max_dispatch_tokens_per_rank: int, num_experts: int, timeout_us: int,
                zero_copy: bool, combined_x_ptr: int, async_finish: bool,
                return_recv_hook: bool, compute_stream_ptr: int
                ) -> Tuple[Optional[EventHandle], Optional[Callable[[], None]]]:
        a = self._cargs
        a.x, a.topk_idx, a.topk_weights = x_ptr, topk_idx_ptr, topk_weights_ptr
        a.src_info, a.layout_range, a.active_ranks = src_info_ptr, layout_range_ptr, active_ranks_ptr
        a.num_local_experts, a.num_combined_tokens = num_local_experts, num_combined_tokens
        a.hidden, a.num_topk = hidden, num_topk
        a.num_max_dispatch_tokens_per_rank = num_max_dispatch_tokens_per_rank
        a.num_experts, a.timeout_us, a.zero_copy = num_experts, timeout_us, int(zero_copy)
        a.combined_x = combined_x_ptr
        a.async_finish, a.return_recv_hook = int(async_finish), int(return_recv_hook)
        a.compute_stream = compute_stream_ptr
        ev, hk = _c.c_void_p(), _c.c_void_p()
        _check(_lib.mcep_combine(self._h, _c.byref(a), _c.byref(ev), _c.byref(hk)))
        return (EventHandle(_adopt=ev.value) if ev.value else None,
                _Hook(hk.value) if hk.value else None)


    # -- elastic-style calls (mooncake-ep/src/mooncake_ep_elastic_buffer.cpp:230-426) -----
    def elastic_dispatch(self, x_ptr: int, x_element_size: int, sf_ptr: int, num_tokens: int,
                         hidden: int, num_sf_packs: int, sf_token_stride: int,
                         sf_hidden_stride: int, topk_idx_ptr: int, num_topk: int,
                         topk_weights_ptr: int, active_ranks_ptr: int, num_experts: int,
                         num_max_tokens_per_rank: int, expert_alignment: int, do_expand: bool,
                         async_with_compute_stream: bool, compute_stream_ptr: int,
                         cached_mode: bool, psum_rank_ptr: int, psum_expert_ptr: int,
                         dst_buffer_slot_idx_ptr: int, recv_x_ptr: int, recv_x_scales_ptr: int,
                         recv_topk_idx_ptr: int, recv_topk_weights_ptr: int,
                         recv_src_metadata_ptr: int, timeout_us: int = -1,
                         copied_topk_idx_ptr: int = 0) -> Optional[EventHandle]:
        a = _ElasticDispatchArgs()
        a.x, a.x_element_size, a.sf = x_ptr, x_element_size, sf_ptr or None
        a.num_tokens, a.hidden, a.num_sf_packs = num_tokens, hidden, num_sf_packs
        a.sf_token_stride, a.sf_hidden_stride = sf_token_stride, sf_hidden_stride
        a.topk_idx, a.num_topk, a.topk_weights = topk_idx_ptr, num_topk, topk_weights_ptr or None
        a.active_ranks = active_ranks_ptr
        a.num_experts, a.num_max_tokens_per_rank = num_experts, num_max_tokens_per_rank
        a.expert_alignment, a.do_expand, a.cached_mode = expert_alignment, int(do_expand), int(cached_mode)
        a.timeout_us = timeout_us
        a.async_with_compute_stream, a.compute_stream = int(async_with_compute_stream), compute_stream_ptr
        a.psum_num_recv_tokens_per_scaleup_rank = psum_rank_ptr
        a.psum_num_recv_tokens_per_expert = psum_expert_ptr
        a.dst_buffer_slot_idx = dst_buffer_slot_idx_ptr
        a.recv_x, a.recv_x_scales = recv_x_ptr, recv_x_scales_ptr or None
        a.recv_topk_idx, a.recv_topk_weights = recv_topk_idx_ptr, recv_topk_weights_ptr or None
        a.recv_src_metadata = recv_src_metadata_ptr
        a.copied_topk_idx = copied_topk_idx_ptr or None
        ev = _c.c_void_p()
        _check(_lib.mcep_elastic_dispatch(self._h, _c.byref(a), _c.byref(ev)))
        return EventHandle(_adopt=ev.value) if ev.value else None

    def elastic_combine(self, x_ptr: int, num_input_tokens: int, hidden: int, topk_idx_ptr: int,
                        num_combined_tokens: int, num_topk: int, topk_weights_ptr: int,
                        psum_rank_ptr: int, recv_src_metadata_ptr: int, active_ranks_ptr: int,
                        num_experts: int, num_max_tokens_per_rank: int, do_expand: bool,
                        async_with_compute_stream: bool, compute_stream_ptr: int,
                        combined_x_ptr: int, timeout_us: int = -1) -> Optional[EventHandle]:
        a = _ElasticCombineArgs()
        a.x, a.num_input_tokens, a.hidden = x_ptr or None, num_input_tokens, hidden
        a.topk_idx, a.num_combined_tokens, a.num_topk = topk_idx_ptr, num_combined_tokens, num_topk
        a.topk_weights = topk_weights_ptr or None
        a.psum_num_recv_tokens_per_scaleup_rank = psum_rank_ptr
        a.recv_src_metadata, a.active_ranks = recv_src_metadata_ptr, active_ranks_ptr
        a.num_experts, a.num_max_tokens_per_rank = num_experts, num_max_tokens_per_rank
        a.do_expand, a.timeout_us = int(do_expand), timeout_us
        a.async_with_compute_stream, a.compute_stream = int(async_with_compute_stream), compute_stream_ptr
        a.combined_x = combined_x_ptr or None
        ev = _c.c_void_p()
        _check(_lib.mcep_elastic_combine(self._h, _c.byref(a), _c.byref(ev)))
        return EventHandle(_adopt=ev.value) if ev.value else None


def elastic_buffer_size_hint(num_max_tokens_per_rank: int, hidden: int, num_ranks: int,
                             num_topk: int) -> int:
    return int(_lib.mcep_elastic_buffer_size_hint(num_max_tokens_per_rank, hidden, num_ranks, num_topk))


def launch_deferred(buffers: List["Buffer"]) -> None:
    """In-process groups: start, as one launch, the calls the given buffers have
    prepared under option "defer_launch" (include/mcep.h: mcep_launch_deferred)."""
    arr = (_c.c_void_p * len(buffers))(*[b._h for b in buffers])
    _check(_lib.mcep_launch_deferred(arr, len(buffers)))


def routing_layout(topk_idx_ptr: int, num_tokens: int, num_topk: int, num_experts: int,
                   num_ranks: int, count_ptr: int, rank_count_ptr: int, expert_prefix_ptr: int,
                   slot_ptr: int, scratch_ptr: int, stream_ptr: int = 0) -> None:
    """The routing-layout kernel on its own (include/mcep.h: mcep_routing_layout)."""
    _check(_lib.mcep_routing_layout(topk_idx_ptr, num_tokens, num_topk, num_experts, num_ranks,
                                    count_ptr, rank_count_ptr, expert_prefix_ptr, slot_ptr,
                                    scratch_ptr, stream_ptr))


def routing_layout_scratch_bytes() -> int:
    return int(_lib.mcep_routing_layout_scratch_bytes())


STATIC_MAX_ENTRIES = 65536  # MCEP_STATIC_MAX_ENTRIES


def combine_single_rank_static(x_ptr: int, topk_idx_ptr: int, topk_weights_ptr: int,
                               src_info_ptr: int, layout_range_ptr: int, num_experts: int,
                               num_combined_tokens: int, hidden: int, num_topk: int,
                               num_max_dispatch_tokens_per_rank: int, combined_x_ptr: int,
                               stream_ptr: int = 0) -> None:
    """Single-rank combine that allocates nothing (include/mcep.h:
    mcep_combine_single_rank_static). For callers that may not call cudaMalloc and
    therefore cannot construct a `Buffer`; the scratch is a static device array
    shared by all calls, so calls that could overlap on the GPU must be ordered.
    At most STATIC_MAX_ENTRIES (token, k) pairs."""
    rc = _lib.mcep_combine_single_rank_static(x_ptr, topk_idx_ptr, topk_weights_ptr, src_info_ptr,
                                              layout_range_ptr, num_experts, num_combined_tokens,
                                              hidden, num_topk, num_max_dispatch_tokens_per_rank,
                                              combined_x_ptr, stream_ptr)
    if rc != 0:
        raise RuntimeError(_lib.mcep_static_last_error().decode())


def static_status() -> int:
    """Anomaly bits the allocation-free combine's kernels recorded on the current
    device since the last call of this function (0 = clean); reading clears them."""
    out = _c.c_int32(0)
    if _lib.mcep_static_status(_c.byref(out)) != 0:
        raise RuntimeError(_lib.mcep_static_last_error().decode())
    return int(out.value)
