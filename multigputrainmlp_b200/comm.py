"""Host side of the data-parallel gradient exchange.

`GradientRangeScheduler` decides WHEN each gradient range is exchanged and updated; it mirrors the
reference's ScheduleGradientAllreduce (native/tools/mgt_native_train_smoke.cu:494-523): ranges
arrive through the gradient-ready callback in backward order, each is cut into chunks of at most
`allreduce_bucket_bytes`, and the exchange runs on a second stream behind an event so that it
overlaps the rest of backward. The exchange is fused with the AdamW update here; that is safe without
holding ranges back because the engine announces a range only after the last kernel that reads its
weights has been enqueued (include/mgt_b200.h). `lag` remains for engines that announce earlier, as the
reference does.

Back-ends:
  PeerBackend  - the library's NVLink peer-to-peer kernels (mgt_comm_* in include/mgt_b200.h)
  NcclBackend  - ncclAllReduce + scale + AdamW kernel, the reference's own scheme (comparison only)
  the tests plug in a CPU back-end over torch.distributed/gloo to exercise the scheduling logic.
"""
from __future__ import annotations

import ctypes as C
import os
from dataclasses import dataclass, field
from typing import Callable, List, Optional, Tuple

from . import _lib
from .api import AdamWKernelConfig, MgtError, _Adam, _ptr, _stream


@dataclass
class ScheduledChunk:
    ready_id: int
    offset: int
    count: int


@dataclass
class GradientRangeScheduler:
    """Orders gradient ranges into exchange launches. Pure host logic, no CUDA."""
    launch: Callable[[int, int], None]               # (param_offset, param_count) -> enqueue exchange(+update) of that range
    wait_for_producer: Callable[[], None]            # make the exchange stream wait for what the compute stream has enqueued so far
    bucket_params: int = (4 << 20) // 4
    expected_ranges: Optional[int] = None
    lag: int = 0                                     # notifications a range is held back (1 = fused update behind an engine that announces a layer before its dX GEMM)
    whole_tail: bool = True                          # ranges left at finish() go out unchunked: nothing remains to overlap with
    launch_early: Optional[Callable[[int, int], None]] = None   # how a range from the early hook is sent (default: like any other)
    coalesce: bool = False                           # join ranges that touch in memory into one launch of at most bucket_params
    scheduled_ranges: int = 0
    scheduled_chunks: int = 0
    log: List[ScheduledChunk] = field(default_factory=list)
    _pending: List[Tuple[int, int, int]] = field(default_factory=list)
    _early: List[Tuple[int, int]] = field(default_factory=list)   # what the early hook already sent this step

    def begin_step(self) -> None:
        self.scheduled_ranges = 0
        self.scheduled_chunks = 0
        self.log = []
        self._pending = []
        self._early = []

    def on_early(self, ready_id: int, param_offset: int, param_count: int) -> int:
        """The engine's early-range hook (mgt_engine_set_early_range_hook): the range that closes backward in the
        reference's order (embedding table + input bias), or a leading part of it, is complete while weight-gradient
        GEMMs of other layers are still to run. It goes out at once and whole, so that its exchange runs under that
        work; the closing gradient-ready call then only sends what is left of the range, if anything."""
        if param_count == 0:
            return 1
        self._flush(0)
        self.wait_for_producer()
        (self.launch_early or self.launch)(param_offset, param_count)
        self.log.append(ScheduledChunk(ready_id, param_offset, param_count))
        self.scheduled_chunks += 1
        self._early.append((param_offset, param_count))
        return 0

    def _flush(self, keep: int, whole: bool = False) -> None:
        if len(self._pending) <= keep:
            return
        self.wait_for_producer()
        while len(self._pending) > keep:
            ready_id, offset, count = self._pending.pop(0)
            remaining = count
            while remaining > 0:
                chunk = remaining if whole else min(remaining, max(1, self.bucket_params))
                self.launch(offset, chunk)
                self.log.append(ScheduledChunk(ready_id, offset, chunk))
                offset += chunk
                remaining -= chunk
                self.scheduled_chunks += 1

    def on_ready(self, ready_id: int, param_offset: int, param_count: int) -> int:
        if param_count == 0 or (self.expected_ranges is not None and ready_id >= self.expected_ranges):
            return 1  # invalid_config, as the reference's callback does (tool:501-504)
        self.scheduled_ranges += 1
        # leading blocks of this range that the early hook has sent already
        end = param_offset + param_count
        for off, cnt in sorted(self._early):
            if off == param_offset and off + cnt <= end:
                param_offset += cnt
        param_count = end - param_offset
        if param_count > 0:
            self._append(ready_id, param_offset, param_count)
        # the range that closes backward waits for finish(), where it goes out whole
        last = self.whole_tail and self.expected_ranges is not None and self.scheduled_ranges == self.expected_ranges
        # with coalescing the newest entry is held back as well: the next range may still join it
        self._flush(max(self.lag, 1 if (last or self.coalesce) else 0))
        return 0

    def _append(self, ready_id: int, offset: int, count: int) -> None:
        """Backward announces the ranges of a layer group end to end (the residual blocks, last to first, then the hidden
        layer below them). Every launch costs a handshake with all peers, so ranges that touch are joined while the sum
        stays within one bucket; the joined range carries the id of its latest member."""
        if self.coalesce and self._pending:
            _, p_off, p_cnt = self._pending[-1]
            touches = offset + count == p_off or p_off + p_cnt == offset
            if touches and p_cnt + count <= max(1, self.bucket_params):
                self._pending[-1] = (ready_id, min(offset, p_off), p_cnt + count)
                return
        self._pending.append((ready_id, offset, count))

    def finish(self) -> None:
        self._flush(0, whole=self.whole_tail)
        if self.expected_ranges is not None and self.scheduled_ranges != self.expected_ranges:
            raise RuntimeError(f"gradient-ready ranges: got {self.scheduled_ranges}, expected {self.expected_ranges}")  # tool:817


class _CudaArrayView:
    def __init__(self, ptr: int, count: int):
        self.__cuda_array_interface__ = {"shape": (count,), "typestr": "<f4", "data": (ptr, False), "version": 3, "strides": None}


class PeerBackend:
    """The library's communicator (one per process). Owns the gradient buffer."""

    def __init__(self, device_index: int, world_size: int, global_rank: int, id_file: Optional[str], gradient_floats: int):
        self._lib = _lib.load()
        lib = self._lib
        lib.mgt_comm_create.argtypes = [C.c_int32, C.c_uint32, C.c_uint32, C.c_char_p, C.c_uint64, C.POINTER(C.c_void_p)]
        lib.mgt_comm_destroy.argtypes = [C.c_void_p]
        lib.mgt_comm_gradient_buffer.restype = C.c_void_p
        lib.mgt_comm_gradient_buffer.argtypes = [C.c_void_p]
        lib.mgt_comm_allreduce_average.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p]
        lib.mgt_comm_allreduce_average_adamw.argtypes = [C.c_void_p, C.c_uint64, C.c_uint64, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p]
        lib.mgt_comm_check.argtypes = [C.c_void_p, C.c_void_p, C.POINTER(C.c_int32)]
        lib.mgt_comm_launch_count.restype = C.c_uint64
        lib.mgt_comm_launch_count.argtypes = [C.c_void_p]
        lib.mgt_comm_set_wait_limit_ms.argtypes = [C.c_void_p, C.c_uint32]
        lib.mgt_comm_host_barrier.argtypes = [C.c_void_p, C.c_uint32]
        handle = C.c_void_p()
        st = lib.mgt_comm_create(device_index, world_size, global_rank, id_file.encode() if id_file else None, gradient_floats, C.byref(handle))
        if st != 0:
            raise MgtError(st, "mgt_comm_create")
        self.handle = handle
        self.world_size = world_size
        self.global_rank = global_rank
        self.gradient_floats = gradient_floats
        self.grad_ptr = int(lib.mgt_comm_gradient_buffer(handle))

    def gradient_tensor(self, device):
        import torch
        return torch.as_tensor(_CudaArrayView(self.grad_ptr, self.gradient_floats), device=device)

    def allreduce_average(self, offset: int, count: int, stream=None, seq: int = 0) -> int:
        class Cfg(C.Structure):
            _fields_ = [("world_size", C.c_uint32), ("global_rank", C.c_uint32), ("collective_seq", C.c_uint64), ("element_count", C.c_uint64)]
        cfg = Cfg(self.world_size, self.global_rank, seq, count)
        return int(self._lib.mgt_comm_allreduce_average(self.handle, C.byref(cfg), C.c_void_p(self.grad_ptr + 4 * offset), _stream(stream)))

    def allreduce_average_adamw(self, offset: int, count: int, adamw: AdamWKernelConfig, w, w_half, m, v, stream=None) -> int:
        cfg = adamw.c()
        return int(self._lib.mgt_comm_allreduce_average_adamw(self.handle, offset, count, C.byref(cfg), _ptr(w), _ptr(w_half), _ptr(m), _ptr(v), _stream(stream)))

    def check(self, stream=None):
        code = C.c_int32(0)
        st = int(self._lib.mgt_comm_check(self.handle, _stream(stream), C.byref(code)))
        return st, int(code.value)

    def set_wait_limit_ms(self, milliseconds: int) -> int:
        """How long an exchange kernel waits for a peer before it gives up (default 1000 ms)."""
        return int(self._lib.mgt_comm_set_wait_limit_ms(self.handle, milliseconds))

    def host_barrier(self, timeout_ms: int = 600000) -> int:
        """Host-side rendezvous of all ranks (files beside the id file); no GPU work."""
        return int(self._lib.mgt_comm_host_barrier(self.handle, timeout_ms))

    @property
    def launch_count(self) -> int:
        return int(self._lib.mgt_comm_launch_count(self.handle))

    def close(self):
        if getattr(self, "handle", None):
            self._lib.mgt_comm_destroy(self.handle)
            self.handle = None


class OverlappedGradientExchange:
    """Wires a back-end, a second CUDA stream and the scheduler to the engine's gradient-ready
    callback, the way the reference trainer's step loop does (tool:785-821). `extra_ranges`: announcements beyond the
    reference's 2 * blocks + 3 (1 with batch normalisation: the scale/shift vectors, announced last)."""

    def __init__(self, backend: PeerBackend, device, bucket_bytes: int = 4 << 20, residual_blocks: int = 16, fused_adamw: bool = True,
                 early_update_after_backward: bool = True, coalesce: bool = True, extra_ranges: int = 0):
        import torch
        self.torch = torch
        self.backend = backend
        self.device = device
        self.comm_stream = torch.cuda.Stream(device=device)
        self.fused = fused_adamw
        self.events = [torch.cuda.Event() for _ in range(2 * residual_blocks + 4)]
        self._ev = 0
        self.done_event = torch.cuda.Event()
        self.early_done_event = torch.cuda.Event()
        self.adamw: Optional[AdamWKernelConfig] = None
        self.state = None
        # The range from the early hook is exchanged while HBM-bound weight-gradient GEMMs run. Its AdamW update (30 bytes of
        # HBM traffic per parameter) would fight them for bandwidth, so by default only the NVLink exchange overlaps and the
        # update of that range follows once backward has ended.
        self.early_update_after_backward = early_update_after_backward and fused_adamw
        self._deferred = []
        self.scheduler = GradientRangeScheduler(self._launch, self._wait_for_producer, bucket_params=max(1, bucket_bytes // 4),
                                                expected_ranges=2 * residual_blocks + 3 + extra_ranges, lag=0, launch_early=self._launch_early,
                                                coalesce=coalesce)

    def _wait_for_producer(self):
        ev = self.events[self._ev % len(self.events)]
        self._ev += 1
        ev.record(self.torch.cuda.current_stream(self.device))
        self.comm_stream.wait_event(ev)

    def _launch(self, offset: int, count: int):
        w, w_half, m, v = self.state
        if self.fused:
            st = self.backend.allreduce_average_adamw(offset, count, self.adamw, w, w_half, m, v, stream=self.comm_stream)
        else:
            st = self.backend.allreduce_average(offset, count, stream=self.comm_stream)
        if st != 0:
            raise MgtError(st, "gradient exchange")

    def _launch_early(self, offset: int, count: int):
        if not self.early_update_after_backward:
            return self._launch(offset, count)
        st = self.backend.allreduce_average(offset, count, stream=self.comm_stream)
        if st != 0:
            raise MgtError(st, "gradient exchange")
        self._deferred.append((offset, count))
        self.early_done_event.record(self.comm_stream)

    def begin_step(self, adamw: AdamWKernelConfig, w, w_half, m, v):
        self.adamw = adamw
        self.state = (w, w_half, m, v)
        self._deferred = []
        self.scheduler.begin_step()

    def callback(self, user, ready_id, offset, count, stream) -> int:
        return self.scheduler.on_ready(int(ready_id), int(offset), int(count))

    def early_callback(self, user, ready_id, offset, count, stream) -> int:
        return self.scheduler.on_early(int(ready_id), int(offset), int(count))

    def finish_step(self):
        self.scheduler.finish()
        self.done_event.record(self.comm_stream)
        compute = self.torch.cuda.current_stream(self.device)
        # the deferred update only needs the early range's own exchange: it runs beside the tail of the exchange
        compute.wait_event(self.early_done_event if self._deferred else self.done_event)
        if self._deferred:
            from .api import launch_adamw_kernel_with_half_mirror
            w, w_half, m, v = self.state
            grad = self.backend.gradient_tensor(self.device)
            for offset, count in self._deferred:
                cfg = AdamWKernelConfig(count, self.adamw.step, self.adamw.learning_rate, self.adamw.beta1, self.adamw.beta2, self.adamw.eps,
                                        self.adamw.weight_decay)
                hi = offset + count
                st = launch_adamw_kernel_with_half_mirror(cfg, w[offset:hi], w_half[offset:hi], grad[offset:hi], m[offset:hi], v[offset:hi])
                if st != 0:
                    raise MgtError(st, "AdamW")
            compute.wait_event(self.done_event)  # tool:820-821


class NcclBackend:
    """The reference's scheme, for comparison only: in-place ncclAllReduce(sum) of each chunk followed
    by a scale kernel, AdamW after all communication (allreduce_nccl.cu:130-148, tool:816-835)."""

    def __init__(self, grad, world_size: int):
        import torch.distributed as dist
        self.dist = dist
        self.grad = grad
        self.world_size = world_size

    def allreduce_average(self, offset: int, count: int, stream=None, seq: int = 0) -> int:
        import torch
        view = self.grad[offset:offset + count]
        with torch.cuda.stream(stream) if stream is not None else _NullCtx():
            self.dist.all_reduce(view, op=self.dist.ReduceOp.SUM)
            if self.world_size > 1:
                view.mul_(1.0 / self.world_size)
        return 0


class _NullCtx:
    def __enter__(self):
        return self

    def __exit__(self, *a):
        return False


def default_id_file() -> str:
    port = os.environ.get("MASTER_PORT", "0")
    return os.path.join(os.environ.get("TMPDIR", "/tmp"), f"mgt_b200_{os.getuid()}_{port}.id")
