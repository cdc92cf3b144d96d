"""The b200 execution adapter: the FFI boundary of a compiled program.

Call convention of the reference's TPU branch (tilelang/jit/adapter/cython/adapter.py:214-246):
the caller passes EVERY parameter, inputs and outputs; outputs named by `out_idx` are overwritten
in place; the call returns the native `int` status.  The reference copies every tensor through
host byte buffers on each call and blocks until the device has finished.

Here tensors that already live on the GPU are used as they are, on the caller's current stream.
Host tensors are staged by the adapter itself:

  * three streams per adapter (copy-in, compute, copy-out) and two sets of device buffers, so the
    host->device copy of call i+1 and the device->host copy of call i-1 overlap the kernels of
    call i (PCIe is full duplex) - the overlap belongs to the product, not to a benchmark loop;
  * pinned host tensors make the call asynchronous, like `cudaMemcpyAsync`: it returns once the
    work is queued, inputs must stay untouched and outputs are complete after
    `adapter.synchronize()` (or `torch.cuda.synchronize()`).  A later call of ANY b200 adapter that
    reads a host tensor which an earlier call still writes waits for that copy on the device;
  * if any host tensor of a call is pageable the call blocks until its results are on the host,
    as the reference does.
"""
from __future__ import annotations

import threading
from typing import Callable, Dict, List, Tuple

import torch

from ...engine.param import CompiledArtifact, KernelParam
from .base import BaseKernelAdapter

# host allocations that an adapter's copy-out stream is still writing: data_ptr -> event
_pending_host_writes: Dict[int, torch.cuda.Event] = {}
_pending_lock = threading.Lock()


def _wait_for_pending_write(stream: torch.cuda.Stream, t: torch.Tensor) -> None:
    with _pending_lock:
        ev = _pending_host_writes.get(t.untyped_storage().data_ptr())
        if ev is not None and ev.query():
            del _pending_host_writes[t.untyped_storage().data_ptr()]
            ev = None
    if ev is not None:
        stream.wait_event(ev)


class _Staging:
    """Streams, events and two sets of device buffers for the host-tensor path of one adapter on one device."""

    def __init__(self, device: torch.device, params: List[KernelParam]):
        self.device = device
        self.s_in, self.s_cmp, self.s_out = (torch.cuda.Stream(device) for _ in range(3))
        self.sets: List[List[torch.Tensor | None]] = [[None] * len(params) for _ in range(2)]
        self.ev_in = [torch.cuda.Event() for _ in range(2)]
        self.ev_cmp = [torch.cuda.Event() for _ in range(2)]
        self.ev_out = [torch.cuda.Event() for _ in range(2)]
        self.calls = 0

    def buffer(self, which: int, i: int, like: torch.Tensor) -> torch.Tensor:
        buf = self.sets[which][i]
        if buf is None or buf.shape != like.shape or buf.dtype != like.dtype:
            buf = self.sets[which][i] = torch.empty(like.shape, dtype=like.dtype, device=self.device)
        return buf

    def streams(self) -> Tuple[torch.cuda.Stream, ...]:
        return self.s_in, self.s_cmp, self.s_out


class B200KernelAdapter(BaseKernelAdapter):

    def __init__(self, artifact: CompiledArtifact, params: List[KernelParam], result_idx, verbose: bool = False):
        self.bound = artifact.rt_mod
        self.verbose = verbose
        self._staging: Dict[int, _Staging] = {}
        super().__init__(artifact, params, result_idx)

    def _check(self, args):
        if len(args) != len(self.params):
            raise ValueError(f"Expected {len(self.params)} inputs, got {len(args)} with "
                             f"{len(self.result_idx)} of them outputs (every parameter is passed)")
        for i, (a, p) in enumerate(zip(args, self.params)):
            if not isinstance(a, torch.Tensor):
                raise ValueError(f"argument {i} is not a torch.Tensor")
            want = p.dtype
            same_bits = {torch.int32, torch.uint32}
            if a.dtype != want and not (a.dtype in same_bits and want in same_bits):
                raise ValueError(f"argument {i}: dtype {a.dtype} does not match the program's {want}")
            if list(a.shape) != list(p.shape):
                raise ValueError(f"argument {i}: shape {list(a.shape)} does not match the program's {list(p.shape)}")

    # ------------------------------------------------------------------ host-tensor path
    def synchronize(self) -> None:
        """Block until every queued host-tensor call of this adapter has delivered its results."""
        for st in self._staging.values():
            for s in st.streams():
                s.synchronize()

    def join(self, stream: torch.cuda.Stream | None = None) -> None:
        """Make `stream` (default: the current stream) wait for this adapter's queued host-tensor calls."""
        stream = stream or torch.cuda.current_stream()
        for st in self._staging.values():
            for s in st.streams():
                stream.wait_stream(s)

    def _run_staged(self, args) -> int:
        dev_index = torch.cuda.current_device()
        st = self._staging.get(dev_index)
        if st is None:
            st = self._staging[dev_index] = _Staging(torch.device("cuda", dev_index), self.params)
        b = st.calls & 1
        again = st.calls >= 2                     # this buffer set has been used by call - 2
        st.calls += 1
        result_idx = self.result_idx
        host = [not a.is_cuda for a in args]
        blocking = any(h and not a.is_pinned() for a, h in zip(args, host))
        # a program that writes every element of its outputs does not need their old contents on the device
        skip_upload = set(result_idx) if getattr(self.bound, "full_outputs", False) else set()
        caller = torch.cuda.current_stream()
        mixed = not all(host)
        staged: List[torch.Tensor] = []
        with torch.cuda.stream(st.s_in):
            if mixed:
                st.s_in.wait_stream(caller)       # device tensors of the call were produced on the caller's stream
            if again:
                st.s_in.wait_event(st.ev_cmp[b])  # the call that last read this set has computed
            for i, a in enumerate(args):
                if not host[i]:
                    staged.append(a if a.is_contiguous() else a.contiguous())
                    continue
                src = a if a.is_contiguous() else a.contiguous()
                buf = st.buffer(b, i, src)
                if i not in skip_upload:          # (other outputs go up too: the program may read or keep parts of them)
                    _wait_for_pending_write(st.s_in, a)
                    buf.copy_(src, non_blocking=True)
                staged.append(buf)
            st.ev_in[b].record(st.s_in)
        with torch.cuda.stream(st.s_cmp):
            st.s_cmp.wait_event(st.ev_in[b])
            if again:
                st.s_cmp.wait_event(st.ev_out[b])  # its previous results have left for the host
            status = self.bound.run(*staged)
            st.ev_cmp[b].record(st.s_cmp)
        with torch.cuda.stream(st.s_out):
            st.s_out.wait_event(st.ev_cmp[b])
            for i in result_idx:
                if staged[i] is args[i]:
                    continue
                if host[i] and args[i].is_contiguous():
                    args[i].copy_(staged[i], non_blocking=True)
                else:
                    args[i].copy_(staged[i])
            ev = st.ev_out[b] = torch.cuda.Event()
            ev.record(st.s_out)
        if mixed:
            caller.wait_event(st.ev_cmp[b])       # device outputs are ordered into the caller's stream
        with _pending_lock:
            for i in result_idx:
                if host[i]:
                    _pending_host_writes[args[i].untyped_storage().data_ptr()] = ev
        if blocking:
            st.s_out.synchronize()                # pageable host memory: results complete on return
        return int(status)

    def _convert_torch_func(self) -> Callable:
        bound = self.bound
        result_idx = self.result_idx

        def forward(*args):
            self._check(args)
            if any(not a.is_cuda for a in args):
                return self._run_staged(args)
            staged = [a if a.is_contiguous() else a.contiguous() for a in args]
            status = bound.run(*staged)
            for i in result_idx:
                if staged[i] is not args[i]:
                    args[i].copy_(staged[i], non_blocking=True)
            return int(status)

        return forward
