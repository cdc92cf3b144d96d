"""The b200 execution adapter: the FFI boundary of a compiled program.

Call convention of the reference's TPU branch (tilelang/jit/adapter/cython/adapter.py:214-246):
the caller passes EVERY parameter, inputs and outputs; outputs named by `out_idx` are overwritten
in place; the call returns the native `int` status.  The reference copies every tensor through
host byte buffers on each call.  Here tensors that already live on the GPU are used as they are;
host tensors are staged through device buffers (inputs up, `out_idx` tensors back) on the current
stream, which is the path the end-to-end benchmark times.
"""
from __future__ import annotations

from typing import Callable, List

import torch

from ...engine.param import CompiledArtifact, KernelParam
from .base import BaseKernelAdapter


class B200KernelAdapter(BaseKernelAdapter):

    def __init__(self, artifact: CompiledArtifact, params: List[KernelParam], result_idx, verbose: bool = False):
        self.bound = artifact.rt_mod
        self.verbose = verbose
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

    def _convert_torch_func(self) -> Callable:
        bound = self.bound
        result_idx = self.result_idx

        def forward(*args):
            self._check(args)
            dev = torch.device("cuda", torch.cuda.current_device())
            staged = []
            for a in args:
                if a.is_cuda:
                    staged.append(a if a.is_contiguous() else a.contiguous())
                else:
                    staged.append(a.contiguous().to(dev, non_blocking=True))
            status = bound.run(*staged)
            for i in result_idx:
                if staged[i] is not args[i]:
                    args[i].copy_(staged[i], non_blocking=args[i].is_pinned() if not args[i].is_cuda else True)
            if any(not args[i].is_cuda for i in result_idx):
                torch.cuda.current_stream().synchronize()      # host results are complete on return
            return int(status)

        return forward
