"""`tilelang.compile(...)` end to end on the GPU: the reference's call convention (all
parameters passed, outputs in place, int status) with host tensors and with device tensors."""
import pytest
import torch

import oracle.ops as O
import tilelang
import tilelang.language as T
from test_frontend import (matmul_program, mlp_program, rms_norm_program, rms_norm_program_f32, swiglu_program_f32,
                           topk_program)

pytestmark = pytest.mark.gpu


def gen(seed):
    return torch.Generator(device="cpu").manual_seed(seed)


def test_rmsnorm_program_host_tensors_like_the_demo(cuda_device):
    kernel = tilelang.compile(rms_norm_program(128, 128, 32), out_idx=-1, target="b200")
    a = torch.randn(128, 128, generator=gen(1)).bfloat16()
    b = torch.zeros(128, 128).bfloat16()
    res = kernel(a, b)                      # host tensors, result written into b
    assert res == 0
    ref = O.rmsnorm(a, eps=1e-12)
    assert torch.allclose(b.float(), ref.float(), atol=5e-2, rtol=5e-2)      # the demo's tolerance
    assert torch.allclose(b.float(), ref.float(), atol=2e-2, rtol=2e-2)


def test_rmsnorm_program_device_tensors_and_pinned_host(cuda_device):
    kernel = tilelang.compile(rms_norm_program(256, 512, 32, eps=1e-6), out_idx=-1, target="b200")
    a = torch.randn(256, 512, generator=gen(2)).bfloat16()
    ref = O.rmsnorm(a, eps=1e-6)
    bd = torch.zeros(256, 512, dtype=torch.bfloat16, device=cuda_device)
    assert kernel(a.to(cuda_device), bd) == 0
    assert torch.allclose(bd.cpu().float(), ref.float(), atol=2e-2, rtol=2e-2)
    bp = torch.zeros(256, 512, dtype=torch.bfloat16).pin_memory()
    assert kernel(a.pin_memory(), bp) == 0
    assert torch.equal(bp, bd.cpu())


@pytest.mark.parametrize("trans_b,bk", [(False, 32), (True, 64), (True, 32)])
def test_matmul_program(cuda_device, trans_b, bk):
    kernel = tilelang.compile(matmul_program(64, 64, 64, 32, 32, bk, trans_b=trans_b), out_idx=-1, target="b200")
    g = gen(3)
    a = torch.randn(64, 64, generator=g).half()
    b = torch.randn(64, 64, generator=g).half()
    c = torch.zeros(64, 64).half()
    assert kernel(a, b, c) == 0
    if trans_b and bk < 64:
        # `C = A B^T` overwrites C on every K iteration in the reference's generated code
        # (src/target/codegen_ppl.cc:1276-1279): what is left is the product over the last K tile
        assert kernel.adapter.bound.program == "generic"
        ref = O.matmul(a[:, -bk:].contiguous(), b[:, -bk:].contiguous(), transpose_b=True)
    else:
        assert kernel.adapter.bound.program == "matmul"
        ref = O.matmul(a, b, transpose_b=trans_b)
    assert torch.allclose(c, ref, atol=1e-2, rtol=1e-2)                      # the demo's tolerance


def test_matmul_anchor_program_1024(cuda_device):
    kernel = tilelang.compile(matmul_program(1024, 1024, 1024, 128, 128, 64), out_idx=-1, target="b200")
    g = gen(0)
    a = torch.randn(1024, 1024, generator=g).half()
    b = torch.randn(1024, 1024, generator=g).half()
    c = torch.zeros(1024, 1024).half()
    assert kernel(a, b, c) == 0
    ref = O.matmul(a, b)
    assert ((c.float() - ref.float()).abs() <= 2e-2 * 32 + 2e-2 * ref.float().abs()).all()


def test_topk_program_two_outputs(cuda_device):
    kernel = tilelang.compile(topk_program(1024, 8), out_idx=[1, 2], target="b200")
    src = torch.randn(1024, generator=gen(4))
    out = torch.zeros(1024)
    idx = torch.zeros(1024, dtype=torch.int32)
    assert kernel(src, out, idx) == 0
    rv, ri = torch.topk(src, 8, largest=True, sorted=True)
    assert torch.equal(idx[:8].long(), ri) and torch.equal(out[:8], rv)
    assert torch.allclose(src[idx[:8].long()], rv, atol=1e-5)               # the demo's look-up check


def test_gather_program_uint32_index(cuda_device):
    @T.prim_func
    def main_kernel_inner(Param: T.Tensor((128, 64), "float32"), Index: T.Tensor((8, 1), "uint32"),
                          Output: T.Tensor((8, 64), "float32")):
        with T.Kernel(1, 1, is_cpu=True) as (bx, by):
            T.ppl_gather(Output, Param, Index, 128)

    kernel = tilelang.compile(main_kernel_inner, out_idx=-1, target="b200")
    g = gen(5)
    param = torch.randn(128, 64, generator=g)
    idx_vals = torch.randint(0, 128, (8, 1), generator=g, dtype=torch.int32)
    out = torch.zeros(8, 64)
    assert kernel(param, idx_vals.view(torch.uint32), out) == 0
    assert torch.equal(out, param[idx_vals.view(-1)])


def test_profiler_consistency_and_bench(cuda_device):
    kernel = tilelang.compile(rms_norm_program(512, 1024, 32), out_idx=-1, target="b200")
    prof = kernel.get_profiler()
    prof.assert_consistent(repeat=3)
    assert prof.do_bench(rep=3) > 0


def test_mlp_program(cuda_device):
    """Output first in the parameter list, as in the reference's MLP program."""
    rows, hidden, inter = 128, 256, 512
    kernel = tilelang.compile(mlp_program(rows, hidden, inter, 64), out_idx=0, target="b200")
    g = gen(8)
    x = torch.randn(rows, hidden, generator=g).bfloat16()
    wg = (torch.randn(inter, hidden, generator=g) / hidden ** 0.5).bfloat16()
    wu = (torch.randn(inter, hidden, generator=g) / hidden ** 0.5).bfloat16()
    wd = (torch.randn(hidden, inter, generator=g) / inter ** 0.5).bfloat16()
    y = torch.zeros(rows, hidden).bfloat16()
    assert kernel(y, x, wg, wu, wd) == 0
    assert torch.allclose(y.float(), O.mlp(x, wg, wu, wd).float(), atol=2e-2, rtol=2e-2)


def test_float32_program_forms(cuda_device):
    g = gen(9)
    x = torch.randn(64, 128, generator=g)
    y = torch.zeros(64, 128)
    assert tilelang.compile(rms_norm_program_f32(64, 128, 32, eps=1e-6), out_idx=-1, target="b200")(x, y) == 0
    assert torch.allclose(y, O.rmsnorm(x, eps=1e-6), atol=1e-5, rtol=1e-5)
    gate, up = torch.randn(64, 128, generator=g), torch.randn(64, 128, generator=g)
    out = torch.zeros(64, 128)
    assert tilelang.compile(swiglu_program_f32(64, 128, 32, 64), out_idx=0, target="b200")(out, gate, up) == 0
    assert torch.allclose(out, O.swiglu(gate, up), atol=1e-5, rtol=1e-5)
