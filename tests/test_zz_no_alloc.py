"""The allocation-free MLA decode entry point against the regular one, through the C ABI.

Collected last on purpose: a run that stops at the first failure has then already run every
other test.  It also has to pass alone in a fresh process (its first call does the one-time
address look-up of the built-in scratch array)."""
import pytest
import torch

from tilelang import _native as N
from tilelang import ops, workloads

pytestmark = pytest.mark.gpu


def test_noalloc_matches_workspace_entry_point_twice(cuda_device):
    lib = N.load()
    ops._prepare(torch.zeros(1, device=cuda_device))          # tl_b200_init for this device
    w = workloads.mla_fp8_paged(batch=5, heads=128, min_len=40, max_len=900, seed=21)
    d = {k: (v.to(cuda_device) if isinstance(v, torch.Tensor) else v) for k, v in w.items()}
    q = d["q"]
    ref = torch.zeros(5, 128, 512, dtype=q.dtype, device=cuda_device)
    ops.mla_decode_paged(q, d["kv_cache"], d["kv_scale"], d["block_table"], d["cache_seqlens"], ref,
                         softmax_scale=w["softmax_scale"])
    torch.cuda.synchronize()
    stream = torch.cuda.current_stream().cuda_stream
    for call in range(2):
        if call == 1:                       # second call: other lengths, same shared scratch
            d["cache_seqlens"] = torch.flip(d["cache_seqlens"], dims=[0]).contiguous()
            # (table slots past a sequence's own pages hold 0, a valid page: both entry points read the same bytes)
            ops.mla_decode_paged(q, d["kv_cache"], d["kv_scale"], d["block_table"], d["cache_seqlens"], ref,
                                 softmax_scale=w["softmax_scale"])
        out = torch.full_like(ref, float("nan"))
        rc = lib.tl_b200_mla_decode_paged_noalloc(
            q.data_ptr(), d["kv_cache"].data_ptr(), d["kv_scale"].data_ptr(), d["block_table"].data_ptr(),
            d["cache_seqlens"].data_ptr(), out.data_ptr(), 5, 128, 64, d["block_table"].shape[1],
            d["kv_cache"].shape[0], float(w["softmax_scale"]), N.TL_BF16, stream)
        assert rc == 0, N.last_error()
        torch.cuda.synchronize()
        assert torch.isfinite(out.float()).all()
        assert torch.allclose(out.float(), ref.float(), atol=2e-2, rtol=2e-2)
        # (the workspace entry point may split short batches along the sequence; this one never does)
        assert (out.float() - ref.float()).norm() <= 5e-3 * ref.float().norm()


def test_noalloc_rejects_oversized_batch(cuda_device):
    lib = N.load()
    rc = lib.tl_b200_mla_decode_paged_noalloc(None, None, None, None, None, None, 5000, 128, 64, 1, 1, 1.0,
                                              N.TL_BF16, None)
    assert rc == -1 and "4096" in N.last_error()
