"""GPU: the allocation-free block-score entry point (psa_block_scores_static).

It exists for hosts that must not allocate device memory when they call in - a server that handed all GPU memory to
its own pools at start-up, a plug-in that is only given input/output buffers.  Its scratch is a fixed device array
inside the library, so the checks here are: same scores as psa_block_scores (same kernels, so bit-equal), on two
calls in a row with different inputs (the array keeps the first call's contents), and a clear refusal when a call
needs more scratch than the array holds.  This file is collected last on purpose.
"""
import ctypes as C

import pytest
import torch

import cases

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def _call_static(lib, q, k, iq, ik, bm, bn):
    from psa_b200 import ops
    B, H, S, D = q.shape
    po = torch.empty((B, H, -(-S // bm), -(-S // bn)), dtype=q.dtype, device=q.device)
    stream = C.c_void_p(torch.cuda.current_stream(q.device).cuda_stream)
    rc = lib.psa_block_scores_static(q.data_ptr(), k.data_ptr(), iq.data_ptr(), ik.data_ptr(), po.data_ptr(), B * H, S, S, D,
                                     bm, bn, ops._DT[q.dtype], 0, stream)
    return rc, po


def test_static_scratch_matches_the_allocating_entry_point_twice():
    from psa_b200 import _lib, ops
    lib = _lib.lib
    assert lib.psa_block_scores_static_capacity() == 64 << 20
    # (seed, S, D, H, bm, bn, dtype): the second call is smaller and of another dtype, so stale scratch would show
    for seed, S, D, H, bm, bn, dt in ((31, 3000, 128, 2, 128, 64, torch.bfloat16), (57, 1111, 64, 3, 128, 32, torch.float32)):
        q, k, _ = (x.to(DEV) for x in cases.qkv(seed, 1, H, S, D, dt))
        iq = cases.sample_idx(seed + 3, 1, H, bm, bm // 4).to(DEV).to(torch.int32).contiguous()
        ik = cases.sample_idx(seed + 4, 1, H, bn, bn // 4).to(DEV).to(torch.int32).contiguous()
        rc, po = _call_static(lib, q, k, iq, ik, bm, bn)
        assert rc == 0, _lib.last_error()
        ref = ops.block_scores(q, k, iq, ik, bm, bn)
        torch.cuda.synchronize()
        assert torch.equal(po, ref)
        # the same call again, output buffer already there: the device's free memory must not move while it runs
        # (the driver's figure, so an allocation by any route would show)
        torch.cuda.synchronize()
        free_before, _ = torch.cuda.mem_get_info()
        stream = C.c_void_p(torch.cuda.current_stream(q.device).cuda_stream)
        rc = lib.psa_block_scores_static(q.data_ptr(), k.data_ptr(), iq.data_ptr(), ik.data_ptr(), po.data_ptr(), H, S, S, D,
                                         bm, bn, ops._DT[q.dtype], 0, stream)
        torch.cuda.synchronize()
        free_after, _ = torch.cuda.mem_get_info()
        assert rc == 0 and free_after == free_before, (free_before, free_after)
        assert torch.equal(po, ref)


def test_static_scratch_capacity_counts_the_calls_own_head_dim():
    """44 heads x 8192 tokens in bf16 would need 66.3 MiB of scratch at head_dim 128 (what the public size query assumes)
    but only ~44 MiB at head_dim 64: the allocation-free entry point must take it."""
    from psa_b200 import _lib, ops
    lib = _lib.lib
    H, S, D, bm, bn = 44, 8192, 64, 128, 64
    assert lib.psa_block_scores_scratch_bytes(H, S, S, bm, bn, 2) > lib.psa_block_scores_static_capacity()
    g = torch.Generator(device=DEV).manual_seed(5)
    q = torch.randn((1, H, S, D), device=DEV, dtype=torch.bfloat16, generator=g)
    k = torch.randn((1, H, S, D), device=DEV, dtype=torch.bfloat16, generator=g)
    iq = cases.sample_idx(3, 1, H, bm, bm // 4).to(DEV).to(torch.int32).contiguous()
    ik = cases.sample_idx(4, 1, H, bn, bn // 4).to(DEV).to(torch.int32).contiguous()
    rc, po = _call_static(lib, q, k, iq, ik, bm, bn)
    assert rc == 0, _lib.last_error()
    torch.cuda.synchronize()
    assert torch.equal(po, ops.block_scores(q, k, iq, ik, bm, bn))


def test_static_scratch_rejects_oversized_calls():
    from psa_b200 import _lib
    lib = _lib.lib
    H, S = 16, 32768                      # needs ~134 MB of scratch in bf16: beyond the 64 MiB array
    need = lib.psa_block_scores_scratch_bytes(H, S, S, 128, 64, 2)
    assert need > lib.psa_block_scores_static_capacity()
    x = torch.zeros(16, dtype=torch.bfloat16, device=DEV)     # never dereferenced: the size check comes first
    i = torch.zeros(64, dtype=torch.int32, device=DEV)
    rc = lib.psa_block_scores_static(x.data_ptr(), x.data_ptr(), i.data_ptr(), i.data_ptr(), x.data_ptr(), H, S, S, 128, 128,
                                     64, 2, 0, None)
    assert rc == _lib.PSA_ERR_ARG
    msg = _lib.last_error()
    assert "scratch" in msg and str(64 << 20) in msg
