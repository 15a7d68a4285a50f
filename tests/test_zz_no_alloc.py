"""The entry point for callers that cannot allocate device memory (an inference plugin that is handed only
its buffers, a server with a frozen memory pool): ``vig_bigla_fwd_noalloc`` keeps the scan's scratch in a
fixed array inside the library.  It runs the same kernels as ``vig_bigla_fwd``, so its output must equal
that entry point's, also on a second call that reuses the array with other data and another shape.
This file is collected last on purpose: a run that stops at the first failure has then run everything else.
"""
import pytest
import torch

import oracle

pytestmark = pytest.mark.gpu


def _inputs(B, H, L, dk, dtype, seed):
    return [t.to("cuda", dtype) for t in oracle.make_bigla_inputs(B, H, L, dk, 64, seed=seed)]


def _setup_call(status):
    """The entry point's first call on a device looks up the scratch array's address; with CUDA's lazy module loading
    that is also when the runtime places the library's device image, the 16 MiB array included, in device memory.
    Callers make this call at start-up, before their memory is frozen; the tests make it before they measure."""
    from vig_b200 import ops
    q, k, v, gf, gb = _inputs(1, 1, 8, 64, torch.bfloat16, seed=0)
    ops.bi_gla_noalloc(q, k, v, gf, gb, torch.empty_like(v), status=status)
    torch.cuda.synchronize()


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
def test_noalloc_matches_workspace_entry_point_twice_in_a_row(dtype):
    import vig_b200
    from vig_b200 import ops
    # both shapes span several segments, so the scratch array is really used; the second call is larger
    status = ops.status_word().tensor                            # the error word exists before the calls under test
    _setup_call(status)
    for call, (B, H, L, dk) in enumerate([(2, 3, 1300, 64), (3, 2, 2100, 32)]):
        q, k, v, gf, gb = _inputs(B, H, L, dk, dtype, seed=40 + call)
        expected = vig_b200.bi_gla(q, k, v, gf, gb, out_scale=0.5)
        out = torch.full_like(expected, float("nan"))
        torch.cuda.synchronize()
        before, free_before = torch.cuda.memory_allocated(), torch.cuda.mem_get_info()[0]
        ops.bi_gla_noalloc(q, k, v, gf, gb, out, out_scale=0.5, status=status)
        torch.cuda.synchronize()
        assert torch.cuda.memory_allocated() == before           # nothing came from torch's allocator ...
        assert torch.cuda.mem_get_info()[0] == free_before       # ... and nothing from cudaMalloc inside the library
        ops.check_status()
        # same arithmetic; for 2048..8192 tokens the workspace entry point runs the tensor-core path as one launch and
        # this one as three, which differ by bf16 rounding of the cross-segment term
        tol = 1e-5 if dtype == torch.float32 else 1e-2
        diff = float((out.float() - expected.float()).abs().max() / expected.float().abs().max())
        assert diff < tol, f"call {call}: relative difference {diff}"
        ref = oracle.naive_bi_gla(*[t.float().cpu() for t in (q, k, v, gf, gb)], out_scale=0.5)
        err = float((out.float().cpu() - ref).abs().max() / ref.abs().max())
        assert err < (1e-4 if dtype == torch.float32 else 2e-2)


def test_noalloc_rejects_problems_beyond_the_fixed_scratch():
    from vig_b200 import _lib, ops
    L_ = _lib.lib()
    limit = L_.vig_bigla_noalloc_scratch_bytes()
    B, H, L, dk = 64, 3, 4096, 64
    assert L_.vig_bigla_workspace_bytes(B, H, L, dk, 64, 1, 0) > limit
    # sizes are checked before any pointer is touched, so tiny placeholder tensors are enough
    x = torch.zeros(1, device="cuda", dtype=torch.bfloat16)
    args = [_lib.ptr(x)] * 6 + [B, H, L, dk, 64, 1] + [None] * 6 + [-1.0, 1.0, 0.0, float("nan"), 0, None, None]
    st = L_.vig_bigla_fwd_noalloc(*args)
    assert st == -8
    assert b"scratch" in L_.vig_strerror(st)
    with pytest.raises(RuntimeError, match="scratch"):
        _lib.check(st, "vig_bigla_fwd_noalloc")


def test_noalloc_limit_is_what_the_call_uses():
    """The scratch limit counts what the kernel family that runs really uses: a single 256-token segment on the
    tensor-core path uses none, however large the batch; fp32 (SIMT path, 64-token chunks) reaches the limit at a
    quarter of the tokens the tensor-core path does."""
    import vig_b200
    from vig_b200 import _lib, ops
    status = ops.status_word().tensor
    # ViG-T at 224x224 with a large batch: one segment per sequence, no scratch, accepted
    q, k, v, gf, gb = _inputs(256, 3, 196, 64, torch.bfloat16, seed=50)
    out = torch.empty_like(v)
    ops.bi_gla_noalloc(q, k, v, gf, gb, out, out_scale=0.5, status=status)
    expected = vig_b200.bi_gla(q, k, v, gf, gb, out_scale=0.5)
    torch.cuda.synchronize()
    ops.check_status()
    assert float((out.float() - expected.float()).abs().max()) == 0.0
    # B*H*ceil(L/256) = 480 <= 504 < B*H*ceil(L/64) = 1920: bf16 runs, the same shape in fp32 is over the SIMT limit
    q, k, v, gf, gb = _inputs(40, 3, 1024, 64, torch.bfloat16, seed=51)
    out = torch.empty_like(v)
    ops.bi_gla_noalloc(q, k, v, gf, gb, out, status=status)
    expected = vig_b200.bi_gla(q, k, v, gf, gb, impl=_lib.IMPL_TC_SPLIT)
    torch.cuda.synchronize()
    ops.check_status()
    assert float((out.float() - expected.float()).abs().max()) == 0.0
    f32 = [t.float() for t in (q, k, v, gf, gb)]
    with pytest.raises(RuntimeError, match="scratch"):
        ops.bi_gla_noalloc(*f32, torch.empty_like(f32[2]), status=status)
