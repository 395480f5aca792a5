"""GPU test of ar_flash_attn_fwd_noalloc, the forward entry point for callers that cannot
allocate device memory at call time (code running where cudaMalloc is forbidden or would stall
the device: a serving loop with a fixed memory budget, a section under an allocator lock).

It must give what ar_flash_attn_fwd gives.  Two calls in a row with different inputs check that
the shared, never-cleared scratch array inside the library carries nothing over from one call
to the next.  The file name sorts last so that a run stopping at the first failure has already
run every other test."""
import ctypes

import numpy as np
import pytest

import autoresearch_b200 as ab
from autoresearch_b200 import _lib
from oracle import oracle as orc
from tests.parity_util import MAX_ABS_TOL, REL_L2_TOL

pytestmark = pytest.mark.gpu


def _call(fn, o, lse, q, k, v, B, T, H, W):
    import torch
    st = fn(o.data_ptr(), lse.data_ptr(), q.data_ptr(), k.data_ptr(), v.data_ptr(), B, T, H, 128, W,
            torch.cuda.current_stream().cuda_stream)
    assert st == _lib.AR_OK, _lib.lib().ar_last_error()


def test_noalloc_forward_matches_allocating_entry_point_twice(cuda_device):
    import torch
    L = ab.lib()
    L.ar_noalloc_status()      # start clean: reads and clears whatever an earlier test left behind
    for call, (B, T, H, W, seed) in enumerate([(2, 384, 4, 100, 21), (1, 1000, 3, 0, 22)]):
        assert B * T * H <= 16384
        g = torch.Generator(device="cuda").manual_seed(seed)
        q, k, v = (torch.randn(B, T, H, 128, device="cuda", generator=g) for _ in range(3))
        o_ref, o_new = torch.empty_like(q), torch.full_like(q, float("nan"))
        lse_ref = torch.empty(B, T, H, device="cuda")
        lse_new = torch.full((B, T, H), float("nan"), device="cuda")
        _call(L.ar_flash_attn_fwd, o_ref, lse_ref, q, k, v, B, T, H, W)
        torch.cuda.synchronize()
        # The property the entry point exists for: the call must not take device memory.  Free
        # bytes are read straight from the driver before and after (the first call on a device
        # only looks a symbol address up, which allocates nothing either).
        free_before = torch.cuda.mem_get_info()[0]
        _call(L.ar_flash_attn_fwd_noalloc, o_new, lse_new, q, k, v, B, T, H, W)
        torch.cuda.synchronize()
        assert torch.cuda.mem_get_info()[0] == free_before, (call, "device memory was allocated")
        assert L.ar_noalloc_status() == _lib.AR_OK, L.ar_last_error()
        assert torch.cuda.mem_get_info()[0] == free_before, (call, "status read allocated device memory")
        for name, got, want in (("o", o_new, o_ref), ("lse", lse_new, lse_ref)):
            max_abs, rel = orc.parity(got.cpu().numpy(), want.cpu().numpy())
            assert max_abs <= MAX_ABS_TOL and rel <= REL_L2_TOL, (call, name, max_abs, rel)
            # same kernels on the same staged operands: in practice the results are identical
            assert torch.equal(got, want), (call, name)
        # and against the CPU oracle on the operands the kernels see (q, k, v rounded to bf16)
        host = [orc.to_bf16_rne(t.cpu().numpy()) for t in (q, k, v)]
        want = orc.attention_path(*host, None, W)
        for name, got in (("o", o_new), ("lse", lse_new)):
            max_abs, rel = orc.parity(got.cpu().numpy(), want[name])
            assert max_abs <= MAX_ABS_TOL and rel <= REL_L2_TOL, (call, name, "oracle", max_abs, rel)


def test_noalloc_rejects_sizes_beyond_its_fixed_scratch(cuda_device):
    import torch
    L = ab.lib()
    B, T, H = 1, 16384 // 4 + 1, 4          # one row more than the limit
    x = torch.zeros(16, device="cuda")      # never touched: the size check comes first
    st = L.ar_flash_attn_fwd_noalloc(x.data_ptr(), x.data_ptr(), x.data_ptr(), x.data_ptr(), x.data_ptr(),
                                     B, T, H, 128, 0, None)
    assert st == _lib.AR_ERR_WORKSPACE
    assert b"AR_NOALLOC_MAX_ROWS" in L.ar_last_error()
