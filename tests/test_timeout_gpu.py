"""GPU test of the time-out path: what the library does after a bounded device-side wait ran out.

Nothing here faults, traps or hangs the GPU: ar_selftest_wait_timeout launches one warp that waits
about a millisecond on a barrier nothing arrives at, gives up, sets the status word the way an
attention kernel would, and returns normally.  The test then checks the three promises of
include/arattn.h: the status call reports AR_ERR_TIMEOUT once and clears the word; while the word
is set, attention kernels return without touching their outputs; afterwards a normal call is
correct again."""
import pytest

import autoresearch_b200 as ab
from autoresearch_b200 import _lib
from oracle import oracle as orc
from tests.parity_util import assert_parity, compare, device_inputs

pytestmark = pytest.mark.gpu


def test_abandoned_wait_is_reported_sticky_and_recoverable(cuda_device):
    import torch
    L = ab.lib()
    ab.check_device_status()                                   # start clean
    B, T, H, W = 2, 300, 2, 64
    host, dev = device_inputs(B, T, H, seed=11)
    p = ab.AttnParams(window=W)
    assert L.ar_selftest_wait_timeout(0, torch.cuda.current_stream().cuda_stream) == _lib.AR_OK
    o = torch.full_like(dev[0], float("nan"))
    lse = torch.full((B, T, H), float("nan"), device="cuda")
    ab.attn_fwd(*dev[:3], p, out=o, lse=lse)                   # enqueued behind the self-test kernel
    torch.cuda.synchronize()
    assert torch.isnan(o.float()).all() and torch.isnan(lse).all(), "kernels must not run while the word is set"
    with pytest.raises(ab.ArattnError) as e:
        ab.check_device_status()
    assert e.value.status == _lib.AR_ERR_TIMEOUT
    ab.check_device_status()                                   # cleared by the read above
    # AR_FLAG_SYNC reports it from the call itself
    assert L.ar_selftest_wait_timeout(0, torch.cuda.current_stream().cuda_stream) == _lib.AR_OK
    with pytest.raises(ab.ArattnError) as e:
        ab.attn_fwd(*dev[:3], ab.AttnParams(window=W, sync=True))
    assert e.value.status == _lib.AR_ERR_TIMEOUT
    # recovery: a normal forward + backward is correct again
    o, lse = ab.attn_fwd(*dev[:3], p)
    dq, dk, dv, _ = ab.attn_bwd(*dev[:3], o, dev[3], lse, p)
    ab.check_device_status()
    want = orc.attention_path(*host[:3], host[3], W)
    assert_parity(compare({"o": o, "lse": lse, "dq": dq, "dk": dk, "dv": dv}, want), what="after recovery")


def test_noalloc_status_word(cuda_device):
    """Same for the allocation-free forward, whose kernels use the library's own status symbol."""
    import torch
    L = ab.lib()
    s = torch.cuda.current_stream().cuda_stream
    assert L.ar_noalloc_status() == _lib.AR_OK
    B, T, H = 1, 256, 2
    g = torch.Generator(device="cuda").manual_seed(3)
    q, k, v = (torch.randn(B, T, H, 128, device="cuda", generator=g) for _ in range(3))
    o = torch.full_like(q, float("nan"))
    lse = torch.full((B, T, H), float("nan"), device="cuda")
    args = (o.data_ptr(), lse.data_ptr(), q.data_ptr(), k.data_ptr(), v.data_ptr(), B, T, H, 128, 0, s)
    assert L.ar_selftest_wait_timeout(1, s) == _lib.AR_OK
    assert L.ar_flash_attn_fwd_noalloc(*args) == _lib.AR_OK
    torch.cuda.synchronize()
    assert torch.isnan(o).all()                                # silent no-op while the word is set ...
    assert L.ar_device_status() == _lib.AR_OK                  # ... which the other family's word does not show
    assert L.ar_noalloc_status() == _lib.AR_ERR_TIMEOUT        # ... and this call does, once
    assert L.ar_noalloc_status() == _lib.AR_OK
    assert L.ar_flash_attn_fwd_noalloc(*args) == _lib.AR_OK
    torch.cuda.synchronize()
    assert torch.isfinite(o).all() and torch.isfinite(lse).all()
    assert L.ar_selftest_wait_timeout(2, s) == _lib.AR_ERR_BAD_ARG
