"""GPU parity of ar_qk_norm_rope_cast, the step before attention in one launch (rope_fwd and
per-head rmsnorm_fwd on q and k, bf16 cast of q, k, v: model.mojo:668-691), against the oracle's
restatement of rope_fwd + rmsnorm_fwd, and the whole flow it feeds: prologue -> ar_attn_fwd ->
ar_attn_bwd on the saved rotated tensors."""
import numpy as np
import pytest

import autoresearch_b200 as ab
from autoresearch_b200 import _lib
from oracle import oracle as orc
from tests.parity_util import assert_parity, compare

pytestmark = pytest.mark.gpu


def _prologue(q, k, v, cos, sin, T, want_rms=True):
    import torch
    B, _, H, D = q.shape
    q_rot, k_rot, v_b = (torch.empty(B, T, H, D, device="cuda", dtype=torch.bfloat16) for _ in range(3))
    rms_q = torch.empty(B, T, H, device="cuda") if want_rms else None
    rms_k = torch.empty(B, T, H, device="cuda") if want_rms else None
    st = ab.lib().ar_qk_norm_rope_cast(
        q_rot.data_ptr(), k_rot.data_ptr(), v_b.data_ptr(), rms_q.data_ptr() if want_rms else None,
        rms_k.data_ptr() if want_rms else None, q.data_ptr(), k.data_ptr(), v.data_ptr(),
        _lib.AR_F32 if q.dtype == torch.float32 else _lib.AR_BF16, cos.data_ptr(),
        sin.data_ptr(), B * T, H, D, T, 1e-5, torch.cuda.current_stream().cuda_stream)
    assert st == _lib.AR_OK, ab.lib().ar_last_error()
    return q_rot, k_rot, v_b, rms_q, rms_k


@pytest.mark.parametrize("B,T,H", [(1, 1, 1), (2, 300, 3), (3, 2049, 4), (16, 2048, 4)])
def test_prologue_matches_rope_then_rmsnorm(cuda_device, B, T, H):
    import torch
    rng = np.random.default_rng(B * 1000 + T)
    qh, kh, vh = (rng.standard_normal((B, T, H, 128), dtype=np.float32) * s for s in (2.0, 0.5, 1.0))
    cos_h, sin_h = orc.rope_table(T, 128)
    q, k, v, cos, sin = (torch.from_numpy(a).cuda() for a in (qh, kh, vh, cos_h, sin_h))
    q_rot, k_rot, v_b, rms_q, rms_k = _prologue(q, k, v, cos, sin, T)
    torch.cuda.synchronize()
    qo, ko, rq, rk = orc.qk_rope_norm(qh, kh, cos_h, sin_h, T)
    # bf16 outputs: each element within half a bf16 ulp (at most 2^-8 of its magnitude) of the oracle's
    # fp32 value, and - up to the rare element where the two summation orders of the mean square
    # land on different sides of a rounding boundary - equal to the oracle's value rounded to bf16
    for name, got, want in (("q_rot", q_rot, qo), ("k_rot", k_rot, ko), ("v", v_b, vh)):
        g = got.float().cpu().numpy()
        assert (np.abs(g - want) <= np.abs(want) / 256 + 1e-6).all(), name
        assert np.mean(g != orc.to_bf16_rne(want)) < 1e-3, name
    assert np.allclose(rms_q.cpu().numpy(), rq, rtol=2e-6) and np.allclose(rms_k.cpu().numpy(), rk, rtol=2e-6)


def test_prologue_feeds_the_attention_path(cuda_device):
    """fp32 q, k, v -> prologue -> forward -> backward with the saved rotated tensors: O, LSE and the
    gradients with respect to the normalised q, k of the reference flow (its backward passes gradients
    straight through the normalisation, model.mojo:937, and then applies rope_bwd)."""
    import torch
    B, T, H, W = 2, 700, 2, 256
    rng = np.random.default_rng(5)
    qh, kh, vh, doh = (rng.standard_normal((B, T, H, 128), dtype=np.float32) for _ in range(4))
    vh, doh = orc.to_bf16_rne(vh), orc.to_bf16_rne(doh)
    cos_h, sin_h = orc.rope_table(T, 128)
    q, k, v, cos, sin = (torch.from_numpy(a).cuda() for a in (qh, kh, vh, cos_h, sin_h))
    q_rot, k_rot, v_b, _, _ = _prologue(q, k, v, cos, sin, T, want_rms=False)
    do = torch.from_numpy(doh).to("cuda", torch.bfloat16)
    o, lse = ab.attn_fwd(q_rot, k_rot, v_b, ab.AttnParams(window=W))
    p = ab.AttnParams(window=W, rope=(cos, sin), q_rot=q_rot, k_rot=k_rot)
    dq, dk, dv, _ = ab.attn_bwd(q_rot, k_rot, v_b, o, do, lse, p)     # q, k arguments are not read
    ab.check_device_status()
    # oracle: rope + norm in fp32, rounded to bf16 as the prologue hands them on, then the reference's
    # attention and its backward on those tensors, then rope_bwd
    qo, ko, _, _ = orc.qk_rope_norm(qh, kh, cos_h, sin_h, T)
    qo, ko = orc.to_bf16_rne(qo), orc.to_bf16_rne(ko)
    want = orc.attention_path(qo, ko, vh, doh, W)
    want["dq"] = orc.rope_bwd(want["dq"], cos_h, sin_h, T)
    want["dk"] = orc.rope_bwd(want["dk"], cos_h, sin_h, T)
    assert_parity(compare({"o": o, "lse": lse, "dq": dq, "dk": dk, "dv": dv}, want), what="prologue flow")
