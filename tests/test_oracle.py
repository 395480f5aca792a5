"""CPU checks of the oracle: restatement vs an independent fp64 dense formulation,
literal vs row form, committed golden vectors, mask/pair counting, RoPE identities."""
import os

import numpy as np
import pytest

from oracle import oracle as orc

GOLDEN = os.path.join(os.path.dirname(__file__), "golden", "attention_golden.npz")
NAMES = ("o", "lse", "d", "dq", "dk", "dv")


@pytest.mark.parametrize("W", [0, 1, 7, 38, 39, 40, 100])
@pytest.mark.parametrize("rope", [False, True])
def test_restatement_matches_fp64_dense(W, rope):
    B, T, H, D = 2, 40, 3, 16
    q, k, v, do = orc.make_inputs(B, T, H, D, seed=1)
    tables = orc.rope_table(T, D) if rope else None
    got = orc.attention_path(q, k, v, do, W, rope=tables)
    want = orc.dense_attention_path(q, k, v, do, W, rope=tables)
    for n in NAMES:
        max_abs, rel = orc.parity(got[n], want[n])
        assert max_abs < 2e-5 and rel < 2e-6, (n, max_abs, rel)


@pytest.mark.parametrize("W", [0, 5, 200])
def test_literal_and_row_forms_are_bit_identical(W):
    B, T, H, D = 1, 48, 2, 32
    q, k, v, do = orc.make_inputs(B, T, H, D, seed=2)
    o, lse = orc.flash_attn_fwd(q, k, v, W)
    d = orc.flash_attn_bwd_precompute_d(o, do)
    assert np.array_equal(orc.flash_attn_bwd_dq(q, k, v, do, lse, d, W, literal=True),
                          orc.flash_attn_bwd_dq(q, k, v, do, lse, d, W))
    dk_l, dv_l = orc.flash_attn_bwd_dkv(q, k, v, do, lse, d, W, literal=True)
    dk_r, dv_r = orc.flash_attn_bwd_dkv(q, k, v, do, lse, d, W)
    assert np.array_equal(dk_l, dk_r) and np.array_equal(dv_l, dv_r)


def test_config1_shape_full_causal_fp32():
    """BASELINE config 1: B=1, H=4, T=256, D=128, fp32, seed 0, full causal, RoPE base 10000."""
    q, k, v, do = orc.make_inputs(1, 256, 4, 128, seed=0)
    tables = orc.rope_table(256, 128)
    got = orc.attention_path(q, k, v, do, 0, rope=tables)
    want = orc.dense_attention_path(q, k, v, do, 0, rope=tables)
    for n in NAMES:
        max_abs, rel = orc.parity(got[n], want[n])
        assert max_abs < 5e-5 and rel < 2e-6, (n, max_abs, rel)


def test_golden_vectors():
    """The committed fixtures were produced by tests/golden/make_golden.py from this oracle;
    they pin it against silent changes (the reference itself has no vectors for this path)."""
    z = np.load(GOLDEN)
    for case in sorted({key.split("/")[0] for key in z.files}):
        B, T, H, D, W, seed, rope = (int(x) for x in z[f"{case}/meta"])
        q, k, v, do = orc.make_inputs(B, T, H, D, seed=seed)
        tables = orc.rope_table(T, D) if rope else None
        got = orc.attention_path(q, k, v, do, W, rope=tables)
        for n in NAMES:
            np.testing.assert_allclose(got[n], z[f"{case}/{n}"], rtol=2e-5, atol=2e-6, err_msg=f"{case}/{n}")


def test_window_admits_w_plus_one_keys_and_pairs_formula():
    for T, W in [(40, 7), (40, 0), (40, 39), (40, 38), (64, 1), (2048, 1024)]:
        m = orc.visible_mask(T, W)
        assert m.sum() == orc.pairs(T, W)
        if 0 < W < T - 1:
            assert m[T - 1].sum() == W + 1
    assert orc.attn_flops(16, 4 and 2048, 4, 128, 1024) == pytest.approx(1.8056e11, rel=1e-3)


def test_lse_is_natural_log_of_scaled_scores():
    B, T, H, D = 1, 33, 2, 16
    q, k, v, _ = orc.make_inputs(B, T, H, D, seed=4)
    o, lse = orc.flash_attn_fwd(q, k, v, 9)
    s = np.einsum("bqhd,bkhd->bhqk", q.astype(np.float64), k.astype(np.float64)) / np.sqrt(D)
    s = np.where(orc.visible_mask(T, 9)[None, None], s, -np.inf)
    total = np.exp(s - np.transpose(lse, (0, 2, 1))[..., None]).sum(-1)
    np.testing.assert_allclose(total, 1.0, atol=1e-5)


def test_rope_roundtrip_table_and_position_shift_invariance():
    B, T, H, D = 2, 24, 2, 32
    q, k, v, do = orc.make_inputs(B, T, H, D, seed=5)
    cos, sin = orc.rope_table(2 * T, D)
    # table: model.mojo:73-78
    t, d = 7, 3
    ang = t / (10000.0 ** (2 * d / D))
    assert cos[t, d] == np.float32(np.cos(ang)) and sin[t, d] == np.float32(np.sin(ang))
    # rope_bwd is the transpose (inverse) of rope_fwd
    x = orc.rope_fwd(q, cos, sin, T)
    np.testing.assert_allclose(orc.rope_bwd(x, cos, sin, T), q, atol=2e-6)
    # literal index (seq_len <= 0) equals token % T for B == 1
    np.testing.assert_array_equal(orc.rope_fwd(q[:1], cos, sin, 0), orc.rope_fwd(q[:1], cos, sin, T))
    # a common position offset leaves O and LSE unchanged (why pos = t may replace pos = b*T + t)
    shifted = (cos[5:5 + T].copy(), sin[5:5 + T].copy())
    a = orc.attention_path(q, k, v, do, 6, rope=(cos[:T].copy(), sin[:T].copy()))
    b = orc.attention_path(q, k, v, do, 6, rope=shifted)
    for n in ("o", "lse", "dv", "dq", "dk"):
        assert orc.parity(a[n], b[n])[0] < 5e-6, n


def test_bf16_rounding_helper():
    x = np.array([1.0, 1.00390625, 1.01171875, -3.1415927, 0.0], np.float32)
    import torch
    want = torch.from_numpy(x).to(torch.bfloat16).float().numpy()
    np.testing.assert_array_equal(orc.to_bf16_rne(x), want)


def test_autograd_agrees_with_manual_backward():
    """Independent derivation: torch CPU autograd through softmax(QK^T)V with RoPE."""
    import torch
    B, T, H, D, W = 1, 20, 2, 16, 6
    q, k, v, do = orc.make_inputs(B, T, H, D, seed=6)
    cos, sin = orc.rope_table(T, D)
    tq, tk, tv = (torch.tensor(a, dtype=torch.float64, requires_grad=True) for a in (q, k, v))
    c = torch.tensor(cos, dtype=torch.float64)[None, :, None, :]
    s = torch.tensor(sin, dtype=torch.float64)[None, :, None, :]

    def rope(x):
        x1, x2 = x[..., : D // 2], x[..., D // 2:]
        return torch.cat([x1 * c + x2 * s, -x1 * s + x2 * c], -1)

    sc = torch.einsum("bqhd,bkhd->bhqk", rope(tq), rope(tk)) / np.sqrt(D)
    sc = sc.masked_fill(~torch.tensor(orc.visible_mask(T, W))[None, None], float("-inf"))
    o = torch.einsum("bhqk,bkhd->bqhd", torch.softmax(sc, -1), tv)
    o.backward(torch.tensor(do, dtype=torch.float64))
    got = orc.attention_path(q, k, v, do, W, rope=(cos, sin))
    for n, t in (("dq", tq), ("dk", tk), ("dv", tv)):
        assert orc.parity(got[n], t.grad.numpy())[0] < 2e-5, n
    assert orc.parity(got["o"], o.detach().numpy())[0] < 2e-6


def test_rmsnorm_matches_the_reference_known_answer_test():
    """The reference's own test of rmsnorm_fwd (test_kernels.mojo:140-181): two rows of four values,
    expected rms = [2.7386, 2.5], out[0,0] = 0.3651, out[1,3] = 2.0, each within 0.01.  This is the
    one kernel of the step before attention for which the reference holds a known answer."""
    x = np.array([[1.0, 2.0, 3.0, 4.0], [0.0, 0.0, 0.0, 5.0]], np.float32)
    y, rms = orc.rmsnorm_fwd(x)
    assert abs(rms[0] - 2.7386) <= 0.01 and abs(rms[1] - 2.5) <= 0.01
    assert abs(y[0, 0] - 1.0 / 2.7386) <= 0.01 and abs(y[1, 3] - 5.0 / 2.5) <= 0.01
    # and exactly: rms = sqrt(mean(x^2) + 1e-5)
    want = np.sqrt((x.astype(np.float64) ** 2).mean(-1) + 1e-5)
    assert np.allclose(rms, want, rtol=1e-6)
    assert np.allclose(y, x / want[:, None], rtol=1e-6)


def test_qk_rope_norm_commutes_with_normalising_first():
    """model.mojo:668-687 rotates q, k and then normalises each head row.  A rotation keeps a row's
    sum of squares, so normalising first gives the same result up to rounding: the property that lets
    a caller hand normalised, un-rotated q, k to the fused entry points."""
    rng = np.random.default_rng(3)
    B, T, H, D = 2, 33, 3, 128
    q = rng.standard_normal((B, T, H, D), dtype=np.float32) * 3
    k = rng.standard_normal((B, T, H, D), dtype=np.float32)
    cos, sin = orc.rope_table(T, D)
    qo, ko, rq, rk = orc.qk_rope_norm(q, k, cos, sin, T)
    qn, rq2 = orc.rmsnorm_fwd(q)
    assert np.abs(orc.rope_fwd(qn, cos, sin, T) - qo).max() < 2e-6
    assert np.allclose(rq, rq2, rtol=1e-6)
    assert np.allclose((qo.astype(np.float64) ** 2).mean(-1), 1.0, atol=1e-4)
    assert np.allclose((ko.astype(np.float64) ** 2).mean(-1), 1.0, atol=1e-4)
