"""GPU parity of the projection GEMMs ar_linear_fwd / ar_linear_bwd_dx / ar_linear_bwd_dw (the
reference's linear_fwd, linear_bwd_dx, linear_bwd_dw: ops.mojo:110-203, 870-950, 953-1033) against
the oracle's restatement of the sums their docstrings state.  The kernels multiply bf16 operands
exactly and accumulate in fp32, so on bf16-valued inputs the only difference from the oracle is
the order of the fp32 sum: the bound is a few fp32 ulps of sum |a||b|."""
import numpy as np
import pytest

import autoresearch_b200 as ab
from oracle import oracle as orc

pytestmark = pytest.mark.gpu

# M, N, K: one tile; ragged rows; ragged rows, columns and depth; several tiles per CTA with
# ragged depth; the QKV and c_proj shapes of the depth-4 model at a reduced token count
SHAPES = [(128, 256, 64), (200, 96, 160), (1, 32, 32), (777, 1184, 864), (4096, 1536, 512), (4096, 512, 512)]


def _rand(rng, shape, bf16_valued=True, scale=1.0):
    a = rng.standard_normal(shape, dtype=np.float32) * scale
    return orc.to_bf16_rne(a) if bf16_valued else a


def _bound(a_abs_b):
    # |fp32 sum in any order - another order| <= depth * eps * sum |a||b| in the worst case; sums of
    # random signs stay far inside 16 ulps of it
    return 16 * 2.0 ** -24 * a_abs_b + 1e-30


def _dev(a, dtype):
    import torch
    return torch.from_numpy(a).cuda().to(dtype)


@pytest.mark.parametrize("M,N,K", SHAPES)
@pytest.mark.parametrize("in_dtype", ["bf16", "f32"])
def test_linear_fwd(cuda_device, M, N, K, in_dtype):
    import torch
    rng = np.random.default_rng(M + N + K)
    x, w = _rand(rng, (M, K)), _rand(rng, (N, K), scale=0.1)
    dt = torch.bfloat16 if in_dtype == "bf16" else torch.float32
    y = torch.full((M, N), float("nan"), device="cuda")
    ab.linear_fwd(y, _dev(x, dt), _dev(w, dt), M, N, K)
    torch.cuda.synchronize()
    want = orc.linear_fwd(x, w)
    lim = _bound(np.abs(x) @ np.abs(w).T)
    assert (np.abs(y.cpu().numpy() - want) <= lim).all()


@pytest.mark.parametrize("M,N,K", SHAPES)
def test_linear_bwd_dx(cuda_device, M, N, K):
    import torch
    rng = np.random.default_rng(M + 2 * N + K)
    dy, w = _rand(rng, (M, N)), _rand(rng, (N, K), scale=0.1)
    dx = torch.full((M, K), float("nan"), device="cuda")
    ab.linear_bwd_dx(dx, _dev(dy, torch.bfloat16), _dev(w, torch.bfloat16), M, N, K)
    torch.cuda.synchronize()
    want = orc.linear_bwd_dx(dy, w)
    assert (np.abs(dx.cpu().numpy() - want) <= _bound(np.abs(dy) @ np.abs(w))).all()


@pytest.mark.parametrize("M,N,K", SHAPES + [(9000, 256, 128)])
def test_linear_bwd_dw_accumulates(cuda_device, M, N, K):
    """dW is added into, twice over: the second call doubles the product on top of the first value."""
    import torch
    rng = np.random.default_rng(M + N + 3 * K)
    dy, x = _rand(rng, (M, N), scale=0.1), _rand(rng, (M, K))
    dw0 = rng.standard_normal((N, K), dtype=np.float32)
    dw = torch.from_numpy(dw0).cuda()
    dyd, xd = _dev(dy, torch.bfloat16), _dev(x, torch.bfloat16)
    ab.linear_bwd_dw(dw, dyd, xd, M, N, K)
    torch.cuda.synchronize()
    want1 = orc.linear_bwd_dw(dw0, dy, x)
    lim = _bound(np.abs(dy).T @ np.abs(x)) + 2.0 ** -22 * np.abs(want1)
    assert (np.abs(dw.cpu().numpy() - want1) <= lim).all()
    ab.linear_bwd_dw(dw, dyd, xd, M, N, K)
    torch.cuda.synchronize()
    want2 = orc.linear_bwd_dw(want1, dy, x)
    assert (np.abs(dw.cpu().numpy() - want2) <= 2 * lim + 2.0 ** -22 * np.abs(want2)).all()


def test_linear_fp32_inputs_and_bf16_output(cuda_device):
    """fp32 operands are rounded to bf16 on the way in (the same result as rounding them first), and
    a bf16 output is the fp32 accumulator rounded once."""
    import torch
    M, N, K = 640, 512, 512
    rng = np.random.default_rng(11)
    x, w = _rand(rng, (M, K), bf16_valued=False), _rand(rng, (N, K), bf16_valued=False, scale=0.1)
    y32 = torch.empty(M, N, device="cuda")
    y16 = torch.empty(M, N, device="cuda", dtype=torch.bfloat16)
    xd, wd = _dev(x, torch.float32), _dev(w, torch.float32)
    ab.linear_fwd(y32, xd, wd, M, N, K)
    ab.linear_fwd(y16, xd, wd, M, N, K)
    torch.cuda.synchronize()
    xr, wr = orc.to_bf16_rne(x), orc.to_bf16_rne(w)
    want = orc.linear_fwd(xr, wr)
    assert (np.abs(y32.cpu().numpy() - want) <= _bound(np.abs(xr) @ np.abs(wr).T)).all()
    assert torch.equal(y16, y32.to(torch.bfloat16))
    # against the unrounded fp32 product: two operand roundings of 2^-9 each
    assert (np.abs(y32.cpu().numpy() - orc.linear_fwd(x, w)) <= 2.0 ** -8 * (np.abs(x) @ np.abs(w).T)).all()


def test_linear_full_token_count_against_fp32_matmul(cuda_device):
    """The headline token count (B*T = 32768) of the QKV projection and its two gradients against an
    fp32 matrix product of the same bf16-valued operands on the device (TF32 off)."""
    import torch
    M, N, K = 32768, 1536, 512
    was = torch.backends.cuda.matmul.allow_tf32
    torch.backends.cuda.matmul.allow_tf32 = False
    try:
        g = torch.Generator(device="cuda").manual_seed(3)
        x = torch.randn(M, K, device="cuda", generator=g).bfloat16()
        w = (torch.randn(N, K, device="cuda", generator=g) * 0.05).bfloat16()
        dy = (torch.randn(M, N, device="cuda", generator=g) * 0.1).bfloat16()
        y, dx, dw = torch.empty(M, N, device="cuda"), torch.empty(M, K, device="cuda"), torch.zeros(N, K, device="cuda")
        ab.linear_fwd(y, x, w, M, N, K)
        ab.linear_bwd_dx(dx, dy, w, M, N, K)
        ab.linear_bwd_dw(dw, dy, x, M, N, K)
        torch.cuda.synchronize()
        for got, want, mag in ((y, x.float() @ w.float().T, x.float().abs() @ w.float().abs().T),
                               (dx, dy.float() @ w.float(), dy.float().abs() @ w.float().abs()),
                               (dw, dy.float().T @ x.float(), dy.float().abs().T @ x.float().abs())):
            assert bool(((got - want).abs() <= 64 * 2.0 ** -24 * mag).all())
    finally:
        torch.backends.cuda.matmul.allow_tf32 = was


def test_linear_rejects_what_it_cannot_tile(cuda_device):
    import torch
    x = torch.zeros(64, 60, device="cuda", dtype=torch.bfloat16)
    w = torch.zeros(32, 60, device="cuda", dtype=torch.bfloat16)
    with pytest.raises(ab.ArattnError):
        ab.linear_fwd(torch.zeros(64, 32, device="cuda"), x, w, 64, 32, 60)   # K not a multiple of 8
    with pytest.raises(ValueError):
        ab.linear_fwd(torch.zeros(64, 32, device="cuda"), x.float(), w, 64, 32, 60)


def test_linear_bwd_dx_in_place_on_fp32(cuda_device):
    """The reference calls linear_bwd_dx with grad_input = grad_output (model.mojo:906, square c_proj):
    with fp32 operands the call stages them first, so the in-place form gives the same result."""
    import torch
    M = N = K = 512
    rng = np.random.default_rng(21)
    dy, w = _rand(rng, (M, N)), _rand(rng, (N, K), scale=0.1)
    buf, wd = _dev(dy, torch.float32), _dev(w, torch.float32)
    ab.linear_bwd_dx(buf, buf, wd, M, N, K)
    torch.cuda.synchronize()
    assert (np.abs(buf.cpu().numpy() - orc.linear_bwd_dx(dy, w)) <= _bound(np.abs(dy) @ np.abs(w))).all()
    b16 = _dev(dy, torch.bfloat16)
    with pytest.raises(ab.ArattnError):
        ab.linear_bwd_dx(b16, b16, _dev(w, torch.bfloat16), M, N, K)
