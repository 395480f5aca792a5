"""Python face of the CPU oracle.  TEST INFRASTRUCTURE ONLY.

Two independent CPU statements of the reference attention path
(kernels/ops.mojo:209-480, 1091-1120; model.mojo:57-81):

* ``CORacle`` functions: ctypes bindings of ``attn_oracle.c``, the loop-for-loop
  fp32 restatement of the reference kernels (the oracle proper).
* ``dense_*`` functions: an fp64 dense masked-softmax formulation in numpy with
  analytically derived gradients.  It shares no code or loop structure with the
  restatement and is used only to cross-check it.

Parity is UNPINNED against the reference itself: the reference cannot be run
(Mojo toolchain absent, GPU-only code) and ships no golden vectors for this path.

Nothing in the shipped package may import this module; only tests, the smoke
check and the benchmark's CPU-baseline leg do.
"""
from __future__ import annotations

import ctypes
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_SO = os.path.join(_HERE, "_build", "liboracle.so")
_lib = None

ROPE_BASE = 10000.0  # config.mojo:87


def build(force: bool = False) -> str:
    """Compile attn_oracle.c into oracle/_build/liboracle.so (gcc, OpenMP)."""
    src = os.path.join(_HERE, "attn_oracle.c")
    if force or not os.path.exists(_SO) or os.path.getmtime(_SO) < os.path.getmtime(src):
        subprocess.check_call(["make", "-C", _HERE, "-s", "-B"])
    return _SO


def lib() -> ctypes.CDLL:
    global _lib
    if _lib is None:
        build()
        _lib = ctypes.CDLL(_SO)
        _lib.oracle_num_threads.restype = ctypes.c_int
    return _lib


def _p(a: np.ndarray):
    assert a.dtype == np.float32 and a.flags["C_CONTIGUOUS"]
    return a.ctypes.data_as(ctypes.POINTER(ctypes.c_float))


def _i(x: int):
    return ctypes.c_int64(int(x))


def num_threads() -> int:
    return int(lib().oracle_num_threads())


def use_all_cores() -> int:
    """Undo OMP_NUM_THREADS=1 (set by torchrun and similar launchers) for the timed CPU legs."""
    n = len(os.sched_getaffinity(0)) if hasattr(os, "sched_getaffinity") else (os.cpu_count() or 1)
    lib().oracle_set_num_threads(ctypes.c_int(n))
    return num_threads()


def rope_table(rows: int, head_dim: int, base: float = ROPE_BASE):
    """cos, sin tables [rows, head_dim//2] fp32 (model.mojo:57-81)."""
    cos = np.empty((rows, head_dim // 2), np.float32)
    sin = np.empty((rows, head_dim // 2), np.float32)
    lib().oracle_rope_table(_p(cos), _p(sin), _i(rows), _i(head_dim), ctypes.c_double(base))
    return cos, sin


def rope_fwd(x: np.ndarray, cos: np.ndarray, sin: np.ndarray, seq_len: int) -> np.ndarray:
    """x: [B, T, H, D] (or [tokens, H, D]); ops.mojo:209-238 with pos = token % seq_len."""
    x = np.ascontiguousarray(x, np.float32)
    out = np.empty_like(x)
    H, D = x.shape[-2], x.shape[-1]
    tokens = x.size // (H * D)
    lib().oracle_rope_fwd(_p(out), _p(x), _p(cos), _p(sin), _i(tokens), _i(H), _i(D), _i(seq_len))
    return out


def rope_bwd(g: np.ndarray, cos: np.ndarray, sin: np.ndarray, seq_len: int) -> np.ndarray:
    """ops.mojo:1091-1120."""
    g = np.ascontiguousarray(g, np.float32)
    out = np.empty_like(g)
    H, D = g.shape[-2], g.shape[-1]
    tokens = g.size // (H * D)
    lib().oracle_rope_bwd(_p(out), _p(g), _p(cos), _p(sin), _i(tokens), _i(H), _i(D), _i(seq_len))
    return out


def rmsnorm_fwd(x: np.ndarray):
    """ops.mojo:61-104 on the last axis.  Returns (y, rms) with rms = sqrt(mean(x^2) + 1e-5) per row."""
    x = np.ascontiguousarray(x, np.float32)
    dim = x.shape[-1]
    rows = x.size // dim
    out = np.empty_like(x)
    rms = np.empty(x.shape[:-1], np.float32)
    lib().oracle_rmsnorm_fwd(_p(out), _p(rms), _p(x), _i(rows), _i(dim))
    return out, rms


def qk_rope_norm(q: np.ndarray, k: np.ndarray, cos: np.ndarray, sin: np.ndarray, seq_len: int):
    """model.mojo:668-687: rope_fwd then the per-head rmsnorm_fwd on q and k [.., H, D].
    Returns (q_out, k_out, rms_q, rms_k)."""
    q, k = (np.ascontiguousarray(a, np.float32) for a in (q, k))
    H, D = q.shape[-2], q.shape[-1]
    tokens = q.size // (H * D)
    qo, ko = np.empty_like(q), np.empty_like(k)
    rq, rk = np.empty(q.shape[:-1], np.float32), np.empty(k.shape[:-1], np.float32)
    lib().oracle_qk_rope_norm(_p(qo), _p(ko), _p(rq), _p(rk), _p(q), _p(k), _p(cos), _p(sin), _i(tokens), _i(H),
                              _i(D), _i(seq_len))
    return qo, ko, rq, rk


def linear_fwd(x: np.ndarray, w: np.ndarray) -> np.ndarray:
    """ops.mojo:110-117: Y = X W^T for X [M,K], W [N,K]."""
    x, w = np.ascontiguousarray(x, np.float32), np.ascontiguousarray(w, np.float32)
    (M, K), N = x.shape, w.shape[0]
    y = np.empty((M, N), np.float32)
    lib().oracle_linear_fwd(_p(y), _p(x), _p(w), _i(M), _i(N), _i(K))
    return y


def linear_bwd_dx(dy: np.ndarray, w: np.ndarray) -> np.ndarray:
    """ops.mojo:870-878: dX = dY W for dY [M,N], W [N,K]."""
    dy, w = np.ascontiguousarray(dy, np.float32), np.ascontiguousarray(w, np.float32)
    (M, N), K = dy.shape, w.shape[1]
    dx = np.empty((M, K), np.float32)
    lib().oracle_linear_bwd_dx(_p(dx), _p(dy), _p(w), _i(M), _i(N), _i(K))
    return dx


def linear_bwd_dw(dw: np.ndarray, dy: np.ndarray, x: np.ndarray) -> np.ndarray:
    """ops.mojo:953-961: dW += dY^T X (returns the updated copy of dw)."""
    dw = np.array(dw, np.float32, order="C")
    dy, x = np.ascontiguousarray(dy, np.float32), np.ascontiguousarray(x, np.float32)
    (M, N), K = dy.shape, x.shape[1]
    lib().oracle_linear_bwd_dw(_p(dw), _p(dy), _p(x), _i(M), _i(N), _i(K))
    return dw


def flash_attn_fwd(q, k, v, window_size: int):
    """ops.mojo:244-323.  q,k,v [B,T,H,D] fp32 -> (O [B,T,H,D], LSE [B,T,H])."""
    q, k, v = (np.ascontiguousarray(a, np.float32) for a in (q, k, v))
    B, T, H, D = q.shape
    o = np.zeros_like(q)
    lse = np.zeros((B, T, H), np.float32)
    lib().oracle_flash_attn_fwd(_p(o), _p(lse), _p(q), _p(k), _p(v), _i(B), _i(T), _i(H), _i(D),
                                _i(window_size))
    return o, lse


def flash_attn_bwd_precompute_d(o, d_o):
    """ops.mojo:329-346."""
    o, d_o = (np.ascontiguousarray(a, np.float32) for a in (o, d_o))
    B, T, H, D = o.shape
    d = np.zeros((B, T, H), np.float32)
    lib().oracle_flash_attn_bwd_precompute_d(_p(d), _p(o), _p(d_o), _i(B), _i(T), _i(H), _i(D))
    return d


def flash_attn_bwd_dq(q, k, v, d_o, lse, d_buf, window_size: int, literal: bool = False):
    """ops.mojo:349-411 (literal=True: one loop iteration per reference thread)."""
    q, k, v, d_o, lse, d_buf = (np.ascontiguousarray(a, np.float32) for a in (q, k, v, d_o, lse, d_buf))
    B, T, H, D = q.shape
    dq = np.zeros_like(q)
    fn = lib().oracle_flash_attn_bwd_dq_literal if literal else lib().oracle_flash_attn_bwd_dq
    fn(_p(dq), _p(q), _p(k), _p(v), _p(d_o), _p(lse), _p(d_buf), _i(B), _i(T), _i(H), _i(D),
       _i(window_size))
    return dq


def flash_attn_bwd_dkv(q, k, v, d_o, lse, d_buf, window_size: int, literal: bool = False):
    """ops.mojo:414-480."""
    q, k, v, d_o, lse, d_buf = (np.ascontiguousarray(a, np.float32) for a in (q, k, v, d_o, lse, d_buf))
    B, T, H, D = q.shape
    dk = np.zeros_like(q)
    dv = np.zeros_like(q)
    fn = lib().oracle_flash_attn_bwd_dkv_literal if literal else lib().oracle_flash_attn_bwd_dkv
    fn(_p(dk), _p(dv), _p(q), _p(k), _p(v), _p(d_o), _p(lse), _p(d_buf), _i(B), _i(T), _i(H),
       _i(D), _i(window_size))
    return dk, dv


def attention_path(q, k, v, d_o=None, window_size: int = 0, rope=None):
    """The whole path in model.mojo's launch order (model.mojo:668-699, 915-964).

    rope = (cos, sin) rotates q and k first (position = t) and returns dq/dk with
    respect to the un-rotated inputs; rope=None treats q, k as already rotated.
    Returns a dict with o, lse and (if d_o is given) d, dq, dk, dv.
    """
    q, k, v = (np.ascontiguousarray(a, np.float32) for a in (q, k, v))
    B, T, H, D = q.shape
    backward = d_o is not None
    d_o = np.ascontiguousarray(d_o, np.float32) if backward else np.zeros(1, np.float32)
    cos, sin = rope if rope is not None else (np.zeros(1, np.float32), np.zeros(1, np.float32))
    out = {n: np.zeros_like(q) for n in ("o", "dq", "dk", "dv", "q_rot", "k_rot")}
    out["lse"] = np.zeros((B, T, H), np.float32)
    out["d"] = np.zeros((B, T, H), np.float32)
    lib().oracle_attention_path(
        _p(out["o"]), _p(out["lse"]), _p(out["d"]), _p(out["dq"]), _p(out["dk"]), _p(out["dv"]),
        _p(out["q_rot"]), _p(out["k_rot"]), _p(q), _p(k), _p(v), _p(d_o), _p(cos), _p(sin),
        _i(B), _i(T), _i(H), _i(D), _i(window_size),
        ctypes.c_int32(1 if rope is not None else 0), ctypes.c_int32(1 if backward else 0))
    if not backward:
        for n in ("dq", "dk", "dv", "d"):
            del out[n]
    return out


# ----------------------------------------------------------------------------
# Independent fp64 dense formulation (cross-check of the restatement)
# ----------------------------------------------------------------------------

def visible_mask(T: int, window_size: int) -> np.ndarray:
    """mask[q, k] = k <= q and (W <= 0 or k >= q - W)   (ops.mojo:290-293)."""
    qi = np.arange(T)[:, None]
    ki = np.arange(T)[None, :]
    m = ki <= qi
    if window_size > 0:
        m &= ki >= qi - window_size
    return m


def pairs(T: int, W: int) -> int:
    """Number of visible (q, k) pairs per (b, h) unit: the work unit of the FLOP count."""
    if W <= 0 or W >= T - 1:
        return T * (T + 1) // 2
    return (W + 1) * (W + 2) // 2 + (T - W - 1) * (W + 1)


def attn_flops(B: int, T: int, H: int, D: int, W: int, fwd: bool = True, bwd: bool = True) -> float:
    """Algorithmic FLOPs: forward 4*D per visible pair, backward 10*D per pair."""
    per_pair = (4 * D if fwd else 0) + (10 * D if bwd else 0)
    return float(per_pair) * pairs(T, W) * B * H


def dense_rope(x, cos, sin, inverse: bool = False):
    x = np.asarray(x, np.float64)
    T, D = x.shape[1], x.shape[3]
    c = np.asarray(cos[:T], np.float64)[None, :, None, :]
    s = np.asarray(sin[:T], np.float64)[None, :, None, :]
    if inverse:
        s = -s
    x1, x2 = x[..., : D // 2], x[..., D // 2:]
    return np.concatenate([x1 * c + x2 * s, -x1 * s + x2 * c], axis=-1)


def dense_attention_path(q, k, v, d_o=None, window_size: int = 0, rope=None):
    """softmax(mask(Q K^T / sqrt(D))) V and its analytic gradients, all in fp64."""
    q, k, v = (np.asarray(a, np.float64) for a in (q, k, v))
    B, T, H, D = q.shape
    if rope is not None:
        q = dense_rope(q, *rope)
        k = dense_rope(k, *rope)
    mask = visible_mask(T, window_size)
    s = np.einsum("bqhd,bkhd->bhqk", q, k) / np.sqrt(D)
    s = np.where(mask[None, None], s, -np.inf)
    mx = s.max(axis=-1, keepdims=True)
    e = np.exp(s - mx)
    l = e.sum(axis=-1, keepdims=True)
    p = e / l
    out = {"o": np.einsum("bhqk,bkhd->bqhd", p, v),
           "lse": np.transpose((mx + np.log(l))[..., 0], (0, 2, 1))}
    if d_o is None:
        return out
    d_o = np.asarray(d_o, np.float64)
    dp = np.einsum("bqhd,bkhd->bhqk", d_o, v)
    delta = (out["o"] * d_o).sum(-1)                      # [B,T,H]
    ds = p * (dp - np.transpose(delta, (0, 2, 1))[..., None])
    dq = np.einsum("bhqk,bkhd->bqhd", ds, k) / np.sqrt(D)
    dk = np.einsum("bhqk,bqhd->bkhd", ds, q) / np.sqrt(D)
    dv = np.einsum("bhqk,bqhd->bkhd", p, d_o)
    if rope is not None:
        dq = dense_rope(dq, *rope, inverse=True)
        dk = dense_rope(dk, *rope, inverse=True)
    out.update(d=delta, dq=dq, dk=dk, dv=dv)
    return out


# ----------------------------------------------------------------------------
# Seeded synthetic inputs and the parity metric
# ----------------------------------------------------------------------------

def to_bf16_rne(x: np.ndarray) -> np.ndarray:
    """Round fp32 to the nearest bf16 (ties to even); returns fp32 holding bf16 values."""
    u = np.ascontiguousarray(x, np.float32).view(np.uint32).astype(np.uint64)
    u = (u + 0x7FFF + ((u >> 16) & 1)) & 0xFFFF0000
    return u.astype(np.uint32).view(np.float32).reshape(x.shape)


def make_inputs(B: int, T: int, H: int, D: int, seed: int = 0, bf16: bool = False):
    """Q, K, V, dO ~ N(0,1) from numpy PCG64(seed), drawn in that order, [B,T,H,D] fp32.

    bf16=True rounds each tensor to bf16 (RNE) so the oracle runs in fp32 on exactly
    the values a bf16 kernel receives."""
    rng = np.random.default_rng(seed)
    ts = [rng.standard_normal((B, T, H, D), dtype=np.float32) for _ in range(4)]
    if bf16:
        ts = [to_bf16_rne(t) for t in ts]
    return ts


def parity(got: np.ndarray, want: np.ndarray):
    """(max-abs error, relative L2 error) of got against want."""
    got = np.asarray(got, np.float64)
    want = np.asarray(want, np.float64)
    diff = got - want
    denom = np.sqrt((want ** 2).sum())
    return float(np.abs(diff).max()), float(np.sqrt((diff ** 2).sum()) / max(denom, 1e-30))


MAX_ABS_TOL = 2e-2   # bf16 inputs against the fp32 oracle
REL_L2_TOL = 1e-2
