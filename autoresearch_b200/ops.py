"""Host-side mirror of the reference's attention kernels (kernels/ops.mojo).

Each function keeps the name, argument order and buffer contract of the Mojo kernel
it stands for: caller-allocated fp32 CUDA tensors, outputs written in place, nothing
returned.  `stream` defaults to torch's current stream.  The reference launches these
with ``ctx.enqueue_function`` (model.mojo:668-699, 915-964); here each is one call
into libarattn.so.
"""
from __future__ import annotations

import torch

from . import _lib


def _ptr(t: torch.Tensor, name: str) -> int:
    if not isinstance(t, torch.Tensor) or not t.is_cuda:
        raise ValueError(f"{name} must be a CUDA tensor")
    if t.dtype != torch.float32:
        raise ValueError(f"{name} must be float32 (got {t.dtype})")
    if not t.is_contiguous():
        raise ValueError(f"{name} must be contiguous")
    return t.data_ptr()


def _stream(stream) -> int:
    if stream is None:
        return torch.cuda.current_stream().cuda_stream
    return stream.cuda_stream if hasattr(stream, "cuda_stream") else int(stream)


def rope_fwd(output, input, cos_buf, sin_buf, num_tokens, num_heads, head_dim, seq_len=0, stream=None):
    """ops.mojo:209-217.  In place when output is input.  seq_len > 0 indexes the table
    with token % seq_len; 0 keeps the reference's literal token index."""
    _lib.check(_lib.lib().ar_rope_fwd(_ptr(output, "output"), _ptr(input, "input"), _ptr(cos_buf, "cos_buf"),
                                      _ptr(sin_buf, "sin_buf"), num_tokens, num_heads, head_dim, seq_len,
                                      _stream(stream)))


def rope_bwd(grad_input, grad_output, cos_buf, sin_buf, num_tokens, num_heads, head_dim, seq_len=0, stream=None):
    """ops.mojo:1091-1099."""
    _lib.check(_lib.lib().ar_rope_bwd(_ptr(grad_input, "grad_input"), _ptr(grad_output, "grad_output"),
                                      _ptr(cos_buf, "cos_buf"), _ptr(sin_buf, "sin_buf"), num_tokens,
                                      num_heads, head_dim, seq_len, _stream(stream)))


def flash_attn_fwd(output, lse_out, q, k, v, B, T, num_heads, head_dim, window_size, stream=None):
    """ops.mojo:244-255."""
    _lib.check(_lib.lib().ar_flash_attn_fwd(_ptr(output, "output"), _ptr(lse_out, "lse_out"), _ptr(q, "q"),
                                            _ptr(k, "k"), _ptr(v, "v"), B, T, num_heads, head_dim,
                                            window_size, _stream(stream)))


def flash_attn_bwd_precompute_d(d_out, output, grad_output, B, T, num_heads, head_dim, stream=None):
    """ops.mojo:329-337."""
    _lib.check(_lib.lib().ar_flash_attn_bwd_precompute_d(_ptr(d_out, "d_out"), _ptr(output, "output"),
                                                         _ptr(grad_output, "grad_output"), B, T, num_heads,
                                                         head_dim, _stream(stream)))


def flash_attn_bwd_dq(grad_q, q, k, v, grad_output, lse, d_buf, B, T, num_heads, head_dim, window_size,
                      stream=None):
    """ops.mojo:349-362."""
    _lib.check(_lib.lib().ar_flash_attn_bwd_dq(_ptr(grad_q, "grad_q"), _ptr(q, "q"), _ptr(k, "k"), _ptr(v, "v"),
                                               _ptr(grad_output, "grad_output"), _ptr(lse, "lse"),
                                               _ptr(d_buf, "d_buf"), B, T, num_heads, head_dim, window_size,
                                               _stream(stream)))


def flash_attn_bwd_dkv(grad_k, grad_v, q, k, v, grad_output, lse, d_buf, B, T, num_heads, head_dim,
                       window_size, stream=None):
    """ops.mojo:414-428."""
    _lib.check(_lib.lib().ar_flash_attn_bwd_dkv(_ptr(grad_k, "grad_k"), _ptr(grad_v, "grad_v"), _ptr(q, "q"),
                                                _ptr(k, "k"), _ptr(v, "v"), _ptr(grad_output, "grad_output"),
                                                _ptr(lse, "lse"), _ptr(d_buf, "d_buf"), B, T, num_heads,
                                                head_dim, window_size, _stream(stream)))


def _mat(t: torch.Tensor, name: str, shape, dtypes=(torch.float32, torch.bfloat16)) -> int:
    if not isinstance(t, torch.Tensor) or not t.is_cuda or not t.is_contiguous():
        raise ValueError(f"{name} must be a contiguous CUDA tensor")
    if tuple(t.shape) != tuple(shape):
        raise ValueError(f"{name} has shape {tuple(t.shape)}, expected {tuple(shape)}")
    if t.dtype not in dtypes:
        raise ValueError(f"{name} has dtype {t.dtype}")
    return t.data_ptr()


def _dt(t: torch.Tensor) -> int:
    return _lib.AR_F32 if t.dtype == torch.float32 else _lib.AR_BF16


def linear_fwd(output, input, weight, M, N, K, stream=None):
    """ops.mojo:110-117: output[M,N] = input[M,K] weight[N,K]^T.  input and weight share a dtype
    (fp32 or bf16); output fp32 or bf16."""
    if input.dtype != weight.dtype:
        raise ValueError("input and weight must share a dtype")
    with torch.cuda.device(input.device):
        _lib.check(_lib.lib().ar_linear_fwd(_mat(output, "output", (M, N)), _mat(input, "input", (M, K)),
                                            _mat(weight, "weight", (N, K)), M, N, K, _dt(input), _dt(output),
                                            _stream(stream)))


def linear_bwd_dx(grad_input, grad_output, weight, M, N, K, stream=None):
    """ops.mojo:870-878: grad_input[M,K] = grad_output[M,N] weight[N,K]."""
    if grad_output.dtype != weight.dtype:
        raise ValueError("grad_output and weight must share a dtype")
    with torch.cuda.device(weight.device):
        _lib.check(_lib.lib().ar_linear_bwd_dx(_mat(grad_input, "grad_input", (M, K)), _mat(grad_output, "grad_output", (M, N)),
                                               _mat(weight, "weight", (N, K)), M, N, K, _dt(weight), _dt(grad_input),
                                               _stream(stream)))


def linear_bwd_dw(grad_weight, grad_output, input, M, N, K, stream=None):
    """ops.mojo:953-961: grad_weight[N,K] += grad_output[M,N]^T input[M,K] (fp32, accumulated)."""
    if grad_output.dtype != input.dtype:
        raise ValueError("grad_output and input must share a dtype")
    with torch.cuda.device(input.device):
        _lib.check(_lib.lib().ar_linear_bwd_dw(_mat(grad_weight, "grad_weight", (N, K), (torch.float32,)),
                                               _mat(grad_output, "grad_output", (M, N)), _mat(input, "input", (M, K)),
                                               M, N, K, _dt(input), _stream(stream)))
