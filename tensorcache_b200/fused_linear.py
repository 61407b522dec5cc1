"""``FusedDequantLinear``: dequantise + GEMM in one tcgen05 kernel, no bf16 intermediate in HBM.

Mirrors ``FusedDequantLinear`` of the reference (src/tensorcache/fused_ops.py:1406-1461):
``forward(q, scales)`` computes ``dequant(q) @ weight.T + bias`` for a quantised
*activation* ``q`` (signed int8 codes, one bf16 scale per ``group_size`` values
along the last dimension) and a dense bf16 ``weight``.  On top of that:

* ``forward(q, scales, zero_points)`` takes AMO-BQ codes (uint8 + zero points);
* ``fused_dequant_matmul(x, wq, ws, wzp)`` is the quantised-*weight* form
  ``x @ dequant(W).T`` used when the weight matrix is what sits in the cache.

Both run the same kernel: the operand whose rows are the output's rows becomes the
M side of the tensor-core tile, so either form stores row-contiguous vectors.  The
inner dimension must be a multiple of the group size.
"""
from __future__ import annotations

import ctypes
import math
from typing import Optional

import torch
import torch.nn as nn

from . import _lib

SUPPORTED_GROUP_SIZES = (16, 32, 64, 128)  # group sizes the tensor-core kernel is instantiated for


def _ptr(t: Optional[torch.Tensor]):
    return ctypes.c_void_p(t.data_ptr() if t is not None else 0)


def _aligned(t: Optional[torch.Tensor], nbytes: int = 16) -> Optional[torch.Tensor]:
    """The TMA descriptors need 16-byte aligned operands.  A contiguous view into a larger tensor (``w[1:]``,
    ``q[3:]``) can start anywhere, so such an operand is copied once; aligned tensors pass through untouched."""
    if t is None or t.data_ptr() % nbytes == 0:
        return t
    return t.clone(memory_format=torch.contiguous_format)


def _launch(dense, q, scales, zp, bias, out, R_d, R_q, K, group_size, quant_is_rhs):
    dense, q = _aligned(dense), _aligned(q)
    dev = dense.device
    with torch.cuda.device(dev):
        stream = ctypes.c_void_p(torch.cuda.current_stream(dev).cuda_stream)
        _lib.check(_lib.lib().tcb_fused_dequant_linear(_ptr(dense), _ptr(q), _ptr(scales), _ptr(zp), _ptr(bias), _ptr(out),
                                                       R_d, R_q, K, group_size, 1 if quant_is_rhs else 0, stream))


def _check_common(codes, scales, zp, K, rows, group_size):
    if group_size not in SUPPORTED_GROUP_SIZES:
        raise ValueError(f"group_size {group_size} is not supported, choose from {SUPPORTED_GROUP_SIZES}")
    if K <= 0 or K % group_size != 0:
        raise ValueError(f"the inner dimension ({K}) must be a positive multiple of the group size {group_size}")
    groups = rows * K // group_size
    if scales.numel() != groups or scales.dtype != torch.bfloat16:
        raise ValueError(f"expected {groups} bf16 scales, got {scales.numel()} of {scales.dtype}")
    if zp is not None:
        if codes.dtype != torch.uint8 or zp.dtype != torch.uint8 or zp.numel() != groups:
            raise ValueError("AMO-BQ operands are uint8 codes with one uint8 zero point per group")
    elif codes.dtype != torch.int8:
        raise ValueError("without zero points the codes must be signed int8 (symmetric quantisation)")
    if not codes.is_cuda:
        raise RuntimeError("FusedDequantLinear runs on CUDA tensors only (no CPU fallback)")


def check_device_status(device=None) -> None:
    """Raises if a bounded wait inside the fused kernel ran out (synchronises the current stream)."""
    dev = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
    with torch.cuda.device(dev):
        _lib.check(_lib.lib().tcb_fused_dequant_linear_check(ctypes.c_void_p(torch.cuda.current_stream(dev).cuda_stream)))


def fused_dequant_matmul(x: torch.Tensor, wq: torch.Tensor, w_scales: torch.Tensor, w_zero_points: Optional[torch.Tensor] = None,
                         bias: Optional[torch.Tensor] = None, group_size: int = 32) -> torch.Tensor:
    """``x @ dequant(W).T (+ bias)`` with W stored as codes ``wq [N, K]`` quantised along K.

    ``x`` is bf16 ``[..., K]``; the result is bf16 ``[..., N]``.
    """
    N, K = wq.shape
    _check_common(wq, w_scales, w_zero_points, K, N, group_size)
    lead = x.shape[:-1]
    x2 = x.reshape(-1, K)
    if x2.dtype != torch.bfloat16:
        raise ValueError("x must be bf16")
    x2 = x2.contiguous()
    M = x2.shape[0]
    out = torch.empty((M, N), dtype=torch.bfloat16, device=x.device)
    if M and N:
        b = None if bias is None else bias.to(torch.bfloat16).contiguous()
        _launch(x2, wq.contiguous(), w_scales.contiguous().view(-1), None if w_zero_points is None else w_zero_points.contiguous().view(-1),
                b, out, M, N, K, group_size, True)
    return out.view(*lead, N)


class FusedDequantLinear(nn.Module):
    """``y = dequant(q) @ weight.T + bias`` with the dequantisation fused into the GEMM."""

    def __init__(self, in_features: int, out_features: int, bias: bool = True, group_size: int = 32):
        super().__init__()
        self.in_features = in_features
        self.out_features = out_features
        self.group_size = group_size
        self.weight = nn.Parameter(torch.empty((out_features, in_features), dtype=torch.bfloat16))
        if bias:
            self.bias = nn.Parameter(torch.empty(out_features, dtype=torch.bfloat16))
        else:
            self.register_parameter("bias", None)
        nn.init.kaiming_uniform_(self.weight, a=math.sqrt(5))
        if self.bias is not None:
            nn.init.zeros_(self.bias)

    def forward(self, q_int8: torch.Tensor, scales: torch.Tensor, zero_points: Optional[torch.Tensor] = None) -> torch.Tensor:
        orig_shape = q_int8.shape[:-1]
        x_2d = q_int8.reshape(-1, self.in_features).contiguous()
        M, K = x_2d.shape
        N = self.out_features
        _check_common(x_2d, scales, zero_points, K, M, self.group_size)
        out = torch.empty((M, N), dtype=torch.bfloat16, device=q_int8.device)
        if M and N:
            _launch(self.weight.detach().contiguous(), x_2d, scales.contiguous().view(-1),
                    None if zero_points is None else zero_points.contiguous().view(-1),
                    None if self.bias is None else self.bias.detach().contiguous(), out, N, M, K, self.group_size, False)
        if len(orig_shape) == 0:
            return out
        return out.view(*orig_shape, N)
