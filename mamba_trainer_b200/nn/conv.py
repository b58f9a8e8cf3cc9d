"""Depthwise causal convolution + SiLU, the step in front of the scan.

Mirrors CausalConv1d of the reference (src/nn/conv.rs:89-232): weight [kernel_size, channels],
optional per-channel bias, apply / apply_with_history / step / empty_history.  The arithmetic runs
in libm3scan (m3_conv_forward / m3_conv_backward); there is no fallback.
"""
from __future__ import annotations

import ctypes as C
from typing import Optional, Tuple

import torch

from .. import _ffi
from ..error import ShapeError, UnsupportedError
from ..ssm.scan import Context, _DTYPES


def _ptr(t: Optional[torch.Tensor]):
    return C.c_void_p(t.data_ptr()) if t is not None else None


def _rows(t: torch.Tensor) -> int:
    """Row stride (elements between consecutive time steps) of a [B, T, C] view whose channels are
    contiguous and whose batches follow each other without a gap."""
    B, T, Cn = t.shape
    if t.stride(2) != 1 and Cn > 1:
        raise ShapeError("channels must be contiguous")
    rs = t.stride(1) if T > 1 else Cn
    if B > 1 and T > 0 and t.stride(0) != T * rs:
        raise ShapeError("batches must follow each other at seq * row stride")
    return rs


class _FusedConv(torch.autograd.Function):
    @staticmethod
    def forward(fctx, x, weight, bias, history, activation, want_history):
        ctx = Context.for_device(x.device)
        B, T, Cn = x.shape
        K = weight.shape[0]
        y = torch.empty((B, T, Cn), device=x.device, dtype=x.dtype)
        new_hist = torch.empty((B, K - 1, Cn), device=x.device, dtype=x.dtype) if want_history else None
        desc = _ffi.ConvDesc(batch=B, seq=T, channels=Cn, kernel_size=K, dtype=_DTYPES[x.dtype],
                             activation=1 if activation else 0, x_stride=_rows(x), y_stride=Cn,
                             x=_ptr(x), history=_ptr(history), weight=_ptr(weight), bias=_ptr(bias))
        ctx.check(ctx.lib.m3_conv_forward(ctx.handle, C.byref(desc), _ptr(y), _ptr(new_hist)))
        fctx.save_for_backward(x, weight, bias, history)
        fctx.activation = activation
        if want_history:
            fctx.mark_non_differentiable(new_hist)
            return y, new_hist
        return y

    @staticmethod
    def backward(fctx, dy, *_unused):
        x, weight, bias, history = fctx.saved_tensors
        ctx = Context.for_device(x.device)
        B, T, Cn = x.shape
        K = weight.shape[0]
        dy = dy.contiguous()
        need = fctx.needs_input_grad
        dx = torch.empty((B, T, Cn), device=x.device, dtype=x.dtype) if need[0] else None
        dw = torch.empty((K, Cn), device=x.device, dtype=torch.float32) if need[1] else None
        db = torch.empty((Cn,), device=x.device, dtype=torch.float32) if (bias is not None and need[2]) else None
        dh = torch.empty_like(history) if (history is not None and need[3]) else None
        xc = x if dx is None else x.contiguous()   # dx is written dense, with x's row stride
        desc = _ffi.ConvDesc(batch=B, seq=T, channels=Cn, kernel_size=K, dtype=_DTYPES[x.dtype],
                             activation=1 if fctx.activation else 0, x_stride=_rows(xc), y_stride=Cn,
                             x=_ptr(xc), history=_ptr(history), weight=_ptr(weight), bias=_ptr(bias))
        ctx.check(ctx.lib.m3_conv_backward(ctx.handle, C.byref(desc), _ptr(dy), _ptr(dx), _ptr(dw), _ptr(db), _ptr(dh)))
        return dx, dw, db, dh, None, None


def causal_conv1d(x: torch.Tensor, weight: torch.Tensor, bias: Optional[torch.Tensor] = None,
                  history: Optional[torch.Tensor] = None, activation: bool = True, want_history: bool = False):
    """y = act(conv(x)) over [batch, seq, channels]; weight [K, channels] float32, bias [channels]
    float32.  `x` may be a column band of a wider tensor (channels contiguous).  With want_history
    also returns the [batch, K-1, channels] inputs the next window continues from."""
    if x.dim() != 3:
        raise ShapeError(f"CausalConv1d expects [batch, seq, channels], got {tuple(x.shape)}")
    if x.dtype not in _DTYPES:
        raise UnsupportedError(f"element type {x.dtype}: float32 and bfloat16 are served")
    K, Cn = weight.shape
    if x.shape[2] != Cn:
        raise ShapeError(f"CausalConv1d expects {Cn} channels, got {tuple(x.shape)}")
    if not 1 <= K <= 8:
        raise UnsupportedError(f"kernel_size {K} outside [1, 8]")
    if history is not None and tuple(history.shape) != (x.shape[0], K - 1, Cn):
        raise ShapeError(f"history has shape {tuple(history.shape)}, expected {(x.shape[0], K - 1, Cn)}")
    try:
        _rows(x)
    except ShapeError:
        x = x.contiguous()
    w32 = weight.to(torch.float32).contiguous()
    b32 = bias.to(torch.float32).contiguous() if bias is not None else None
    hist = history.to(x.dtype).contiguous() if history is not None else None
    return _FusedConv.apply(x, w32, b32, hist, bool(activation), bool(want_history))


class CausalConv1d(torch.nn.Module):
    """src/nn/conv.rs:89-232.  Parameters are float32 masters; activations may be bfloat16."""

    def __init__(self, channels: int, kernel_size: int, bias: bool = True, device=None):
        super().__init__()
        self.channels, self.kernel_size = channels, kernel_size
        bound = 1.0 / kernel_size ** 0.5
        self.weight = torch.nn.Parameter((torch.rand(kernel_size, channels, device=device) * 2 - 1) * bound)
        self.bias = torch.nn.Parameter(torch.zeros(channels, device=device)) if bias else None

    def apply_conv(self, x: torch.Tensor, activation: bool = False) -> torch.Tensor:
        """CausalConv1d::apply (:143-150); activation=True fuses the mixer's SiLU."""
        return causal_conv1d(x, self.weight, self.bias, None, activation)

    forward = apply_conv

    def apply_with_history(self, x: torch.Tensor, history: torch.Tensor, activation: bool = False
                           ) -> Tuple[torch.Tensor, torch.Tensor]:
        """:185-203: the output for the new positions and the history to carry forward."""
        return causal_conv1d(x, self.weight, self.bias, history, activation, want_history=True)

    def step(self, x: torch.Tensor, history: torch.Tensor, activation: bool = False):
        """:206-212: one decoding step; x holds a single position."""
        return self.apply_with_history(x, history, activation)

    def empty_history(self, batch: int, device=None, dtype=torch.float32) -> torch.Tensor:
        """:215-221."""
        return torch.zeros((batch, self.kernel_size - 1, self.channels), device=device, dtype=dtype)
