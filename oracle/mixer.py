"""CPU restatement (torch, any float dtype) of the mixer steps either side of the scan.

TEST INFRASTRUCTURE ONLY: imported by tests/, the smoke check and the CPU-baseline leg of the
benchmark; the product path never touches this module.

Pinned by tests/golden/conv_silu.npz and tests/golden/mixer_core.npz, which hold outputs of the
reference's own PyTorch port (bench/torch_mamba3.py:165-207) - see tests/golden/make_golden.py.
"""
from __future__ import annotations

from typing import Optional

import torch
import torch.nn.functional as F

from . import m3_oracle as O


def causal_conv1d(x, weight, bias=None, history=None, activation: bool = True):
    """Depthwise causal convolution as a sum of zero-padded shifts, each scaled by its tap:
    CausalConv1d::apply_composed, src/nn/conv.rs:152-176 (tap k pairs with delay K-1-k), continued
    from `history` [B, K-1, C] as apply_with_history (:185-203), then the mixer's SiLU
    (src/models/mamba3.rs:401).  x [B, T, C]; weight [K, C]; bias [C].
    Returns (y [B, T, C], new_history [B, K-1, C])."""
    B, T, C = x.shape
    K = weight.shape[0]
    past = history if history is not None else x.new_zeros(B, K - 1, C)
    full = torch.cat([past, x], dim=1)                     # time index t maps to t + K - 1
    acc = None
    for delay in range(K):
        term = full[:, K - 1 - delay: K - 1 - delay + T] * weight[K - 1 - delay].reshape(1, 1, C)
        acc = term if acc is None else acc + term
    if bias is not None:
        acc = acc + bias.reshape(1, 1, C)
    y = F.silu(acc) if activation else acc
    return y, full[:, full.shape[1] - (K - 1):]
