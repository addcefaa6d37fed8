"""Mamba-2 mixer on the ragged recurrent kernels: one projection ``[z | x | B | C | dt]``, a short causal convolution (+ bias, SiLU) over
``[x | B | C]``, and per head the state-space recurrence

    dt_t = softplus(dt_t + dt_bias)                           (no clamp)
    S_t  = exp(-exp(A_log) dt_t) S_(t-1) + dt_t B_t x_t^T      S: [state, head_dim], fp32
    y_t  = S_t^T C_t + D x_t

with head ``h`` reading B / C group ``h // (heads / groups)``; then ``y * silu(z)`` (gate first), an RMS norm in ``norm_groups`` equal parts of
the inner width times a weight, and the output projection.

The framework's other Mamba-2 path (``models/mamba.py``) runs prompts through a chunked PyTorch formulation and keeps one stacked state
tensor for equal layers.  This mixer serves prompt portions, single decode tokens and mixed batches with the same two kernels
(``ops.causal_conv1d`` and ``ops.mamba2_scan``, csrc/kernels/mamba.cu) and takes the convolution history and the matrix state from a
``LayeredStatePool`` row per request slot, addressed by ``state_idx``: a layer that runs several times per forward (weight-shared loops) owns
one pool entry per run.  Step size, decay, state, skip and gate are fp32; the projection and the convolution inputs are in the model dtype.
"""
from __future__ import annotations

from typing import Optional

import torch
from torch import nn

from .. import ops
from ..model_executor.forward_batch import ForwardBatch


class Mamba2ScanMixer(nn.Module):
    def __init__(self, width: int, heads: int, head_dim: int, state: int, groups: int, taps: int, norm_groups: int, eps: float, dtype,
                 conv_bias: bool = True):
        super().__init__()
        assert heads % groups == 0 and (heads * head_dim) % norm_groups == 0
        self.H, self.P, self.N, self.G, self.taps, self.norm_groups, self.eps = heads, head_dim, state, groups, taps, norm_groups, eps
        self.inner = heads * head_dim
        self.conv_dim = self.inner + 2 * groups * state
        self.dtype = dtype
        mk = lambda *s: nn.Parameter(torch.zeros(*s, dtype=dtype), requires_grad=False)
        f32 = lambda *s: nn.Parameter(torch.zeros(*s, dtype=torch.float32), requires_grad=False)
        self.in_weight = mk(2 * self.inner + 2 * groups * state + heads, width)          # rows [z | x | B | C | dt]
        self.conv_weight = mk(self.conv_dim, taps)
        self.conv_bias = mk(self.conv_dim) if conv_bias else None
        self.dt_bias, self.A_log, self.D = f32(heads), f32(heads), f32(heads)
        self.norm_weight = nn.Parameter(torch.ones(self.inner, dtype=dtype), requires_grad=False)
        self.o_weight = mk(width, self.inner)

    # ---- geometry for the recurrent-state pool: (conv channels, taps, heads, state rows, head_dim)
    def state_geometry(self):
        return (self.conv_dim, self.taps, self.H, self.N, self.P)

    def load(self, leaf: str, w: torch.Tensor) -> bool:
        name = {"in": "in_weight", "conv": "conv_weight", "conv.b": "conv_bias", "dt_bias": "dt_bias", "A_log": "A_log", "D": "D", "norm": "norm_weight",
                "o": "o_weight"}.get(leaf)
        if name is None or getattr(self, name) is None:
            return False
        p = getattr(self, name)
        p.data.copy_(w.to(p.dtype).reshape(p.shape))
        return True

    def forward(self, h: torch.Tensor, fb: ForwardBatch, state_idx: int) -> torch.Tensor:
        pool = fb.kv_pool.mamba
        inner, cd = self.inner, self.conv_dim
        proj = ops.linear(h, self.in_weight)                                     # [T, z | x B C | dt]
        xbc = proj[:, inner:inner + cd]
        if self.taps > 1:
            u = ops.causal_conv1d(xbc, self.conv_weight, self.conv_bias, pool.conv[state_idx], fb.cu_q, fb.req_slots, fb.seq_lens, fb.max_q_len, silu=True)
        else:
            a = xbc.float() * self.conv_weight[:, 0].float()
            u = torch.nn.functional.silu(a + self.conv_bias.float() if self.conv_bias is not None else a).contiguous()
        y = ops.mamba2_scan(u, proj[:, :inner], proj[:, inner + cd:], self.dt_bias, self.A_log, self.D, pool.ssm[state_idx], fb.req_slots, fb.seq_lens,
                            fb.cu_q, fb.q_lens, self.H, self.P, self.N, self.G)
        y = ops.grouped_rmsnorm(y, self.norm_weight, self.norm_groups, self.eps, h.dtype)
        return ops.linear(y, self.o_weight)
