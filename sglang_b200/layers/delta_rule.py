"""Gated delta-rule mixer: a linear-attention layer whose per-head matrix state ``S`` [key_dim, value_dim] is corrected, not just
accumulated, by every token:

    S <- g_t * S                      (decay: one number per head, or one per head and key channel acting on the rows of S)
    w  = beta_t * (v_t - S^T k_t)     (what the state gets wrong about v_t, scaled by the write strength)
    S <- S + k_t w^T
    o_t = S^T q_t                     (read after the write)

with ``q``, ``k``, ``v`` = projection -> short causal convolution over time -> SiLU, ``q`` and ``k`` unit vectors per head (``q`` also divided by
sqrt(key_dim)), ``beta = sigmoid(W_b h)``, ``g = exp(-exp(A_log) * softplus(a + dt_bias))``, and the output normalised per head (RMS over
value_dim, a weight shared by the heads) and gated.  Two parameterisations share the module:

* ``decay="head"``:    ``a = W_a h`` (one per head), gate ``silu(W_g h)``;
* ``decay="channel"``: ``a = W_a2 (W_a1 h)`` (low rank, one per head and key channel), gate ``sigmoid(W_g2 (W_g1 h))``.

Serving layout: the q/k/v projections are one GEMM and one convolution over the concatenated channels ([q | k | v]); the small projections
(gate, beta, decay) are a second GEMM.  The convolution's last ``taps - 1`` inputs and the fp32 matrix state live in the recurrent-state
pool by request slot (``mem_cache/memory_pool.py``), so a prompt cut into portions, decoding, and mixed batches all run the same two
kernels: ``ops.causal_conv1d`` (csrc/kernels/mamba.cu) and ``ops.gated_delta_rule`` (csrc/kernels/delta_rule.cu: normalisation, decay,
recurrence, output norm and gate fused; everything that enters the recurrence is fp32).
"""
from __future__ import annotations

from typing import Optional

import torch
from torch import nn

from .. import ops
from ..model_executor.forward_batch import ForwardBatch


class GatedDeltaMixer(nn.Module):
    def __init__(self, width: int, heads: int, kv_heads: int, dim: int, vdim: int, taps: int, decay: str, eps: float, state_idx: int, dtype,
                 rank: Optional[int] = None):
        super().__init__()
        assert decay in ("head", "channel") and heads % kv_heads == 0
        self.H, self.Hk, self.Dk, self.Dv, self.taps, self.decay, self.eps = heads, kv_heads, dim, vdim, taps, decay, eps
        self.state_idx = state_idx                      # index into the recurrent-state pool
        self.key_dim, self.value_dim = kv_heads * dim, heads * vdim
        self.conv_dim = 2 * self.key_dim + self.value_dim
        self.width, self.dtype = width, dtype
        mk = lambda *s: nn.Parameter(torch.zeros(*s, dtype=dtype), requires_grad=False)
        f32 = lambda *s: nn.Parameter(torch.zeros(*s, dtype=torch.float32), requires_grad=False)
        self.qkv_weight = mk(self.conv_dim, width)
        self.conv_weight = mk(self.conv_dim, taps)
        self.A_log = f32(heads)
        self.norm_weight = nn.Parameter(torch.ones(vdim, dtype=dtype), requires_grad=False)
        self.o_weight = mk(width, self.value_dim)
        self.b_weight = mk(heads, width)
        if decay == "head":
            self.g_weight, self.a_weight = mk(self.value_dim, width), mk(heads, width)
            self.dt_bias = f32(heads)
            self.gate_act = "silu"
        else:
            # low-rank decay and gate: the inner widths are properties of the checkpoint's tensors (``load`` resizes to them)
            r = rank or 16
            self.g_weight, self.g_up = mk(r, width), mk(self.value_dim, r)
            self.a_weight, self.a_up = mk(r, width), mk(heads * dim, r)
            self.dt_bias = f32(heads * dim)
            self.gate_act = "sigmoid"
        self._aux = None                 # [gate | decay | beta] projection rows stacked for one GEMM (built on first use)

    def _fit(self, name: str, w: torch.Tensor) -> None:
        p = getattr(self, name)
        if tuple(p.shape) != tuple(w.shape):
            assert self.decay == "channel" and name in ("g_weight", "g_up", "a_weight", "a_up"), (name, tuple(p.shape), tuple(w.shape))
            setattr(self, name, nn.Parameter(torch.zeros(*w.shape, dtype=p.dtype, device=p.device), requires_grad=False))
        getattr(self, name).data.copy_(w)
        self._aux = None

    # ---- geometry for the recurrent-state pool: (conv channels, taps, heads, key dim, value dim)
    def state_geometry(self):
        return (self.conv_dim, self.taps, self.H, self.Dk, self.Dv)

    def load(self, leaf: str, w: torch.Tensor) -> bool:
        kd, vd, H = self.key_dim, self.value_dim, self.H
        rows = {"q": (0, kd), "k": (kd, 2 * kd), "v": (2 * kd, 2 * kd + vd)}
        if leaf in rows:
            a, b = rows[leaf]
            self.qkv_weight.data[a:b].copy_(w)
        elif leaf.endswith(".conv") and leaf[:-5] in rows:
            a, b = rows[leaf[:-5]]
            self.conv_weight.data[a:b].copy_(w)
        elif leaf in ("A_log", "dt_bias"):
            getattr(self, leaf).data.copy_(w.float())
        elif leaf == "norm":
            self.norm_weight.data.copy_(w)
        elif leaf == "o":
            self.o_weight.data.copy_(w)
        elif leaf == "b":
            self._fit("b_weight", w)
        elif self.decay == "head" and leaf in ("g", "a"):
            self._fit(leaf + "_weight", w)
        elif self.decay == "channel" and leaf in ("g1", "a1", "g2", "a2"):
            self._fit(leaf[0] + ("_weight" if leaf[1] == "1" else "_up"), w)
        else:
            return False
        return True

    def forward(self, h: torch.Tensor, fb: ForwardBatch) -> torch.Tensor:
        pool = fb.kv_pool.mamba
        T, H, vd = h.shape[0], self.H, self.value_dim
        mixed = ops.linear(h, self.qkv_weight)                                  # [T, q | k | v]
        if self.taps > 1:
            u = ops.causal_conv1d(mixed, self.conv_weight, None, pool.conv[self.state_idx], fb.cu_q, fb.req_slots, fb.seq_lens, fb.max_q_len, silu=True)
        else:
            u = torch.nn.functional.silu(mixed.float() * self.conv_weight[:, 0].float())
        if self._aux is None or self._aux.device != h.device:
            self._aux = torch.cat([self.g_weight.data, self.a_weight.data, self.b_weight.data], 0).contiguous()
        aux = ops.linear(h, self._aux)
        ng, na = self.g_weight.shape[0], self.a_weight.shape[0]
        gate_raw, a_raw, b_raw = aux[:, :ng], aux[:, ng:ng + na], aux[:, ng + na:]
        if self.decay == "channel":
            gate_raw = ops.linear(gate_raw.contiguous(), self.g_up)
            a_raw = ops.linear(a_raw.contiguous(), self.a_up)
        o = ops.gated_delta_rule(u, self.Hk, self.Dk, H, self.Dv, a_raw, self.A_log, self.dt_bias, b_raw, pool.ssm[self.state_idx], fb.req_slots,
                                 fb.seq_lens, fb.cu_q, fb.q_lens, gate_raw, self.norm_weight, self.eps, self.gate_act, self.decay == "channel")
        return ops.linear(o.view(T, vd).to(h.dtype), self.o_weight)
