"""Grouped-query attention without positional rotation whose scores carry the position instead:

    q, k      each head divided by its root mean square (no weight);  q_i also times  1 + coef * ln(floor((i + 1) / every) + 1)
    s_ij      = cap * tanh(q_i . k_j * scale / cap)  -  slope_h * (i - j)            slope_h = 2^(-8 (h + 1) / H)
    visible   0 <= i - j < window
    p_ij      = exp(s_ij) / (exp(sink_h) + sum_j' exp(s_ij'))                          the sink has no key and no value

The projections are one GEMM with their biases in the epilogue; ``ops.qk_norm_cache_write`` normalises q and k, applies the query
temperature and writes k / v rows into the paged pool; ``ops.window_attention`` (csrc/kernels/window_attention.cu) is the attention itself,
one kernel for prompt portions and decode tokens.  Cap, bias, mask, sink and soft-max are fp32; the cache is in the model dtype.  bf16
models whose key and value heads are at most 128 wide run the framework's tcgen05 attention kernels instead (``ops.paged_attention`` with
``slopes``: the distance bias joins their score pass behind the cap, the sink enters through the log-sum-exp).  Those kernels have 128-wide
heads, so such a layer lays its heads out 128 columns wide in q and in the cache rows, zeros behind the values (``pad``): the scores do not
change, the output's first ``vdim`` columns are the result, and a 64-wide head pays twice the cache bytes and tensor-core work for leaving
the CUDA-core kernel (about 3x faster on prompts at that size).  Every other size (heads wider than 128, group sizes that do not divide 128),
fp32 serving, and any call the tcgen05 kernels do not take stay on the general kernel, which reads the same layout.

The paged pool holds one flat row per token and plane (``cache_width`` columns, the widest layer's ``kv_heads * max(dim, vdim)``, or
``kv_heads * 128`` for padded layers): a layer reads the first columns of the key plane as its key heads, so layers of different head counts
and sizes share one pool.
``cache_idx`` selects the pool layer: a layer that runs several times per forward owns one pool layer per run.  The window only masks — pages
behind the window stay with the request until it ends.
"""
from __future__ import annotations

from typing import Optional

import torch
from torch import nn

from .. import ops
from ..model_executor.forward_batch import ForwardBatch


class FlatCacheSpec:
    """what the model runner reads to size the paged pool: one "KV head" of ``cache_width`` per token in a key and a value plane"""

    def __init__(self, num_heads: int, cache_width: int, layer_id: int, scale: float, window: int):
        self.num_heads, self.num_kv_heads, self.head_dim, self.kv_head_dim = num_heads, 1, cache_width, cache_width
        self.latent_v_dim = 0
        self.layer_id, self.scale, self.window, self.logit_cap, self.rope, self.sinks = layer_id, scale, window, 0.0, None, None


def distance_slopes(heads: int, base: float = 8.0) -> torch.Tensor:
    """slope_h = 2^(-base (h + 1) / heads), h = 0 .. heads - 1"""
    return torch.pow(2.0, -base * torch.arange(1, heads + 1, dtype=torch.float64) / heads).float()


class BiasedWindowAttention(nn.Module):
    tc_route = True            # class-wide switch of the tcgen05 route (tests compare it with the general kernel)

    def __init__(self, width: int, heads: int, kv_heads: int, dim: int, vdim: int, scale: Optional[float], softcap: float, window: int, eps: float,
                 dtype, temp_coef: float = 0.0, temp_every: int = 1, qk_norm: bool = True, distance_bias: bool = True, sinks: bool = True,
                 bias: bool = True):
        super().__init__()
        assert heads % kv_heads == 0
        self.H, self.G, self.D, self.Dv = heads, kv_heads, dim, vdim
        self.eps, self.softcap, self.window = eps, float(softcap or 0.0), int(window or -1)
        self.scale = float(scale) if scale is not None else dim ** -0.5
        self.temp_coef, self.temp_every, self.qk_norm = float(temp_coef), int(temp_every), qk_norm
        n = heads * dim + kv_heads * dim + kv_heads * vdim
        self.qkv_weight = nn.Parameter(torch.zeros(n, width, dtype=dtype), requires_grad=False)          # rows [q | k | v]: one GEMM
        self.qkv_bias = nn.Parameter(torch.zeros(n, dtype=dtype), requires_grad=False) if bias else None
        self.o_weight = nn.Parameter(torch.zeros(width, heads * vdim, dtype=dtype), requires_grad=False)
        self.sinks = nn.Parameter(torch.zeros(heads, dtype=torch.float32), requires_grad=False) if sinks else None
        self.slopes = nn.Parameter(distance_slopes(heads), requires_grad=False) if distance_bias else None
        self.pad = 0                 # 128: heads laid out 128 columns wide for the tcgen05 kernels (the model decides, see ``wants_padding``)

    def wants_padding(self, dtype) -> bool:
        """whether this layer would run the tcgen05 kernels if its pool rows are ``kv_heads * 128`` wide"""
        return bool(self.tc_route and dtype == torch.bfloat16 and self.D <= 128 and self.Dv <= 128 and 128 % (self.H // self.G) == 0)

    @property
    def cache_width(self) -> int:
        return self.G * (self.pad if self.pad else max(self.D, self.Dv))

    def load(self, leaf: str, w: torch.Tensor) -> bool:
        hd, gd = self.H * self.D, self.G * self.D
        rows = {"q": (0, hd), "k": (hd, hd + gd), "v": (hd + gd, hd + gd + self.G * self.Dv)}
        if leaf in rows:
            a, b = rows[leaf]
            self.qkv_weight.data[a:b].copy_(w)
        elif leaf.endswith(".b") and leaf[:-2] in rows and self.qkv_bias is not None:
            a, b = rows[leaf[:-2]]
            self.qkv_bias.data[a:b].copy_(w)
        elif leaf == "sink" and self.sinks is not None:
            self.sinks.data.copy_(w.float())
        elif leaf == "o":
            self.o_weight.data.copy_(w)
        else:
            return False
        return True

    def forward(self, h: torch.Tensor, fb: ForwardBatch, cache_idx: int) -> torch.Tensor:
        T = h.shape[0]
        qkv = ops.linear(h, self.qkv_weight, self.qkv_bias)
        kc, vc = fb.kv_pool.k(cache_idx), fb.kv_pool.v(cache_idx)                  # [slots, 1, cache_width] each
        pad = self.pad
        q = ops.qk_norm_cache_write(qkv, self.H, self.G, self.D, self.Dv, fb.positions, self.eps, self.temp_coef, self.temp_every, kc, vc,
                                    fb.out_cache_loc, self.qk_norm, pad)
        if pad == 128 and kc.shape[-1] == self.G * 128:
            k4, v4 = kc.view(-1, self.G, 128), vc.view(-1, self.G, 128)
            if ops.tc_attention_ok(q, k4, v4, fb.page_size):
                # bf16, 128-wide heads: the framework's tcgen05 attention kernels (prompt tiles and split-KV decode) with the bias folded into
                # their score pass; the sink enters through the log-sum-exp: o * exp(lse) / (exp(lse) + exp(sink))
                lse = torch.empty(T, self.H, dtype=torch.float32, device=q.device) if self.sinks is not None else None
                dec = fb.cu_q is None
                o = ops.paged_attention(q, k4, v4, fb.page_table, fb.req_slots, fb.seq_lens, fb.cu_q, fb.q_lens, fb.max_q_len, fb.page_size, self.scale,
                                        causal=True, window=self.window, logit_cap=self.softcap, num_splits=fb.num_splits if dec else 1,
                                        workspace=fb.attn_workspace if dec else None, lse=lse, slopes=self.slopes)
                if lse is not None:
                    o = ops.attention_sink_gate(o, lse, self.sinks, self.Dv)
                elif self.Dv < 128:
                    o = o[:, :, : self.Dv]
                return ops.linear(o.reshape(T, self.H * self.Dv), self.o_weight)
        o = ops.window_attention(q, kc, vc, self.G, self.Dv, fb.page_table, fb.req_slots, fb.seq_lens, fb.cu_q, fb.q_lens, fb.max_q_len, fb.page_size,
                                 self.scale, self.softcap, self.window, self.slopes, self.sinks, self.D, pad)
        return ops.linear(o.view(T, self.H * self.Dv), self.o_weight)
