"""Rirotar: a decoder whose configuration lists its layers one by one.  Each layer is pre-norm,

    x <- x + mixer(norm1(x));   x <- x + ff(norm2(x))        (no second half when the layer has no feed-forward)

with the mixer one of

* ``latent_attention``: position-free latent attention with a sliding window and soft-max sinks (``layers/latent_attention.py``);
* ``delta``:            gated delta rule, one decay per head, SiLU output gate (``layers/delta_rule.py``, ``decay="head"``);
* ``channel_delta``:    gated delta rule, low-rank decay per head and key channel, sigmoid output gate (``decay="channel"``);

and the feed-forward either dense or a mixture of experts behind a group-limited sigmoid router (``layers/moe.py``), both with the clamped
GLU ``min(g, limit) * sigmoid(1.702 g) * (clamp(u, +-limit) + 1)``.  Norms are RMS norms with weights stored around zero (``1 + w``).  The
logits pass a tanh soft cap.

How it sits in the engine: the residual stream is fp32 on every path (``ops.add_rmsnorm_f32`` adds a branch's output to it and emits the next
norm in the GEMM dtype in one kernel); attention layers cache one latent row per token in the paged pool (``KVPool`` latent plane, width =
the largest ``kv_rank``); recurrent layers keep convolution history and matrix state in a ``LayeredStatePool`` by request slot, each
layer with its own geometry.  Prompt portions, decode steps and mixed batches are the same forward: every kernel is ragged over
``cu_q`` / ``seq_lens``.  Prefix caching is off (recurrent state has no page-aligned snapshot).  Tensor parallelism is not split for this
family (one rank holds the model).

Checkpoint names: ``embed``, ``l<i>.norm1|norm2``, ``l<i>.mix.*``, ``l<i>.mlp.{gate,up,down}`` or ``l<i>.mlp.e<j>.{gate,up,down}`` +
``l<i>.mlp.router``, ``final.norm``, ``head``; linear weights are [out, in].
"""
from __future__ import annotations

import zlib
from typing import Iterable, List, Optional, Tuple

import torch
from torch import nn

from .. import ops
from ..configs.model_config import ModelConfig
from ..layers.delta_rule import GatedDeltaMixer
from ..layers.latent_attention import WindowedLatentAttention
from ..layers.moe import FusedMoE, grouped_sigmoid_route
from ..mem_cache.memory_pool import LayeredStatePool
from ..model_executor.forward_batch import ForwardBatch
from ..parallel.parallel_state import get_pp_group, get_tp_group
from .llama import _DT

GLU_ALPHA = 1.702


class ZeroCentredNorm(nn.Module):
    """weight holder; the norm itself runs fused with the residual update (``ops.add_rmsnorm_f32``)"""

    def __init__(self, n: int, dtype):
        super().__init__()
        self.weight = nn.Parameter(torch.zeros(n, dtype=dtype), requires_grad=False)


class ClampedGLU(nn.Module):
    def __init__(self, width: int, ff: int, limit: float, dtype):
        super().__init__()
        self.gate_up = nn.Parameter(torch.zeros(2 * ff, width, dtype=dtype), requires_grad=False)        # rows [gate | up]: one GEMM
        self.down = nn.Parameter(torch.zeros(width, ff, dtype=dtype), requires_grad=False)
        self.ff, self.limit = ff, float(limit)

    def load(self, leaf: str, w: torch.Tensor) -> bool:
        if leaf == "gate":
            self.gate_up.data[: self.ff].copy_(w)
        elif leaf == "up":
            self.gate_up.data[self.ff:].copy_(w)
        elif leaf == "down":
            self.down.data.copy_(w)
        else:
            return False
        return True

    def forward(self, h: torch.Tensor) -> torch.Tensor:
        return ops.linear(ops.clamped_glu(ops.linear(h, self.gate_up), self.limit, GLU_ALPHA), self.down)


class GroupRoutedMoE(nn.Module):
    def __init__(self, width: int, mlp: dict, dtype, layer_id: int):
        super().__init__()
        r = mlp["router"]
        self.E, self.top, self.scale = int(r["experts"]), int(r["top"]), float(r.get("scale", 1.0))
        gr = r.get("groups") or {}
        self.n_groups, self.keep = int(gr.get("count", 1)), int(gr.get("keep", gr.get("count", 1)))
        self.limit = float(mlp["expert"]["limit"])
        self.router = nn.Parameter(torch.zeros(self.E, width, dtype=dtype), requires_grad=False)
        self.experts = FusedMoE(self.E, self.top, width, int(mlp["expert"]["ff"]), dtype, True, 1, None, layer_id)
        self.experts.act = ("clamped_glu", self.limit, GLU_ALPHA)
        self._router32 = None

    def load(self, leaf: str, w: torch.Tensor) -> bool:
        if leaf == "router":
            self.router.data.copy_(w)
            self._router32 = None
            return True
        head, _, proj = leaf.partition(".")
        if head[:1] == "e" and head[1:].isdigit() and proj in ("gate", "up", "down"):
            ex = self.experts
            ex.weight_loader(ex.w2 if proj == "down" else ex.w13, w, int(head[1:]), {"gate": "w1", "up": "w3", "down": "w2"}[proj])
            return True
        return False

    def forward(self, h: torch.Tensor) -> torch.Tensor:
        if self._router32 is None or self._router32.device != h.device:
            self._router32 = self.router.detach().float()
        logits = torch.nn.functional.linear(h.float(), self._router32)          # router in fp32 on the (possibly bf16-rounded) input
        w, ids = grouped_sigmoid_route(logits, self.top, self.n_groups, self.keep, self.scale)
        y = self.experts.forward_routed(h, w, ids)
        return y.resolve() if hasattr(y, "resolve") else y


class RirotarBlock(nn.Module):
    def __init__(self, cfg: ModelConfig, spec: dict, idx: int, local_idx: int, dtype, cache_width: int):
        super().__init__()
        W, m, eps = cfg.hidden_size, spec["mixer"], cfg.rms_norm_eps
        kind = spec["type"]
        self.norm1 = ZeroCentredNorm(W, dtype)
        if kind == "latent_attention":
            self.kind = "attention"
            self.self_attn = WindowedLatentAttention(W, int(m["heads"]), int(m["dim"]), int(m["vdim"]), int(m["kv_rank"]), m.get("scale"),
                                                     int((m.get("mask") or {}).get("size") or -1), eps, local_idx, dtype, cache_width)
            self.mix = self.self_attn
        elif kind in ("delta", "channel_delta"):
            self.kind = "mamba"
            self.mix = GatedDeltaMixer(W, int(m["heads"]), int(m.get("kv_heads", m["heads"])), int(m["dim"]), int(m["vdim"]), int(m.get("conv", 1)),
                                       "head" if kind == "delta" else "channel", eps, local_idx, dtype, m.get("rank"))
        else:
            raise ValueError(f"Rirotar: unknown mixer type {kind!r} in layer {idx}")
        mlp = spec.get("mlp")
        self.norm2 = self.mlp = None
        if mlp:
            self.norm2 = ZeroCentredNorm(W, dtype)
            if mlp["kind"] == "dense":
                self.mlp = ClampedGLU(W, int(mlp["ff"]), mlp["limit"], dtype)
            elif mlp["kind"] == "moe":
                self.mlp = GroupRoutedMoE(W, mlp, dtype, idx)
            else:
                raise ValueError(f"Rirotar: unknown feed-forward kind {mlp['kind']!r} in layer {idx}")


class RirotarForCausalLM(nn.Module):
    supports_cuda_graph = False          # the ragged kernels read lengths from device memory, but the expert loop syncs on the host
    disable_radix_cache = True           # recurrent state per request: no page-aligned prefix to share

    def __init__(self, cfg: ModelConfig, quant_name: Optional[str] = None, device="cpu"):
        super().__init__()
        assert get_tp_group().world_size == 1 and get_pp_group().world_size == 1, "Rirotar runs on one rank"
        assert cfg.hybrid and cfg.hybrid.get("layers") is not None, "Rirotar needs the per-layer list of its configuration"
        self.cfg = cfg
        dtype = _DT[cfg.dtype]
        self.dtype = dtype
        specs = cfg.hybrid["layers"]
        cache_width = max([int(s["mixer"]["kv_rank"]) for s in specs if s["type"] == "latent_attention"] or [0])
        bb = nn.Module()
        bb.embed_tokens = nn.Embedding(cfg.vocab_size, cfg.hidden_size, dtype=dtype)
        bb.embed_tokens.weight.requires_grad_(False)
        blocks, n_attn, n_rec = [], 0, 0
        for i, s in enumerate(specs):
            rec = s["type"] != "latent_attention"
            blocks.append(RirotarBlock(cfg, s, i, n_rec if rec else n_attn, dtype, cache_width))
            n_rec, n_attn = n_rec + int(rec), n_attn + int(not rec)
        bb.all_layers = nn.ModuleList(blocks)
        bb.layers = [b for b in blocks if b.kind == "attention"]          # what the runner sizes the paged pool from
        bb.norm = ZeroCentredNorm(cfg.hidden_size, dtype)
        self.model = bb
        self.lm_head = nn.Parameter(torch.zeros(cfg.vocab_size, cfg.hidden_size, dtype=dtype), requires_grad=False)
        self.layer_tap = None            # callable(layer index, fp32 residual [T, width]) after every layer (debugging / tests)
        if dtype == torch.float32:
            torch.backends.cuda.matmul.allow_tf32 = False          # fp32 serving means fp32 products

    # ---- forward: fp32 residual stream; every norm is fused with the residual add that precedes it
    def forward(self, fb: ForwardBatch, inputs_embeds=None):
        m, eps, dt = self.model, self.cfg.rms_norm_eps, self.dtype
        if inputs_embeds is None:          # decode gathers the last sampled token of every request slot on the device
            inputs_embeds = ops.embedding(m.embed_tokens.weight, fb.next_token_buf, fb.req_slots) if fb.input_ids is None \
                else ops.embedding(m.embed_tokens.weight, fb.input_ids)
        x = inputs_embeds.float().contiguous()
        y = None                          # branch output not yet added to the residual
        for i, blk in enumerate(m.all_layers):
            h = ops.add_rmsnorm_f32(x, y, blk.norm1.weight, eps, True, dt)
            y = blk.mix(h, fb)
            if blk.mlp is not None:
                h = ops.add_rmsnorm_f32(x, y, blk.norm2.weight, eps, True, dt)
                y = blk.mlp(h)
            if self.layer_tap is not None:
                self.layer_tap(i, x + y.float())
        return ops.add_rmsnorm_f32(x, y, m.norm.weight, eps, True, dt)

    def compute_logits(self, hidden: torch.Tensor, key: str = "logits") -> torch.Tensor:
        y = ops.linear(hidden, self.lm_head).float()
        cap = self.cfg.final_logit_softcapping
        return torch.tanh(y / cap) * cap if cap > 0 else y

    # ---- recurrent state
    def make_mamba_pool(self, slots: int, device) -> Optional[LayeredStatePool]:
        geo = [b.mix.state_geometry() for b in self.model.all_layers if b.kind == "mamba"]
        return LayeredStatePool(slots, geo, self.dtype, device) if geo else None

    # ---- weights
    def load_weights(self, weights: Iterable[Tuple[str, torch.Tensor]]) -> List[str]:
        loaded = []
        L = self.model.all_layers
        for name, w in weights:
            ok = False
            if name == "embed":
                self.model.embed_tokens.weight.data.copy_(w)
                ok = True
            elif name == "head":
                self.lm_head.data.copy_(w)
                ok = True
            elif name == "final.norm":
                self.model.norm.weight.data.copy_(w)
                ok = True
            elif name[:1] == "l" and "." in name and name[1:name.index(".")].isdigit():
                i, rest = int(name[1:name.index(".")]), name[name.index(".") + 1:]
                if i < len(L):
                    blk = L[i]
                    if rest in ("norm1", "norm2") and getattr(blk, rest) is not None:
                        getattr(blk, rest).weight.data.copy_(w)
                        ok = True
                    elif rest.startswith("mix."):
                        ok = blk.mix.load(rest[4:], w)
                    elif rest.startswith("mlp.") and blk.mlp is not None:
                        ok = blk.mlp.load(rest[4:], w)
            if ok:
                loaded.append(name)
        return loaded

    @staticmethod
    def dummy_checkpoint(cfg: ModelConfig, device, dtype, seed: int = 0, scale: float = 0.02):
        """random tensors under the checkpoint names (name-seeded), scaled so that activations stay O(1) through many layers"""
        def rnd(name: str, *shape: int, s: float = 1.0, off: float = 0.0) -> torch.Tensor:
            g = torch.Generator(device="cpu").manual_seed((seed * 1000003 + zlib.crc32(name.encode())) & 0x7FFFFFFF)
            return (torch.randn(*shape, generator=g) * s + off).to(dtype)

        lin = lambda name, o, i, s=1.0: rnd(name, o, i, s=s * i ** -0.5)
        W = cfg.hidden_size
        yield "embed", rnd("embed", cfg.vocab_size, W)
        for i, sp in enumerate(cfg.hybrid["layers"]):
            p, m = f"l{i}.", sp["mixer"]
            yield p + "norm1", rnd(p + "norm1", W, s=0.1)
            if sp["type"] == "latent_attention":
                H, D, Dv, R = int(m["heads"]), int(m["dim"]), int(m["vdim"]), int(m["kv_rank"])
                yield p + "mix.q", lin(p + "q", H * D, W, 2.0)
                yield p + "mix.dkv", lin(p + "dkv", R, W)
                yield p + "mix.dkv.norm", rnd(p + "dkvn", R, s=0.1, off=1.0)
                yield p + "mix.uk", lin(p + "uk", H * D, R, 2.0)
                yield p + "mix.uv", lin(p + "uv", H * Dv, R)
                yield p + "mix.sink", rnd(p + "sink", H).float()
                yield p + "mix.o", lin(p + "o", W, H * Dv)
            else:
                H, Hk, Dk, Dv, taps = int(m["heads"]), int(m.get("kv_heads", m["heads"])), int(m["dim"]), int(m["vdim"]), int(m.get("conv", 1))
                for nm, n in (("q", Hk * Dk), ("k", Hk * Dk), ("v", H * Dv)):
                    yield p + "mix." + nm, lin(p + nm, n, W)
                    yield p + f"mix.{nm}.conv", rnd(p + nm + "c", n, taps, s=0.5)
                yield p + "mix.b", lin(p + "b", H, W)
                yield p + "mix.A_log", rnd(p + "A", H, s=0.5, off=-1.0).float()
                yield p + "mix.norm", rnd(p + "n", Dv, s=0.1, off=1.0)
                if sp["type"] == "channel_delta":
                    r = int(m.get("rank") or 16)
                    yield p + "mix.a1", lin(p + "a1", r, W)
                    yield p + "mix.a2", lin(p + "a2", H * Dk, r)
                    yield p + "mix.dt_bias", rnd(p + "dt", H * Dk, s=0.5).float()
                    yield p + "mix.g1", lin(p + "g1", r, W)
                    yield p + "mix.g2", lin(p + "g2", H * Dv, r)
                else:
                    yield p + "mix.a", lin(p + "a", H, W)
                    yield p + "mix.dt_bias", rnd(p + "dt", H, s=0.5).float()
                    yield p + "mix.g", lin(p + "g", H * Dv, W)
                yield p + "mix.o", lin(p + "o", W, H * Dv)
            mlp = sp.get("mlp")
            if not mlp:
                continue
            yield p + "norm2", rnd(p + "norm2", W, s=0.1)
            if mlp["kind"] == "dense":
                ff = int(mlp["ff"])
                yield p + "mlp.gate", lin(p + "mg", ff, W)
                yield p + "mlp.up", lin(p + "mu", ff, W)
                yield p + "mlp.down", lin(p + "md", W, ff)
            else:
                ff = int(mlp["expert"]["ff"])
                for e in range(int(mlp["router"]["experts"])):
                    q = p + f"mlp.e{e}."
                    yield q + "gate", lin(q + "g", ff, W)
                    yield q + "up", lin(q + "u", ff, W)
                    yield q + "down", lin(q + "d", W, ff)
                yield p + "mlp.router", lin(p + "r", int(mlp["router"]["experts"]), W, 2.0)
        yield "final.norm", rnd("fn", W, s=0.1)
        yield "head", lin("head", cfg.vocab_size, W)
