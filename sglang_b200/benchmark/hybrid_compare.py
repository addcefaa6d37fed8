"""Rirotar beside the closest existing family at equal size (``python bench.py --hybrid-compare``).

Two parts, random weights, one GPU:

1. **engine**: prefill and decode throughput of a four-layer Rirotar slice (delta + dense, latent attention + MoE, channel delta + dense,
   delta + MoE) and of a Qwen3-Next slice of the same width, head counts, head sizes, feed-forward sizes and expert counts (three gated
   DeltaNet layers + one gated softmax-attention layer), both through ``Scheduler.replay_step`` (the serving step).
2. **kernels**: each new kernel beside the like op of the closest model on the same shapes, with the algorithmic bytes over the measured
   copy bandwidth as the roofline: gated delta rule (prefill, decode) vs Qwen3-Next's chunked prefill path and ``gated_delta_update``;
   latent window attention (prefill, decode) vs the latent attention DeepSeek models run (``torch_ref.paged_attention`` over the
   latent rows, no window); fp32-residual add+norm vs ``fused_add_rmsnorm``; clamped GLU vs ``silu_and_mul``.

Timing: CUDA events on the launching stream, >= 3 warm-ups, an L2 flush (a 256 MB write) between timed iterations.
Prints one JSON line per measurement and a closing summary line.
"""
from __future__ import annotations

import json
import os
import tempfile
from typing import Callable, Dict, List

import torch


def _peaks() -> Dict[str, float]:
    p = os.path.join(os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))), "MEASURED_PEAKS.json")
    try:
        with open(p) as f:
            d = json.load(f)
        return {"hbm_gbs": float(d["hbm_gbs"]), "bf16_tflops": float(d["bf16_tflops"]), "src": "measured"}
    except Exception:
        return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "src": "fallback"}


class _Timer:
    def __init__(self):
        self.flush = torch.empty(256 << 20, dtype=torch.uint8, device="cuda")

    def __call__(self, fn: Callable[[], None], iters: int = 5, warmup: int = 3) -> float:
        for _ in range(warmup):
            fn()
        ts = []
        for _ in range(iters):
            self.flush.fill_(1)
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            torch.cuda.synchronize()
            a.record()
            fn()
            b.record()
            torch.cuda.synchronize()
            ts.append(a.elapsed_time(b))
        return sorted(ts)[len(ts) // 2]


def _rirotar_cfg(width: int, heads: int, ff: int, experts: int, top: int, eff: int, rank: int, window: int) -> dict:
    delta = lambda kind: {"type": kind, "mixer": {"heads": heads, "kv_heads": heads // 2, "dim": 128, "vdim": 128, "conv": 4}}
    attn = {"type": "latent_attention", "mixer": {"heads": heads, "dim": 128, "vdim": 128, "kv_rank": rank, "mask": {"size": window}, "scale": 128 ** -0.5}}
    dense = {"kind": "dense", "ff": ff, "limit": 7.0}
    moe = {"kind": "moe", "expert": {"ff": eff, "limit": 7.0}, "router": {"experts": experts, "top": top, "scale": 1.0, "groups": {"count": 4, "keep": 2}}}
    return {"architecture": "Rirotar", "width": width, "vocab": 32000, "norm": {"eps": 1e-6}, "logit_softcap": 30.0,
            "layers": [dict(delta("delta"), mlp=dense), dict(attn, mlp=moe), dict(delta("channel_delta"), mlp=dense), dict(delta("delta"), mlp=moe)]}


def _qwen3_next_cfg(width: int, heads: int, ff: int, experts: int, top: int, eff: int) -> dict:
    return {"architectures": ["Qwen3NextForCausalLM"], "hidden_size": width, "num_hidden_layers": 4, "num_attention_heads": heads,
            "num_key_value_heads": max(1, heads // 8), "head_dim": 128, "vocab_size": 32000, "rms_norm_eps": 1e-6, "intermediate_size": ff,
            "linear_num_key_heads": heads // 2, "linear_num_value_heads": heads, "linear_key_head_dim": 128, "linear_value_head_dim": 128,
            "linear_conv_kernel_dim": 4, "layer_types": ["linear_attention", "full_attention", "linear_attention", "linear_attention"],
            "num_experts": experts, "num_experts_per_tok": top, "moe_intermediate_size": eff, "shared_expert_intermediate_size": 0,
            "decoder_sparse_step": 1, "mlp_only_layers": [0, 2], "norm_topk_prob": True, "max_position_embeddings": 32768,
            "rope_theta": 10000.0, "partial_rotary_factor": 0.25, "tie_word_embeddings": False}


def _engine(cfg: dict, tokens: int, slots: int):
    import sglang_b200 as sgl

    d = tempfile.mkdtemp(prefix="hybrid_cmp_")
    with open(os.path.join(d, "config.json"), "w") as f:
        json.dump(cfg, f)
    return sgl.Engine(model_path=d, load_format="dummy", skip_tokenizer_init=True, page_size=64, max_total_tokens=tokens, max_running_requests=slots,
                      context_length=8192, disable_radix_cache=True, disable_cuda_graph=True, disable_overlap_schedule=True,
                      chunked_prefill_size=-1, max_prefill_tokens=tokens, log_level="warning")


def _engine_numbers(name: str, cfg: dict, B: int, S: int, dec_B: int, dec_steps: int, timer: _Timer) -> List[dict]:
    import numpy as np

    eng = _engine(cfg, max(B * S, dec_B * (S + 64)) + 4096, max(B, dec_B))
    sch = eng.scheduler
    rng = np.random.default_rng(0)
    out = []
    n = [0]

    def prefill():
        ids = [f"p{n[0]}_{i}" for i in range(B)]
        n[0] += 1
        sch.replay_step([(r, rng.integers(0, 32000, S).tolist(), []) for r in ids], ids)

    ms = timer(prefill, iters=3, warmup=3)
    out.append({"part": "engine", "model": name, "phase": "prefill", "batch": B, "seq_len": S, "ms": round(ms, 3), "tokens_per_s": round(B * S / ms * 1e3)})
    ids = [f"d{i}" for i in range(dec_B)]
    sch.replay_step([(r, rng.integers(0, 32000, S).tolist(), []) for r in ids], [])

    def decode():
        for _ in range(dec_steps):
            sch.replay_step([(r, [int(rng.integers(0, 32000))], []) for r in ids], [])

    ms = timer(decode, iters=3, warmup=3)
    out.append({"part": "engine", "model": name, "phase": "decode", "batch": dec_B, "context": S, "ms_per_step": round(ms / dec_steps, 3),
                "tokens_per_s": round(dec_B * dec_steps / ms * 1e3)})
    sch.replay_step([], ids)
    eng.shutdown()
    del eng
    torch.cuda.empty_cache()
    return out


def _kernel_numbers(timer: _Timer, hbm_gbs: float) -> List[dict]:
    import torch.nn.functional as F

    from .. import ops
    from ..models.qwen3_next import gated_delta_chunked
    from ..ops import torch_ref

    dev, out = "cuda", []

    def rec(kernel, phase, shape, ms, nbytes, like=None, like_ms=None):
        r = {"part": "kernel", "kernel": kernel, "phase": phase, "shape": shape, "ms": round(ms, 4), "algorithmic_mb": round(nbytes / 1e6, 2),
             "roofline_frac": round(nbytes / (ms * 1e-3) / (hbm_gbs * 1e9), 4)}
        if like is not None:
            r.update(like=like, like_ms=round(like_ms, 4), like_roofline_frac=round(nbytes / (like_ms * 1e-3) / (hbm_gbs * 1e9), 4),
                     distance_ratio=round(ms / like_ms, 3))
        out.append(r)

    # ---- gated delta rule
    H, Hk, Dk, Dv = 32, 16, 128, 128
    g = torch.Generator(device=dev).manual_seed(0)
    A_log, dtb, nw = torch.zeros(H, device=dev), torch.zeros(H, device=dev), torch.ones(Dv, device=dev)
    for B, S in ((8, 1024), (1, 4096)):
        T = B * S
        u = torch.randn(T, 2 * Hk * Dk + H * Dv, device=dev, generator=g)
        a, b, gate = (torch.randn(T, n, device=dev, generator=g) for n in (H, H, H * Dv))
        state = torch.zeros(B + 1, H, Dk, Dv, device=dev)
        slots = torch.arange(B, dtype=torch.int32, device=dev)
        sl = torch.full((B,), S, dtype=torch.int32, device=dev)
        cu = torch.arange(0, T + 1, S, dtype=torch.int32, device=dev)
        ms = timer(lambda: ops.gated_delta_rule(u, Hk, Dk, H, Dv, a, A_log, dtb, b, state, slots, sl, cu, sl, gate, nw, 1e-6, "silu", False))
        qh = u[:, :Hk * Dk].view(T, Hk, Dk).repeat_interleave(2, 1)
        kh = u[:, Hk * Dk:2 * Hk * Dk].view(T, Hk, Dk).repeat_interleave(2, 1)
        vh = u[:, 2 * Hk * Dk:].view(T, H, Dv)
        gl, be = -F.softplus(a), torch.sigmoid(b)

        def chunked():
            for i in range(B):
                s = slice(i * S, (i + 1) * S)
                o, st = gated_delta_chunked(qh[s], kh[s], vh[s], gl[s], be[s], state[i])
                o = o * torch.rsqrt(o.pow(2).mean(-1, keepdim=True) + 1e-6) * F.silu(gate[s].view(S, H, Dv))

        like = timer(chunked)
        nbytes = u.numel() * 4 + gate.numel() * 4 + T * H * Dv * 4 + 2 * state[:B].numel() * 4
        rec("gated_delta_rule", "prefill", f"B{B} S{S} H{H} Dk{Dk} Dv{Dv}", ms, nbytes, "qwen3_next.gated_delta_chunked (torch)", like)
    for B in (32, 256):
        u = torch.randn(B, 2 * Hk * Dk + H * Dv, device=dev, generator=g)
        a, b, gate = (torch.randn(B, n, device=dev, generator=g) for n in (H, H, H * Dv))
        state = torch.randn(B + 1, H, Dk, Dv, device=dev, generator=g)
        slots = torch.arange(B, dtype=torch.int32, device=dev)
        sl = torch.full((B,), 999, dtype=torch.int32, device=dev)
        ms = timer(lambda: ops.gated_delta_rule(u, Hk, Dk, H, Dv, a, A_log, dtb, b, state, slots, sl, None, None, gate, nw, 1e-6, "silu", False))
        gl, be = -F.softplus(a), torch.sigmoid(b)

        def upd():
            o = ops.gated_delta_update(state, slots, u, gl, be, Hk)
            o = o * torch.rsqrt(o.pow(2).mean(-1, keepdim=True) + 1e-6) * F.silu(gate.view(B, H, Dv))

        like = timer(upd)
        rec("gated_delta_rule", "decode", f"B{B} H{H} Dk{Dk} Dv{Dv}", ms, 2 * state[:B].numel() * 4, "gated_delta_update + torch norm/gate", like)
    # ---- latent attention
    H, R, ps, W = 32, 512, 64, 1024
    for B, S, Q in ((4, 2048, 2048), (64, 2048, 1)):
        pages = B * S // ps
        cache = torch.randn((pages + 1) * ps, 1, R, device=dev, generator=g).to(torch.bfloat16)
        pt = (torch.arange(pages, dtype=torch.int32, device=dev) + 1).view(B, S // ps).contiguous()
        slots = torch.arange(B, dtype=torch.int32, device=dev)
        sl = torch.full((B,), S, dtype=torch.int32, device=dev)
        ql = torch.full((B,), Q, dtype=torch.int32, device=dev)
        cu = None if Q == 1 else torch.arange(0, B * Q + 1, Q, dtype=torch.int32, device=dev)
        q = torch.randn(B * Q, H, R, device=dev, generator=g) * 0.05
        sinks = torch.zeros(H, device=dev)
        ms = timer(lambda: ops.latent_attention(q, cache, R, pt, slots, sl, cu, None if Q == 1 else ql, Q, ps, 0.06, W, sinks))
        qb = q.to(torch.bfloat16)
        like = timer(lambda: torch_ref.paged_attention(qb, cache, cache, pt, slots, sl, None if Q == 1 else ql, ps, 0.06, True, -1, 0.0), iters=3, warmup=1)
        nbytes = q.numel() * 4 * 2 + B * min(S, W + Q) * R * 2
        rec("latent_attention", "prefill" if Q > 1 else "decode", f"B{B} S{S} q{Q} H{H} R{R} window{W}", ms, nbytes,
            "deepseek latent path (torch_ref.paged_attention, no window)", like)
        if Q > 1:          # the route bf16 prompts with 128-wide heads take: up-projection GEMMs + tcgen05 flash attention over the window rows
            import types

            from ..layers.latent_attention import WindowedLatentAttention

            layer = WindowedLatentAttention(4096, H, 128, 128, R, 128 ** -0.5, W, 1e-6, 0, torch.bfloat16).to(dev)
            for prm in (layer.uk, layer.uv):
                prm.data.normal_(0.0, 0.03)
            fb = types.SimpleNamespace(page_size=ps, seq_lens_cpu=[S] * B, q_lens_cpu=[Q] * B, req_slots=slots, page_table=pt, seq_lens=sl, cu_q=cu,
                                       q_lens=ql, max_q_len=Q)
            q128 = torch.randn(B * Q, H * 128, device=dev, generator=g).to(torch.bfloat16)

            def expanded():
                fb.__dict__.pop("_latent_expand", None)
                layer._forward_expanded(q128, cache, fb)

            ms2 = timer(expanded)
            rec("latent_attention (expanded: GEMMs + tcgen05 flash attention)", "prefill", f"B{B} S{S} q{Q} H{H} D128 R{R} window{W}", ms2, nbytes,
                "deepseek latent path (torch_ref.paged_attention, no window)", like)
    # ---- elementwise
    T, Wd = 8192, 4096
    res, d16 = torch.randn(T, Wd, device=dev), torch.randn(T, Wd, device=dev).to(torch.bfloat16)
    w16 = torch.zeros(Wd, device=dev, dtype=torch.bfloat16)
    ms = timer(lambda: ops.add_rmsnorm_f32(res, d16, w16, 1e-6, True, torch.bfloat16))
    r16 = res.to(torch.bfloat16)
    x16 = d16.clone()
    like = timer(lambda: ops.fused_add_rmsnorm(x16, r16, w16, 1e-6, True))
    rec("add_rmsnorm_f32", "any", f"T{T} W{Wd} (fp32 residual: 12 B/elem)", ms, T * Wd * (4 + 4 + 2 + 2), "fused_add_rmsnorm (bf16 residual: 8 B/elem)", like)
    out[-1]["like_roofline_frac"] = round(T * Wd * 8 / (like * 1e-3) / (hbm_gbs * 1e9), 4)
    out[-1]["distance_ratio"] = round(out[-1]["like_roofline_frac"] / max(out[-1]["roofline_frac"], 1e-9), 3)
    gu = torch.randn(T, 2 * 14336, device=dev).to(torch.bfloat16)
    ms = timer(lambda: ops.clamped_glu(gu, 7.0))
    like = timer(lambda: ops.silu_and_mul(gu))
    rec("clamped_glu", "any", f"T{T} I14336", ms, gu.numel() * 2 * 1.5, "silu_and_mul", like)
    return out


def main(sizes: str = "2048,4096") -> None:
    pk = _peaks()
    timer = _Timer()
    rows: List[dict] = []
    for w in [int(x) for x in sizes.split(",") if x]:
        heads = w // 128
        kw = dict(width=w, heads=heads, ff=3 * w, experts=16, top=4, eff=w // 2)
        for name, cfg in (("rirotar", _rirotar_cfg(rank=512, window=1024, **kw)), ("qwen3_next", _qwen3_next_cfg(**kw))):
            for r in _engine_numbers(name, cfg, 4, 2048, 32, 8, timer):
                r["width"] = w
                rows.append(r)
                print(json.dumps(r), flush=True)
    for r in _kernel_numbers(timer, pk["hbm_gbs"]):
        rows.append(r)
        print(json.dumps(r), flush=True)
    worst = max((r.get("distance_ratio", 0.0) for r in rows if r["part"] == "kernel"), default=0.0)
    print(json.dumps({"metric": "hybrid_compare", "roofline": f"{pk['hbm_gbs']} GB/s ({pk['src']})", "worst_kernel_distance_ratio": worst,
                      "rows": len(rows), "data": "synthetic", "dtype": "bf16"}), flush=True)
