"""Zaparax beside the closest existing family at equal size (``python bench.py --hybrid-compare --hybrid-family zaparax``).

Two parts, random weights, one GPU:

1. **engine**: prefill and decode throughput of a four-layer Zaparax slice (Mamba-2 + MoE, window attention + MoE, twice) and of a
   Nemotron-H slice of the same width, head counts, head sizes, state size, groups and taps (pattern ``M-*-M-*-``; its dense feed-forward is as
   wide as the experts a Zaparax token runs: ``top * expert ff + shared ff``), both through ``Scheduler.replay_step`` (the serving step).
2. **kernels**: each new kernel beside the like op of the closest model on the same shapes: the ragged Mamba-2 scan vs the chunked PyTorch
   scan Nemotron-H prompts run and vs ``selective_state_update`` (+ its PyTorch softplus / gate) in decode; biased window attention vs the
   tcgen05 paged attention kernel with the same window; q/k norm + cache write vs ``rope_kv_write``; the sandwich-norm residual kernel vs
   ``add_rmsnorm_f32`` and ``fused_add_rmsnorm``; the identity-expert router vs ``topk_softmax``; the bigram embedding vs ``embedding``.
   Roofline: algorithmic bytes over the measured copy bandwidth; for prompt attention also FLOPs over the measured bf16 GEMM rate.

Timing: CUDA events on the launching stream, >= 3 warm-ups, an L2 flush (a 256 MB write) between timed iterations.
Prints one JSON line per measurement and a closing summary line.
"""
from __future__ import annotations

import json
from typing import List

import torch

from .hybrid_compare import _engine_numbers, _peaks, _Timer


def _zaparax_cfg(width: int, heads: int, experts: int, top: int, eff: int, shared: int, window: int, state: int) -> dict:
    mamba = {"type": "mamba2", "mixer": {"heads": 2 * width // 64, "vdim": 64, "state": state, "groups": 8, "conv": 4, "norm_groups": 8}}
    attn = {"type": "attention", "mixer": {"heads": heads, "kv_heads": max(1, heads // 8), "dim": 128, "vdim": 128, "mask": {"size": window},
                                           "q_temp": {"coef": 0.1, "every": 1024}, "scale": 128 ** -0.5, "softcap": 30.0}}
    moe = {"kind": "moe", "expert": {"ff": eff}, "router": {"experts": experts, "identity": 2, "top": top}, "shared": {"ff": shared}}
    return {"architecture": "Zaparax", "width": width, "vocab": 32000, "norm": {"eps": 1e-6},
            "embedding": {"scale": 1.0, "bigram": {"buckets": 65521, "mul_prev": 31, "mul_cur": 13}},
            "layers": [dict(mamba, mlp=moe), dict(attn, mlp=moe), dict(mamba, mlp=moe), dict(attn, mlp=moe)]}


def _nemotron_h_cfg(width: int, heads: int, ff: int, state: int) -> dict:
    return {"architectures": ["NemotronHForCausalLM"], "hidden_size": width, "num_hidden_layers": 8, "hybrid_override_pattern": "M-*-M-*-",
            "mamba_num_heads": 2 * width // 64, "mamba_head_dim": 64, "ssm_state_size": state, "conv_kernel": 4, "n_groups": 8, "chunk_size": 128,
            "num_attention_heads": heads, "num_key_value_heads": max(1, heads // 8), "attention_head_dim": 128, "intermediate_size": ff,
            "vocab_size": 32000, "layer_norm_epsilon": 1e-6, "max_position_embeddings": 32768, "tie_word_embeddings": False}


def _kernel_numbers(timer: _Timer, hbm_gbs: float, tflops: float) -> List[dict]:
    import torch.nn.functional as F

    from .. import ops
    from ..models.mamba import ssd_chunk_scan
    from ..ops import moe_ops

    dev, out = "cuda", []

    def rec(kernel, phase, shape, ms, nbytes, like=None, like_ms=None, like_bytes=None, flops=None):
        r = {"part": "kernel", "kernel": kernel, "phase": phase, "shape": shape, "ms": round(ms, 4), "algorithmic_mb": round(nbytes / 1e6, 2),
             "roofline_frac": round(nbytes / (ms * 1e-3) / (hbm_gbs * 1e9), 4)}
        if flops is not None:
            r["tensor_frac"] = round(flops / (ms * 1e-3) / (tflops * 1e12), 4)
        if like is not None:
            lb = nbytes if like_bytes is None else like_bytes
            r.update(like=like, like_ms=round(like_ms, 4), like_roofline_frac=round(lb / (like_ms * 1e-3) / (hbm_gbs * 1e9), 4))
            r["distance_ratio"] = round(r["like_roofline_frac"] / max(r["roofline_frac"], 1e-9), 3)
        out.append(r)

    g = torch.Generator(device=dev).manual_seed(0)
    # ---- Mamba-2 scan
    H, P, N, G = 64, 64, 128, 8
    inner = H * P
    dtb, A_log, D = torch.zeros(H, device=dev), torch.zeros(H, device=dev), torch.ones(H, device=dev)
    for B, S in ((4, 2048), (1, 4096)):
        T = B * S
        u = torch.randn(T, inner + 2 * G * N, device=dev, generator=g)
        proj = torch.randn(T, inner + H, device=dev, generator=g).to(torch.bfloat16)
        z, dt_raw = proj[:, :inner], proj[:, inner:]
        state = torch.zeros(B + 1, H, N, P, device=dev)
        slots = torch.arange(B, dtype=torch.int32, device=dev)
        sl = torch.full((B,), S, dtype=torch.int32, device=dev)
        cu = torch.arange(0, T + 1, S, dtype=torch.int32, device=dev)
        ms = timer(lambda: ops.mamba2_scan(u, z, dt_raw, dtb, A_log, D, state, slots, sl, cu, sl, H, P, N, G))
        st2 = torch.zeros(B + 1, H, P, N, device=dev)
        x = u[:, :inner].view(T, H, P)
        Bm = u[:, inner:inner + G * N].view(T, G, N).repeat_interleave(H // G, 1)
        Cm = u[:, inner + G * N:].view(T, G, N).repeat_interleave(H // G, 1)

        def chunked():
            dt = F.softplus(dt_raw.float() + dtb)
            for i in range(B):
                s = slice(i * S, (i + 1) * S)
                y, fin = ssd_chunk_scan(x[s], dt[s], -A_log.exp(), Bm[s], Cm[s], st2[i], 128)
                y = (y + D[None, :, None] * x[s]).reshape(S, inner) * F.silu(z[s].float())
                st2[i].copy_(fin)

        like = timer(chunked, iters=3, warmup=2)
        nbytes = u.numel() * 4 + proj.numel() * 2 + T * inner * 4 + 2 * state[:B].numel() * 4
        rec("mamba2_scan", "prefill", f"B{B} S{S} H{H} P{P} N{N} G{G}", ms, nbytes, "mamba.ssd_chunk_scan + gate (torch)", like)
    for B in (32, 256):
        u = torch.randn(B, inner + 2 * G * N, device=dev, generator=g)
        proj = torch.randn(B, inner + H, device=dev, generator=g).to(torch.bfloat16)
        z, dt_raw = proj[:, :inner], proj[:, inner:]
        state = torch.randn(B + 1, H, N, P, device=dev, generator=g)
        st2 = torch.randn(B + 1, H, P, N, device=dev, generator=g)
        slots = torch.arange(B, dtype=torch.int32, device=dev)
        sl = torch.full((B,), 999, dtype=torch.int32, device=dev)
        ms = timer(lambda: ops.mamba2_scan(u, z, dt_raw, dtb, A_log, D, state, slots, sl, None, None, H, P, N, G))
        negA = -A_log.exp()

        def upd():
            dt = F.softplus(dt_raw.float() + dtb)
            y = ops.selective_state_update(st2, slots, u[:, :inner], dt, negA, u[:, inner:inner + G * N], u[:, inner + G * N:], D)
            y = y.reshape(B, inner) * F.silu(z.float())

        like = timer(upd)
        rec("mamba2_scan", "decode", f"B{B} H{H} P{P} N{N} G{G}", ms, 2 * state[:B].numel() * 4, "selective_state_update + torch softplus/gate", like)
    # ---- window attention
    H, Gk, Dh, ps, W = 32, 4, 128, 64, 1024
    slopes = (2.0 ** (-8.0 * torch.arange(1, H + 1, device=dev) / H)).float()
    sinks = torch.zeros(H, device=dev)
    for B, S, Q in ((4, 2048, 2048), (64, 2048, 1)):
        pages = B * S // ps
        kc = torch.randn((pages + 1) * ps, 1, Gk * Dh, device=dev, generator=g).to(torch.bfloat16)
        vc = torch.randn((pages + 1) * ps, 1, Gk * Dh, device=dev, generator=g).to(torch.bfloat16)
        pt = (torch.arange(pages, dtype=torch.int32, device=dev) + 1).view(B, S // ps).contiguous()
        slots = torch.arange(B, dtype=torch.int32, device=dev)
        sl = torch.full((B,), S, dtype=torch.int32, device=dev)
        ql = torch.full((B,), Q, dtype=torch.int32, device=dev)
        cu = None if Q == 1 else torch.arange(0, B * Q + 1, Q, dtype=torch.int32, device=dev)
        q = torch.randn(B * Q, H, Dh, device=dev, generator=g).to(torch.bfloat16)
        ms = timer(lambda: ops.window_attention(q, kc, vc, Gk, Dh, pt, slots, sl, cu, None if Q == 1 else ql, Q, ps, Dh ** -0.5, 30.0, W, slopes, sinks))
        k4, v4 = kc.view(-1, Gk, Dh), vc.view(-1, Gk, Dh)
        like = timer(lambda: ops.paged_attention(q, k4, v4, pt, slots, sl, cu, None if Q == 1 else ql, Q, ps, Dh ** -0.5, True, W, 30.0))
        keys = sum(min(i + 1, W) for i in range(S - Q, S))
        nbytes = q.numel() * 2 * 2 + B * min(S, W + Q) * Gk * Dh * 2 * 2
        ph = "prefill" if Q > 1 else "decode"
        rec("window_attention (general kernel: any head size, fp32 serving)", ph, f"B{B} S{S} q{Q} H{H} G{Gk} D{Dh} window{W} cap bias sink", ms, nbytes,
            "paged_attention (tcgen05 / split-KV decode kernel, same window and cap)", like, flops=4.0 * B * keys * H * Dh)
        lse = torch.empty(B * Q, H, dtype=torch.float32, device=dev)
        ns = 1 if Q > 1 else 4

        def tc_route():          # what bf16 serving with 128-wide heads runs: the same tcgen05 kernels with the bias in the score pass + the sink
            o = ops.paged_attention(q, k4, v4, pt, slots, sl, cu, None if Q == 1 else ql, Q, ps, Dh ** -0.5, True, W, 30.0, num_splits=ns, lse=lse,
                                    slopes=slopes)
            return ops.attention_sink_gate(o, lse, sinks)

        ms2 = timer(tc_route)
        like2 = timer(lambda: ops.paged_attention(q, k4, v4, pt, slots, sl, cu, None if Q == 1 else ql, Q, ps, Dh ** -0.5, True, W, 30.0, num_splits=ns))
        rec("window attention on the tcgen05 kernels (bias in the score pass, sink through the lse)", ph,
            f"B{B} S{S} q{Q} H{H} G{Gk} D{Dh} window{W} cap bias sink splits{ns}", ms2, nbytes, "paged_attention (same kernels, no bias, no sink)", like2,
            flops=4.0 * B * keys * H * Dh)
    # ---- the general kernel beside the framework's own general-shape attention (64-wide heads: neither takes the tcgen05 kernels)
    Dh = 64
    for B, S, Q in ((4, 2048, 2048), (64, 2048, 1)):
        pages = B * S // ps
        kc = torch.randn((pages + 1) * ps, 1, Gk * Dh, device=dev, generator=g).to(torch.bfloat16)
        vc = torch.randn((pages + 1) * ps, 1, Gk * Dh, device=dev, generator=g).to(torch.bfloat16)
        pt = (torch.arange(pages, dtype=torch.int32, device=dev) + 1).view(B, S // ps).contiguous()
        slots = torch.arange(B, dtype=torch.int32, device=dev)
        sl = torch.full((B,), S, dtype=torch.int32, device=dev)
        ql = torch.full((B,), Q, dtype=torch.int32, device=dev)
        cu = None if Q == 1 else torch.arange(0, B * Q + 1, Q, dtype=torch.int32, device=dev)
        q = torch.randn(B * Q, H, Dh, device=dev, generator=g).to(torch.bfloat16)
        ms = timer(lambda: ops.window_attention(q, kc, vc, Gk, Dh, pt, slots, sl, cu, None if Q == 1 else ql, Q, ps, Dh ** -0.5, 30.0, W, slopes, sinks))
        k4, v4 = kc.view(-1, Gk, Dh), vc.view(-1, Gk, Dh)
        like = timer(lambda: ops.paged_attention(q, k4, v4, pt, slots, sl, cu, None if Q == 1 else ql, Q, ps, Dh ** -0.5, True, W, 30.0, impl=1))
        keys = sum(min(i + 1, W) for i in range(S - Q, S))
        nbytes = q.numel() * 2 * 2 + B * min(S, W + Q) * Gk * Dh * 2 * 2
        rec("window_attention (general kernel)", "prefill" if Q > 1 else "decode", f"B{B} S{S} q{Q} H{H} G{Gk} D{Dh} window{W} cap bias sink", ms, nbytes,
            "paged_attention impl=1 (the framework's kernel for head sizes other than 128)", like, flops=4.0 * B * keys * H * Dh)
        # what bf16 serving runs for these heads: the same rows laid out 128 columns wide (zeros behind the 64 values) on the tcgen05 kernels
        kp = torch.nn.functional.pad(k4, (0, 128 - Dh)).contiguous()
        vp = torch.nn.functional.pad(v4, (0, 128 - Dh)).contiguous()
        qp = torch.nn.functional.pad(q, (0, 128 - Dh)).contiguous()
        lse = torch.empty(B * Q, H, dtype=torch.float32, device=dev)
        ns = 1 if Q > 1 else 4

        def padded_tc():
            o = ops.paged_attention(qp, kp, vp, pt, slots, sl, cu, None if Q == 1 else ql, Q, ps, Dh ** -0.5, True, W, 30.0, num_splits=ns, lse=lse,
                                    slopes=slopes)
            return ops.attention_sink_gate(o, lse, sinks, Dh)

        ms3 = timer(padded_tc)
        rec("window attention, 64-wide heads laid out 128 wide on the tcgen05 kernels", "prefill" if Q > 1 else "decode",
            f"B{B} S{S} q{Q} H{H} G{Gk} D{Dh}->128 window{W} cap bias sink splits{ns}", ms3, 2 * nbytes, "window_attention (general kernel) on the plain layout",
            ms, like_bytes=nbytes, flops=4.0 * B * keys * H * Dh)
    Dh = 128
    # ---- q/k norm + cache write
    T = 8192
    qkv = torch.randn(T, (H + 2 * Gk) * Dh, device=dev, generator=g).to(torch.bfloat16)
    kc = torch.zeros(T + 64, 1, Gk * Dh, device=dev, dtype=torch.bfloat16)
    vc = torch.zeros_like(kc)
    pos = torch.arange(T, dtype=torch.int32, device=dev)
    loc = pos + 64
    ms = timer(lambda: ops.qk_norm_cache_write(qkv, H, Gk, Dh, Dh, pos, 1e-6, 0.1, 1024, kc, vc, loc))
    q3 = qkv[:, :H * Dh].clone().view(T, H, Dh)
    k3, v3 = qkv[:, H * Dh:(H + Gk) * Dh].clone().view(T, Gk, Dh), qkv[:, (H + Gk) * Dh:].clone().view(T, Gk, Dh)
    cs = torch.randn(T, Dh, device=dev)
    like = timer(lambda: ops.rope_kv_write(q3, k3, v3, pos, cs, kc.view(-1, Gk, Dh), vc.view(-1, Gk, Dh), loc))
    rec("qk_norm_cache_write", "any", f"T{T} H{H} G{Gk} D{Dh}", ms, qkv.numel() * 2 * 2, "rope_kv_write", like)
    # ---- sandwich norm on the fp32 residual
    Wd = 4096
    res, d16 = torch.randn(T, Wd, device=dev), torch.randn(T, Wd, device=dev).to(torch.bfloat16)
    w16 = torch.zeros(Wd, device=dev, dtype=torch.bfloat16)
    ms = timer(lambda: ops.add_rmsnorm_f32(res, d16, w16, 1e-6, True, torch.bfloat16, w16))
    like = timer(lambda: ops.add_rmsnorm_f32(res, d16, w16, 1e-6, True, torch.bfloat16))
    rec("add_rmsnorm_f32(post_weight)", "any", f"T{T} W{Wd} (post-norm + add + pre-norm, 12 B/elem)", ms, T * Wd * 12, "add_rmsnorm_f32 (add + pre-norm)", like)
    y32 = torch.randn(T, Wd, device=dev)
    ms = timer(lambda: ops.grouped_rmsnorm(y32, w16, 8, 1e-6, torch.bfloat16))
    y16 = y32.to(torch.bfloat16)
    like = timer(lambda: ops.rmsnorm(y16, w16, 1e-6))
    rec("grouped_rmsnorm", "any", f"T{T} C{Wd} groups8 (fp32 in, 6 B/elem)", ms, T * Wd * 6, "rmsnorm (bf16 in, 4 B/elem)", like, like_bytes=T * Wd * 4)
    # ---- router, combine, embedding
    E = 66
    logits = torch.randn(T, E, device=dev, generator=g)
    corr = torch.zeros(E, device=dev)
    ms = timer(lambda: moe_ops.softmax_bias_route(logits, corr, 4, 64))
    like = timer(lambda: moe_ops.topk_softmax(logits, 4, False))
    rec("softmax_bias_route", "any", f"T{T} E{E} top4", ms, T * (E * 4 + 4 * 8 + 4), "topk_softmax", like)
    emb = torch.randn(32000, Wd, device=dev).to(torch.bfloat16)
    bg = torch.randn(65522, Wd, device=dev).to(torch.bfloat16)
    ids = torch.randint(0, 32000, (T,), device=dev, dtype=torch.int32)
    prev = torch.zeros(8, dtype=torch.int32, device=dev)
    cu = torch.arange(0, T + 1, 2048, dtype=torch.int32, device=dev)
    slots = torch.arange(4, dtype=torch.int32, device=dev)
    sl = torch.full((4,), 2048, dtype=torch.int32, device=dev)
    ms = timer(lambda: ops.bigram_embedding(emb, bg, ids, prev, cu, slots, sl, 2048, 1.0, 31, 13, 65521))
    like = timer(lambda: ops.embedding(emb, ids))
    rec("bigram_embedding", "any", f"T{T} W{Wd} (two rows in, fp32 out: 8 B/elem)", ms, T * Wd * 8, "embedding (one row in, bf16 out: 4 B/elem)", like,
        like_bytes=T * Wd * 4)
    return out


def main(sizes: str = "2048,4096") -> None:
    pk = _peaks()
    timer = _Timer()
    rows: List[dict] = []
    for w in [int(x) for x in sizes.split(",") if x]:
        heads = w // 128
        experts, top, eff, shared = 16, 4, w // 2, w
        cfgs = (("zaparax", _zaparax_cfg(w, heads, experts, top, eff, shared, 1024, 128)),
                ("nemotron_h", _nemotron_h_cfg(w, heads, top * eff + shared, 128)))
        for name, cfg in cfgs:
            for r in _engine_numbers(name, cfg, 4, 2048, 32, 8, timer):
                r["width"] = w
                rows.append(r)
                print(json.dumps(r), flush=True)
    for r in _kernel_numbers(timer, pk["hbm_gbs"], pk["bf16_tflops"]):
        rows.append(r)
        print(json.dumps(r), flush=True)
    worst = max((r.get("distance_ratio", 0.0) for r in rows if r["part"] == "kernel"), default=0.0)
    print(json.dumps({"metric": "hybrid_compare", "family": "zaparax", "roofline": f"{pk['hbm_gbs']} GB/s, {pk['bf16_tflops']} TFLOP/s ({pk['src']})",
                      "worst_kernel_distance_ratio": worst, "rows": len(rows), "data": "synthetic", "dtype": "bf16"}), flush=True)
