"""Plain, slow oracle for the Rirotar design: one function per mechanism, straight from the equations, token by token where the
mechanism is recurrent.  It shares no code with the serving path (no pools, no kernels, no batching) and runs in float64 by default.

Notation: ``x`` [T, width] is one sequence's residual stream; linear weights are [out, in] and applied as ``x @ W.T``.
"""
from __future__ import annotations

import math
from typing import Dict, List, Optional

import torch


def rms_unit(x: torch.Tensor, eps: float) -> torch.Tensor:
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def norm_zero_centred(x, w, eps):
    return rms_unit(x, eps) * (1.0 + w)


def norm_plain(x, w, eps):
    return rms_unit(x, eps) * w


def short_conv_silu(x: torch.Tensor, w: torch.Tensor) -> torch.Tensor:
    """x [T, C], w [C, taps]; the last tap multiplies the current token, zeros before the sequence start"""
    T, C = x.shape
    taps = w.shape[1]
    out = torch.zeros_like(x)
    for t in range(T):
        for j in range(taps):
            s = t - (taps - 1) + j
            if s >= 0:
                out[t] += w[:, j] * x[s]
    return out * torch.sigmoid(out)


def unit_vec(x: torch.Tensor) -> torch.Tensor:
    return x / torch.sqrt((x * x).sum(-1, keepdim=True) + 1e-6)


def delta_recurrence(q, k, v, beta, g):
    """q, k [T, H, Dk] (already unit / scaled), v [T, H, Dv], beta [T, H], g [T, H] or [T, H, Dk] -> o [T, H, Dv]"""
    T, H, Dk = q.shape
    Dv = v.shape[-1]
    o = torch.zeros(T, H, Dv, dtype=q.dtype)
    for h in range(H):
        S = torch.zeros(Dk, Dv, dtype=q.dtype)
        for t in range(T):
            gt = g[t, h]
            S = S * (gt[:, None] if gt.dim() == 1 else gt)
            u = beta[t, h] * (v[t, h] - S.t() @ k[t, h])
            S = S + torch.outer(k[t, h], u)
            o[t, h] = S.t() @ q[t, h]
    return o


def delta_mixer(h: torch.Tensor, P: Dict[str, torch.Tensor], m: dict, eps: float, per_channel: bool) -> torch.Tensor:
    T = h.shape[0]
    H, Hk, Dk, Dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = short_conv_silu(h @ P["q"].t(), P["q.conv"]).view(T, Hk, Dk)
    k = short_conv_silu(h @ P["k"].t(), P["k.conv"]).view(T, Hk, Dk)
    v = short_conv_silu(h @ P["v"].t(), P["v.conv"]).view(T, H, Dv)
    q = unit_vec(q) * Dk ** -0.5
    k = unit_vec(k)
    rep = H // Hk
    q = q.repeat_interleave(rep, 1)
    k = k.repeat_interleave(rep, 1)
    beta = torch.sigmoid(h @ P["b"].t())
    if per_channel:
        a = (h @ P["a1"].t()) @ P["a2"].t() + P["dt_bias"]
        g = torch.exp(-torch.exp(P["A_log"])[None, :, None] * torch.nn.functional.softplus(a).view(T, H, Dk))
        gate = torch.sigmoid((h @ P["g1"].t()) @ P["g2"].t())
    else:
        a = h @ P["a"].t() + P["dt_bias"]
        g = torch.exp(-torch.exp(P["A_log"])[None, :] * torch.nn.functional.softplus(a))
        z = h @ P["g"].t()
        gate = z * torch.sigmoid(z)
    o = delta_recurrence(q, k, v, beta, g)
    o = rms_unit(o, eps) * P["norm"]
    o = o * gate.view(T, H, Dv)
    return o.reshape(T, H * Dv) @ P["o"].t()


def latent_attention(h: torch.Tensor, P: Dict[str, torch.Tensor], m: dict, eps: float) -> torch.Tensor:
    T = h.shape[0]
    H, D, Dv = m["heads"], m["dim"], m["vdim"]
    window = int(m["mask"]["size"]) if m.get("mask") else None
    q = (h @ P["q"].t()).view(T, H, D)
    c = norm_plain(h @ P["dkv"].t(), P["dkv.norm"], eps)
    k = (c @ P["uk"].t()).view(T, H, D)
    v = (c @ P["uv"].t()).view(T, H, Dv)
    out = torch.zeros(T, H, Dv, dtype=h.dtype)
    for i in range(T):
        lo = 0 if window is None else max(0, i - window + 1)
        for hh in range(H):
            s = (k[lo:i + 1, hh] @ q[i, hh]) * m["scale"]
            mx = torch.maximum(s.max(), P["sink"][hh])
            e = torch.exp(s - mx)
            den = e.sum() + torch.exp(P["sink"][hh] - mx)
            out[i, hh] = (e[:, None] * v[lo:i + 1, hh]).sum(0) / den
    return out.reshape(T, H * Dv) @ P["o"].t()


def clamped_glu(h, wg, wu, wd, limit):
    g = torch.clamp(h @ wg.t(), max=limit)
    u = torch.clamp(h @ wu.t(), -limit, limit)
    return (g * torch.sigmoid(1.702 * g) * (u + 1.0)) @ wd.t()


def route(h, w_router, r: dict):
    """-> (weights [T, top], expert ids [T, top])"""
    s = torch.sigmoid(h @ w_router.t())
    T, E = s.shape
    allowed = torch.ones(T, E, dtype=torch.bool)
    gr = r.get("groups")
    if gr:
        n, keep = int(gr["count"]), int(gr["keep"])
        per = E // n
        sg = s.view(T, n, per)
        score = sg.topk(min(2, per), dim=-1).values.sum(-1)
        best = score.topk(keep, dim=-1).indices
        ok = torch.zeros(T, n, dtype=torch.bool)
        ok.scatter_(1, best, True)
        allowed = ok[:, :, None].expand(T, n, per).reshape(T, E)
    ids = s.masked_fill(~allowed, -1.0).topk(int(r["top"]), dim=-1).indices
    w = s.gather(1, ids)
    w = w / (w.sum(-1, keepdim=True) + 1e-20) * float(r.get("scale", 1.0))
    return w, ids


def moe(h, P, mlp: dict):
    r = mlp["router"]
    w, ids = route(h, P["router"], r)
    out = torch.zeros(h.shape[0], P["e0.down"].shape[0], dtype=h.dtype)
    for t in range(h.shape[0]):
        for j in range(ids.shape[1]):
            e = int(ids[t, j])
            out[t] += w[t, j] * clamped_glu(h[t:t + 1], P[f"e{e}.gate"], P[f"e{e}.up"], P[f"e{e}.down"], mlp["expert"]["limit"])[0]
    return out


def sub(weights: Dict[str, torch.Tensor], prefix: str) -> Dict[str, torch.Tensor]:
    return {k[len(prefix):]: v for k, v in weights.items() if k.startswith(prefix)}


def forward(cfg: dict, weights: Dict[str, torch.Tensor], tokens: List[int], dtype=torch.float64, layers_out: Optional[list] = None) -> torch.Tensor:
    """whole sequence -> logits [T, vocab]"""
    W = {k: (v.to(dtype) if v.is_floating_point() else v) for k, v in weights.items()}
    eps = float(cfg["norm"]["eps"])
    x = W["embed"][torch.tensor(tokens)]
    for i, layer in enumerate(cfg["layers"]):
        pre = f"l{i}."
        h = norm_zero_centred(x, W[pre + "norm1"], eps)
        P = sub(W, pre + "mix.")
        kind = layer["type"]
        if kind == "latent_attention":
            y = latent_attention(h, P, layer["mixer"], eps)
        elif kind == "delta":
            y = delta_mixer(h, P, layer["mixer"], eps, False)
        elif kind == "channel_delta":
            y = delta_mixer(h, P, layer["mixer"], eps, True)
        else:
            raise ValueError(kind)
        x = x + y
        mlp = layer.get("mlp")
        if mlp:
            h = norm_zero_centred(x, W[pre + "norm2"], eps)
            M = sub(W, pre + "mlp.")
            x = x + (clamped_glu(h, M["gate"], M["up"], M["down"], mlp["limit"]) if mlp["kind"] == "dense" else moe(h, M, mlp))
        if layers_out is not None:
            layers_out.append(x.clone())
    x = norm_zero_centred(x, W["final.norm"], eps)
    logits = x @ W["head"].t()
    cap = cfg.get("logit_softcap")
    if cap:
        logits = cap * torch.tanh(logits / cap)
    return logits


def random_weights(cfg: dict, seed: int = 0, dtype=torch.float32) -> Dict[str, torch.Tensor]:
    """tensors under the checkpoint names for a configuration, sized so that activations stay O(1)"""
    g = torch.Generator().manual_seed(seed)
    W: Dict[str, torch.Tensor] = {}

    def lin(name, o, i, s=1.0):
        W[name] = (torch.randn(o, i, generator=g) * s / math.sqrt(i)).to(dtype)

    def vec(name, n, s=0.2, off=0.0):
        W[name] = (torch.randn(n, generator=g) * s + off).to(dtype)

    width, V = cfg["width"], cfg["vocab"]
    W["embed"] = torch.randn(V, width, generator=g).to(dtype)
    for i, layer in enumerate(cfg["layers"]):
        p, m = f"l{i}.", layer["mixer"]
        vec(p + "norm1", width)
        if layer["type"] == "latent_attention":
            H, D, Dv, R = m["heads"], m["dim"], m["vdim"], m["kv_rank"]
            lin(p + "mix.q", H * D, width, 2.0)
            lin(p + "mix.dkv", R, width)
            vec(p + "mix.dkv.norm", R, 0.2, 1.0)
            lin(p + "mix.uk", H * D, R, 2.0)
            lin(p + "mix.uv", H * Dv, R)
            vec(p + "mix.sink", H, 1.0)
            lin(p + "mix.o", width, H * Dv)
        else:
            H, Hk, Dk, Dv, taps = m["heads"], m["kv_heads"], m["dim"], m["vdim"], m["conv"]
            for nm, n in (("q", Hk * Dk), ("k", Hk * Dk), ("v", H * Dv)):
                lin(p + "mix." + nm, n, width)
                W[p + f"mix.{nm}.conv"] = (torch.randn(n, taps, generator=g) * 0.5).to(dtype)
            lin(p + "mix.b", H, width)
            vec(p + "mix.A_log", H, 0.5, -1.0)
            vec(p + "mix.norm", Dv, 0.2, 1.0)
            if layer["type"] == "channel_delta":
                r = m.get("rank", 8)
                lin(p + "mix.a1", r, width)
                lin(p + "mix.a2", H * Dk, r)
                vec(p + "mix.dt_bias", H * Dk, 0.5)
                lin(p + "mix.g1", r, width)
                lin(p + "mix.g2", H * Dv, r)
            else:
                lin(p + "mix.a", H, width)
                vec(p + "mix.dt_bias", H, 0.5)
                lin(p + "mix.g", H * Dv, width)
            lin(p + "mix.o", width, H * Dv)
        mlp = layer.get("mlp")
        if mlp:
            vec(p + "norm2", width)
            if mlp["kind"] == "dense":
                lin(p + "mlp.gate", mlp["ff"], width, 2.0)
                lin(p + "mlp.up", mlp["ff"], width, 2.0)
                lin(p + "mlp.down", width, mlp["ff"])
            else:
                ff = mlp["expert"]["ff"]
                for e in range(mlp["router"]["experts"]):
                    lin(p + f"mlp.e{e}.gate", ff, width, 2.0)
                    lin(p + f"mlp.e{e}.up", ff, width, 2.0)
                    lin(p + f"mlp.e{e}.down", width, ff)
                lin(p + "mlp.router", mlp["router"]["experts"], width, 3.0)
    vec("final.norm", width)
    lin("head", V, width)
    return W
