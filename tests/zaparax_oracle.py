"""A plain, slow restatement of the Zaparax decoder, written from its equations with one function per mechanism.  It shares no code with the
serving path: every token is visited one by one, every sum is spelled out, everything is float64.  The tests compare the engine with it.

Notation: ``h`` the normed input of a sublayer, ``p`` a position (from 0), ``W x`` a stored [out, in] matrix applied to a vector.
"""
import math

import torch

F64 = torch.float64


def rms(x, eps):
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def norm(x, w, eps):
    """weights stored around zero"""
    return rms(x, eps) * (1.0 + w)


def silu(z):
    return z * torch.sigmoid(z)


def layer_runs(cfg):
    """which layer runs when: the looped stretch is repeated with the same weights, every run keeps its own cache or state"""
    n = len(cfg["layers"])
    lp = cfg.get("loop") or {}
    a, b, times = int(lp.get("start", 0)), int(lp.get("stop", 0)), int(lp.get("times", 1))
    if not lp or b <= a:
        return list(range(n))
    return list(range(a)) + list(range(a, b)) * times + list(range(b, n))


def embed(cfg, W, tokens):
    e = cfg["embedding"]
    x = W["embed"][tokens] * float(e.get("scale", 1.0))
    bg = e.get("bigram")
    if bg:
        nb = int(bg["buckets"])
        for t, tok in enumerate(tokens):
            row = nb if t == 0 else (tokens[t - 1] * int(bg["mul_prev"]) + tok * int(bg["mul_cur"])) % nb
            x[t] = x[t] + W["bigram"][row]
    return x


def mamba2(h, m, W, pre, eps):
    """h [T, width] -> [T, width]; state and convolution history start at zero"""
    T = h.shape[0]
    H, P, N, G, taps = int(m["heads"]), int(m["vdim"]), int(m["state"]), int(m["groups"]), int(m["conv"])
    ng = int(m.get("norm_groups", 1))
    inner = H * P
    proj = h @ W[pre + "in"].t()
    z, xbc, dt = proj[:, :inner], proj[:, inner:2 * inner + 2 * G * N], proj[:, 2 * inner + 2 * G * N:]
    cw, cb = W[pre + "conv"], W[pre + "conv.b"]
    conv = torch.zeros_like(xbc)
    for t in range(T):
        acc = cb.clone()
        for j in range(taps):
            src = t - (taps - 1) + j
            if src >= 0:
                acc = acc + cw[:, j] * xbc[src]
        conv[t] = silu(acc)
    x = conv[:, :inner].reshape(T, H, P)
    B = conv[:, inner:inner + G * N].reshape(T, G, N)
    C = conv[:, inner + G * N:].reshape(T, G, N)
    dt = torch.nn.functional.softplus(dt + W[pre + "dt_bias"], threshold=1e9)
    a = torch.exp(W[pre + "A_log"])
    S = torch.zeros(H, N, P, dtype=h.dtype)
    y = torch.zeros(T, H, P, dtype=h.dtype)
    for t in range(T):
        for hd in range(H):
            g = hd // (H // G)
            S[hd] = math.exp(-float(a[hd]) * float(dt[t, hd])) * S[hd] + float(dt[t, hd]) * torch.outer(B[t, g], x[t, hd])
            y[t, hd] = S[hd].t() @ C[t, g] + W[pre + "D"][hd] * x[t, hd]
    y = y.reshape(T, inner) * silu(z)
    y = rms(y.reshape(T, ng, inner // ng), eps).reshape(T, inner) * W[pre + "norm"]
    return y @ W[pre + "o"].t()


def attention(h, m, W, pre, eps):
    T = h.shape[0]
    H, G, D, Dv = int(m["heads"]), int(m["kv_heads"]), int(m["dim"]), int(m["vdim"])
    q = (h @ W[pre + "q"].t() + W[pre + "q.b"]).reshape(T, H, D)
    k = (h @ W[pre + "k"].t() + W[pre + "k.b"]).reshape(T, G, D)
    v = (h @ W[pre + "v"].t() + W[pre + "v.b"]).reshape(T, G, Dv)
    q, k = rms(q, eps), rms(k, eps)
    qt = m.get("q_temp")
    window = int((m.get("mask") or {}).get("size") or 0)
    cap = float(m.get("softcap") or 0.0)
    scale = float(m["scale"]) if m.get("scale") is not None else D ** -0.5
    out = torch.zeros(T, H, Dv, dtype=h.dtype)
    for i in range(T):
        temp = 1.0 + float(qt["coef"]) * math.log((i + 1) // int(qt["every"]) + 1) if qt else 1.0
        for hd in range(H):
            g = hd // (H // G)
            slope = 2.0 ** (-8.0 * (hd + 1) / H)
            lo = max(0, i - window + 1) if window > 0 else 0
            s = []
            for j in range(lo, i + 1):
                sc = float((q[i, hd] * temp) @ k[j, g]) * scale
                if cap > 0:
                    sc = cap * math.tanh(sc / cap)
                s.append(sc - slope * (i - j))
            s = torch.tensor(s, dtype=h.dtype)
            sink = W.get(pre + "sink")
            mx = max(float(s.max()), float(sink[hd])) if sink is not None else float(s.max())
            e = torch.exp(s - mx)
            den = e.sum() + (math.exp(float(sink[hd]) - mx) if sink is not None else 0.0)
            out[i, hd] = (e[:, None] * v[lo:i + 1, g]).sum(0) / den
    return out.reshape(T, H * Dv) @ W[pre + "o"].t()


def glu(h, W, pre):
    return (silu(h @ W[pre + "gate"].t()) * (h @ W[pre + "up"].t())) @ W[pre + "down"].t()


def route(h, W, pre, r):
    """-> (weights [T, top], chosen [T, top]) over experts + identity experts"""
    s = torch.softmax(h @ W[pre + "router"].t(), -1)
    choice = s + W[pre + "correction"] if (pre + "correction") in W else s
    idx = torch.topk(choice, int(r["top"]), dim=-1).indices
    return s.gather(1, idx), idx


def moe(h, mlp, W, pre):
    r = mlp["router"]
    E, n_id = int(r["experts"]), int(r.get("identity", 0))
    w, idx = route(h, W, pre, r)
    out = torch.zeros_like(h)
    for t in range(h.shape[0]):
        for j in range(idx.shape[1]):
            e = int(idx[t, j])
            if e >= E:
                assert e < E + n_id
                out[t] = out[t] + w[t, j] * h[t]
            else:
                out[t] = out[t] + w[t, j] * glu(h[t:t + 1], W, pre + f"e{e}.")[0]
    if mlp.get("shared"):
        out = out + torch.sigmoid(h @ W[pre + "shared.sg"].t()) * glu(h, W, pre + "shared.")
    return out


def forward(cfg, W, tokens, tap=None, dtype=F64):
    """logits [T, vocab] of one sequence; ``tap(run, x)`` sees the residual stream after every layer run"""
    W = {k: (v.to(dtype) if v.is_floating_point() else v) for k, v in W.items()}
    eps = float(cfg["norm"]["eps"])
    x = embed(cfg, W, list(tokens))
    for run, i in enumerate(layer_runs(cfg)):
        sp, p = cfg["layers"][i], f"l{i}."
        h = norm(x, W[p + "norm1"], eps)
        y = mamba2(h, sp["mixer"], W, p + "mix.", eps) if sp["type"] == "mamba2" else attention(h, sp["mixer"], W, p + "mix.", eps)
        x = x + norm(y, W[p + "norm1b"], eps)
        if sp.get("mlp"):
            h = norm(x, W[p + "norm2"], eps)
            x = x + norm(moe(h, sp["mlp"], W, p + "mlp."), W[p + "norm2b"], eps)
        if tap is not None:
            tap(run, x)
    return norm(x, W["final.norm"], eps) @ W["head"].t()


def random_weights(cfg, seed=0):
    """random tensors under the checkpoint names, scaled so that every mechanism matters in the logits"""
    g = torch.Generator().manual_seed(seed)
    rn = lambda *s, sc=1.0, off=0.0: torch.randn(*s, generator=g) * sc + off
    lin = lambda o, i, sc=1.0: rn(o, i, sc=sc * i ** -0.5)
    Wd, V = int(cfg["width"]), int(cfg["vocab"])
    W = {"embed": rn(V, Wd, sc=0.3), "final.norm": rn(Wd, sc=0.2), "head": lin(V, Wd)}
    bg = cfg["embedding"].get("bigram")
    if bg:
        W["bigram"] = rn(int(bg["buckets"]) + 1, Wd, sc=2.0)
    for i, sp in enumerate(cfg["layers"]):
        p, m = f"l{i}.", sp["mixer"]
        for nm in ("norm1", "norm1b") + (("norm2", "norm2b") if sp.get("mlp") else ()):
            W[p + nm] = rn(Wd, sc=0.2)
        if sp["type"] == "mamba2":
            H, P, N, G, taps = int(m["heads"]), int(m["vdim"]), int(m["state"]), int(m["groups"]), int(m["conv"])
            inner, ch = H * P, H * P + 2 * G * N
            W[p + "mix.in"] = lin(2 * inner + 2 * G * N + H, Wd, 1.5)
            W[p + "mix.conv"] = rn(ch, taps, sc=0.6)
            W[p + "mix.conv.b"] = rn(ch, sc=0.2)
            W[p + "mix.dt_bias"] = rn(H, sc=1.0, off=-1.5)
            W[p + "mix.A_log"] = rn(H, sc=0.7, off=-1.0)
            W[p + "mix.D"] = rn(H, sc=0.5, off=0.5)
            W[p + "mix.norm"] = rn(inner, sc=0.2, off=1.0)
            W[p + "mix.o"] = lin(Wd, inner)
        else:
            H, G, D, Dv = int(m["heads"]), int(m["kv_heads"]), int(m["dim"]), int(m["vdim"])
            W[p + "mix.q"], W[p + "mix.q.b"] = lin(H * D, Wd, 2.0), rn(H * D, sc=0.3)
            W[p + "mix.k"], W[p + "mix.k.b"] = lin(G * D, Wd, 2.0), rn(G * D, sc=0.3)
            W[p + "mix.v"], W[p + "mix.v.b"] = lin(G * Dv, Wd), rn(G * Dv, sc=0.3)
            W[p + "mix.sink"] = rn(H, sc=1.0)
            W[p + "mix.o"] = lin(Wd, H * Dv)
        mlp = sp.get("mlp")
        if not mlp:
            continue
        r = mlp["router"]
        E, n_id, ff = int(r["experts"]), int(r.get("identity", 0)), int(mlp["expert"]["ff"])
        for e in range(E):
            q = p + f"mlp.e{e}."
            W[q + "gate"], W[q + "up"], W[q + "down"] = lin(ff, Wd, 2.0), lin(ff, Wd, 2.0), lin(Wd, ff, 2.0)
        W[p + "mlp.router"] = lin(E + n_id, Wd, 3.0)
        W[p + "mlp.correction"] = rn(E + n_id, sc=0.05)
        if mlp.get("shared"):
            fs = int(mlp["shared"]["ff"])
            q = p + "mlp.shared."
            W[q + "gate"], W[q + "up"], W[q + "down"], W[q + "sg"] = lin(fs, Wd, 2.0), lin(fs, Wd, 2.0), lin(Wd, fs, 2.0), lin(1, Wd, 2.0)
    return W
