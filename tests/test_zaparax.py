"""Zaparax through the serving engine (CPU tier, fp32) against the plain oracle in ``zaparax_oracle.py``: every mechanism alone, prefill against
token-by-token decoding, prompt portions down to two tokens, unequal batches, page and slot reuse, window and page edges, far keys, the first
tokens, long decoding, weight-shared loops, sizes that differ from layer to layer, and greedy generation through ``Engine.generate``."""
import json
import math
import os

import numpy as np
import pytest
import torch

import sglang_b200 as sgl
import zaparax_oracle as O
from sglang_b200.layers.moe import softmax_bias_route
from sglang_b200.ops import torch_ref

PAGE = 8


def _mamba(heads=4, vdim=6, state=5, groups=2, conv=3, norm_groups=2):
    return {"type": "mamba2", "mixer": dict(heads=heads, vdim=vdim, state=state, groups=groups, conv=conv, norm_groups=norm_groups)}


def _attn(heads=4, kv_heads=2, dim=6, vdim=5, window=7, scale=0.6, softcap=4.0, coef=0.4, every=5):
    m = dict(heads=heads, kv_heads=kv_heads, dim=dim, vdim=vdim, scale=scale)
    if window:
        m["mask"] = {"size": window}
    if softcap:
        m["softcap"] = softcap
    if coef:
        m["q_temp"] = {"coef": coef, "every": every}
    return {"type": "attention", "mixer": m}


def _moe(experts=5, identity=2, top=2, ff=10, shared=14):
    m = {"kind": "moe", "expert": {"ff": ff}, "router": {"experts": experts, "identity": identity, "top": top}}
    if shared:
        m["shared"] = {"ff": shared}
    return m


def _cfg(layers, width=24, vocab=50, loop=None, eps=1e-5, bigram=True, scale=3.0):
    c = {"architecture": "Zaparax", "layers": layers, "norm": {"eps": eps}, "vocab": vocab, "width": width, "embedding": {"scale": scale}}
    if bigram:
        c["embedding"]["bigram"] = {"buckets": 37, "mul_prev": 11, "mul_cur": 5}
    if loop:
        c["loop"] = dict(zip(("start", "stop", "times"), loop))
    return c


def L(mix, mlp):
    return dict(mix, mlp=mlp)


# layers 1-2 (an attention and a Mamba-2 layer) run three times with the same weights; sizes differ from layer to layer
MIXED = _cfg([L(_attn(), _moe()), L(_attn(heads=3, kv_heads=3, dim=4, vdim=8, window=19, scale=0.9, softcap=0.0, every=3), None),
              L(_mamba(), _moe(experts=3, identity=0, top=1, shared=0)), L(_mamba(heads=2, vdim=9, state=12, groups=1, conv=4, norm_groups=3), None),
              L(_attn(heads=2, kv_heads=1, dim=8, vdim=8, window=0, coef=0.0), _moe(experts=4, identity=3, top=3, ff=6, shared=5))], loop=(1, 3, 3))
# every expert is chosen: nothing depends on which side of a near-tie a rounded router input falls (bf16 runs)
EVERY_EXPERT = _cfg([L(_mamba(), _moe(experts=3, identity=1, top=4)), L(_attn(), _moe(experts=2, identity=2, top=4, shared=0)),
                     L(_attn(heads=2, kv_heads=2, dim=8, vdim=4, window=30, every=7), None)], loop=(0, 2, 2))


def _wide(top_all):
    moe = lambda: _moe(experts=4, identity=2, top=6 if top_all else 2, ff=64, shared=128)
    return _cfg([L(_mamba(heads=4, vdim=64, state=64, groups=2, conv=4, norm_groups=4), moe()),
                 L(_attn(heads=4, kv_heads=2, dim=64, vdim=128, window=40, scale=0.125, softcap=30.0, every=16), moe())], width=128, vocab=192, loop=(0, 2, 2))


WIDE, WIDE_EVERY_EXPERT = _wide(False), _wide(True)
HEADS128_EVERY_EXPERT = _cfg([L(_attn(heads=4, kv_heads=2, dim=128, vdim=128, window=40, scale=0.09, softcap=30.0, every=16), _moe(experts=4, identity=2, top=6, ff=64, shared=128)),
                              L(_mamba(heads=4, vdim=64, state=64, groups=2, conv=4, norm_groups=4), None)], width=128, vocab=192, loop=(0, 1, 2))


def drawn_config(seed, every_expert=False, friendly=False):
    """a randomly drawn stack: order of layers, head counts and sizes, state sizes, taps, windows from 1 to beyond the prompt, expert counts,
    identity and shared experts, loop bounds and passes, bigram constants.  ``friendly``: sizes in multiples of 16 (vector lanes, GEMM tiles)"""
    rng = np.random.default_rng(seed)
    pick = lambda *a: a[int(rng.integers(len(a)))]
    u = 16 if friendly else 1
    layers = []
    for _ in range(int(rng.integers(2, 6))):
        if rng.random() < 0.5:
            g = pick(1, 2, 3)
            h = g * pick(1, 2, 4)
            vd = pick(8, 16, 32) if friendly else pick(3, 4, 7, 10)
            ng = pick(*[k for k in (1, 2, 3, 4, 6) if (h * vd) % k == 0])
            mix = _mamba(heads=h, vdim=vd, state=pick(16, 32) if friendly else pick(2, 5, 9, 17, 33), groups=g, conv=pick(1, 2, 3, 4, 5), norm_groups=ng)
        else:
            g = pick(1, 2, 3)
            mix = _attn(heads=g * pick(1, 2, 3, 5), kv_heads=g, dim=pick(16, 32) if friendly else pick(2, 5, 8, 12), vdim=pick(16, 48) if friendly else pick(3, 6, 9),
                        window=pick(0, 1, 2, 5, 16, 33, 200), scale=pick(0.3, 0.7, 1.1), softcap=pick(0.0, 2.0, 6.0), coef=pick(0.0, 0.3), every=pick(1, 4, 9))
        if rng.random() < 0.25:
            layers.append(L(mix, None))
            continue
        E, n_id = pick(1, 2, 4, 7), pick(0, 1, 3)
        top = E + n_id if every_expert else int(rng.integers(1, E + n_id + 1))
        layers.append(L(mix, _moe(experts=E, identity=n_id, top=top, ff=pick(16, 32) if friendly else pick(3, 8, 11), shared=pick(0, 16 if friendly else 5, 32 if friendly else 12))))
    n = len(layers)
    a = int(rng.integers(0, n))
    b = int(rng.integers(a + 1, n + 1))
    loop = pick(None, (a, b, pick(1, 2, 3)))
    c = _cfg(layers, width=pick(32, 64) if friendly else pick(10, 24, 36), vocab=pick(64, 128) if friendly else pick(19, 50, 131), loop=loop,
             bigram=rng.random() < 0.7, scale=pick(1.0, 2.5, 8.0))
    if "bigram" in c["embedding"]:
        c["embedding"]["bigram"] = {"buckets": pick(5, 37, 101), "mul_prev": pick(1, 11, 1000003), "mul_cur": pick(1, 5, 77)}
    return c


class Harness:
    """a model folder with random weights, an engine on it, and the oracle's logits for any token sequence"""

    def __init__(self, tmp, cfg, seed=0, slots=4, max_tokens=512, device="cpu", dtype="float32", page=PAGE):
        from safetensors.torch import save_file

        self.cfg = cfg
        self.W = O.random_weights(cfg, seed)
        d = os.path.join(str(tmp), f"m{seed}")
        os.makedirs(d, exist_ok=True)
        with open(os.path.join(d, "config.json"), "w") as f:
            json.dump({**cfg, "dtype": dtype}, f)
        if dtype == "bfloat16":          # the oracle sees the rounded weights the engine serves
            self.W = {k: v.to(torch.bfloat16).float() for k, v in self.W.items()}
        save_file({k: v.contiguous() for k, v in self.W.items()}, os.path.join(d, "model.safetensors"))
        self.dir = d
        self.eng = sgl.Engine(model_path=d, device=device, skip_tokenizer_init=True, page_size=page, max_total_tokens=max_tokens,
                              max_running_requests=slots, context_length=max_tokens, disable_radix_cache=True, chunked_prefill_size=-1,
                              max_prefill_tokens=max_tokens, log_level="warning")
        self.sched = self.eng.scheduler
        self._oracle = {}

    def oracle(self, tokens):
        k = tuple(tokens)
        if k not in self._oracle:
            self._oracle[k] = O.forward(self.cfg, self.W, list(tokens)).float().numpy()
        return self._oracle[k]

    def step(self, entries, end=()):
        return self.sched.replay_step([(i, list(t), list(w)) for i, t, w in entries], list(end))

    def run_cut(self, rid, tokens, cuts):
        """feed one request in portions of the given sizes (the rest token by token); returns logits of every position"""
        out, at = [], 0
        sizes = list(cuts) + [1] * (len(tokens) - sum(cuts))
        for n in sizes:
            last = at + n == len(tokens)
            out.append(self.step([(rid, tokens[at:at + n], range(n))], [rid] if last else []))
            at += n
        return np.concatenate(out, 0)

    def close(self):
        self.eng.shutdown()


def _tokens(n, vocab, seed):
    return np.random.default_rng(seed).integers(0, vocab, size=n).tolist()


def _close(a, b, tol=2e-4):
    err = np.abs(a - b).max()
    assert err < tol, err


# ------------------------------------------------------------------ mechanisms alone (functions of the serving path against the oracle's)
def test_router_against_oracle():
    g = torch.Generator().manual_seed(0)
    for E, n_id, top in ((5, 2, 2), (3, 0, 1), (4, 3, 3), (6, 1, 7), (1, 1, 1)):
        h, wr = torch.randn(40, 16, generator=g), torch.randn(E + n_id, 16, generator=g)
        W = {"r.router": wr.double(), "r.correction": (torch.randn(E + n_id, generator=g) * 0.3).double()}
        w1, i1, d1 = softmax_bias_route(h @ wr.t(), W["r.correction"].float(), top, E)
        w2, i2 = O.route(h.double(), W, "r.", {"top": top})
        o1, o2 = i1.long().sort(-1), i2.sort(-1)
        assert torch.equal(o1.values, o2.values)
        real = (o2.values < E)
        torch.testing.assert_close(w1.gather(1, o1.indices).double(), w2.gather(1, o2.indices) * real, rtol=1e-5, atol=1e-6)
        torch.testing.assert_close(d1.double(), (w2.gather(1, o2.indices) * ~real).sum(-1), rtol=1e-5, atol=1e-6)
    # the correction steers the choice only: a large correction on a weak expert gets it chosen, with its small plain score as the weight
    z = torch.tensor([[4.0, 0.0, -3.0]])
    w, i, _ = softmax_bias_route(z, torch.tensor([0.0, 0.0, 5.0]), 1, 3)
    assert int(i[0, 0]) == 2 and abs(float(w[0, 0]) - float(torch.softmax(z, -1)[0, 2])) < 1e-7


def test_mamba2_reference_op_against_oracle_and_far_memory():
    """the ragged reference op in two portions against the oracle's mixer; then one early write that must be read back 400 tokens later"""
    g = torch.Generator().manual_seed(1)
    m = dict(heads=4, vdim=3, state=5, groups=2, conv=1, norm_groups=1)
    H, P, N, G = 4, 3, 5, 2
    inner, T = H * P, 40
    u = torch.randn(T, inner + 2 * G * N, generator=g)
    z, dt_raw = torch.randn(T, inner, generator=g), torch.randn(T, H, generator=g)
    dtb, A_log, D = torch.randn(H, generator=g), torch.randn(H, generator=g) * 0.3, torch.randn(H, generator=g)
    state = torch.randn(3, H, N, P, generator=g)          # a used slot: a fresh request must not see it
    outs = []
    for lo, hi in ((0, 13), (13, 40)):
        outs.append(torch_ref.mamba2_scan(u[lo:hi], z[lo:hi], dt_raw[lo:hi], dtb, A_log, D, state, torch.tensor([2]), torch.tensor([hi]),
                                          torch.tensor([hi - lo]), H, P, N, G))
    got = torch.cat(outs)
    x, Bm, Cm = u[:, :inner].double().view(T, H, P), u[:, inner:inner + G * N].double().view(T, G, N), u[:, inner + G * N:].double().view(T, G, N)
    dt = torch.nn.functional.softplus(dt_raw.double() + dtb.double())
    S = torch.zeros(H, N, P, dtype=torch.float64)
    ref = torch.zeros(T, H, P, dtype=torch.float64)
    for t in range(T):
        for h in range(H):
            S[h] = math.exp(-math.exp(float(A_log[h])) * float(dt[t, h])) * S[h] + float(dt[t, h]) * torch.outer(Bm[t, h // 2], x[t, h])
            ref[t, h] = S[h].t() @ Cm[t, h // 2] + float(D[h]) * x[t, h]
    ref = ref.reshape(T, inner) * (z.double() * torch.sigmoid(z.double()))
    torch.testing.assert_close(got.double(), ref, rtol=1e-4, atol=1e-5)
    # far memory: slow decay, one large B x^T write at t = 3, C along the same direction only at the very end
    T = 404
    u = torch.randn(T, inner + 2 * G * N, generator=g) * 0.02
    u[3, inner] = 6.0                      # B, group 0, row 0
    u[3, 0:P] = torch.tensor([5.0, -4.0, 3.0])
    u[-1, inner + G * N] = 7.0             # C, group 0, row 0
    dt_raw = torch.zeros(T, H)
    state = torch.zeros(1, H, N, P)
    y = torch_ref.mamba2_scan(u, None, dt_raw, torch.zeros(H), torch.full((H,), -9.0), None, state, torch.tensor([0]), torch.tensor([T]),
                              torch.tensor([T]), H, P, N, G)
    want = math.log(2.0) * 6.0 * 7.0 * torch.tensor([5.0, -4.0, 3.0]) * math.exp(-math.exp(-9.0) * math.log(2.0) * (T - 4))
    assert (y[-1, :P] - want).abs().max() < 0.02 * want.abs().max()


def test_window_attention_reference_op_edges_sink_and_bias():
    """one key's value is made to stand out; it must count when it is the oldest key inside the window and vanish one step later, in a prompt
    portion and in a decode step, across a page border; the sink and the distance bias are checked against sums written out by hand"""
    H, G, D, Dv, W, ps = 2, 1, 6, 3, 11, 4
    g = torch.Generator().manual_seed(2)
    kc = torch.randn(64 * ps, 1, 8, generator=g) * 0.1
    vc = torch.randn(64 * ps, 1, 8, generator=g) * 0.1
    pages = torch.randperm(60, generator=g)[:16] + 1
    pt = torch.zeros(3, 20, dtype=torch.int32)
    pt[1, :16] = pages.int()
    slot_of = lambda pos: int(pages[pos // ps]) * ps + pos % ps
    mark = 19                                                   # position of the standout key: the last slot of a page
    kc[slot_of(mark), 0, :D] = torch.tensor([5.0, 0, 0, 0, 0, 0])
    vc[slot_of(mark), 0, :Dv] = 50.0
    sinks, slopes = torch.tensor([0.3, -0.2]), torch.tensor([0.5, 0.03])
    for qpos in (mark + W - 1, mark + W):                       # last position that sees it / first that does not
        q = torch.zeros(1, H, D)
        q[0, :, 0] = 3.0
        L_ = qpos + 1
        args = (kc, vc, G, Dv, pt, torch.tensor([1]), torch.tensor([L_]))
        out = torch_ref.window_attention(q, *args, None, ps, 0.7, 2.5, W, slopes, sinks)                                           # decode step
        out2 = torch_ref.window_attention(torch.cat([torch.zeros(3, H, D), q]), *args, torch.tensor([4]), ps, 0.7, 2.5, W, slopes, sinks)[-1:]
        torch.testing.assert_close(out, out2)
        lo = max(0, qpos - W + 1)
        K = torch.stack([kc[slot_of(p), 0, :D] for p in range(lo, L_)]).double()
        V = torch.stack([vc[slot_of(p), 0, :Dv] for p in range(lo, L_)]).double()
        for h in range(H):
            s = 2.5 * torch.tanh(K @ q[0, h].double() * 0.7 / 2.5) - slopes[h].double() * torch.arange(qpos - lo, -1, -1).double()
            den = torch.exp(s).sum() + torch.exp(sinks[h].double())
            torch.testing.assert_close(out[0, h].double(), (torch.exp(s)[:, None] * V).sum(0) / den, rtol=1e-5, atol=1e-6)
        assert (out[0, 1, 0].item() > 1.0) == (qpos == mark + W - 1)


def test_padded_head_layout_reference_ops():
    """heads laid out 16 columns wide (zeros behind the values) give the same q, the same cache contents under the padding and the same output"""
    g = torch.Generator().manual_seed(5)
    H, G, D, Dv, ps, T, pad = 4, 2, 6, 5, 4, 21, 16
    qkv = torch.randn(T, (H + G) * D + G * Dv, generator=g)
    pos = torch.arange(T, dtype=torch.int32)
    pt = torch.zeros(2, 8, dtype=torch.int32)
    pt[1, :6] = torch.tensor([3, 1, 6, 2, 5, 4], dtype=torch.int32)
    loc = (pt[1, (pos // ps).long()] * ps + pos % ps).int()
    k1, v1 = torch.zeros(8 * ps, 1, G * 6), torch.zeros(8 * ps, 1, G * 6)
    k2, v2 = torch.full((8 * ps, 1, G * pad), 9.0), torch.full((8 * ps, 1, G * pad), 9.0)          # stale numbers the padding has to overwrite
    q1 = torch_ref.qk_norm_cache_write(qkv, H, G, D, Dv, pos, 1e-5, 0.3, 4, k1, v1, loc)
    q2 = torch_ref.qk_norm_cache_write(qkv, H, G, D, Dv, pos, 1e-5, 0.3, 4, k2, v2, loc, True, pad)
    assert q2.shape == (T, H, pad) and torch.equal(q2[:, :, :D], q1) and float(q2[:, :, D:].abs().max()) == 0.0
    assert torch.equal(k2[loc.long(), 0].view(T, G, pad)[:, :, :D], k1[loc.long(), 0, :G * D].view(T, G, D))
    assert float(k2[loc.long(), 0].view(T, G, pad)[:, :, D:].abs().max()) == 0.0 and float(v2[loc.long(), 0].view(T, G, pad)[:, :, Dv:].abs().max()) == 0.0
    args = (pt, torch.tensor([1]), torch.tensor([T]), torch.tensor([T]), ps, 0.8, 3.0, 7, torch.tensor([0.5, 0.1, 0.03, 0.01]), torch.randn(H, generator=g))
    o1 = torch_ref.window_attention(q1, k1, v1, G, Dv, *args)
    o2 = torch_ref.window_attention(q2, k2, v2, G, Dv, *args, D, pad)
    torch.testing.assert_close(o2, o1)


def test_far_key_without_a_window():
    """no window: a key 300 positions back still wins when its score stands out (small slope head), and loses on the steep-slope head"""
    H, G, D, Dv, ps = 2, 1, 4, 2, 8
    g = torch.Generator().manual_seed(3)
    n = 330
    kc, vc = torch.randn(64 * ps, 1, 4, generator=g) * 0.05, torch.randn(64 * ps, 1, 4, generator=g) * 0.05
    pt = torch.zeros(2, 64, dtype=torch.int32)
    pt[1, :42] = torch.arange(1, 43).int()
    far = 9
    kc[ps + far, 0, :D] = torch.tensor([9.0, 0, 0, 0])
    vc[ps + far, 0, :Dv] = 10.0
    q = torch.zeros(1, H, D)
    q[0, :, 0] = 2.0
    out = torch_ref.window_attention(q, kc, vc, G, Dv, pt, torch.tensor([1]), torch.tensor([n]), None, ps, 1.0, 0.0, -1,
                                     torch.tensor([0.4, 0.001]), torch.zeros(H))
    assert out[0, 1, 0].item() > 9.0 and abs(out[0, 0, 0].item()) < 0.5


def test_bigram_embedding_reference_op_keeps_the_previous_token():
    g = torch.Generator().manual_seed(4)
    V, Wd, NB = 30, 6, 13
    emb, bg = torch.randn(V, Wd, generator=g), torch.randn(NB + 1, Wd, generator=g)
    cfg = {"embedding": {"scale": 2.0, "bigram": {"buckets": NB, "mul_prev": 7, "mul_cur": 3}}}
    toks = _tokens(23, V, 1)
    ref = O.embed(cfg, {"embed": emb.double(), "bigram": bg.double()}, toks)
    prev = torch.full((4,), 17, dtype=torch.int32)              # stale entries of earlier requests
    out, at = [], 0
    for n in (1, 2, 9, 1, 1, 9):
        ids = torch.tensor(toks[at:at + n], dtype=torch.int32)
        out.append(torch_ref.bigram_embedding(emb, bg, ids, prev, torch.tensor([0, n]) if n > 1 else None, torch.tensor([2]), torch.tensor([at + n]),
                                              2.0, 7, 3, NB))
        at += n
    torch.testing.assert_close(torch.cat(out).double(), ref, rtol=1e-6, atol=1e-6)
    assert int(prev[2]) == toks[-1] and int(prev[0]) == 17


def test_layer_runs_and_config_reader(tmp_path):
    from sglang_b200.configs.model_config import load_model_config
    from sglang_b200.models.zaparax import layer_runs

    assert layer_runs(5, {"start": 1, "stop": 3, "times": 3}) == [0, 1, 2, 1, 2, 1, 2, 3, 4] == O.layer_runs({"layers": [0] * 5, "loop": MIXED["loop"]})
    assert layer_runs(3, None) == [0, 1, 2] and layer_runs(3, {"start": 0, "stop": 3, "times": 2}) == [0, 1, 2, 0, 1, 2]
    assert layer_runs(2, {"start": 1, "stop": 2, "times": 1}) == [0, 1]
    d = tmp_path / "cfg"
    d.mkdir()
    (d / "config.json").write_text(json.dumps(MIXED))
    c = load_model_config(str(d))
    assert c.architecture == "Zaparax" and c.hidden_size == 24 and c.vocab_size == 50 and c.num_hidden_layers == 5 and c.rms_norm_eps == 1e-5
    assert c.hybrid["layers"][1]["mixer"]["mask"]["size"] == 19 and c.hybrid["loop"]["times"] == 3 and c.hybrid["embedding"]["bigram"]["buckets"] == 37


# ------------------------------------------------------------------ single mechanisms through the engine
@pytest.mark.parametrize("cfg", [
    _cfg([L(_mamba(), None)]), _cfg([L(_mamba(heads=3, vdim=4, state=9, groups=3, conv=1, norm_groups=1), None)], bigram=False),
    _cfg([L(_mamba(heads=2, vdim=8, state=3, groups=1, conv=6, norm_groups=4), _moe())]),
    _cfg([L(_attn(), None)]), _cfg([L(_attn(window=1), _moe(identity=0))]), _cfg([L(_attn(heads=6, kv_heads=1, window=0, softcap=0.0, coef=0.0), None)]),
    _cfg([L(_attn(heads=2, kv_heads=2, dim=3, vdim=11, window=4, every=1), _moe(experts=2, identity=4, top=3, shared=0))], loop=(0, 1, 4)),
    _cfg([L(_mamba(), _moe(experts=6, identity=1, top=1))], loop=(0, 1, 2), scale=1.0)])
def test_one_layer_models(tmp_path, cfg):
    h = Harness(tmp_path, cfg)
    toks = _tokens(37, 50, 5)
    ref = h.oracle(toks)
    _close(h.step([("a", toks, range(len(toks)))], ["a"]), ref)                    # whole prompt
    _close(h.run_cut("b", toks, []), ref)                                          # token by token from the first token
    h.close()


# ------------------------------------------------------------------ the mixed model: cuts, batches, reuse
@pytest.fixture(scope="module")
def mixed(tmp_path_factory):
    h = Harness(tmp_path_factory.mktemp("zaparax"), MIXED, seed=3, slots=4, max_tokens=40 * PAGE)
    yield h
    h.close()


def test_residual_after_every_layer_run(mixed):
    toks = _tokens(17, 50, 6)
    want, got = [], []
    O.forward(mixed.cfg, mixed.W, toks, tap=lambda run, x: want.append(x.float()))
    model = mixed.sched.worker.runner.model if hasattr(mixed.sched.worker, "runner") else mixed.sched.worker.model
    model.layer_tap = lambda run, x: got.append(x.clone())
    try:
        mixed.step([("t", toks, [])], ["t"])
    finally:
        model.layer_tap = None
    assert len(got) == len(want) == 9
    for a, b in zip(got, want):
        torch.testing.assert_close(a.cpu(), b, rtol=1e-4, atol=1e-4)


def test_first_tokens_and_prefill_against_decode(mixed):
    toks = _tokens(61, 50, 7)
    ref = mixed.oracle(toks)
    whole = mixed.step([("w", toks, range(len(toks)))], ["w"])
    _close(whole, ref)
    _close(whole[:3], ref[:3], 1e-4)                                               # positions 0, 1, 2: zero history, the bigram's start row
    _close(mixed.run_cut("d", toks, [30]), ref)                                    # 30 at once, then 31 decode steps (windows 7 and 19 pass over them)


@pytest.mark.parametrize("cuts", [[2, 2, 2, 3, 2], [7, 8, 9, 2, 16], [1, 2, 17, 2, 2, 23], [PAGE, PAGE, 2 * PAGE], [PAGE - 1, 2, PAGE + 1, 19]])
def test_portions_of_many_sizes(mixed, cuts):
    toks = _tokens(70, 50, 11)
    _close(mixed.run_cut("c", toks, cuts), mixed.oracle(toks))


def test_unequal_batches_and_reuse_of_pages_and_slots(mixed):
    rng = np.random.default_rng(5)
    lens = [53, 9, 31, 2, 44, 18, 27]
    seqs = [_tokens(n, 50, 100 + i) for i, n in enumerate(lens)]
    at = [0] * len(seqs)
    got = [[] for _ in seqs]
    waiting, live = list(range(len(seqs))), []
    rounds = 0
    while waiting or live:
        while waiting and len(live) < 4:                                           # four slots: later requests take over freed slots and pages
            live.append(waiting.pop(0))
        entries, end = [], []
        for i in live:
            left = len(seqs[i]) - at[i]
            n = int(min(left, rng.choice([1, 1, 2, 3, 5, 11, 16])))
            if at[i] and rng.random() < 0.2:
                continue                                                           # a request may sit a step out
            entries.append((f"r{i}", seqs[i][at[i]:at[i] + n], range(n)))
        if not entries:
            continue
        for rid, t, _ in entries:
            i = int(rid[1:])
            if at[i] + len(t) == len(seqs[i]):
                end.append(rid)
        out = mixed.step(entries, end)
        o = 0
        for rid, t, _ in entries:
            i = int(rid[1:])
            got[i].append(out[o:o + len(t)])
            o += len(t)
            at[i] += len(t)
            if at[i] == len(seqs[i]):
                live.remove(i)
        rounds += 1
    assert rounds > 10
    for i, s in enumerate(seqs):
        _close(np.concatenate(got[i], 0), mixed.oracle(s))
    assert mixed.sched.kv.allocator.available_pages() == mixed.sched.kv.allocator.total_pages        # everything was given back
    assert mixed.sched.kv.slots.available() == 4


def test_long_decoding_past_every_window(mixed):
    toks = _tokens(5 + 90, 50, 13)
    _close(mixed.run_cut("l", toks, [5]), mixed.oracle(toks), 3e-4)


def test_greedy_generation_through_the_engine(mixed):
    prompts = [_tokens(n, 50, 40 + n) for n in (12, 3, 25)]
    outs = mixed.eng.generate(input_ids=prompts, sampling_params={"max_new_tokens": 10, "temperature": 0, "ignore_eos": True})
    for p, o in zip(prompts, outs):
        seq = list(p)
        for _ in range(10):
            seq.append(int(mixed.oracle(seq)[-1].argmax()))
        assert o["output_ids"] == seq[len(p):]
    mixed.sched.check_invariants()


def test_other_sizes_whole_portions_and_batch(tmp_path):
    h = Harness(tmp_path, EVERY_EXPERT, seed=9, max_tokens=30 * PAGE)
    a, b = _tokens(58, 50, 1), _tokens(21, 50, 2)
    ra, rb = h.oracle(a), h.oracle(b)
    _close(h.run_cut("a", a, [29, 2, 2]), ra)
    out = h.step([("a", a[:40], range(40)), ("b", b, range(len(b)))], ["b"])
    _close(out[:40], ra[:40]); _close(out[40:], rb)
    _close(h.step([("a", a[40:], range(18))], ["a"]), ra[40:])
    h.close()


def test_text_prompts_on_a_weights_only_folder(tmp_path):
    """a folder with only config.json and model.safetensors serves text through the byte tokenizer (what `cli generate` and the HTTP server do)"""
    h = Harness(tmp_path, _cfg([L(_mamba(), _moe()), L(_attn(), None)], vocab=300), seed=8)
    h.close()
    eng = sgl.Engine(model_path=h.dir, device="cpu", page_size=PAGE, max_total_tokens=256, max_running_requests=2, log_level="warning")
    out = eng.generate("hello there", {"max_new_tokens": 4, "temperature": 0.7, "top_k": 5, "ignore_eos": True})
    assert len(out["output_ids"]) == 4 and isinstance(out["text"], str)
    eng.shutdown()


@pytest.mark.parametrize("seed", [1, 2, 3])
def test_randomly_drawn_stacks(tmp_path, seed):
    cfg = drawn_config(seed)
    h = Harness(tmp_path, cfg, seed=50 + seed, max_tokens=30 * PAGE)
    V = cfg["vocab"]
    a, b = _tokens(45, V, 1), _tokens(14, V, 2)
    ra, rb = h.oracle(a), h.oracle(b)
    _close(h.step([("w", a, range(len(a)))], ["w"]), ra, 3e-4)
    _close(h.run_cut("c", a, [19, 2, 9, 2]), ra, 3e-4)
    out = h.step([("a", a[:30], range(30)), ("b", b, range(len(b)))], ["b"])
    _close(out[:30], ra[:30], 3e-4); _close(out[30:], rb, 3e-4)
    _close(h.step([("a", a[30:], range(15))], ["a"]), ra[30:], 3e-4)
    h.close()
