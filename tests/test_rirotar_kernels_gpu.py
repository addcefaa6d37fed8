"""CUDA kernels of the Rirotar mechanisms against plain fp32 PyTorch references of the same ops (``ops.torch_ref``), which the CPU tests in
``test_rirotar.py`` check against the token-by-token oracle."""
import pytest
import torch

from sglang_b200 import ops
from sglang_b200.ops import torch_ref

pytestmark = pytest.mark.gpu
DEV = "cuda"


def _native():
    assert ops.load_native(), "CUDA extension not built"


@pytest.mark.parametrize("H", [96, 256, 1000])
@pytest.mark.parametrize("ddt,odt", [(torch.bfloat16, torch.bfloat16), (torch.float32, torch.float32), (None, torch.bfloat16)])
def test_add_rmsnorm_f32(H, ddt, odt):
    _native()
    g = torch.Generator(device=DEV).manual_seed(H)
    res = torch.randn(7, H, device=DEV, generator=g) * 3
    delta = None if ddt is None else torch.randn(7, H, device=DEV, generator=g).to(ddt)
    w = (torch.randn(H, device=DEV, generator=g) * 0.2).to(odt)
    for zc in (True, False):
        r1, r2 = res.clone(), res.clone()
        o1 = ops.add_rmsnorm_f32(r1, delta, w, 1e-5, zc, odt)
        o2 = torch_ref.add_rmsnorm_f32(r2, delta, w, 1e-5, zc, odt)
        assert o1.dtype == odt
        torch.testing.assert_close(r1, r2, rtol=0, atol=0)
        torch.testing.assert_close(o1.float(), o2.float(), rtol=1e-2 if odt == torch.bfloat16 else 2e-6, atol=1e-2 if odt == torch.bfloat16 else 2e-6)


@pytest.mark.parametrize("dt", [torch.bfloat16, torch.float32])
def test_clamped_glu(dt):
    _native()
    gu = (torch.randn(33, 2 * 70, device=DEV) * 3).to(dt)
    a = ops.clamped_glu(gu, 1.5)
    b = torch_ref.clamped_glu(gu, 1.5)
    torch.testing.assert_close(a.float(), b.float(), rtol=1e-2 if dt == torch.bfloat16 else 1e-6, atol=1e-2 if dt == torch.bfloat16 else 1e-6)


def _paged(seq_lens, page_size, width, dtype, seed):
    """a page table whose pages are scattered over the pool, and a cache full of values"""
    g = torch.Generator().manual_seed(seed)
    need = [(-(-L // page_size)) for L in seq_lens]
    total = sum(need) + 3
    perm = (torch.randperm(total - 1, generator=g) + 1).tolist()
    pt = torch.zeros(len(seq_lens) + 2, max(need) + 1, dtype=torch.int32)
    slots = [2, 0, 3, 1][: len(seq_lens)]
    for b, n in enumerate(need):
        for c in range(n):
            pt[slots[b], c] = perm.pop()
    cache = torch.randn(total * page_size, 1, width, generator=g).to(dtype)
    return pt.to(DEV), torch.tensor(slots, dtype=torch.int32, device=DEV), cache.to(DEV)


@pytest.mark.parametrize("cdt", [torch.bfloat16, torch.float32])
@pytest.mark.parametrize("R,H,window", [(40, 5, 19), (72, 7, 141), (128, 3, -1), (24, 17, 1)])
def test_latent_attention_prefill_and_decode(cdt, R, H, window):
    _native()
    ps = 16
    seq = [75, 203, 9, 130]
    ql = [75, 37, 2, 1]
    pt, slots, cache = _paged(seq, ps, R + 8, cdt, R)
    g = torch.Generator(device=DEV).manual_seed(1)
    sinks = torch.randn(H, device=DEV, generator=g)
    sl = torch.tensor(seq, dtype=torch.int32, device=DEV)
    q_lens = torch.tensor(ql, dtype=torch.int32, device=DEV)
    cu = torch.zeros(5, dtype=torch.int32, device=DEV)
    cu[1:] = torch.cumsum(q_lens, 0)
    q = torch.randn(sum(ql), H, R, device=DEV, generator=g) * 0.5
    for sk in (sinks, None):
        a = ops.latent_attention(q, cache, R, pt, slots, sl, cu, q_lens, max(ql), ps, 0.3, window, sk)
        b = torch_ref.latent_attention(q, cache, R, pt, slots, sl, q_lens, ps, 0.3, window, sk)
        torch.testing.assert_close(a, b, rtol=2e-5, atol=2e-5)
    # decode: one query per request
    qd = torch.randn(4, H, R, device=DEV, generator=g) * 0.5
    a = ops.latent_attention(qd, cache, R, pt, slots, sl, None, None, 1, ps, 0.3, window, sinks)
    b = torch_ref.latent_attention(qd, cache, R, pt, slots, sl, None, ps, 0.3, window, sinks)
    torch.testing.assert_close(a, b, rtol=2e-5, atol=2e-5)


@pytest.mark.parametrize("Hk,H,Dk,Dv,chan", [(1, 2, 32, 32, False), (4, 4, 32, 32, True), (2, 6, 24, 40, True), (2, 4, 128, 128, False),
                                             (1, 2, 64, 256, True), (1, 1, 200, 64, False), (3, 3, 8, 16, True)])
def test_gated_delta_rule(Hk, H, Dk, Dv, chan):
    _native()
    g = torch.Generator(device=DEV).manual_seed(Dk * 7 + Dv)
    ql = [19, 1, 30, 3]
    seq = [19, 50, 44, 3]            # requests 0 and 3 are fresh, 1 is a decode step, 2 continues a prompt
    T = sum(ql)
    u = torch.randn(T, 2 * Hk * Dk + H * Dv, device=DEV, generator=g)
    a_raw = torch.randn(T, H * Dk if chan else H, device=DEV, generator=g)
    A_log = torch.randn(H, device=DEV, generator=g) * 0.5 - 1
    dtb = torch.randn(H * Dk if chan else H, device=DEV, generator=g) * 0.5
    b_raw = torch.randn(T, H, device=DEV, generator=g)
    gate = torch.randn(T, H * Dv, device=DEV, generator=g)
    nw = torch.randn(Dv, device=DEV, generator=g) * 0.2 + 1
    state = torch.randn(6, H, Dk, Dv, device=DEV, generator=g) * 0.3
    slots = torch.tensor([4, 1, 0, 5], dtype=torch.int32, device=DEV)
    sl = torch.tensor(seq, dtype=torch.int32, device=DEV)
    q_lens = torch.tensor(ql, dtype=torch.int32, device=DEV)
    cu = torch.zeros(5, dtype=torch.int32, device=DEV)
    cu[1:] = torch.cumsum(q_lens, 0)
    for act in ("silu", "sigmoid"):
        s1, s2 = state.clone(), state.clone()
        o1 = ops.gated_delta_rule(u, Hk, Dk, H, Dv, a_raw, A_log, dtb, b_raw, s1, slots, sl, cu, q_lens, gate, nw, 1e-5, act, chan)
        o2 = torch_ref.gated_delta_rule(u, Hk, Dk, H, Dv, a_raw, A_log, dtb, b_raw, s2, slots, sl, q_lens, gate, nw, 1e-5, act, chan)
        torch.testing.assert_close(o1, o2, rtol=1e-4, atol=1e-5)
        torch.testing.assert_close(s1, s2, rtol=1e-4, atol=1e-5)
    # decode form (no cu_q) and raw read-out (no norm)
    ud = u[:4].contiguous()
    s1, s2 = state.clone(), state.clone()
    sld = torch.tensor([7, 2, 9, 31], dtype=torch.int32, device=DEV)
    o1 = ops.gated_delta_rule(ud, Hk, Dk, H, Dv, a_raw[:4].contiguous(), A_log, dtb, b_raw[:4].contiguous(), s1, slots, sld, None, None,
                              per_channel=chan)
    o2 = torch_ref.gated_delta_rule(ud, Hk, Dk, H, Dv, a_raw[:4], A_log, dtb, b_raw[:4], s2, slots, sld, None, per_channel=chan)
    torch.testing.assert_close(o1, o2, rtol=1e-4, atol=1e-5)
    torch.testing.assert_close(s1, s2, rtol=1e-4, atol=1e-5)


def test_latent_attention_standout_key_at_the_window_edge():
    """a key whose latent row dominates the scores is seen by the last query inside the window and not by the next one (decode and portion)"""
    _native()
    R, H, W, ps = 48, 3, 33, 16
    g = torch.Generator().manual_seed(4)
    pages = torch.randperm(40, generator=g)[:12] + 1
    pt = torch.zeros(3, 16, dtype=torch.int32)
    pt[2, :12] = pages.int()
    cache = torch.randn(48 * ps, 1, R, generator=g) * 0.1
    mark = 63                                                   # last slot of a page
    cache[int(pages[mark // ps]) * ps + mark % ps, 0, 0] = 5.0
    cache, pt = cache.to(DEV), pt.to(DEV)
    slots = torch.tensor([2], dtype=torch.int32, device=DEV)
    for qpos in (mark + W - 1, mark + W):
        q = torch.zeros(5, H, R, device=DEV)
        q[-1, :, 0] = 6.0
        sl = torch.tensor([qpos + 1], dtype=torch.int32, device=DEV)
        dec = ops.latent_attention(q[-1:].contiguous(), cache, R, pt, slots, sl, None, None, 1, ps, 1.0, W, None)
        ql = torch.tensor([5], dtype=torch.int32, device=DEV)
        cu = torch.tensor([0, 5], dtype=torch.int32, device=DEV)
        por = ops.latent_attention(q, cache, R, pt, slots, sl, cu, ql, 5, ps, 1.0, W, None)
        ref = torch_ref.latent_attention(q, cache, R, pt, slots, sl, ql, ps, 1.0, W, None)
        torch.testing.assert_close(por, ref, rtol=2e-5, atol=2e-5)
        torch.testing.assert_close(dec, ref[-1:], rtol=2e-5, atol=2e-5)
        assert (dec[0, 0, 0].item() > 4.0) == (qpos == mark + W - 1)


@pytest.mark.parametrize("dtype,tol", [("float32", 3e-4), ("bfloat16", 0.08)])
def test_engine_on_cuda_against_the_oracle(tmp_path, dtype, tol):
    """the serving engine on the GPU (own kernels) against the token-by-token oracle: whole prompt, portions, decode, a mixed batch"""
    import numpy as np

    from test_rirotar import L, Harness, _attn, _cfg, _delta, _dense, _moe, _tokens

    cfg = _cfg([L(_delta("delta", heads=4, kv_heads=2, dim=16, vdim=24), _dense(ff=64)), L(_attn(heads=4, dim=16, vdim=24, kv_rank=40, window=21), _moe(ff=32)),
                L(_delta("channel_delta", heads=2, kv_heads=2, dim=40, vdim=16, conv=4, rank=8), _moe(experts=4, top=1, count=2, keep=2)),
                L(_attn(heads=2, dim=8, vdim=8, kv_rank=24, window=70, scale=0.5), None)], width=64, vocab=96)
    h = Harness(tmp_path, cfg, seed=9, device="cuda", dtype=dtype, page=16, max_tokens=1024)
    a, b = _tokens(150, 96, 1), _tokens(77, 96, 2)
    ra, rb = h.oracle(a), h.oracle(b)
    if dtype == "float32":
        err = lambda x, y: float(np.abs(x - y).max())
    else:      # bf16 rounding can flip a close expert choice, and the recurrent layers carry the difference on: judge the median position
        err = lambda x, y: float(np.quantile(np.sqrt(((x - y) ** 2).mean(-1)), 0.5))
    assert err(h.step([("w", a, range(len(a)))], ["w"]), ra) < tol
    assert err(h.run_cut("c", a, [2, 31, 16, 3, 64]), ra) < tol
    # two requests interleaved: a portion of one beside single tokens of the other
    o1 = h.step([("x", a[:100], range(100)), ("y", b[:5], range(5))])
    got_a, got_b = [o1[:100]], [o1[100:]]
    for i in range(50):
        e = [("x", a[100 + i:101 + i], [0])]
        if 5 + i < len(b):
            e.append(("y", b[5 + i:6 + i], [0]))
        o = h.step(e)
        got_a.append(o[:1])
        if len(e) > 1:
            got_b.append(o[1:])
    o = h.step([("y", b[55:], range(len(b) - 55))], ["x", "y"])
    got_b.append(o)
    assert err(np.concatenate(got_a), ra) < tol
    assert err(np.concatenate(got_b), rb) < tol
    outs = h.eng.generate(input_ids=[a[:20]], sampling_params={"max_new_tokens": 6, "temperature": 0, "ignore_eos": True})
    assert len(outs[0]["output_ids"]) == 6
    if dtype == "float32":
        seq = list(a[:20])
        for _ in range(6):
            seq.append(int(h.oracle(seq)[-1].argmax()))
        assert outs[0]["output_ids"] == seq[20:]
    h.close()


def test_expanded_prompt_route_for_128_wide_heads_matches_the_absorbed_kernel(tmp_path):
    """bf16 prompts with 128-wide key and value heads run the tcgen05 flash-attention kernel over up-projected keys and values; the result
    has to agree with the absorbed latent kernel (same engine, route switched off) and with the oracle, for whole prompts, portions that
    start inside the window, and a batch of unequal requests"""
    import numpy as np

    from sglang_b200.layers.latent_attention import WindowedLatentAttention as WLA
    from test_rirotar import L, Harness, _attn, _cfg, _delta, _dense, _tokens

    cfg = _cfg([L(_attn(heads=2, dim=128, vdim=128, kv_rank=64, window=50, scale=128 ** -0.5), _dense(ff=64)),
                L(_delta("delta", heads=2, kv_heads=1, dim=16, vdim=16), None),
                L(_attn(heads=3, dim=128, vdim=128, kv_rank=40, window=300, scale=128 ** -0.5), None)], width=64, vocab=96)
    h = Harness(tmp_path, cfg, seed=4, device="cuda", dtype="bfloat16", page=16, max_tokens=2048)
    a, b = _tokens(333, 96, 1), _tokens(120, 96, 2)
    rms = lambda x, y: float(np.quantile(np.sqrt(((x - y) ** 2).mean(-1)), 0.9))

    def run():
        whole = h.step([("w", a, range(len(a)))], ["w"])
        cut = h.run_cut("c", a, [70, 3, 130, 64, 60])
        o1 = h.step([("x", a[:200], range(200)), ("y", b[:7], range(7))])
        o2 = h.step([("x", a[200:], range(133)), ("y", b[7:], range(113))], ["x", "y"])
        return whole, cut, np.concatenate([o1[:200], o2[:133]]), np.concatenate([o1[200:], o2[133:]])

    assert WLA.expand_prefill
    got = run()
    WLA.expand_prefill = False
    try:
        ref = run()
    finally:
        WLA.expand_prefill = True
    for x, y in zip(got, ref):
        assert rms(x, y) < 0.05
    ra, rb = h.oracle(a), h.oracle(b)
    for x, y in zip(got, (ra, ra, ra, rb)):
        assert rms(x, y) < 0.06
    h.close()


@pytest.mark.parametrize("dtype,tol", [("float32", 3e-4), ("bfloat16", 0.1)])
def test_engine_on_cuda_with_sizes_no_vector_lane_divides(tmp_path, dtype, tol):
    """widths, ranks, head sizes, expert sizes and a vocabulary that are multiples of nothing convenient: every op has to take its general path"""
    import numpy as np

    from test_rirotar import L, Harness, _attn, _cfg, _delta, _dense, _moe, _tokens

    cfg = _cfg([L(_attn(heads=5, dim=24, vdim=40, kv_rank=36, window=9, scale=0.3), _moe(experts=6, top=3, count=2, keep=1, ff=20)),
                L(_delta("channel_delta", heads=3, kv_heads=1, dim=20, vdim=12, conv=2, rank=5), _dense(ff=100)),
                L(_delta("delta", heads=2, kv_heads=2, dim=72, vdim=36, conv=7), None),
                L(_attn(heads=1, dim=10, vdim=6, kv_rank=14, window=400, scale=0.9), _dense(ff=36))], width=100, vocab=301, softcap=0.0)
    h = Harness(tmp_path, cfg, seed=21, device="cuda", dtype=dtype, page=16, max_tokens=1024)
    a = _tokens(130, 301, 3)
    ra = h.oracle(a)
    if dtype == "float32":
        err = lambda x, y: float(np.abs(x - y).max())
    else:
        err = lambda x, y: float(np.quantile(np.sqrt(((x - y) ** 2).mean(-1)), 0.5))
    assert err(h.step([("w", a, range(len(a)))], ["w"]), ra) < tol
    assert err(h.run_cut("c", a, [3, 40, 2, 17]), ra) < tol
    h.close()


@pytest.mark.parametrize("seed", [0, 1, 2, 3])
def test_engine_on_cuda_with_randomly_drawn_stacks(tmp_path, seed):
    """layer order, head counts, head sizes, ranks, windows, taps, expert counts and groups drawn at random (fp32, so the oracle is a strict
    reference): a whole prompt, portions, and three requests batched with one of them decoding beside the others' portions"""
    import numpy as np

    from test_rirotar import L, Harness, _attn, _cfg, _delta, _dense, _moe, _tokens

    rng = np.random.default_rng(500 + seed)
    ch = lambda xs: xs[int(rng.integers(0, len(xs)))]
    layers = []
    for _ in range(int(rng.integers(2, 6))):
        kind = ch(["delta", "channel_delta", "latent_attention"])
        if kind == "latent_attention":
            mix = _attn(heads=ch([1, 2, 3, 5, 8, 12]), dim=ch([16, 24, 48, 64, 128]), vdim=ch([16, 40, 64, 96, 128]), kv_rank=ch([16, 24, 48, 96, 192]),
                        window=ch([1, 2, 17, 64, 100, 200, 1000]), scale=ch([0.125, 0.25, 0.09]))
        else:
            kvh = ch([1, 2, 3, 4])
            mix = _delta(kind, heads=kvh * ch([1, 2, 3]), kv_heads=kvh, dim=ch([16, 48, 64, 128]), vdim=ch([16, 48, 64, 128]), conv=ch([2, 4, 5]),
                         **({"rank": ch([4, 8, 16])} if kind == "channel_delta" else {}))
        m = ch(["dense", "moe", "moe", None])
        if m == "moe":
            cnt, per = ch([1, 2, 4]), ch([1, 2, 3, 4])
            keep = int(rng.integers(1, cnt + 1))
            mlp = _moe(experts=cnt * per, top=int(rng.integers(1, min(keep * per, 6) + 1)), count=cnt, keep=keep, ff=ch([32, 48, 40, 128]),
                       limit=ch([1.0, 3.0]), scale=ch([1.0, 2.5]))
        else:
            mlp = _dense(ff=ch([96, 200]), limit=ch([1.0, 7.0])) if m else None
        layers.append(L(mix, mlp))
    V = ch([160, 300, 512])
    cfg = _cfg(layers, width=ch([48, 96, 160, 256]), vocab=V, softcap=ch([0.0, 15.0]), eps=ch([1e-5, 1e-6]))
    h = Harness(tmp_path, cfg, seed=seed, device="cuda", dtype="float32", page=64, max_tokens=1024)
    a, b, c = _tokens(230, V, seed), _tokens(70, V, seed + 50), _tokens(110, V, seed + 99)
    ra, rb, rc = h.oracle(a), h.oracle(b), h.oracle(c)
    err = lambda x, y: float(np.abs(x - y).max())
    assert err(h.step([("w", a, range(len(a)))], ["w"]), ra) < 5e-4
    assert err(h.run_cut("c", a[:200], [2, 61, 3, 64, 37, 5]), ra[:200]) < 5e-4
    got = {"a": [], "b": [], "c": [h.step([("c", c[:100], range(100))])]}
    pa = pb = 0
    for i, (sa, sb) in enumerate(zip([50, 2, 77, 1, 1, 64, 35], [0, 33, 2, 35, 0, 0, 0])):
        ent = [(r, t[p:p + n], range(n)) for r, t, p, n in (("a", a, pa, sa), ("b", b, pb, sb)) if n] + [("c", c[100 + i:101 + i], range(1))]
        out = h.step(ent, [r for r, t, p, n in (("a", a, pa, sa), ("b", b, pb, sb)) if n and p + n == len(t)])
        at = 0
        for r, toks, _ in ent:
            got[r].append(out[at:at + len(toks)])
            at += len(toks)
        pa, pb = pa + sa, pb + sb
    h.step([("c", c[107:108], [0])], ["c"])
    assert err(np.concatenate(got["a"]), ra) < 5e-4 and err(np.concatenate(got["b"]), rb) < 5e-4 and err(np.concatenate(got["c"]), rc[:107]) < 5e-4
    h.close()


@pytest.mark.parametrize("H,I,E,K,T", [(256, 64, 8, 4, 300), (64, 16, 3, 1, 50), (96, 48, 5, 3, 129), (32, 32, 2, 2, 1), (128, 80, 16, 4, 1000)])
def test_clamped_glu_experts_grouped_against_the_per_expert_loop(H, I, E, K, T):
    """expert-sorted rows through the grouped tcgen05 GEMMs with the clamped GLU between them == one GEMM pair per expert"""
    _native()
    from sglang_b200.ops import moe_ops

    g = torch.Generator(device=DEV).manual_seed(H + I)
    x = torch.randn(T, H, device=DEV, generator=g).to(torch.bfloat16)
    w13 = (torch.randn(E, 2 * I, H, device=DEV, generator=g) * H ** -0.5).to(torch.bfloat16)
    w2 = (torch.randn(E, H, I, device=DEV, generator=g) * I ** -0.5).to(torch.bfloat16)
    ids = torch.stack([torch.randperm(E, device=DEV, generator=g)[:K] for _ in range(T)]).to(torch.int32)
    w = torch.rand(T, K, device=DEV, generator=g) + 0.1
    act = ("clamped_glu", 1.5, 1.702)
    a = moe_ops.fused_moe(x, w13, w2, w, ids, 0, act)
    fn = lambda gu: ops.clamped_glu(gu.contiguous(), 1.5, 1.702)
    b = moe_ops._fused_moe_sorted(x, w13, w2, w, ids, 0, fn)
    ref = torch_ref.fused_moe(x.float(), w13.float(), w2.float(), w, ids, 0, lambda gu: torch_ref.clamped_glu(gu, 1.5, 1.702))
    scale = ref.abs().max().item()
    assert (a.float() - ref).abs().max().item() < 0.03 * scale
    assert (b.float() - ref).abs().max().item() < 0.03 * scale
