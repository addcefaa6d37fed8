"""Rirotar through the serving engine (CPU tier, fp32) against the plain oracle in ``rirotar_oracle.py``: every mechanism alone, prefill against
token-by-token decoding, prompt portions down to two tokens, unequal batches, page and slot reuse, window and page edges, the first tokens,
long decoding, sizes that differ from layer to layer, and greedy generation through ``Engine.generate``."""
import json
import os

import numpy as np
import pytest
import torch

import rirotar_oracle as O
import sglang_b200 as sgl
from sglang_b200.layers.moe import grouped_sigmoid_route
from sglang_b200.ops import torch_ref

PAGE = 8


def _delta(kind, heads=2, kv_heads=1, dim=8, vdim=12, conv=3, **kw):
    return {"type": kind, "mixer": dict(heads=heads, kv_heads=kv_heads, dim=dim, vdim=vdim, conv=conv, **kw)}


def _attn(heads=3, dim=8, vdim=10, kv_rank=12, window=7, scale=0.4):
    return {"type": "latent_attention", "mixer": dict(heads=heads, dim=dim, vdim=vdim, kv_rank=kv_rank, mask={"size": window}, scale=scale)}


def _dense(ff=40, limit=1.0):
    return {"kind": "dense", "ff": ff, "limit": limit}


def _moe(experts=6, top=2, count=3, keep=2, ff=12, limit=0.8, scale=1.5):
    return {"kind": "moe", "expert": {"ff": ff, "limit": limit}, "router": {"experts": experts, "top": top, "scale": scale, "groups": {"count": count, "keep": keep}}}


def _cfg(layers, width=24, vocab=50, softcap=8.0, eps=1e-5):
    c = {"architecture": "Rirotar", "layers": layers, "norm": {"eps": eps}, "vocab": vocab, "width": width}
    if softcap:
        c["logit_softcap"] = softcap
    return c


def L(mix, mlp):
    return dict(mix, mlp=mlp)


MIXED = _cfg([L(_delta("delta"), _dense()), L(_attn(), _moe()), L(_delta("channel_delta", heads=4, kv_heads=2, dim=6, vdim=5, conv=4, rank=3), None),
              L(_attn(heads=2, dim=6, vdim=4, kv_rank=9, window=19, scale=0.7), _dense(ff=16, limit=2.5)),
              L(_delta("delta", heads=3, kv_heads=3, dim=5, vdim=7, conv=2), _moe(experts=4, top=1, count=1, keep=1, scale=1.0))])


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
        for j, n in enumerate(sizes):
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
    for E, top, n, keep in ((8, 4, 4, 3), (6, 2, 3, 1), (5, 5, 1, 1), (12, 3, 4, 4), (4, 1, 4, 2)):
        logits = torch.randn(40, E, generator=g) * 2
        h, wr = torch.randn(40, 16, generator=g), torch.randn(E, 16, generator=g)
        logits = h @ wr.t()
        w1, i1 = grouped_sigmoid_route(logits, top, n, keep, 2.0)
        w2, i2 = O.route(h.double(), wr.double(), {"experts": E, "top": top, "scale": 2.0, "groups": {"count": n, "keep": keep}})
        o1, o2 = i1.long().sort(-1), i2.sort(-1)
        assert torch.equal(o1.values, o2.values)
        torch.testing.assert_close(w1.gather(1, o1.indices).double(), w2.gather(1, o2.indices), rtol=1e-5, atol=1e-6)


def test_delta_rule_reference_op_against_oracle_and_far_memory():
    g = torch.Generator().manual_seed(1)
    for chan in (False, True):
        T, Hk, H, Dk, Dv = 300, 1, 2, 6, 5
        u = torch.randn(T, 2 * Hk * Dk + H * Dv, generator=g)
        # one early write that must still be readable hundreds of tokens later: a large key at t = 3, the same direction queried at the end,
        # orthogonal small keys in between, and decays close to one
        u[:, Hk * Dk:2 * Hk * Dk] *= 0.05
        u[3, Hk * Dk:2 * Hk * Dk] = torch.tensor([9.0, 0, 0, 0, 0, 0])
        u[4:, Hk * Dk] = 0.0
        u[-1, :Hk * Dk] = torch.tensor([7.0, 0, 0, 0, 0, 0])
        a_raw = torch.randn(T, H * Dk if chan else H, generator=g) - 12.0
        A_log, dtb = torch.zeros(H), torch.zeros(H * Dk if chan else H)
        b_raw = torch.randn(T, H, generator=g) + 3
        state = torch.zeros(2, H, Dk, Dv)
        o = torch_ref.gated_delta_rule(u, Hk, Dk, H, Dv, a_raw, A_log, dtb, b_raw, state, torch.tensor([1]), torch.tensor([T]), torch.tensor([T]),
                                       per_channel=chan)
        q = O.unit_vec(u[:, :Hk * Dk].double().view(T, Hk, Dk)) * Dk ** -0.5
        k = O.unit_vec(u[:, Hk * Dk:2 * Hk * Dk].double().view(T, Hk, Dk))
        v = u[:, 2 * Hk * Dk:].double().view(T, H, Dv)
        sp = torch.nn.functional.softplus(a_raw.double())
        gd = torch.exp(-sp.view(T, H, Dk)) if chan else torch.exp(-sp)
        ref = O.delta_recurrence(q.repeat_interleave(H, 1), k.repeat_interleave(H, 1), v, torch.sigmoid(b_raw.double()), gd)
        torch.testing.assert_close(o.double(), ref, rtol=1e-4, atol=1e-5)
        # the read-out at the end is dominated by what was written at t = 3
        want = torch.sigmoid(b_raw[3].double())[:, None] * v[3] * Dk ** -0.5
        assert (ref[-1] - want).abs().max() < 0.15 * want.abs().max()


def test_latent_attention_reference_op_window_edges_with_a_standout_key():
    """one key's latent row is made to dominate the scores; it must count when it is the oldest key inside the window and vanish one step
    later, in a prompt portion and in a decode step, across a page border"""
    R, H, W, ps = 6, 2, 11, 4
    g = torch.Generator().manual_seed(2)
    cache = torch.randn(64 * ps, 1, R + 2, generator=g) * 0.1
    pages = torch.randperm(60, generator=g)[:16] + 1
    pt = torch.zeros(3, 20, dtype=torch.int32)
    pt[1, :16] = pages.int()
    slot_of = lambda pos: int(pages[pos // ps]) * ps + pos % ps
    mark = 17                                                   # position of the standout key
    cache[slot_of(mark), 0, :R] = torch.tensor([5.0, 0, 0, 0, 0, 0])
    sinks = torch.tensor([0.3, -0.2])
    for qpos in (mark + W - 1, mark + W):                       # last position that sees it / first that does not
        q = torch.zeros(1, H, R)
        q[0, :, 0] = 6.0
        L_ = qpos + 1
        out = torch_ref.latent_attention(q, cache, R, pt, torch.tensor([1]), torch.tensor([L_]), None, ps, 1.0, W, sinks)          # decode step
        out2 = torch_ref.latent_attention(torch.cat([torch.zeros(3, H, R), q]), cache, R, pt, torch.tensor([1]), torch.tensor([L_]),
                                          torch.tensor([4]), ps, 1.0, W, sinks)[-1:]                                               # end of a portion
        torch.testing.assert_close(out, out2)
        C = torch.stack([cache[slot_of(p), 0, :R] for p in range(L_)]).double()
        lo = max(0, qpos - W + 1)
        for h in range(H):
            s = C[lo:] @ q[0, h].double()
            den = torch.exp(s).sum() + torch.exp(sinks[h].double())
            ref = (torch.exp(s)[:, None] * C[lo:]).sum(0) / den
            torch.testing.assert_close(out[0, h].double(), ref, rtol=1e-5, atol=1e-6)
        seen = out[0, 0, 0].item() > 4.0
        assert seen == (qpos == mark + W - 1)


# ------------------------------------------------------------------ single mechanisms through the engine
@pytest.mark.parametrize("layer", [L(_delta("delta"), None), L(_delta("channel_delta", heads=4, kv_heads=4, dim=6, vdim=6, rank=5), None),
                                   L(_attn(), None), L(_attn(window=1), _dense()), L(_delta("delta", conv=1), _moe()),
                                   L(_delta("delta", heads=6, kv_heads=2, conv=5), _moe(experts=8, top=4, count=4, keep=3))])
def test_one_layer_models(tmp_path, layer):
    h = Harness(tmp_path, _cfg([layer], softcap=0.0 if layer["mlp"] is None else 6.0))
    toks = _tokens(37, 50, 5)
    ref = h.oracle(toks)
    _close(h.step([("a", toks, range(len(toks)))], ["a"]), ref)                    # whole prompt
    _close(h.run_cut("b", toks, []), ref)                                          # token by token from the first token
    h.close()


# ------------------------------------------------------------------ the mixed model: cuts, batches, reuse
@pytest.fixture(scope="module")
def mixed(tmp_path_factory):
    h = Harness(tmp_path_factory.mktemp("rirotar"), MIXED, seed=3, slots=4, max_tokens=40 * PAGE)
    yield h
    h.close()


def test_first_tokens_and_prefill_against_decode(mixed):
    toks = _tokens(61, 50, 7)
    ref = mixed.oracle(toks)
    whole = mixed.step([("w", toks, range(len(toks)))], ["w"])
    _close(whole, ref)
    _close(whole[:3], ref[:3], 1e-4)                                               # positions 0, 1, 2: zero history of the convolutions
    _close(mixed.run_cut("d", toks, [30]), ref)                                    # 30 at once, then 31 decode steps (window 19 and 7 pass over them)


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


def test_config_reader_takes_every_size_from_the_file(tmp_path):
    from sglang_b200.configs.model_config import load_model_config

    d = tmp_path / "cfg"
    d.mkdir()
    (d / "config.json").write_text(json.dumps(MIXED))
    c = load_model_config(str(d))
    assert c.architecture == "Rirotar" and c.hidden_size == 24 and c.vocab_size == 50 and c.num_hidden_layers == 5
    assert c.final_logit_softcapping == 8.0 and c.rms_norm_eps == 1e-5 and c.hybrid["layers"][3]["mixer"]["mask"]["size"] == 19


def test_text_prompts_on_a_weights_only_folder(tmp_path):
    """a folder with only config.json and model.safetensors serves text through the byte tokenizer (what `cli generate` and the HTTP server do)"""
    h = Harness(tmp_path, _cfg([L(_delta("delta"), _dense()), L(_attn(), None)], vocab=300), seed=8)
    h.close()
    eng = sgl.Engine(model_path=os.path.join(str(tmp_path), "m8"), device="cpu", page_size=PAGE, max_total_tokens=256, max_running_requests=2,
                     log_level="warning")
    out = eng.generate("hello there", {"max_new_tokens": 4, "temperature": 0.7, "top_k": 5, "ignore_eos": True})
    assert len(out["output_ids"]) == 4 and isinstance(out["text"], str)
    eng.shutdown()
