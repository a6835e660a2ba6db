"""Zigivik through the framework (kernels, page pool and state slots, ragged steps, scheduler) against the plain oracle
(oracle/zigivik_oracle.py): every mechanism alone, then whole models under every way of cutting and batching the work."""
import json
import os
import struct
import sys

import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)
from oracle import zigivik_oracle as O  # noqa: E402

pytestmark = pytest.mark.gpu

F32_TOL, BF16_TOL = 2e-4, 4e-2


def latent(heads=3, dim=24, rot_dim=8, vdim=20, q_rank=28, kv_rank=36, size=37, scaling=True, base=5000.0, scale=None, kv_from=None):
    rot = {"base": base, "dims": rot_dim}
    if scaling:
        rot["scaling"] = {"factor": 4.0, "original": 64, "fast": 8.0, "slow": 1.0}
    m = {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "q_rank": q_rank, "kv_rank": kv_rank, "rot": rot,
         "scale": scale if scale is not None else (dim + rot_dim) ** -0.5, "mask": {"size": size}}
    if kv_from is not None:
        m["kv_from"] = kv_from
    return {"type": "latent_attention", "mixer": m}


def attention(heads=6, kv_heads=3, dim=20, rot_dims=12, base=300.0, scale=None):
    m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": dim, "rot": {"base": base, "dims": rot_dims}, "scale": scale if scale is not None else dim ** -0.5}
    return {"type": "attention", "mixer": m}


def with_ff(l, ff=80):
    return dict(l, mlp={"kind": "dense", "ff": ff} if ff else None)


def make_cfg(layers, width=72, vocab=90, eps=1e-5, taps=4, mult=0.6):
    return {"architecture": "Zigivik", "vocab": vocab, "width": width, "norm": {"eps": eps}, "canon": {"taps": taps}, "residual_mult": mult, "layers": layers}


# both mixer types, grouped and ungrouped key heads, a layer without a feed-forward, a borrowing layer whose window differs from its source's
BASE_CFG = make_cfg([with_ff(attention()), with_ff(latent(size=37)), with_ff(attention(heads=4, kv_heads=4, dim=16, rot_dims=16), 0),
                     with_ff(latent(heads=5, dim=12, vdim=16, q_rank=20, size=90, kv_from=1), 48), with_ff(latent(heads=2, dim=16, rot_dim=16, vdim=8, kv_rank=24, size=20, scaling=False), 33)])


def build(cfg, w, dtype):
    from paligemma_multimodal_system_b200.modeling_zigivik import ZigivikConfig, ZigivikForCausalLM
    return ZigivikForCausalLM(ZigivikConfig(cfg), dtype).load_weights({k: v.to(torch.bfloat16) for k, v in w.items()})


def engine_for(cfg, w, dtype, max_tokens=1024, slots=4):
    from paligemma_multimodal_system_b200.engine import SequenceEngine
    return SequenceEngine(build(cfg, w, dtype), max_tokens, slots)


def poison(engine):
    """Stale memory must never be read: pages and state slots start as huge values instead of zeros."""
    for t in engine.store.k_pages + engine.store.v_pages + engine.store.state:
        if t is not None:
            t.fill_(1e4)


def rel_err(got, ref):
    got, ref = got.double().cpu(), ref.double()
    return float((got - ref).pow(2).mean().sqrt() / ref.pow(2).mean().sqrt())


def worst_row(got, ref):
    """The largest error of any row, relative to the typical row's size (one wrong position must not drown among hundreds)."""
    got, ref = got.double().cpu().reshape(ref.shape[0], -1), ref.double().reshape(ref.shape[0], -1)
    return float(((got - ref).pow(2).mean(-1).sqrt() / ref.pow(2).mean().sqrt()).max())


def close(got, ref, dtype):
    """fp32: every row within F32_TOL.  bf16: the tensor within BF16_TOL / 2 and no row beyond twice BF16_TOL (in the smallest test
    models a single row's rounding reaches past BF16_TOL, alone and in a batch alike)."""
    if dtype == torch.float32:
        return worst_row(got, ref) < F32_TOL
    return rel_err(got, ref) < BF16_TOL / 2 and worst_row(got, ref) < 2 * BF16_TOL


def toks(n, vocab, seed):
    g = torch.Generator().manual_seed(seed)
    return torch.randint(0, vocab, (n,), generator=g).tolist()


def run_cut(engine, rid, tokens, cuts):
    """Feeds `tokens` in portions of the given sizes (the last size repeats); returns logits of every position."""
    out, pos, i = [], 0, 0
    while pos < len(tokens):
        k = min(cuts[min(i, len(cuts) - 1)], len(tokens) - pos)
        out.append(engine.step([(rid, tokens[pos:pos + k], list(range(k)))], [rid] if pos + k == len(tokens) else []))
        pos, i = pos + k, i + 1
    return torch.cat(out)


def one_store(layout, T, dtype, skip_pages=2):
    """A store with one admitted sequence of up to T tokens whose pages do not start at page 0 and whose slot is not slot 0."""
    from paligemma_multimodal_system_b200.cache import SequenceStore
    store = SequenceStore(layout, max_tokens=(T + 63) // 64 * 64 + 64 * skip_pages, num_slots=2, dtype=dtype)
    store.pool.take(skip_pages)
    store.admit("skipped")
    store.admit(0)
    store.reserve(0, T)
    for t in store.k_pages + store.v_pages + store.state:
        if t is not None:
            t.fill_(1e4)
    return store


def run_mixer(mx, layout, h, cuts, dtype, prec, li=0, store=None):
    """h [T, D] through a mixer in portions; returns fp32 [T, D] on the CPU."""
    from paligemma_multimodal_system_b200 import seq_ops
    T = h.shape[0]
    store = store or one_store(layout, T, dtype)
    rec, pos, outs, i = store.live[0], 0, [], 0
    while pos < T:
        k = min(cuts[min(i, len(cuts) - 1)], T - pos)
        b = seq_ops.make_step_batch([dict(tokens=[0] * k, ctx=pos, slot=rec.slot, pages=rec.pages)])
        outs.append(mx(h[pos:pos + k].cuda().to(dtype).contiguous(), b, store, li, prec).float().cpu())
        pos, i = pos + k, i + 1
    return torch.cat(outs)


def load_mixer(cfg, w, i=0):
    from paligemma_multimodal_system_b200.modeling_zigivik import _mixer
    l = cfg["layers"][i]
    mx = _mixer(cfg["width"], l["type"], l["mixer"], cfg["norm"]["eps"])
    left = {k: v.to(torch.bfloat16) for k, v in w.items()}
    mx.load(lambda name, shape: left.pop(name), f"l{i}.mix.")
    return mx


# ----------------------------------------------------------------------------------------------------------------------
# mechanisms alone
# ----------------------------------------------------------------------------------------------------------------------
@pytest.mark.parametrize("D,taps,scalar", [(40, 3, True), (72, 2, True), (257, 4, False), (1024, 8, True), (64, 1, True), (96, 5, False)])
@pytest.mark.parametrize("f32", [True, False])
def test_norm_and_causal_convolution_in_portions(D, taps, scalar, f32):
    """Three sequences advance together in unequal portions -- one token by token, one in portions shorter than the convolution's
    reach -- and both outputs must equal the whole-sequence oracle at every position, whatever the state slots held before."""
    from paligemma_multimodal_system_b200 import seq_ops
    from paligemma_multimodal_system_b200.cache import SequenceStore
    lens, plans = [23, 9, 14], [[5, 1, 2, 15], [1] * 9, [2, 2, 1, 3, 6]]
    g = torch.Generator().manual_seed(D + taps)
    eps = 1e-5
    xs = [3.0 * torch.randn(n, D, generator=g) for n in lens]
    wn = torch.randn(() if scalar else (D,), generator=g) + 1.5
    cw = torch.randn(D, taps, generator=g)
    ref_h = [O.unit_rms(x, eps) * wn for x in xs]
    ref_c = [h + O.causal_conv(h, cw) for h in ref_h]
    store = SequenceStore([("state", (taps - 1, D)) if taps > 1 else None], max_tokens=512, num_slots=4, dtype=torch.float32)
    if taps > 1:
        store.state[0].fill_(1e4)
    store.admit("unused")
    for i in range(3):
        store.admit(i)
    dt = torch.float32 if f32 else torch.bfloat16
    got_h, got_c = [[] for _ in lens], [[] for _ in lens]
    fed, step = [0, 0, 0], 0
    while any(fed[i] < lens[i] for i in range(3)):
        es, rows = [], []
        for i in range(3):
            if fed[i] < lens[i] and step < len(plans[i]):
                k = plans[i][step]
                rec = store.reserve(i, k)
                es.append(dict(tokens=[0] * k, ctx=rec.length, slot=rec.slot, pages=rec.pages))
                rows.append((i, k))
        b = seq_ops.make_step_batch(es)
        x = torch.cat([xs[i][fed[i]:fed[i] + k] for i, k in rows]).cuda().contiguous()
        oh, oc = torch.empty(b.T, D, device="cuda", dtype=dt), torch.empty(b.T, D, device="cuda", dtype=dt)
        seq_ops.rmsnorm_conv(x, wn.reshape(-1).cuda().contiguous(), oh, oc, eps, conv_w=cw.t().contiguous().cuda(), state=store.state[0], b=b)
        r = 0
        for i, k in rows:
            got_h[i].append(oh[r:r + k].float().cpu())
            got_c[i].append(oc[r:r + k].float().cpu())
            store.commit(i, k)
            fed[i] += k
            r += k
        step += 1
    tol = 1e-5 if f32 else 8e-3
    for i in range(3):
        assert worst_row(torch.cat(got_h[i]), ref_h[i]) < tol and worst_row(torch.cat(got_c[i]), ref_c[i]) < tol, i
    # a bare norm (the embedding's and the model's last one): one output, fp32 or the activation type, no state
    o = torch.empty(lens[0], D, device="cuda", dtype=dt)
    seq_ops.rmsnorm_conv(xs[0].cuda().contiguous(), wn.reshape(-1).cuda().contiguous(), o, None, eps)
    assert worst_row(o.float(), ref_h[0]) < tol


@pytest.mark.parametrize("D,taps,lens,plans", [(72, 4, [5000, 9, 2703], [[4000, 1, 2, 997], [1] * 9, [700, 2001, 2]]),
                                               (1280, 3, [2500, 3, 1301], [[1, 2400, 99], [1, 1, 1], [1300, 1]]),
                                               (250, 8, [3000, 5, 3000], [[2999, 1], [5], [3, 2997]])])
@pytest.mark.parametrize("f32", [True, False])
def test_norm_and_convolution_in_steps_of_thousands_of_rows(D, taps, lens, plans, f32):
    """Long portions walk chunks of consecutive rows per CTA: chunk borders fall inside entries, on their first rows and on their last
    ones; the entries' first rows and the state slots come from a launch of their own."""
    from paligemma_multimodal_system_b200 import seq_ops
    from paligemma_multimodal_system_b200.cache import SequenceStore
    g = torch.Generator().manual_seed(D)
    eps = 1e-5
    xs = [2.0 * torch.randn(n, D, generator=g) for n in lens]
    wn, cw = torch.tensor([1.3]), torch.randn(D, taps, generator=g)
    ref_h = [O.unit_rms(x, eps) * wn for x in xs]
    ref_c = []
    for h in ref_h:  # the convolution as shifted sums (the oracle's loop, vectorised over time)
        acc = h.clone()
        for j in range(taps):
            s = taps - 1 - j
            if s < h.shape[0]:
                acc[s:] += cw[:, j] * h[:h.shape[0] - s]
        ref_c.append(acc)
    assert torch.allclose(ref_c[1], ref_h[1] + O.causal_conv(ref_h[1], cw), atol=1e-5)
    store = SequenceStore([("state", (taps - 1, D))], max_tokens=sum(lens) + 256, num_slots=4, dtype=torch.float32)
    store.state[0].fill_(1e4)
    store.admit("unused")
    for i in range(3):
        store.admit(i)
    dt = torch.float32 if f32 else torch.bfloat16
    got_h, got_c = [[] for _ in lens], [[] for _ in lens]
    fed, step = [0, 0, 0], 0
    while any(fed[i] < lens[i] for i in range(3)):
        es, rows = [], []
        for i in range(3):
            if fed[i] < lens[i] and step < len(plans[i]):
                k = plans[i][step]
                rec = store.reserve(i, k)
                es.append(dict(tokens=[0] * k, ctx=rec.length, slot=rec.slot, pages=rec.pages))
                rows.append((i, k))
        b = seq_ops.make_step_batch(es)
        x = torch.cat([xs[i][fed[i]:fed[i] + k] for i, k in rows]).cuda().contiguous()
        oh, oc = torch.empty(b.T, D, device="cuda", dtype=dt), torch.empty(b.T, D, device="cuda", dtype=dt)
        seq_ops.rmsnorm_conv(x, wn.cuda(), oh, oc, eps, conv_w=cw.t().contiguous().cuda(), state=store.state[0], b=b)
        r = 0
        for i, k in rows:
            got_h[i].append(oh[r:r + k].float().cpu())
            got_c[i].append(oc[r:r + k].float().cpu())
            store.commit(i, k)
            fed[i] += k
            r += k
        step += 1
    tol = 1e-5 if f32 else 8e-3
    for i in range(3):
        assert worst_row(torch.cat(got_h[i]), ref_h[i]) < tol and worst_row(torch.cat(got_c[i]), ref_c[i]) < tol, i


def test_convolution_state_survives_a_step_the_sequence_sits_out():
    """A sequence left out of a step finds its own last rows again, not those another sequence wrote in between."""
    from paligemma_multimodal_system_b200 import seq_ops
    from paligemma_multimodal_system_b200.cache import SequenceStore
    D, taps, eps = 48, 4, 1e-6
    g = torch.Generator().manual_seed(1)
    xa, xb = torch.randn(12, D, generator=g), torch.randn(7, D, generator=g)
    wn, cw = torch.tensor([0.8]), torch.randn(D, taps, generator=g)
    ref = {0: None, 1: None}
    for i, x in ((0, xa), (1, xb)):
        h = O.unit_rms(x, eps) * wn
        ref[i] = h + O.causal_conv(h, cw)
    store = SequenceStore([("state", (taps - 1, D))], max_tokens=256, num_slots=2, dtype=torch.float32)
    store.state[0].fill_(-7e3)
    store.admit(0), store.admit(1)
    got = {0: [], 1: []}
    for plan in ([(0, 5)], [(1, 2)], [(1, 1), (0, 1)], [(1, 4)], [(0, 6)]):
        es, xs = [], []
        for i, k in plan:
            rec = store.reserve(i, k)
            es.append(dict(tokens=[0] * k, ctx=rec.length, slot=rec.slot, pages=rec.pages))
            xs.append((xa if i == 0 else xb)[rec.length:rec.length + k])
        b = seq_ops.make_step_batch(es)
        oc = torch.empty(b.T, D, device="cuda")
        seq_ops.rmsnorm_conv(torch.cat(xs).cuda().contiguous(), wn.cuda(), None, oc, eps, conv_w=cw.t().contiguous().cuda(), state=store.state[0], b=b)
        r = 0
        for i, k in plan:
            got[i].append(oc[r:r + k].cpu())
            store.commit(i, k)
            r += k
    assert worst_row(torch.cat(got[0]), ref[0]) < 1e-5 and worst_row(torch.cat(got[1]), ref[1]) < 1e-5


@pytest.mark.parametrize("T,F", [(1, 8), (37, 50), (5, 1000), (300, 257)])
@pytest.mark.parametrize("f32", [True, False])
def test_polynomial_of_norms(T, F, f32):
    from paligemma_multimodal_system_b200 import seq_ops
    g = torch.Generator().manual_seed(F)
    z = (1.5 * torch.randn(T, F, generator=g)).to(torch.bfloat16).float()
    coef = torch.tensor([0.7, -0.4, 0.25, 0.1])
    dt = torch.float32 if f32 else torch.bfloat16
    zd = z.cuda().to(dt)
    out = seq_ops.polynorm(zd, coef.cuda(), torch.empty_like(zd), 1e-5)
    assert worst_row(out.float(), O.poly_norm(z, coef, 1e-5)) < (1e-5 if f32 else 8e-3)
    assert torch.equal(seq_ops.polynorm(zd, coef.cuda(), zd, 1e-5), out)  # in place


def test_ramped_frequencies_and_pair_order():
    from paligemma_multimodal_system_b200.mixers import half_to_pair_order, ramped_rotary_frequencies
    for base, dims, sc in ((5000.0, 8, dict(factor=4.0, original=64, fast=8.0, slow=1.0)), (1e6, 64, dict(factor=40.0, original=4096, fast=32.0, slow=1.0)),
                           (100.0, 6, dict(factor=2.0, original=16, fast=1.0, slow=1.0))):
        f, gain = ramped_rotary_frequencies(base, dims, sc["factor"], sc["original"], sc["fast"], sc["slow"])
        rf, rg = O.rescaled_frequencies(base, dims, sc)
        assert torch.allclose(f, torch.tensor(rf, dtype=torch.float64), rtol=1e-12, atol=0) and abs(gain - rg) < 1e-12
    # turning the reordered vector in neighbouring pairs = reordering the vector turned in half-split pairs
    v, freqs = torch.randn(3, 14, dtype=torch.float64), [0.3, 0.02, 1.1, 0.5]
    order = half_to_pair_order(14, 8)
    assert torch.allclose(O.turn_pairs(v[:, order], 11, freqs), O.turn_half(v, 11, freqs, 1.0)[:, order], atol=1e-12)


LATENTS = [dict(), dict(scaling=False), dict(heads=1, dim=8, rot_dim=4, vdim=8, q_rank=8, kv_rank=8, size=1),
           dict(heads=4, dim=64, rot_dim=32, vdim=64, q_rank=48, kv_rank=64, size=70),    # a head size the tensor-core prompt kernel has: explicit-head form
           dict(heads=4, dim=128, rot_dim=64, vdim=128, q_rank=64, kv_rank=128, size=129, base=1e6),
           dict(heads=5, dim=10, rot_dim=6, vdim=14, q_rank=9, kv_rank=11, size=1000)]     # odd sizes, a window longer than the sequence


@pytest.mark.parametrize("kw", LATENTS)
@pytest.mark.parametrize("dtype,tol", [(torch.float32, 1e-4), (torch.bfloat16, 3e-2)])
def test_latent_attention_alone(kw, dtype, tol):
    """One mixer over 200 positions: as one portion, and as context + portion + single tokens (decode kernel)."""
    from paligemma_multimodal_system_b200 import seq_ops
    D, T, eps = 56, 200, 1e-5
    cfg = make_cfg([with_ff(latent(**kw), 0)], width=D, eps=eps)
    w = O.random_weights(cfg, seed=len(str(kw)))
    h = torch.randn(T, D, generator=torch.Generator().manual_seed(3)).to(torch.bfloat16).float()
    m = cfg["layers"][0]["mixer"]
    ref = O.latent_attention(h, w, "l0.mix.", m, eps, O.latent_rows(h, w, "l0.mix.", m, eps))
    mx = load_mixer(cfg, w)
    prec = seq_ops.Precision(dtype)
    mx.pack(prec)
    for cuts in ([T], [131, 67, 1], [2]):
        assert worst_row(run_mixer(mx, [mx.cache_spec()], h, cuts, dtype, prec), ref) < tol, cuts


@pytest.mark.parametrize("kw", [dict(), dict(heads=4, kv_heads=4, dim=64, rot_dims=64), dict(heads=8, kv_heads=1, dim=64, rot_dims=20), dict(heads=4, kv_heads=2, dim=128, rot_dims=128, base=1e6),
                                dict(heads=3, kv_heads=3, dim=10, rot_dims=0), dict(heads=2, kv_heads=1, dim=7, rot_dims=4)])
@pytest.mark.parametrize("dtype,tol", [(torch.float32, 1e-4), (torch.bfloat16, 3e-2)])
def test_keys_as_values_attention_alone(kw, dtype, tol):
    from paligemma_multimodal_system_b200 import seq_ops
    D, T, eps = 56, 200, 1e-5
    cfg = make_cfg([with_ff(attention(**kw), 0)], width=D, eps=eps)
    w = O.random_weights(cfg, seed=len(str(kw)))
    h = torch.randn(T, D, generator=torch.Generator().manual_seed(4)).to(torch.bfloat16).float()
    ref = O.key_value_attention(h, w, "l0.mix.", cfg["layers"][0]["mixer"])
    mx = load_mixer(cfg, w)
    prec = seq_ops.Precision(dtype)
    mx.pack(prec)
    for cuts in ([T], [131, 67, 1], [2]):
        assert worst_row(run_mixer(mx, [mx.cache_spec()], h, cuts, dtype, prec), ref) < tol, cuts


_EDGE_CASES = [(dict(), 37), (dict(heads=4, dim=64, rot_dim=32, vdim=64, q_rank=48, kv_rank=64), 64), (dict(heads=4, dim=64, rot_dim=32, vdim=64, q_rank=48, kv_rank=64), 65), (dict(), 130)]
_EDGE_REFS = {}


def _edge_ref(case, needle):
    """Config, weights, input and oracle output of a window-edge case (made once per case and needle)."""
    if (case, needle) not in _EDGE_REFS:
        kw, window = _EDGE_CASES[case]
        D, T, eps = 56, 400, 1e-5
        cfg = make_cfg([with_ff(latent(size=window, scaling=False, **kw), 0)], width=D, eps=eps)
        w = O.random_weights(cfg, seed=5)
        m = cfg["layers"][0]["mixer"]
        h = torch.randn(T, D, generator=torch.Generator().manual_seed(needle)).to(torch.bfloat16).float()
        h[needle] *= 10.0
        rows = O.latent_rows(h, w, "l0.mix.", m, eps)
        ref = O.latent_attention(h, w, "l0.mix.", m, eps, rows)
        for other in (window - 1, window + 1):  # a window one key shorter or longer would show far above the tolerance
            if other >= 1:
                off = O.latent_attention(h, w, "l0.mix.", dict(m, mask={"size": other}), eps, rows)
                assert worst_row(off, ref) > 0.15, (case, needle, other)  # three times the widest tolerance used below
        _EDGE_REFS[(case, needle)] = (cfg, w, h, ref)
    return _EDGE_REFS[(case, needle)]


@pytest.mark.parametrize("case", range(len(_EDGE_CASES)))
@pytest.mark.parametrize("dtype,tol", [(torch.float32, 2e-4), (torch.bfloat16, 5e-2)])
@pytest.mark.parametrize("cuts", [[400], [190, 1], [137, 63, 2, 2, 1], [64], [3]])
def test_latent_window_edge_with_a_key_that_dominates(case, dtype, tol, cuts):
    """The input of one token is ten times larger: its rotated key part dominates every softmax that sees it.  The last query that
    still sees it and the first that no longer does sit in prompts and among decoded tokens, at page borders and portion starts."""
    from paligemma_multimodal_system_b200 import seq_ops
    window = _EDGE_CASES[case][1]
    mx = None
    for needle in (0, 63, 200 - window, 255):
        cfg, w, h, ref = _edge_ref(case, needle)
        if mx is None:
            mx = load_mixer(cfg, w)
            prec = seq_ops.Precision(dtype)
            mx.pack(prec)
        assert worst_row(run_mixer(mx, [mx.cache_spec()], h, cuts, dtype, prec), ref) < tol, needle


@pytest.mark.parametrize("needle", [0, 63, 64, 700, 1023, 1024, 1087])
@pytest.mark.parametrize("dtype,tol", [(torch.float32, 2e-4), (torch.bfloat16, 8e-2)])
def test_far_key_among_a_thousand_in_keys_as_values_attention(needle, dtype, tol):
    """One token's input is five times larger, so its key (and value) weighs heavily wherever it is seen: from the end of a prompt of
    1100 tokens, from a portion that starts on a page border and from decoded tokens.  (bf16: the rows next to the large token carry its
    rounding, hence the wider bound on them.)"""
    from paligemma_multimodal_system_b200 import seq_ops
    D, T, eps = 40, 1100, 1e-5
    cfg = make_cfg([with_ff(attention(heads=2, kv_heads=1, dim=64, rot_dims=32, base=1e4), 0)], width=D, eps=eps)
    w = O.random_weights(cfg, seed=8)
    h = torch.randn(T, D, generator=torch.Generator().manual_seed(needle)).to(torch.bfloat16).float()
    plain = O.key_value_attention(h, w, "l0.mix.", cfg["layers"][0]["mixer"])
    h[needle] *= 5.0
    ref = O.key_value_attention(h, w, "l0.mix.", cfg["layers"][0]["mixer"])
    assert worst_row(plain[-40:], ref[-40:]) > 0.5  # the far token matters to the last rows
    mx = load_mixer(cfg, w)
    prec = seq_ops.Precision(dtype)
    mx.pack(prec)
    for cuts in ([T], [1088, 1], [1024, 70, 2]):
        got = run_mixer(mx, [mx.cache_spec()], h, cuts, dtype, prec)
        assert worst_row(got[-40:], ref[-40:]) < min(tol, 5e-2) and worst_row(got, ref) < tol, cuts


def test_first_positions_share_the_softmax_with_the_unit_in_the_denominator():
    """With tiny scores every weight is 1 / (keys + 1): position 0 returns half its value, position 1 a third of each."""
    from paligemma_multimodal_system_b200 import seq_ops
    D, eps = 32, 1e-5
    cfg = make_cfg([with_ff(attention(heads=2, kv_heads=2, dim=16, rot_dims=8, scale=1e-9), 0)], width=D, eps=eps)
    w = O.random_weights(cfg, seed=3)
    h = torch.randn(3, D, generator=torch.Generator().manual_seed(1)).to(torch.bfloat16).float()
    k = h @ w["l0.mix.k"].T + w["l0.mix.k.b"]
    expect = torch.stack([k[0] / 2, (k[0] + k[1]) / 3, (k[0] + k[1] + k[2]) / 4]) @ w["l0.mix.o"].T
    mx = load_mixer(cfg, w)
    prec = seq_ops.Precision(torch.float32)
    mx.pack(prec)
    for cuts in ([3], [1], [2, 1]):
        assert worst_row(run_mixer(mx, [mx.cache_spec()], h, cuts, torch.float32, prec), expect) < 1e-5


@pytest.mark.parametrize("ff", [80, 33, 256])
@pytest.mark.parametrize("dtype,tol,T", [(torch.float32, 1e-5, 77), (torch.bfloat16, 2e-2, 77), (torch.float32, 1e-5, 1), (torch.bfloat16, 2e-2, 300)])
def test_feed_forward_alone_and_into_a_scaled_residual(ff, dtype, tol, T):
    from paligemma_multimodal_system_b200 import seq_ops
    from paligemma_multimodal_system_b200.mixers import PolyNormFeedForward
    D, eps = 64, 1e-5
    cfg = make_cfg([with_ff(attention(), ff)], width=D, eps=eps)
    w = O.random_weights(cfg, seed=T)
    g = torch.Generator().manual_seed(5)
    h = torch.randn(T, D, generator=g).to(torch.bfloat16).float()
    x0 = torch.randn(T, D, generator=g)
    ref = O.feed_forward(h, w, "l0.mlp.", eps)
    f = PolyNormFeedForward(D, ff, eps)
    left = {k: v.to(torch.bfloat16) for k, v in w.items()}
    f.load(lambda name, shape: left.pop(name), "l0.mlp.")
    prec = seq_ops.Precision(dtype)
    f.pack(prec)
    hd = h.cuda().to(dtype).contiguous()
    assert worst_row(f(hd, None, prec), ref) < tol
    x = x0.cuda().contiguous()
    f(hd, None, prec, resid=x, resid_scale=0.35)
    assert worst_row(x.cpu() - x0, 0.35 * ref) < tol


def test_causal_edge_and_stale_rows():
    """Position i must see row i and not row i + 1: a changed LAST token leaves every earlier position's logits bit-identical."""
    w = O.random_weights(BASE_CFG, seed=2)
    tk = toks(80, BASE_CFG["vocab"], 6)
    eng = engine_for(BASE_CFG, w, torch.float32)
    poison(eng)
    got = eng.step([("a", tk, list(range(80)))], ["a"])
    tk2 = tk[:-1] + [(tk[-1] + 1) % BASE_CFG["vocab"]]
    got2 = eng.step([("b", tk2, list(range(80)))], ["b"])
    assert torch.equal(got[:-1], got2[:-1]) and not torch.equal(got[-1], got2[-1])
    assert close(got, O.forward(BASE_CFG, w, tk), torch.float32)


# ----------------------------------------------------------------------------------------------------------------------
# whole models
# ----------------------------------------------------------------------------------------------------------------------
@pytest.fixture(scope="module")
def base():
    w = O.random_weights(BASE_CFG, seed=1)
    tk = toks(150, BASE_CFG["vocab"], 2)
    return w, tk, O.forward(BASE_CFG, w, tk)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_whole_prompt_every_layer(base, dtype):
    w, tk, ref = base
    eng = engine_for(BASE_CFG, w, dtype)
    poison(eng)
    trace = []
    got = eng.step([("a", tk, list(range(len(tk))))], ["a"], trace=trace)
    _, layers = O.forward(BASE_CFG, w, tk, return_layers=True)
    assert len(trace) == len(BASE_CFG["layers"])
    for i, x in enumerate(trace):
        assert close(x, layers[i], dtype), f"residual after layer {i}"
    assert close(got, ref, dtype)


@pytest.mark.parametrize("cuts", [[1], [2], [3, 5, 2], [31, 33], [32], [64, 1], [65, 2, 2, 1], [100, 7], [20, 21, 22]])
def test_portions_and_token_by_token_equal_the_whole_prompt(base, cuts):
    w, tk, ref = base
    eng = engine_for(BASE_CFG, w, torch.float32)
    poison(eng)
    assert close(run_cut(eng, "a", tk, cuts), ref, torch.float32)


def test_portions_in_bf16(base):
    w, tk, ref = base
    eng = engine_for(BASE_CFG, w, torch.bfloat16)
    poison(eng)
    assert close(run_cut(eng, "a", tk, [37, 2, 64, 1]), ref, torch.bfloat16)


def test_unequal_batch_equals_each_alone_and_pages_and_slots_are_reused(base):
    """Four live requests of different lengths, portions beside single tokens, in a pool that only holds them because finished
    requests give their pages and slots back; every request's logits equal its solo run."""
    w, _, _ = base
    V = BASE_CFG["vocab"]
    prompts = {i: toks(n, V, 10 + i) for i, n in enumerate([130, 70, 1, 45, 90, 64, 3])}
    refs = {i: O.forward(BASE_CFG, w, p) for i, p in prompts.items()}
    eng = engine_for(BASE_CFG, w, torch.float32, max_tokens=6 * 64, slots=4)
    poison(eng)
    fed = {i: 0 for i in prompts}
    got = {i: [] for i in prompts}
    waiting, live, step = list(prompts), [], 0
    seen_pages, seen_slots = {}, {}
    while waiting or live:
        while waiting and len(live) < 4 and sum((len(prompts[i]) + 63) // 64 for i in live + waiting[:1]) <= 6:
            live.append(waiting.pop(0))
        entries, end = [], []
        for k, i in enumerate(live):
            left = len(prompts[i]) - fed[i]
            n = 1 if (step + k) % 3 == 0 else min(left, [17, 2, 40][(step + k) % 3])
            n = min(n, left)
            entries.append((i, prompts[i][fed[i]:fed[i] + n], list(range(n))))
            fed[i] += n
            if fed[i] == len(prompts[i]):
                end.append(i)
        out = eng.step(entries, end)
        for i in live:
            if i in eng.store.live:
                seen_pages[i], seen_slots[i] = list(eng.store.live[i].pages), eng.store.live[i].slot
        r = 0
        for i, tk, _ in entries:
            got[i].append(out[r:r + len(tk)])
            r += len(tk)
        live = [i for i in live if i not in end]
        step += 1
    for i in prompts:
        assert close(torch.cat(got[i]), refs[i], torch.float32), i
    all_pages = [p for ps in seen_pages.values() for p in ps]
    assert len(all_pages) > len(set(all_pages)), "no page was handed out twice"
    assert len(set(seen_slots.values())) < len(seen_slots), "no slot was handed out twice"
    assert not eng.store.live and len(eng.store.pool.free) == 6


def test_long_decoding_across_page_borders_and_out_of_every_window(base):
    w, _, _ = base
    tk = toks(260, BASE_CFG["vocab"], 77)
    ref = O.forward(BASE_CFG, w, tk)
    for dtype in (torch.float32, torch.bfloat16):
        eng = engine_for(BASE_CFG, w, dtype)
        poison(eng)
        assert close(run_cut(eng, "a", tk, [60, 1]), ref, dtype)  # 200 single-token steps: eager, captured, then replayed graphs


def test_first_tokens_of_a_sequence(base):
    """One-token prompts, a one-token first portion, two-token portions from the start."""
    w, tk, ref = base
    eng = engine_for(BASE_CFG, w, torch.float32)
    poison(eng)
    one = eng.step([("x", tk[:1], [0])], ["x"])
    assert close(one, ref[:1], torch.float32)
    assert close(run_cut(eng, "y", tk[:9], [1, 2, 2, 1, 3]), ref[:9], torch.float32)
    assert close(run_cut(eng, "z", tk[:8], [2]), ref[:8], torch.float32)


OTHER_SIZES = [
    # one key head per query head, two taps, no residual multiplier, odd sizes the 16-byte paths cannot take, a borrowing layer right after its source
    make_cfg([with_ff(latent(heads=5, dim=10, rot_dim=6, vdim=14, q_rank=9, kv_rank=11, size=17), 25), with_ff(latent(heads=2, dim=6, rot_dim=6, vdim=5, q_rank=7, kv_rank=11, size=9, kv_from=0), 0),
              with_ff(attention(heads=3, kv_heads=3, dim=14, rot_dims=6), 25)], width=34, vocab=41, taps=2, mult=1.0),
    # sizes the tensor-core kernels like (explicit-head latent form, 64- and 128-wide heads); a latent layer first; eight taps
    make_cfg([with_ff(latent(heads=4, dim=64, rot_dim=32, vdim=64, q_rank=96, kv_rank=64, size=48), 256), with_ff(attention(heads=4, kv_heads=1, dim=128, rot_dims=64), 0),
              with_ff(attention(heads=8, kv_heads=2, dim=64, rot_dims=64), 128), with_ff(latent(heads=8, dim=64, rot_dim=32, vdim=64, q_rank=64, kv_rank=64, size=100, kv_from=0), 256)],
             width=128, vocab=256, eps=1e-6, taps=8, mult=0.25),
    # a single head everywhere, one tap (no state), windows of one and of more than anything fed
    make_cfg([with_ff(attention(heads=1, kv_heads=1, dim=32, rot_dims=32), 12), with_ff(latent(heads=1, dim=8, rot_dim=8, vdim=8, q_rank=8, kv_rank=8, size=1), 12),
              with_ff(latent(heads=1, dim=16, rot_dim=2, vdim=4, q_rank=5, kv_rank=8, size=5000, scaling=False), 0)], width=24, vocab=20, taps=1, mult=0.9),
]


@pytest.mark.parametrize("ci", range(len(OTHER_SIZES)))
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_other_sizes(ci, dtype):
    cfg = OTHER_SIZES[ci]
    w = O.random_weights(cfg, seed=20 + ci)
    tk = toks(100, cfg["vocab"], ci)
    ref = O.forward(cfg, w, tk)
    eng = engine_for(cfg, w, dtype)
    poison(eng)
    assert close(run_cut(eng, "a", tk, [70, 2, 1, 1, 20, 1]), ref, dtype)
    two = [toks(n, cfg["vocab"], 50 + n) for n in (66, 30)]
    out = eng.step([(i, p, list(range(len(p)))) for i, p in enumerate(two)], [0, 1])
    assert close(out[:66], O.forward(cfg, w, two[0]), dtype) and close(out[66:], O.forward(cfg, w, two[1]), dtype)


def test_greedy_generation_through_the_scheduler():
    """engine.generate: more prompts than slots, a pool smaller than the sum of all requests, portions of 48 rows; the tokens
    equal the oracle's greedy continuation of each prompt alone."""
    cfg = make_cfg([with_ff(latent(heads=2, dim=16, rot_dim=8, vdim=16, q_rank=16, kv_rank=16, size=30), 48), with_ff(attention(heads=2, kv_heads=1, dim=16, rot_dims=8), 32),
                    with_ff(latent(heads=4, dim=8, rot_dim=8, vdim=8, q_rank=16, kv_rank=16, size=25, kv_from=0), 0)], width=48, vocab=60)
    w = O.random_weights(cfg, seed=31)
    prompts = [toks(n, 60, 40 + n) for n in (70, 5, 33, 1, 90, 12)]
    new = 10
    eng = engine_for(cfg, w, torch.float32, max_tokens=5 * 64, slots=3)
    poison(eng)
    got = eng.generate(prompts, new, step_tokens=48)
    for p, g in zip(prompts, got):
        seq = list(p)
        for _ in range(new):
            lg = O.forward(cfg, w, seq)[-1]
            top2 = lg.topk(2).values
            assert float(top2[0] - top2[1]) > 1e-3, "test weights give a near tie"
            seq.append(int(lg.argmax()))
        assert g == seq[len(p):]
    assert not eng.store.live and len(eng.store.pool.free) == 5


def test_sampled_generation_stays_in_vocabulary_and_stops_at_eos():
    cfg = make_cfg([with_ff(attention(heads=2, kv_heads=1, dim=16, rot_dims=8), 32), with_ff(latent(heads=2, dim=16, rot_dim=8, vdim=16, q_rank=16, kv_rank=16, size=12), 0)], width=48, vocab=60)
    w = O.random_weights(cfg, seed=9)
    eng = engine_for(cfg, w, torch.bfloat16, max_tokens=256, slots=2)
    out = eng.generate([toks(20, 60, 1), toks(3, 60, 2), toks(40, 60, 3)], 10, do_sample=True, temperature=0.9, top_p=0.8, eos_token_id=7, seed=3)
    for g in out:
        assert 1 <= len(g) <= 10 and all(0 <= t < 60 for t in g)
        assert 7 not in g[:-1]


def test_registry_loads_a_checkpoint_folder(tmp_path):
    """config.json + model.safetensors on disk -> registry.load_model -> the same logits as the in-memory model."""
    from paligemma_multimodal_system_b200.engine import SequenceEngine
    from paligemma_multimodal_system_b200.registry import load_model
    cfg = OTHER_SIZES[0]
    w = O.random_weights(cfg, seed=11)
    meta, blobs, off = {}, [], 0
    for name, t in w.items():
        raw = t.to(torch.bfloat16).contiguous().view(torch.int16).numpy().tobytes()
        meta[name] = {"dtype": "BF16", "shape": list(t.shape), "data_offsets": [off, off + len(raw)]}
        blobs.append(raw)
        off += len(raw)
    head = json.dumps(meta).encode()
    (tmp_path / "model.safetensors").write_bytes(struct.pack("<Q", len(head)) + head + b"".join(blobs))
    (tmp_path / "config.json").write_text(json.dumps(cfg))
    tk = toks(50, cfg["vocab"], 5)
    eng = SequenceEngine(load_model(str(tmp_path), dtype=torch.float32), 128, 1)
    assert close(eng.step([("a", tk, list(range(50)))], ["a"]), O.forward(cfg, w, tk), torch.float32)


def test_wider_model_long_prompt_reaches_the_large_tile_paths():
    """Width 512, a 2048-wide feed-forward, 64-wide key heads and the explicit-head latent form over 1100 tokens in bf16, every window
    edge inside the prompt; then 20 decoded tokens."""
    cfg = make_cfg([with_ff(latent(heads=8, dim=64, rot_dim=32, vdim=64, q_rank=192, kv_rank=128, size=300, base=1e5), 2048),
                    with_ff(attention(heads=8, kv_heads=2, dim=64, rot_dims=32), 1024),
                    with_ff(latent(heads=8, dim=64, rot_dim=32, vdim=64, q_rank=128, kv_rank=128, size=200, base=1e5, kv_from=0), 512)], width=512, vocab=1000, taps=4)
    w = O.random_weights(cfg, seed=77)
    tk = toks(1120, 1000, 3)
    ref = O.forward(cfg, w, tk)
    eng = engine_for(cfg, w, torch.bfloat16, max_tokens=1280, slots=2)
    poison(eng)
    assert close(run_cut(eng, "a", tk, [1100, 1]), ref, torch.bfloat16)


@pytest.mark.parametrize("kv_rank,rot_dim,heads", [(64, 32, 8), (128, 32, 40), (256, 32, 32), (128, 64, 64), (512, 32, 32), (512, 64, 72)])
@pytest.mark.parametrize("window", [1, 63, 64, 65, 200, 5000])
def test_windowed_decode_of_cached_latent_rows_on_the_tensor_cores(kv_rank, rot_dim, heads, window):
    """Row widths the tensor-core decode kernel of the absorbed form has, bf16: three sequences of unequal context decode together, the
    window's first key at every place of a 64-key tile, a dominating key just inside and just outside the window."""
    from paligemma_multimodal_system_b200 import seq_ops
    from paligemma_multimodal_system_b200.cache import SequenceStore
    kd, R, scale = kv_rank + rot_dim, kv_rank, 0.05
    assert (kd, R) in seq_ops.LATENT_MMA_SIZES
    ctxs = [700, 130, 5]
    g = torch.Generator().manual_seed(window + kd)
    store = SequenceStore([("latent", kd)], max_tokens=1024, num_slots=4, dtype=torch.bfloat16)
    store.k_pages[0].fill_(1e4)
    store.pool.take(1)
    rows, qs, es = [], [], []
    for i, c in enumerate(ctxs):
        store.admit(i)
        rec = store.reserve(i, c + 1)
        keys = (0.5 * torch.randn(c + 1, kd, generator=g)).to(torch.bfloat16)
        q = (0.5 * torch.randn(heads, kd, generator=g)).to(torch.bfloat16)
        for needle in (c + 1 - window, c - window):  # the oldest key still seen, and the one before it
            if needle >= 0:
                keys[needle, 0] = 30.0 if needle == c + 1 - window else -30.0
                keys[needle, 1:R] = 3.0 if needle == c + 1 - window else -3.0
        q[:, 0] = 2.0
        for j in range(c + 1):
            store.k_pages[0][rec.pages[j // 64], j % 64] = keys[j].cuda()
        rows.append(keys.double())
        qs.append(q)
        es.append(dict(tokens=[0], ctx=c, slot=rec.slot, pages=rec.pages))
    b = seq_ops.make_step_batch(es)
    out = torch.empty(3, heads * R, device="cuda", dtype=torch.bfloat16)
    seq_ops.attn_ragged(torch.stack(qs).reshape(3, -1).cuda(), store.k_pages[0], store.k_pages[0], None, out, b, heads, 1, kd, R, scale, 0.0, 64, krow=kd, vrow=kd,
                        gate_per_head=True, score=seq_ops.ScoreOptions(heads, window))
    for i, c in enumerate(ctxs):
        lo = max(0, c + 1 - window)
        s = (qs[i].double() @ rows[i][lo:].T) * scale
        ref = torch.softmax(s, -1) @ rows[i][lo:, :R]
        assert worst_row(out[i].float().reshape(heads, R), ref) < 2e-2, (i, c)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_trace_runner_replays_a_mixed_schedule(tmp_path, dtype):
    """bin/trace_run on a checkpoint folder: portions beside single tokens, a step that wants nothing, a request that sits out a step,
    a finished request's page and slot taken over by a later one; the written logits equal the oracle's for each request alone."""
    import subprocess
    import numpy as np
    cfg = OTHER_SIZES[0]
    w = O.random_weights(cfg, seed=13)
    meta, blobs, off = {}, [], 0
    for name, t in w.items():
        raw = t.to(torch.bfloat16).contiguous().view(torch.int16).numpy().tobytes()
        meta[name] = {"dtype": "BF16", "shape": list(t.shape), "data_offsets": [off, off + len(raw)]}
        blobs.append(raw)
        off += len(raw)
    head = json.dumps(meta).encode()
    (tmp_path / "model").mkdir()
    (tmp_path / "model" / "model.safetensors").write_bytes(struct.pack("<Q", len(head)) + head + b"".join(blobs))
    (tmp_path / "model" / "config.json").write_text(json.dumps(cfg))
    V = cfg["vocab"]
    tk = {"a": toks(70, V, 1), "b": toks(33, V, 2), "c": toks(1, V, 3), "d": toks(20, V, 4)}
    steps = [
        {"step": 0, "entries": [{"id": "a", "tokens": tk["a"][:40], "want": [0, 39]}, {"id": "b", "tokens": tk["b"][:2], "want": [1]}], "end": []},
        {"step": 1, "entries": [{"id": "a", "tokens": tk["a"][40:41], "want": [0]}, {"id": "c", "tokens": tk["c"], "want": [0]}], "end": ["c"]},
        {"step": 2, "entries": [{"id": "b", "tokens": tk["b"][2:32], "want": []}, {"id": "a", "tokens": tk["a"][41:42], "want": []}], "end": []},
        {"step": 3, "entries": [{"id": "d", "tokens": tk["d"][:19], "want": [18]}, {"id": "a", "tokens": tk["a"][42:], "want": [27]}, {"id": "b", "tokens": tk["b"][32:], "want": [0]}],
         "end": ["a", "b"]},
        {"step": 4, "entries": [{"id": "d", "tokens": tk["d"][19:], "want": [0]}], "end": ["d"]},
    ]
    out = tmp_path / "out"
    r = subprocess.run([sys.executable, os.path.join(ROOT, "bin", "trace_run"), "--model", str(tmp_path / "model"), "--dtype", dtype, "--out", str(out),
                        "--max-tokens", "256"], input="".join(json.dumps(s) + "\n" for s in steps), capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stderr[-2000:]
    assert [l for l in r.stdout.splitlines() if l.startswith("done ")] == [f"done {i}" for i in range(5)]
    assert not (out / "2.f32").exists()
    ref = {k: O.forward(cfg, w, v) for k, v in tk.items()}
    want = {0: [("a", 0), ("a", 39), ("b", 1)], 1: [("a", 40), ("c", 0)], 3: [("d", 18), ("a", 69), ("b", 32)], 4: [("d", 19)]}
    dt = torch.float32 if dtype == "float32" else torch.bfloat16
    for step, rows in want.items():
        got = torch.from_numpy(np.fromfile(out / f"{step}.f32", dtype="<f4").reshape(len(rows), V).copy())
        assert close(got, torch.stack([ref[k][p] for k, p in rows]), dt), step
