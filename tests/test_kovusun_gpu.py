"""Kovusun through the framework (kernels, page pool and state slots, ragged steps, scheduler) against the plain oracle
(oracle/kovusun_oracle.py): every mechanism alone, then whole models under every way of cutting and batching the work."""
import copy
import json
import os
import struct
import sys

import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)
from oracle import kovusun_oracle as O  # noqa: E402

pytestmark = pytest.mark.gpu

F32_TOL, BF16_TOL = 2e-4, 4e-2


def mixer(kind, heads=6, kv_heads=3, dim=24, vdim=40, size=37, keep_first=None, scale=None, rot=None, kv_from=None):
    m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale if scale is not None else dim ** -0.5, "mask": {"size": size}}
    if kind == "attention_3":
        m["mask"]["keep_first"] = 5 if keep_first is None else keep_first
        m["rot"] = rot or {"base": 5000.0, "dims": dim // 2 // 2 * 2}
    if kv_from is not None:
        m["kv_from"] = kv_from
    return m


def dense(ff=80, limit=1.5):
    return {"kind": "dense", "ff": ff, "limit": limit}


def moe(experts=7, top=3, ff=24, shared=40):
    m = {"kind": "moe", "expert": {"ff": ff}, "router": {"experts": experts, "top": top}}
    if shared:
        m["shared"] = {"ff": shared}
    return m


def layer(kind, mlp, **kw):
    return {"type": kind, "mixer": mixer(kind, **kw), "mlp": mlp}


def make_cfg(layers, width=72, vocab=90, eps=1e-5):
    return {"architecture": "Kovusun", "vocab": vocab, "width": width, "norm": {"eps": eps}, "layers": layers}


# every mixer type, a borrowing layer whose window differs from its source's, both feed-forward kinds and a layer without one
BASE_CFG = make_cfg([layer("attention_2", dense(), size=70), layer("attention_3", moe(), heads=4, kv_heads=2, dim=32, vdim=16, size=90, keep_first=3),
                     layer("attention", moe(experts=5, top=2, shared=0), heads=3, kv_heads=3, dim=20, vdim=28, size=33),
                     layer("attention_2", None, heads=2, kv_heads=1, dim=16, vdim=16, size=50),
                     layer("attention", dense(48, 0.7), heads=6, kv_heads=3, dim=20, vdim=28, size=21, kv_from=2)])


def build(cfg, w, dtype):
    from paligemma_multimodal_system_b200.modeling_kovusun import KovusunConfig, KovusunForCausalLM
    return KovusunForCausalLM(KovusunConfig(cfg), dtype).load_weights({k: v.to(torch.bfloat16) for k, v in w.items()})


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


def close(got, ref, dtype):
    """fp32: the whole tensor within F32_TOL.  bf16: nine rows in ten within BF16_TOL -- a routed layer may hand a token whose
    best logits nearly tie to another expert, which moves that token's row and nothing else."""
    if dtype == torch.float32:
        return rel_err(got, ref) < F32_TOL
    got, ref = got.double().cpu(), ref.double()
    rows = (got - ref).pow(2).mean(-1).sqrt() / ref.pow(2).mean(-1).sqrt()
    return float(rows.quantile(0.9)) < BF16_TOL and float(rows.median()) < BF16_TOL / 2


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


def _entries(layout, lens_ctx, dtype, skip_pages=2):
    """A store and a step batch of entries (new tokens, context) whose pages do not start at page 0."""
    from paligemma_multimodal_system_b200 import seq_ops
    from paligemma_multimodal_system_b200.cache import SequenceStore
    total = sum((c + n + 63) // 64 * 64 for n, c in lens_ctx) + 64 * skip_pages
    store = SequenceStore(layout, max_tokens=total, num_slots=len(lens_ctx) + 1, dtype=dtype)
    store.pool.take(skip_pages)
    store.admit("skipped")
    es = []
    for i, (n, c) in enumerate(lens_ctx):
        store.admit(i)
        rec = store.reserve(i, c + n)
        es.append(dict(tokens=[0] * n, ctx=c, slot=rec.slot, pages=rec.pages))
    return store, seq_ops.make_step_batch(es), es


# ----------------------------------------------------------------------------------------------------------------------
# mechanisms alone
# ----------------------------------------------------------------------------------------------------------------------
@pytest.mark.parametrize("D,lens,plans", [(40, [23, 9, 14], [[5, 1, 2, 15], [1] * 9, [14]]), (72, [23, 9, 14], [[5, 1, 2, 15], [1] * 9, [14]]),
                                          (257, [23, 9, 14], [[5, 1, 2, 15], [1] * 9, [14]]), (1024, [23, 9, 14], [[5, 1, 2, 15], [1] * 9, [14]]),
                                          # steps of thousands of rows: the kernel walks chunks of consecutive rows per CTA, chunk borders fall
                                          # inside entries, on their first rows and on their last ones
                                          (72, [5000, 9, 2703], [[4000, 1, 2, 997], [1] * 9, [700, 2001, 2]]),
                                          (1280, [2500, 3, 1301], [[1, 2400, 99], [1, 1, 1], [1300, 1]])])
@pytest.mark.parametrize("f32", [True, False])
def test_two_norms_and_token_shift_in_portions(D, lens, plans, f32):
    """Three sequences advance together in unequal portions (one of them token by token); the mixer's input must equal the
    whole-sequence oracle at every position, whatever the state slots held before."""
    from paligemma_multimodal_system_b200 import seq_ops
    from paligemma_multimodal_system_b200.cache import SequenceStore
    g = torch.Generator().manual_seed(D)
    eps = 1e-5
    xs = [3.0 + 2.0 * torch.randn(n, D, generator=g) for n in lens]
    w1, b1, w2, b2 = (torch.randn(D, generator=g) for _ in range(4))
    sh = torch.rand(D, generator=g)
    ref1 = [O.token_shift(O.layer_norm(x, w1, b1, eps), sh) for x in xs]
    ref2 = [O.layer_norm(x, w2, b2, eps) for x in xs]
    store = SequenceStore([("state", (D,))], max_tokens=sum(lens) + 256, num_slots=4, dtype=torch.float32)
    store.state[0].fill_(1e4)
    store.admit("unused")
    for i in range(3):
        store.admit(i)
    dt = torch.float32 if f32 else torch.bfloat16
    got1, got2 = [[] for _ in lens], [[] for _ in lens]
    fed = [0, 0, 0]
    step = 0
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
        o1, o2 = torch.empty(b.T, D, device="cuda", dtype=dt), torch.empty(b.T, D, device="cuda", dtype=dt)
        seq_ops.layernorm_shift(x, w1.cuda(), b1.cuda(), o1, eps, shift=sh.cuda(), state=store.state[0], b=b, w2=w2.cuda(), b2=b2.cuda(), out2=o2)
        r = 0
        for i, k in rows:
            got1[i].append(o1[r:r + k].float().cpu())
            got2[i].append(o2[r:r + k].float().cpu())
            store.commit(i, k)
            fed[i] += k
            r += k
        step += 1
    tol = 1e-5 if f32 else 6e-3
    for i in range(3):
        assert rel_err(torch.cat(got1[i]), ref1[i]) < tol and rel_err(torch.cat(got2[i]), ref2[i]) < tol, i
    # a bare norm (the model's last one): one output, no state
    o = torch.empty(lens[0], D, device="cuda", dtype=dt)
    seq_ops.layernorm_shift(xs[0].cuda().contiguous(), w2.cuda(), b2.cuda(), o, eps)
    assert rel_err(o.float(), ref2[0]) < tol


@pytest.mark.parametrize("kind,limit", [(1, 0.0), (2, 0.8), (2, 3.0)])
@pytest.mark.parametrize("f32", [True, False])
def test_gated_activations(kind, limit, f32):
    from paligemma_multimodal_system_b200 import seq_ops
    g = torch.Generator().manual_seed(kind)
    T, F = 37, 50
    gu = (2.5 * torch.randn(T, 2 * F, generator=g)).to(torch.bfloat16).float()
    ga, up = gu[:, :F], gu[:, F:]
    if kind == 1:
        ref = ga * torch.sigmoid(ga) * up
    else:
        gc = torch.clamp(ga, max=limit)
        ref = gc * torch.sigmoid(1.702 * gc) * (torch.clamp(up, -limit, limit) + 1.0)
    dt = torch.float32 if f32 else torch.bfloat16
    out = seq_ops.glu(gu.cuda().to(dt), torch.empty(T, F, device="cuda", dtype=dt), kind, limit, 1.702)
    assert rel_err(out.float(), ref) < (1e-6 if f32 else 5e-3)


MIXERS = [("attention", dict()), ("attention_2", dict()), ("attention_3", dict()),
          ("attention", dict(heads=4, kv_heads=4, dim=64, vdim=64, size=70)),               # tensor-core head size, one k/v head per query head
          ("attention_2", dict(heads=8, kv_heads=1, dim=64, vdim=64, size=129)),            # one k/v head for all, groups of 8
          ("attention_3", dict(heads=4, kv_heads=2, dim=128, vdim=128, size=64, keep_first=70, rot={"base": 1e4, "dims": 128})),  # kept keys outnumber the window
          ("attention_3", dict(heads=2, kv_heads=2, dim=10, vdim=6, size=1, keep_first=0, rot={"base": 100.0, "dims": 4})),        # a window of one
          ("attention_2", dict(heads=5, kv_heads=5, dim=18, vdim=30, size=1000))]           # a window longer than the sequence


@pytest.mark.parametrize("kind,kw", MIXERS)
@pytest.mark.parametrize("dtype,tol", [(torch.float32, 1e-4), (torch.bfloat16, 3e-2)])
def test_windowed_attention_alone(kind, kw, dtype, tol):
    """One mixer over 200 positions: as one portion, and as context + portion + two single tokens (decode kernel)."""
    from paligemma_multimodal_system_b200 import seq_ops
    from paligemma_multimodal_system_b200.modeling_kovusun import _mixer
    D, T, eps = 56, 200, 1e-5
    m = mixer(kind, **kw)
    cfg = make_cfg([{"type": kind, "mixer": m, "mlp": None}], width=D)
    w = O.random_weights(cfg, seed=len(str(kw)))
    g = torch.Generator().manual_seed(3)
    h = torch.randn(T, D, generator=g).to(torch.bfloat16).float()
    ref = O.attention(h, w, "l0.mix.", kind, m, eps, O.keys_values(h, w, "l0.mix.", kind, m, eps))
    mx = _mixer(D, kind, m, eps)
    left = {k: v.to(torch.bfloat16) for k, v in w.items()}
    mx.load(lambda name, shape: left.pop(name), "l0.mix.")
    prec = seq_ops.Precision(dtype)
    mx.pack(prec)
    for cuts in ([T], [131, 67, 1, 1]):
        store, _, _ = _entries([mx.cache_spec()], [(T, 0)], dtype)
        for t in (store.k_pages[0], store.v_pages[0]):
            t.fill_(1e4)
        rec, pos, outs = store.live[0], 0, []
        for k in cuts:
            b = seq_ops.make_step_batch([dict(tokens=[0] * k, ctx=pos, slot=rec.slot, pages=rec.pages)])
            outs.append(mx(h[pos:pos + k].cuda().to(dtype).contiguous(), b, store, 0, prec).float().cpu())
            pos += k
        assert rel_err(torch.cat(outs), ref) < tol, cuts


def _needle_case(window, keep, ctx, n, needle, H=4, G=2, dim=16, vdim=8, sink=None, f32=True):
    """Every key is orthogonal to the queries but the needle, whose score stands out; its value is a marker.  Returns the
    kernel's output and the oracle's for the entry's new rows."""
    from paligemma_multimodal_system_b200 import seq_ops
    dt = torch.float32 if f32 else torch.bfloat16
    N = ctx + n
    g = torch.Generator().manual_seed(needle + 7 * ctx + n)
    keys = 0.05 * torch.randn(N, G, dim, generator=g)
    vals = 0.1 * torch.randn(N, G, vdim, generator=g)
    keys[needle] = 0.0
    keys[needle, :, 0] = 8.0
    vals[needle] = 50.0
    q = 0.05 * torch.randn(n, H, dim, generator=g)
    q[:, :, 0] = 4.0
    keys, vals, q = (t.to(torch.bfloat16).float() for t in (keys, vals, q))
    sk = None if sink is None else torch.full((H,), float(sink))
    ref = O.attend(q, keys, vals, 1.0, window, keep, sink=sk, first_pos=ctx)
    store, b, _ = _entries([("kv", G * dim, G * vdim)], [(3, 70), (n, ctx)], dt)
    kp, vp = store.k_pages[0], store.v_pages[0]
    kp.fill_(1e4)
    vp.fill_(1e4)
    pages = store.live[1].pages
    for j in range(N):
        kp[pages[j // 64], j % 64] = keys[j].reshape(-1).to(dt)
        vp[pages[j // 64], j % 64] = vals[j].reshape(-1).to(dt)
    for j in range(73):  # the other entry of the batch: harmless small keys
        kp[store.live[0].pages[j // 64], j % 64] = 0.01
        vp[store.live[0].pages[j // 64], j % 64] = 0.01
    qq = torch.zeros(b.T, H * dim, device="cuda", dtype=dt)
    qq[3:] = q.reshape(n, -1).to(dt)
    out = torch.empty(b.T, H * vdim, device="cuda", dtype=dt)
    score = seq_ops.ScoreOptions(H, window, keep, sink=None if sk is None else sk.cuda())
    seq_ops.attn_ragged(qq, kp, vp, None, out, b, H, G, dim, vdim, 1.0, 0.0, 64, score=score)
    return out[3:].float().cpu().reshape(n, H, vdim), ref


@pytest.mark.parametrize("window,keep", [(96, 0), (64, 0), (65, 6), (130, 3), (1, 0), (40, 64)])
@pytest.mark.parametrize("ctx,n", [(0, 300), (250, 50), (299, 1), (256, 1), (255, 2), (1300, 1), (1250, 40)])
def test_needle_just_inside_and_just_outside_the_window(window, keep, ctx, n):
    """The needle sits `window - 1` keys back from the last query (seen), `window` keys back (not seen), on the last kept first
    position (seen from anywhere) and right after it (seen only from inside the window); prompts and decoded tokens, key
    splits, page borders."""
    last = ctx + n - 1
    for needle, seen in ((last - window + 1, True), (last - window, False), (keep - 1, True), (keep, last - keep < window)):
        if not 0 <= needle <= last:
            continue
        got, ref = _needle_case(window, keep, ctx, n, needle)
        assert rel_err(got, ref) < 1e-4, (needle, seen)
        assert bool(got[-1].abs().max() > 25.0) == seen, (needle, seen)


@pytest.mark.parametrize("needle", [0, 63, 64, 127, 128, 1000, 1023, 1024, 1087, 1088, 1099])
@pytest.mark.parametrize("ctx,n,f32", [(0, 1100, True), (1099, 1, True), (1030, 70, False), (1099, 1, False)])
def test_far_key_at_page_borders_is_found_through_a_long_window(needle, ctx, n, f32):
    got, ref = _needle_case(2000, 0, ctx, n, needle, dim=64, vdim=64, f32=f32)
    assert rel_err(got, ref) < (1e-4 if f32 else 2e-2)
    assert float(got[-1].abs().max()) > 25.0


@pytest.mark.parametrize("ctx,n", [(0, 90), (89, 1), (700, 1)])
@pytest.mark.parametrize("f32", [True, False])
def test_sink_takes_its_share_once(ctx, n, f32):
    """A large sink halves or nearly cancels the output; key splits must not count it once per split."""
    for sink in (-30.0, 0.0, 12.0, 40.0):
        got, ref = _needle_case(64, 0, ctx, n, ctx + n - 5, sink=sink, dim=64, vdim=64, f32=f32)
        assert (got - ref).abs().max() < (1e-3 if f32 else 0.3) and rel_err(got, ref) < (1e-4 if f32 else 2e-2), sink


@pytest.mark.parametrize("dim,vdim", [(32, 32), (64, 64), (128, 128), (64, 128), (128, 64)])
@pytest.mark.parametrize("gsz", [1, 3, 8])
def test_tensor_core_prompt_kernel_with_every_optional_part(dim, vdim, gsz):
    """bf16 prompt portions of the head sizes the tensor-core kernel is built for, all score options at once, against float64."""
    from paligemma_multimodal_system_b200 import seq_ops
    G, ctx, n, window, keep = 2, 150, 170, 100, 9
    H, N = G * gsz, ctx + n
    g = torch.Generator().manual_seed(dim + gsz)
    keys, vals = torch.randn(N, G, dim, generator=g), torch.randn(N, G, vdim, generator=g)
    q = torch.randn(n, H, dim, generator=g)
    keys, vals, q = (t.to(torch.bfloat16).double() for t in (keys, vals, q))
    sink, r1, r2, temp = torch.randn(H, generator=g), torch.rand(H, generator=g), torch.rand(H, generator=g) + 0.1, torch.rand(H, generator=g) + 0.5
    ref = O.attend(q, keys, vals, dim ** -0.5, window, keep, sink=sink.double(), r1=r1.double(), r2=r2.double(), temp=temp.double(), first_pos=ctx)
    store, b, _ = _entries([("kv", G * dim, G * vdim)], [(n, ctx)], torch.bfloat16)
    kp, vp = store.k_pages[0], store.v_pages[0]
    kp.fill_(1e4)
    vp.fill_(1e4)
    pages = store.live[0].pages
    for j in range(N):
        kp[pages[j // 64], j % 64] = keys[j].reshape(-1).to(torch.bfloat16)
        vp[pages[j // 64], j % 64] = vals[j].reshape(-1).to(torch.bfloat16)
    out = torch.empty(n, H * vdim, device="cuda", dtype=torch.bfloat16)
    score = seq_ops.ScoreOptions(H, window, keep, sink=sink.cuda(), dist_a=r1.cuda(), dist_b=r2.cuda(), head_scale=temp.cuda())
    seq_ops.attn_ragged(q.reshape(n, -1).to(torch.bfloat16).cuda(), kp, vp, None, out, b, H, G, dim, vdim, dim ** -0.5, 0.0, 64, score=score)
    assert rel_err(out.float().reshape(n, H, vdim), ref) < 6e-3  # the bf16 rounding of the output alone is 2e-3


@pytest.mark.parametrize("n_all,top", [(7, 3), (12, 1), (5, 5), (40, 6)])
def test_router_takes_the_largest_biased_logits_and_softmaxes_them_alone(n_all, top):
    from paligemma_multimodal_system_b200 import seq_ops
    g = torch.Generator().manual_seed(n_all)
    T = 50
    z, bias = 3.0 * torch.randn(T, n_all, generator=g), 2.0 * torch.randn(n_all, generator=g)
    ids, wts, counts = seq_ops.moe_route(z.cuda(), None, n_all, top, 1, 1, 1.0, logit_bias=bias.cuda())
    zb = z + bias
    best = zb.topk(top, dim=-1)
    assert torch.equal(ids.cpu().long(), best.indices)
    assert torch.allclose(wts.cpu(), torch.softmax(best.values, -1), atol=1e-6, rtol=1e-5)
    assert torch.equal(counts.cpu().long(), torch.bincount(best.indices.reshape(-1), minlength=n_all))


@pytest.mark.parametrize("mlp", [dense(), dense(33, 0.4), moe(), moe(experts=4, top=4, ff=10, shared=0), moe(experts=9, top=1, ff=64, shared=16)])
@pytest.mark.parametrize("dtype,tol,T", [(torch.float32, 1e-5, 77), (torch.bfloat16, 2e-2, 77), (torch.float32, 1e-5, 1), (torch.bfloat16, 2e-2, 300)])
def test_feed_forwards_alone(mlp, dtype, tol, T):
    from paligemma_multimodal_system_b200 import seq_ops
    from paligemma_multimodal_system_b200.modeling_kovusun import _feed_forward
    D = 64
    cfg = make_cfg([{"type": "attention_2", "mixer": mixer("attention_2"), "mlp": mlp}], width=D)
    w = O.random_weights(cfg, seed=T)
    g = torch.Generator().manual_seed(5)
    h = torch.randn(T, D, generator=g).to(torch.bfloat16).float()
    x0 = torch.randn(T, D, generator=g)
    ref = O.feed_forward(h, w, "l0.mlp.", mlp)
    ff = _feed_forward(D, mlp)
    left = {k: v.to(torch.bfloat16) for k, v in w.items()}
    ff.load(lambda name, shape: left.pop(name), "l0.mlp.")
    prec = seq_ops.Precision(dtype)
    ff.pack(prec)
    hd = h.cuda().to(dtype).contiguous()
    assert close(ff(hd, None, prec), ref, dtype) and (dtype == torch.bfloat16 or rel_err(ff(hd, None, prec), ref) < tol)
    x = x0.cuda().contiguous()
    ff(hd, None, prec, resid=x)  # the same, added into a residual
    assert close(x - x0.cuda(), ref, dtype)


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
    assert rel_err(got, O.forward(BASE_CFG, w, tk)) < F32_TOL


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
    assert rel_err(run_cut(eng, "a", tk, cuts), ref) < F32_TOL


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
        assert rel_err(torch.cat(got[i]), refs[i]) < F32_TOL, i
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


def test_long_context_decode_with_key_splits_and_kept_first_keys():
    cfg = make_cfg([layer("attention_3", dense(32), heads=2, kv_heads=1, dim=16, vdim=16, size=700, keep_first=40),
                    layer("attention", moe(experts=4, top=2, ff=16, shared=16), heads=2, kv_heads=2, dim=16, vdim=16, size=1100),
                    layer("attention_2", None, heads=2, kv_heads=2, dim=16, vdim=16, size=64)], width=32, vocab=50)
    w = O.random_weights(cfg, seed=5)
    tk = toks(1300, 50, 9)
    full = O.forward(cfg, w, tk)
    eng = engine_for(cfg, w, torch.float32, max_tokens=1344, slots=1)
    poison(eng)
    got = run_cut(eng, "a", tk, [1260, 1])  # a portion long enough for the row-chunked norm kernel, then 40 decoded tokens
    assert rel_err(got[-40:], full[-40:]) < F32_TOL and rel_err(got, full) < F32_TOL


def test_first_tokens_of_a_sequence(base):
    """One-token prompts, a one-token first portion, two-token portions from the start."""
    w, tk, ref = base
    eng = engine_for(BASE_CFG, w, torch.float32)
    poison(eng)
    one = eng.step([("x", tk[:1], [0])], ["x"])
    assert rel_err(one, ref[:1]) < F32_TOL
    assert rel_err(run_cut(eng, "y", tk[:9], [1, 2, 2, 1, 3]), ref[:9]) < F32_TOL
    assert rel_err(run_cut(eng, "z", tk[:8], [2]), ref[:8]) < F32_TOL


OTHER_SIZES = [
    # one k/v head per query head everywhere, top = 1, odd sizes the 16-byte paths cannot take
    make_cfg([layer("attention", moe(experts=3, top=1, ff=10, shared=6), heads=5, kv_heads=5, dim=10, vdim=14, size=17),
              layer("attention_3", dense(25, 5.0), heads=3, kv_heads=3, dim=14, vdim=6, size=9, keep_first=11, rot={"base": 77.0, "dims": 6})], width=34, vocab=41),
    # sizes the tensor-core kernels like; borrowing across a layer of another type; no feed-forward on the first layer
    make_cfg([layer("attention_2", None, heads=4, kv_heads=2, dim=64, vdim=64, size=48), layer("attention_3", dense(256), heads=4, kv_heads=1, dim=128, vdim=128, size=80, keep_first=2),
              layer("attention_2", moe(experts=8, top=8, ff=64, shared=128), heads=8, kv_heads=2, dim=64, vdim=64, size=100, kv_from=0)], width=128, vocab=256, eps=1e-6),
    # a single head, a single expert
    make_cfg([layer("attention", moe(experts=1, top=1, ff=12, shared=0), heads=1, kv_heads=1, dim=32, vdim=8, size=3),
              layer("attention", None, heads=2, kv_heads=1, dim=32, vdim=8, size=200, kv_from=0)], width=24, vocab=20),
    # full rotation, a window wider than anything fed, kept keys without effect
    make_cfg([layer("attention_3", moe(experts=16, top=5, ff=8, shared=8), heads=6, kv_heads=2, dim=16, vdim=24, size=500, keep_first=4, rot={"base": 1e6, "dims": 16})],
             width=48, vocab=64),
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
    cfg = make_cfg([layer("attention_2", dense(48), heads=2, kv_heads=1, dim=16, vdim=16, size=30), layer("attention_3", moe(experts=4, top=2, ff=16, shared=16), heads=2, kv_heads=2, dim=16, vdim=16, size=25, keep_first=2),
                    layer("attention", None, heads=4, kv_heads=2, dim=16, vdim=16, size=40, kv_from=1)], width=48, vocab=60)
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
    cfg = make_cfg([layer("attention_2", moe(experts=4, top=2, ff=16, shared=0), heads=2, kv_heads=1, dim=16, vdim=16, size=12)], width=48, vocab=60)
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
    cfg = copy.deepcopy(OTHER_SIZES[0])
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
    assert rel_err(eng.step([("a", tk, list(range(50)))], ["a"]), O.forward(cfg, w, tk)) < F32_TOL


@pytest.mark.parametrize("T", [40, 300])
def test_gated_experts_as_dense_runs_per_expert(T, monkeypatch):
    """Long prompt portions hand every expert's tokens to dense tensor-core products with the gated unit in the epilogue;
    forced here at a small size and compared with the grouped kernel and the oracle."""
    from paligemma_multimodal_system_b200 import seq_ops
    from paligemma_multimodal_system_b200.mixers import RoutedFeedForward
    from paligemma_multimodal_system_b200.modeling_kovusun import _feed_forward
    D, mlp = 64, moe(experts=5, top=2, ff=128, shared=0)
    cfg = make_cfg([{"type": "attention_2", "mixer": mixer("attention_2"), "mlp": mlp}], width=D)
    w = O.random_weights(cfg, seed=T)
    h = torch.randn(T, D, generator=torch.Generator().manual_seed(8)).to(torch.bfloat16).float()
    ref = O.feed_forward(h, w, "l0.mlp.", mlp)
    ff = _feed_forward(D, mlp)
    left = {k: v.to(torch.bfloat16) for k, v in w.items()}
    ff.load(lambda name, shape: left.pop(name), "l0.mlp.")
    prec = seq_ops.Precision(torch.bfloat16)
    ff.pack(prec)
    assert ff.w_up_dense is not None
    hd = h.cuda().to(torch.bfloat16).contiguous()
    grouped = ff(hd, None, prec)
    monkeypatch.setattr(RoutedFeedForward, "DENSE_SEGMENT_ROWS", 1)
    assert ff._dense_segments(T, prec)
    dense_runs = ff(hd, None, prec)
    assert close(dense_runs, ref, torch.bfloat16) and rel_err(dense_runs, grouped.cpu()) < 1e-2


def test_wider_model_long_prompt_reaches_the_large_tile_paths():
    """Width 512, 64-wide heads, a 2048-wide dense feed-forward and 256-wide experts over 1100 tokens in bf16: the prompt runs the
    paired-CTA products with bias and gated epilogues, the tensor-core attention with every window edge inside the prompt and
    the per-expert dense runs; then 20 decoded tokens."""
    cfg = make_cfg([layer("attention_2", dense(2048, 2.5), heads=8, kv_heads=2, dim=64, vdim=64, size=300),
                    layer("attention", moe(experts=4, top=2, ff=256, shared=512), heads=8, kv_heads=4, dim=64, vdim=64, size=200),
                    layer("attention_3", moe(experts=4, top=2, ff=256, shared=0), heads=4, kv_heads=1, dim=128, vdim=128, size=500, keep_first=7)],
                   width=512, vocab=1000)
    w = O.random_weights(cfg, seed=77)
    tk = toks(1120, 1000, 3)
    ref = O.forward(cfg, w, tk)
    eng = engine_for(cfg, w, torch.bfloat16, max_tokens=1280, slots=2)
    poison(eng)
    got = run_cut(eng, "a", tk, [1100, 1])
    assert close(got, ref, torch.bfloat16)


@pytest.mark.parametrize("window,keep,ctx,n", [(4500, 0, 5000, 1), (3000, 6, 5000, 1), (4097, 2, 4990, 11)])
def test_needle_at_window_edges_in_a_long_context_with_many_key_splits(window, keep, ctx, n):
    last = ctx + n - 1
    for needle, seen in ((last - window + 1, True), (last - window, False), (keep - 1, True), (keep, False)):
        if needle < 0:
            continue
        got, ref = _needle_case(window, keep, ctx, n, needle, dim=64, vdim=64)
        assert rel_err(got, ref) < 1e-4, (needle, seen)
        assert bool(got[-1].abs().max() > 25.0) == seen, (needle, seen)
