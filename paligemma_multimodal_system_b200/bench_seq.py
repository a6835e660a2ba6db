"""`bench.py --arch mapedra`: prefill and decode throughput of the Mapedra decoder at layer sizes of a real model (random
weights), beside the Gemma decoder of this package at equal width / heads / feed-forward / depth, plus a per-kernel table
(CUDA events, L2 flushed between launches) with each kernel's distance from its roofline and the like kernel of Gemma.

Rooflines use MEASURED_PEAKS.json (copy bandwidth, cuBLAS bf16 burst rate) when present.  Matrix products are the same
tcgen05 kernels in both models and are not listed again.
"""
import json
import os
import time

import torch

from . import _lib, seq_ops
from .cache import SequenceStore
from .engine import SequenceEngine
from .modeling_gemma import PAGE, GemmaConfig, GemmaForCausalLM, KVCache
from .modeling_mapedra import MapedraConfig, MapedraForCausalLM

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        p = json.load(open(path))
        return float(p["hbm_gbs"]) * 1e9, float(p["bf16_tflops"]) * 1e12, "measured"
    return 6650e9, 1590e12, "fallback"


def mapedra_config(width, heads, kv_heads, dim, ff, vocab, layers, every=4):
    """`every`-th layer softmax attention, the others lightning; feed-forward on every layer; a 64-wide token side table."""
    ls = []
    for i in range(layers):
        mlp = {"kind": "dense", "ff": ff}
        if (i + 1) % every == 0:
            ls.append({"type": "attention", "mlp": mlp,
                       "mixer": {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": dim, "scale": dim ** -0.5, "softcap": 50.0,
                                 "rot": {"base": 1e6, "dims": dim // 2, "scaling": {"factor": 8.0, "low": 1.0, "high": 4.0, "original": 8192}}}})
        else:
            ls.append({"type": "lightning", "mlp": mlp,
                       "mixer": {"heads": heads, "dim": dim, "vdim": dim, "decay": [1.0 - 2.0 ** (-5 - 3 * h / heads) for h in range(heads)]}})
    return {"architecture": "Mapedra", "vocab": vocab, "width": width, "embedding": {"scale": width ** 0.5}, "norm": {"eps": 1e-6, "groups": 4},
            "token_side": {"dim": 64}, "layers": ls}


def random_mapedra(cfg, seed=0):
    g = torch.Generator(device="cuda").manual_seed(seed)
    c = MapedraConfig(cfg)
    model = MapedraForCausalLM(c, torch.bfloat16)
    shapes = {}

    def take(name, shape):
        shapes[name] = shape
        std = 1.0 if len(shape) == 1 else shape[-1] ** -0.5
        t = torch.randn(*shape, device="cuda", generator=g) * std
        return (t + 1.0 if len(shape) == 1 else t).to(torch.bfloat16)

    model.embed = take("embed", (c.vocab, c.width)) * 0.05
    model.side_embed = take("side.embed", (c.vocab, c.side_dim * len(c.layers))) if c.side_dim else None
    for blk in model.blocks:
        blk.load(take)
    model.final_norm, model.head = take("final.norm", (c.width,)), take("head", (c.vocab, c.width))
    model.pack()
    return model


def timed(fn, iters=5, warmup=2, flush=None):
    """Median device time of fn() in seconds; `flush` (a > L2 buffer) is rewritten before every timed launch."""
    for _ in range(warmup):
        fn()
    ts = []
    for _ in range(iters):
        if flush is not None:
            flush.add_(1)
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        a.record()
        fn()
        b.record()
        torch.cuda.synchronize()
        ts.append(a.elapsed_time(b) * 1e-3)
    return sorted(ts)[len(ts) // 2]


def run(args):
    _lib.require_device()
    torch.cuda.set_device(0)
    hbm, tflops, src = peaks()
    W, H, G, dh, F, V, L = args.width, args.heads, args.kv_heads, args.head_dim, args.ff, args.vocab, args.layers
    B_pre, S, B_dec, ctx = args.prefill_batch, args.seq_len, args.decode_batch, args.context
    flush = torch.zeros(64 * 1024 * 1024, device="cuda", dtype=torch.float32)  # 256 MB > L2
    out = {"metric": "mapedra_vs_gemma_tokens_per_s", "dtype": "bf16", "data": "synthetic", "peaks": src,
           "config": {"width": W, "heads": H, "kv_heads": G, "head_dim": dh, "ff": F, "vocab": V, "layers": L, "prefill": [B_pre, S],
                      "decode": [B_dec, ctx], "l2": "256 MB buffer rewritten before every timed launch"}}

    # ---------------------------------------------------------------- Mapedra end to end
    cfg = mapedra_config(W, H, G, dh, F, V, L)
    model = random_mapedra(cfg)
    n_att = sum(l["type"] == "attention" for l in cfg["layers"])
    eng = SequenceEngine(model, max_tokens=max(B_pre * S, B_dec * (ctx + PAGE)) + PAGE, num_slots=max(B_pre, B_dec))
    gen = torch.Generator().manual_seed(1)
    prompts = [torch.randint(0, V, (S,), generator=gen).tolist() for _ in range(B_pre)]

    def prefill():
        eng.step([(i, p, [S - 1]) for i, p in enumerate(prompts)], list(range(B_pre)))

    t = timed(prefill, iters=args.steps, warmup=args.warmup, flush=flush)
    out["mapedra_prefill_tok_s"] = B_pre * S / t
    # decode: B_dec sequences with `ctx` tokens each, then single-token steps
    long = [torch.randint(0, V, (ctx,), generator=gen).tolist() for _ in range(B_dec)]
    for i0 in range(0, B_dec, 8):
        eng.step([(("d", i), long[i], []) for i in range(i0, min(B_dec, i0 + 8))])

    def decode():
        eng.step([(("d", i), [7], [0]) for i in range(B_dec)])

    t = timed(decode, iters=max(args.steps, 8), warmup=args.warmup, flush=flush)
    out["mapedra_decode_tok_s"] = B_dec / t
    out["mapedra_decode_ms_per_step"] = t * 1e3
    for i in range(B_dec):
        eng.release(("d", i))

    # ---------------------------------------------------------------- Mapedra kernels
    prec, k = model.prec, {}
    att = next(b.mixer for b in model.blocks if hasattr(b.mixer, "G"))
    lin = next(b.mixer for b in model.blocks if hasattr(b.mixer, "decay"))
    li_att = next(i for i, b in enumerate(model.blocks) if hasattr(b.mixer, "G"))
    li_lin = next(i for i, b in enumerate(model.blocks) if hasattr(b.mixer, "decay"))
    store = eng.store

    def entries(n_seq, n_new, c0):
        es = []
        for i in range(n_seq):
            store.admit(("k", i))
            rec = store.reserve(("k", i), c0 + n_new)
            es.append(dict(tokens=[1] * n_new, ctx=c0, slot=rec.slot, pages=rec.pages))
        b = seq_ops.make_step_batch(es)
        return b

    def drop(n_seq):
        for i in range(n_seq):
            store.release(("k", i))

    for name, (n_seq, n_new, c0) in {"prefill": (B_pre, S, 0), "decode": (B_dec, 1, ctx)}.items():
        b = entries(n_seq, n_new, c0)
        T = b.T
        proj = torch.randn(T, att.w_in.shape[0], device="cuda").to(torch.bfloat16)
        q, o = prec.empty(T, H * dh), prec.empty(T, H * dh)
        kp, vp = store.k_pages[li_att], store.v_pages[li_att]
        kp.normal_()
        vp.normal_()
        gate = proj[:, (H + G) * dh + G * dh:]
        k[f"attn_prepare_{name}"] = dict(
            s=timed(lambda: seq_ops.attn_prepare(proj, b, att.freq_d, att.qn, att.kn, q, kp, vp, H, G, dh, dh, att.rot_dims, 1e-6, PAGE), flush=flush),
            bytes=T * (H + 2 * G) * dh * 2 * 2)
        pairs = n_seq * (n_new * c0 + n_new * (n_new + 1) // 2)
        k[f"attention_{name}"] = dict(
            s=timed(lambda: seq_ops.attn_ragged(q, kp, vp, gate, o, b, H, G, dh, dh, att.scale, att.softcap, PAGE), flush=flush),
            flops=4 * dh * H * pairs, bytes=n_seq * (c0 + n_new) * G * 2 * dh * 2 + 3 * T * H * dh * 2)
        projl = torch.randn(T, lin.w_in.shape[0], device="cuda").to(torch.bfloat16)
        ol = torch.empty(T, H * dh, device="cuda", dtype=torch.float32)
        k[f"lightning_{name}"] = dict(
            s=timed(lambda: seq_ops.linear_attn(projl, store.state[li_lin], lin.decay_d, ol, b, H, dh, dh), flush=flush),
            flops=T * H * 2 * (32 * dh + 32 * dh + 2 * dh * dh) if n_new > 1 else T * H * 4 * dh * dh,
            bytes=n_seq * H * dh * dh * 4 * 2 + T * H * dh * (3 * 2 + 4))
        attl = prec.empty(T, H * dh)
        k[f"lightning_norm_gate_{name}"] = dict(
            s=timed(lambda: seq_ops.rmsnorm_gate(ol, lin.norm, projl[:, 3 * H * dh:], attl, 1e-6), flush=flush), bytes=T * H * dh * (4 + 2 + 2))
        y, x, xa = torch.randn(T, W, device="cuda"), torch.randn(T, W, device="cuda"), prec.empty(T, W)
        w1 = torch.ones(W, device="cuda")
        k[f"group_norm_residual_{name}"] = dict(s=timed(lambda: seq_ops.group_rmsnorm_add(y, w1, x, xa, 4, 1e-6), flush=flush), bytes=T * W * (4 + 4 + 4 + 2))
        drop(n_seq)
    del eng, model, store
    torch.cuda.empty_cache()

    # ---------------------------------------------------------------- Gemma at equal size
    gc = GemmaConfig(hidden_size=W, intermediate_size=F, num_hidden_layers=L, num_attention_heads=H, num_key_value_heads=G, head_dim=dh,
                     vocab_size=V, rms_norm_eps=1e-6)
    gm = GemmaForCausalLM(gc, device="cuda", dtype=torch.bfloat16).eval()
    with torch.no_grad():
        for p in gm.parameters():
            if p.dim() == 2:
                p.normal_(0, p.shape[1] ** -0.5)
    gm.pack()
    L_ = _lib.lib()
    pos = torch.arange(S, device="cuda", dtype=torch.int32).repeat(B_pre)

    def g_prefill():
        h = torch.randn(B_pre * S, W, device="cuda")
        kv = KVCache()
        gm.prefill(h, pos, B_pre, S, kv, last_only=True)

    t = timed(g_prefill, iters=args.steps, warmup=args.warmup, flush=flush)
    out["gemma_prefill_tok_s"] = B_pre * S / t
    kv = KVCache()
    kv.allocate(B_dec, L, G, dh, ctx + PAGE)
    kv.k_pages.normal_()
    kv.v_pages.normal_()
    kv._set_len(ctx, L)
    kv.counters[0].fill_(ctx)
    kv.counters[1].fill_(ctx)
    kv.counters[2].fill_(ctx + 1)
    bufs = gm.decode_buffers(B_dec, private=True)

    def g_decode():
        bufs["h"].normal_()
        gm.decode_layers(bufs, kv, B_dec)

    t = timed(g_decode, iters=max(args.steps, 8), warmup=args.warmup, flush=flush)
    out["gemma_decode_tok_s"] = B_dec / t
    out["gemma_decode_ms_per_step"] = t * 1e3
    # Gemma kernels
    T = B_pre * S
    Wq = (H + 2 * G) * dh
    qkv = torch.randn(T, Wq, device="cuda").to(torch.bfloat16)
    qb, kb, vb = qkv, qkv[:, H * dh:], qkv[:, (H + G) * dh:]
    ao = torch.empty(T, H * dh, device="cuda", dtype=torch.bfloat16)
    Gq = H // G
    k["gemma_attention_prefill"] = dict(
        s=timed(lambda: _lib.check(L_.pg_attention_prefill(qb.data_ptr(), kb.data_ptr(), vb.data_ptr(), ao.data_ptr(), B_pre, G, S * Gq, S, dh, Gq,
                                                          S * Wq, Wq, dh, Gq * dh, S * Wq, Wq, dh, S * H * dh, H * dh, dh, Gq * dh, dh ** -0.5,
                                                          _lib.stream()), "attn"), flush=flush),
        flops=4 * dh * H * B_pre * S * S, bytes=T * Wq * 2 + T * H * dh * 2)
    qkvf = torch.randn(B_dec, Wq, device="cuda")
    ad = torch.empty(B_dec, H * dh, device="cuda", dtype=torch.bfloat16)
    k["gemma_attention_decode"] = dict(
        s=timed(lambda: _lib.check(L_.pg_attention_decode_fused(qkvf.data_ptr(), kv.counters[0].data_ptr(), kv.counters[2].data_ptr(),
                                                               gm._packed["inv_freq"].data_ptr(), kv.k_pages[0].data_ptr(), kv.v_pages[0].data_ptr(),
                                                               kv.page_table.data_ptr(), ad.data_ptr(), B_dec, H, G, dh, PAGE, kv.k_pages.shape[1],
                                                               kv.page_table.shape[1], dh ** -0.5, _lib.stream()), "attn_dec"), flush=flush),
        bytes=B_dec * (ctx + 1) * G * 2 * dh * 2)
    for name, rows in (("prefill", T), ("decode", B_dec)):
        hx, hn = torch.randn(rows, W, device="cuda"), torch.empty(rows, W, device="cuda", dtype=torch.bfloat16)
        w1 = torch.zeros(W, device="cuda")
        k[f"gemma_rmsnorm_{name}"] = dict(s=timed(lambda: _lib.rmsnorm(hx, w1, hn), flush=flush), bytes=rows * W * 6)
    for name, d in k.items():
        d["us"] = round(d.pop("s") * 1e6, 2)
        if "bytes" in d:
            d["hbm_frac"] = round(d["bytes"] / (d["us"] * 1e-6) / hbm, 4)
        if "flops" in d:
            d["tflops"] = round(d["flops"] / (d["us"] * 1e-6) / 1e12, 2)
            d["tensor_frac"] = round(d["flops"] / (d["us"] * 1e-6) / tflops, 5)
    out["kernels"] = k
    out["value"] = out["mapedra_decode_tok_s"]
    out["unit"] = "tokens/s"
    out["n_gpus"] = 1
    for key in list(out):
        if key.endswith("tok_s"):
            out[key] = round(out[key], 1)
    print(json.dumps(out), flush=True)
    return out


# ----------------------------------------------------------------------------------------------------------------------
# `bench.py --arch pukerax`: the Pukerax decoder beside the Mapedra decoder (the closest model of the package: same engine, same
# ragged step, softmax attention over pages) at equal width / heads / feed-forward / depth
# ----------------------------------------------------------------------------------------------------------------------
def pukerax_config(width, heads, ff, vocab, layers, streams=4, experts=14, top=4):
    """Latent attention with 64 plain + 32 rotated query / key dimensions per head, values of 64, a kv latent of 256 and a q
    latent of 768; the first layer's feed-forward dense, the others routed (expert width ff / 8, shared expert ff / 4, two
    identity outputs, four groups of which two are kept)."""
    mixer = {"heads": heads, "dim": 64, "rot_dim": 32, "vdim": 64, "kv_rank": 256, "q_rank": 768, "rot": {"base": 1e6, "dims": 32}, "scale": 96 ** -0.5}
    ls = []
    for i in range(layers):
        if i == 0:
            mlp = {"kind": "dense", "ff": ff}
        else:
            mlp = {"kind": "moe", "expert": {"ff": ff // 8}, "shared": {"ff": ff // 4},
                   "router": {"experts": experts, "identity": 2, "top": top, "scale": 2.5, "groups": {"count": 4, "keep": 2}}}
        ls.append({"type": "latent_attention", "mixer": dict(mixer), "mlp": mlp})
    return {"architecture": "Pukerax", "vocab": vocab, "width": width, "norm": {"eps": 1e-6}, "streams": streams, "layers": ls}


def random_pukerax(cfg, seed=0):
    from .modeling_pukerax import PukeraxConfig, PukeraxForCausalLM
    g = torch.Generator(device="cuda").manual_seed(seed)
    c = PukeraxConfig(cfg)
    model = PukeraxForCausalLM(c, torch.bfloat16)

    def take(name, shape):
        if name.endswith(("norm1", "norm2", "final.norm", "correction")):
            t = torch.randn(*shape, device="cuda", generator=g) * 0.05
        elif name.endswith(("dq.norm", "dkv.norm")):
            t = 1.0 + torch.randn(*shape, device="cuda", generator=g) * 0.05
        elif name.endswith(".in"):
            t = torch.full(shape, 1.0 / c.streams, device="cuda")
        elif name.endswith(".out"):
            t = torch.ones(*shape, device="cuda")
        elif name.endswith(".mix"):
            t = torch.eye(shape[0], device="cuda") + 0.05 * torch.randn(*shape, device="cuda", generator=g)
        else:
            t = torch.randn(*shape, device="cuda", generator=g) * shape[-1] ** -0.5
        return t.to(torch.bfloat16)

    model.embed = take("embed", (c.vocab, c.width))
    for blk in model.blocks:
        blk.load(take)
    model.final_norm, model.head = take("final.norm", (c.width,)), take("head", (c.vocab, c.width))
    model.pack()
    return model


def _throughput(model, args, flush, V, tag, out):
    B_pre, S, B_dec, ctx = args.prefill_batch, args.seq_len, args.decode_batch, args.context
    eng = SequenceEngine(model, max_tokens=max(B_pre * S, B_dec * (ctx + PAGE)) + PAGE, num_slots=max(B_pre, B_dec))
    gen = torch.Generator().manual_seed(1)
    prompts = [torch.randint(0, V, (S,), generator=gen).tolist() for _ in range(B_pre)]
    t = timed(lambda: eng.step([(i, p, [S - 1]) for i, p in enumerate(prompts)], list(range(B_pre))), iters=args.steps, warmup=args.warmup, flush=flush)
    out[f"{tag}_prefill_tok_s"] = B_pre * S / t
    long = [torch.randint(0, V, (ctx,), generator=gen).tolist() for _ in range(B_dec)]
    for i0 in range(0, B_dec, 8):
        eng.step([(("d", i), long[i], []) for i in range(i0, min(B_dec, i0 + 8))])
    t = timed(lambda: eng.step([(("d", i), [7], [0]) for i in range(B_dec)]), iters=max(args.steps, 8), warmup=args.warmup, flush=flush)
    out[f"{tag}_decode_tok_s"] = B_dec / t
    out[f"{tag}_decode_ms_per_step"] = t * 1e3
    for i in range(B_dec):
        eng.release(("d", i))
    return eng


def _entries(store, n_seq, n_new, c0):
    es = []
    for i in range(n_seq):
        store.admit(("k", i))
        rec = store.reserve(("k", i), c0 + n_new)
        es.append(dict(tokens=[1] * n_new, ctx=c0, slot=rec.slot, pages=rec.pages))
    return seq_ops.make_step_batch(es)


def run_pukerax(args):
    _lib.require_device()
    torch.cuda.set_device(0)
    hbm, tflops, src = peaks()
    W, H, F, V, L = args.width, args.heads, args.ff, args.vocab, args.layers
    B_pre, S, B_dec, ctx = args.prefill_batch, args.seq_len, args.decode_batch, args.context
    flush = torch.zeros(64 * 1024 * 1024, device="cuda", dtype=torch.float32)  # 256 MB > L2
    cfg = pukerax_config(W, H, F, V, L)
    m0 = cfg["layers"][0]["mixer"]
    out = {"metric": "pukerax_vs_mapedra_tokens_per_s", "dtype": "bf16", "data": "synthetic", "peaks": src,
           "config": {"width": W, "heads": H, "latent": {k: m0[k] for k in ("dim", "rot_dim", "vdim", "kv_rank", "q_rank")}, "ff": F, "vocab": V,
                      "layers": L, "streams": cfg["streams"], "router": cfg["layers"][-1]["mlp"]["router"] if L > 1 else None,
                      "prefill": [B_pre, S], "decode": [B_dec, ctx], "l2": "256 MB buffer rewritten before every timed launch"}}
    model = random_pukerax(cfg)
    eng = _throughput(model, args, flush, V, "pukerax", out)

    # ---------------------------------------------------------------- Pukerax kernels
    prec, k, store = model.prec, {}, eng.store
    mix = model.blocks[0].mixer
    dim, rot, vdim, R, Q = mix.dim, mix.rot, mix.vdim, mix.R, mix.Q
    kd = R + rot
    Sn = cfg["streams"]
    ff = next((b.ff for b in model.blocks if hasattr(b.ff, "n_real")), None)
    for name, (n_seq, n_new, c0) in {"prefill": (B_pre, S, 0), "decode": (B_dec, 1, ctx)}.items():
        b = _entries(store, n_seq, n_new, c0)
        T = b.T
        pages = store.k_pages[0]
        pages.normal_()
        xs, y, ha = torch.randn(T, Sn, W, device="cuda"), torch.randn(T, W, device="cuda"), prec.empty(T, W)
        hc, nw = model.blocks[0].hc1, model.blocks[0].norm1_d
        k[f"stream_mix_norm_{name}"] = dict(s=timed(lambda: seq_ops.stream_mix_norm(xs, y, hc.mix, hc.write, read=hc.read, norm_w=nw, out_act=ha), flush=flush),
                                            bytes=T * W * (2 * Sn * 4 + 4 + 2))
        proj = torch.randn(T, mix.w_in.shape[0], device="cuda").to(torch.bfloat16)
        cq = prec.empty(T, Q)
        k[f"latent_prepare_{name}"] = dict(
            s=timed(lambda: seq_ops.latent_prepare(proj, b, mix.freq_d, mix.qn, mix.cn, cq, pages, Q, R, rot, mix.rot_dims, 1e-6, PAGE), flush=flush),
            bytes=T * (Q + kd) * 2 * 2)
        q = torch.randn(T, H, dim + rot, device="cuda").to(torch.bfloat16)
        gate = proj[:, Q + kd:]
        att = prec.empty(T, H, vdim)
        pairs = n_seq * (n_new * c0 + n_new * (n_new + 1) // 2)
        if name == "prefill":
            k["latent_expand_prefill"] = dict(s=timed(lambda: seq_ops.latent_expand(pages, b, mix.w_ukv, H, dim, rot, vdim, R, PAGE, prec), flush=flush),
                                              flops=2 * T * R * H * (dim + vdim), bytes=T * (kd * 2 + 2 * H * (dim + vdim) * 2 + H * (dim + rot + vdim) * 2))
            kx, vx = seq_ops.latent_expand(pages, b, mix.w_ukv, H, dim, rot, vdim, R, PAGE, prec)
            k["attention_prefill"] = dict(
                s=timed(lambda: seq_ops.attn_ragged(q.view(T, -1), kx, vx, gate, att.view(T, -1), seq_ops.dense_view(b), H, H, dim + rot, vdim, mix.scale, 0.0,
                                                    PAGE, gate_per_head=True, skip_singles=True), flush=flush),
                flops=2 * (dim + rot + vdim) * H * pairs, bytes=T * H * (2 * (dim + rot) + 2 * vdim) * 2)
        else:
            qlat, olat = prec.empty(T, H, kd), prec.empty(T, H, R)
            k["absorb_query_decode"] = dict(s=timed(lambda: seq_ops.linear_batched(q[:, :, :dim], mix.w_ukT, qlat[:, :, :R]), flush=flush),
                                            bytes=H * R * dim * 2 + T * H * (dim + R) * 2)
            k["attention_decode"] = dict(
                s=timed(lambda: seq_ops.attn_ragged(qlat.view(T, -1), pages, pages, gate, olat.view(T, -1), b, H, 1, kd, R, mix.scale, 0.0, PAGE, krow=kd, vrow=kd,
                                                    gate_per_head=True), flush=flush),
                flops=2 * (kd + R) * H * pairs, bytes=n_seq * (c0 + 1) * kd * 2 + T * H * (kd + R) * 2)
            k["value_up_decode"] = dict(s=timed(lambda: seq_ops.linear_batched(olat, mix.w_uv, att), flush=flush), bytes=H * R * vdim * 2 + T * H * (vdim + R) * 2)
        if ff is not None:
            h = torch.randn(T, W, device="cuda").to(torch.bfloat16)
            z = torch.randn(T, ff.n_all, device="cuda")

            def route():
                ids, wts, counts = seq_ops.moe_route(z, ff.correction, ff.n_real, ff.top, ff.group_count, ff.group_keep, ff.scale)
                return ids, wts, seq_ops.MoePlan(ids, counts, ff.n_real)

            k[f"moe_route_plan_{name}"] = dict(s=timed(route, flush=flush), bytes=T * (ff.n_all * 4 + ff.top * 16))
            ids, wts, plan = route()
            counts = seq_ops.moe_route(z, ff.correction, ff.n_real, ff.top, ff.group_count, ff.group_keep, ff.scale)[2]
            real = int((ids < ff.n_real).sum())
            wbytes = 2 * ff.n_real * ff.F * W * 2
            # the path the model takes at this size (prompt: one dense run per expert on tcgen05; decode: the grouped kernel)
            k[f"moe_expert_products_{name}"] = dict(s=timed(lambda: ff.expert_products(h, plan, counts, prec), flush=flush), flops=4 * real * ff.F * W,
                                                    bytes=wbytes + real * (W * 2 + ff.F * 4 + W * 4))
            if name == "prefill":
                mid, eo2 = prec.empty(plan.pairs, ff.F), torch.empty(plan.pairs, W, device="cuda", dtype=torch.float32)
                k["moe_grouped_kernel_prefill"] = dict(
                    s=timed(lambda: (seq_ops.moe_gemm(h, plan, ff.w_up, mid, gather=True, act=seq_ops.ACT_RELU2), seq_ops.moe_gemm(mid, plan, ff.w_down, eo2, gather=False)),
                            flush=flush), flops=4 * real * ff.F * W)
            eo = ff.expert_products(h, plan, counts, prec)
            yy = torch.empty(T, W, device="cuda")
            k[f"moe_combine_{name}"] = dict(s=timed(lambda: seq_ops.moe_combine(eo, plan, ids, wts, h, y, yy), flush=flush), bytes=T * W * (ff.top * 4 + 4 + 4 + 2))
        for i in range(n_seq):
            store.release(("k", i))
    del eng, model, store
    torch.cuda.empty_cache()

    # ---------------------------------------------------------------- Mapedra (softmax attention on every layer) at equal size
    mc = mapedra_config(W, H, 8, 64, F, V, L, every=1)
    mm = random_mapedra(mc)
    eng = _throughput(mm, args, flush, V, "mapedra", out)
    store, prec = eng.store, mm.prec
    att_m = mm.blocks[0].mixer
    G, dh = att_m.G, att_m.dim
    for name, (n_seq, n_new, c0) in {"prefill": (B_pre, S, 0), "decode": (B_dec, 1, ctx)}.items():
        b = _entries(store, n_seq, n_new, c0)
        T = b.T
        proj = torch.randn(T, att_m.w_in.shape[0], device="cuda").to(torch.bfloat16)
        q, o = prec.empty(T, H * dh), prec.empty(T, H * dh)
        kp, vp = store.k_pages[0], store.v_pages[0]
        kp.normal_()
        vp.normal_()
        gate = proj[:, (H + G) * dh + G * dh:]
        k[f"mapedra_attn_prepare_{name}"] = dict(
            s=timed(lambda: seq_ops.attn_prepare(proj, b, att_m.freq_d, att_m.qn, att_m.kn, q, kp, vp, H, G, dh, dh, att_m.rot_dims, 1e-6, PAGE), flush=flush),
            bytes=T * (H + 2 * G) * dh * 2 * 2)
        pairs = n_seq * (n_new * c0 + n_new * (n_new + 1) // 2)
        k[f"mapedra_attention_{name}"] = dict(
            s=timed(lambda: seq_ops.attn_ragged(q, kp, vp, gate, o, b, H, G, dh, dh, att_m.scale, att_m.softcap, PAGE), flush=flush),
            flops=4 * dh * H * pairs, bytes=n_seq * (c0 + n_new) * G * 2 * dh * 2 + 3 * T * H * dh * 2)
        y, x, xa = torch.randn(T, W, device="cuda"), torch.randn(T, W, device="cuda"), prec.empty(T, W)
        w1 = torch.ones(W, device="cuda")
        k[f"mapedra_group_norm_residual_{name}"] = dict(s=timed(lambda: seq_ops.group_rmsnorm_add(y, w1, x, xa, 4, 1e-6), flush=flush), bytes=T * W * (4 + 4 + 4 + 2))
        for i in range(n_seq):
            store.release(("k", i))
    for name, d in k.items():
        d["us"] = round(d.pop("s") * 1e6, 2)
        if "bytes" in d:
            d["hbm_frac"] = round(d["bytes"] / (d["us"] * 1e-6) / hbm, 4)
        if "flops" in d:
            d["tflops"] = round(d["flops"] / (d["us"] * 1e-6) / 1e12, 2)
            d["tensor_frac"] = round(d["flops"] / (d["us"] * 1e-6) / tflops, 5)
    out["kernels"] = k
    out["value"] = out["pukerax_decode_tok_s"]
    out["unit"] = "tokens/s"
    out["n_gpus"] = 1
    for key in list(out):
        if key.endswith("tok_s"):
            out[key] = round(out[key], 1)
    print(json.dumps(out), flush=True)
    return out


# ----------------------------------------------------------------------------------------------------------------------
# `bench.py --arch kovusun`: the Kovusun decoder beside the Mapedra decoder with softmax attention on every layer (the closest model
# of the package: same engine, grouped-query softmax attention over pages, gated feed-forward) at equal width / heads / k/v heads /
# feed-forward / depth; the routed experts beside the grouped kernel as Pukerax's squared-relu experts use it
# ----------------------------------------------------------------------------------------------------------------------
def kovusun_config(width, heads, kv_heads, dim, ff, vocab, layers, experts=14, top=4):
    """Layer types in turn: sink + gate attention (window 1024), rotated attention with kept first tokens (window 2048), biased
    attention with the distance penalty (window 512), and a layer that borrows the previous layer's keys / values (window 256).
    The first layer's feed-forward is dense (clamped gated unit), the others routed (expert width ff / 8, shared expert ff / 4)."""
    base = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": dim, "scale": dim ** -0.5}
    ls = []
    for i in range(layers):
        mlp = {"kind": "dense", "ff": ff, "limit": 7.0} if i == 0 else {"kind": "moe", "expert": {"ff": ff // 8}, "shared": {"ff": ff // 4},
                                                                        "router": {"experts": experts, "top": top}}
        k = i % 4
        if k == 0:
            ls.append({"type": "attention_2", "mixer": dict(base, mask={"size": 1024}), "mlp": mlp})
        elif k == 1:
            ls.append({"type": "attention_3", "mixer": dict(base, mask={"size": 2048, "keep_first": 4}, rot={"base": 1e6, "dims": dim}), "mlp": mlp})
        elif k == 2:
            ls.append({"type": "attention", "mixer": dict(base, mask={"size": 512}), "mlp": mlp})
        else:
            ls.append({"type": "attention", "mixer": dict(base, mask={"size": 256}, kv_from=i - 1), "mlp": mlp})
    return {"architecture": "Kovusun", "vocab": vocab, "width": width, "norm": {"eps": 1e-5}, "layers": ls}


def random_kovusun(cfg, seed=0):
    from .modeling_kovusun import KovusunConfig, KovusunForCausalLM
    g = torch.Generator(device="cuda").manual_seed(seed)
    c = KovusunConfig(cfg)
    model = KovusunForCausalLM(c, torch.bfloat16)

    def take(name, shape):
        r = torch.randn(*shape, device="cuda", generator=g)
        if name.endswith(("norm1", "norm2", "final.norm")):
            t = 1.0 + 0.05 * r
        elif name.endswith("shift"):
            t = torch.rand(*shape, device="cuda", generator=g)
        elif name.endswith((".b", "sink")):
            t = 0.1 * r
        elif name.endswith(("r1", "r2", "temp")):
            t = 0.5 + torch.rand(*shape, device="cuda", generator=g)
        else:
            t = r * shape[-1] ** -0.5
        return t.to(torch.bfloat16)

    model.embed = take("embed", (c.vocab, c.width))
    for blk in model.blocks:
        blk.load(take, lambda name: name.endswith("shift"))
    model.final_norm, model.final_norm_b = take("final.norm", (c.width,)), take("final.norm.b", (c.width,))
    model.head = take("head", (c.vocab, c.width))
    model.pack()
    return model


def run_kovusun(args):
    _lib.require_device()
    torch.cuda.set_device(0)
    hbm, tflops, src = peaks()
    W, H, G, dh, F, V, L = args.width, args.heads, args.kv_heads, args.head_dim, args.ff, args.vocab, args.layers
    B_pre, S, B_dec, ctx = args.prefill_batch, args.seq_len, args.decode_batch, args.context
    flush = torch.zeros(64 * 1024 * 1024, device="cuda", dtype=torch.float32)  # 256 MB > L2
    cfg = kovusun_config(W, H, G, dh, F, V, L)
    out = {"metric": "kovusun_vs_mapedra_tokens_per_s", "dtype": "bf16", "data": "synthetic", "peaks": src,
           "config": {"width": W, "heads": H, "kv_heads": G, "head_dim": dh, "ff": F, "vocab": V, "layers": L,
                      "windows": [l["mixer"]["mask"] for l in cfg["layers"][:4]], "router": cfg["layers"][-1]["mlp"].get("router") if L > 1 else None,
                      "prefill": [B_pre, S], "decode": [B_dec, ctx], "l2": "256 MB buffer rewritten before every timed launch"}}
    model = random_kovusun(cfg)
    eng = _throughput(model, args, flush, V, "kovusun", out)

    # ---------------------------------------------------------------- Kovusun kernels
    prec, k, store = model.prec, {}, eng.store
    ff = next((b.ff for b in model.blocks if hasattr(b.ff, "n_real")), None)
    blk0 = model.blocks[0]
    for name, (n_seq, n_new, c0) in {"prefill": (B_pre, S, 0), "decode": (B_dec, 1, ctx)}.items():
        b = _entries(store, n_seq, n_new, c0)
        T = b.T
        x, a1, a2 = torch.randn(T, W, device="cuda"), prec.empty(T, W), prec.empty(T, W)
        k[f"two_norms_shift_{name}"] = dict(
            s=timed(lambda: seq_ops.layernorm_shift(x, blk0.norm1_d, blk0.norm1_bd, a1, 1e-5, shift=blk0.shift_d, state=store.state[L], b=b, w2=blk0.norm2_d,
                                                    b2=blk0.norm2_bd, out2=a2), flush=flush), bytes=T * W * (4 + 2 + 2))
        for li, blk in enumerate(model.blocks[:4]):
            mx = blk.mixer
            tag = cfg["layers"][li]["type"] + ("_borrowed" if mx.kv_from is not None else "")
            src_li = li if mx.kv_from is None else mx.kv_from
            kp, vp = store.k_pages[src_li], store.v_pages[src_li]
            kp.normal_()
            vp.normal_()
            proj = torch.randn(T, mx.w_in.shape[0], device="cuda").to(torch.bfloat16)
            q, o = prec.empty(T, H * dh), prec.empty(T, H * dh)
            own = mx.kv_from is None
            k[f"attn_prepare_{tag}_{name}"] = dict(
                s=timed(lambda: seq_ops.attn_prepare(proj, b, mx.freq_d, None, None, q, kp if own else None, vp if own else None, H, G, dh, dh, mx.rot_dims, 1e-5,
                                                     PAGE, norm_qk=mx.qk_norm, norm_v=False), flush=flush), bytes=T * (H + (2 * G if own else 0)) * dh * 2 * 2)
            win, keep = mx.window, mx.keep_first
            # (query, key) pairs inside the window (+ kept first keys) and the key rows a sequence's queries read
            if n_new > 1:
                pairs = n_seq * sum(min(i + 1, win) + max(0, min(keep, i + 1 - win)) for i in range(c0, c0 + n_new))
                keys_read = c0 + n_new
            else:
                pairs = n_seq * min(c0 + 1, win + keep)
                keys_read = min(c0 + 1, win + keep)
            gate = proj[:, mx.gate_col:] if mx.head_gate else None
            k[f"attention_{tag}_{name}"] = dict(
                s=timed(lambda: seq_ops.attn_ragged(q, kp, vp, gate, o, b, H, G, dh, dh, mx.scale, 0.0, PAGE, gate_per_head=True, score=mx.score), flush=flush),
                flops=4 * dh * H * pairs, bytes=n_seq * keys_read * G * 2 * dh * 2 + 2 * T * H * dh * 2)
        if ff is not None:
            h = torch.randn(T, W, device="cuda").to(torch.bfloat16)
            z = torch.randn(T, ff.w_router.shape[0], device="cuda")

            def route():
                ids, wts, counts = seq_ops.moe_route(z[:, :ff.n_all], None, ff.n_real, ff.top, 1, 1, 1.0, logit_bias=ff.router_b)
                return ids, wts, counts, seq_ops.MoePlan(ids, counts, ff.n_real)

            k[f"moe_route_plan_{name}"] = dict(s=timed(lambda: route(), flush=flush), bytes=T * (ff.n_all * 4 + ff.top * 16))
            ids, wts, counts, plan = route()
            wbytes = 3 * ff.n_real * ff.F * W * 2
            k[f"moe_expert_products_{name}"] = dict(s=timed(lambda: ff.expert_products(h, plan, counts, prec), flush=flush), flops=6 * plan.pairs * ff.F * W,
                                                    bytes=wbytes + plan.pairs * (W * 2 + ff.F * 4 + W * 4))
            # the same grouped kernel as squared-relu experts use it (one up projection of the same total width: 2 F rows)
            mid2 = prec.empty(plan.pairs, 2 * ff.F)
            eo2 = torch.empty(plan.pairs, W, device="cuda", dtype=torch.float32)
            w_dn2 = torch.randn(ff.n_real, W, 2 * ff.F, device="cuda").to(torch.bfloat16)
            k[f"moe_relu2_same_kernel_{name}"] = dict(
                s=timed(lambda: (seq_ops.moe_gemm(h, plan, ff.w_up, mid2, gather=True, act=seq_ops.ACT_RELU2), seq_ops.moe_gemm(mid2, plan, w_dn2, eo2, gather=False)),
                        flush=flush), flops=8 * plan.pairs * ff.F * W, bytes=4 * ff.n_real * ff.F * W * 2 + plan.pairs * (W * 2 + ff.F * 8 + W * 4))
            eo = ff.expert_products(h, plan, counts, prec)
            sh, xr = torch.randn(T, W, device="cuda"), torch.randn(T, W, device="cuda")
            k[f"moe_combine_residual_{name}"] = dict(
                s=timed(lambda: seq_ops.moe_combine(eo, plan, ids, wts, h, sh, xr, shared_gate=z[:, ff.n_all:ff.n_all + 1], accumulate=True), flush=flush),
                bytes=T * W * (ff.top * 4 + 4 + 4 + 4))
        dense_ff = blk0.ff
        if dense_ff is not None and hasattr(dense_ff, "limit"):
            h = torch.randn(T, W, device="cuda").to(torch.bfloat16)
            xr = torch.randn(T, W, device="cuda")
            k[f"clamped_glu_feed_forward_{name}"] = dict(s=timed(lambda: dense_ff(h, b, prec, resid=xr), flush=flush), flops=6 * T * W * dense_ff.F,
                                                         bytes=3 * W * dense_ff.F * 2 + T * (W * 2 + dense_ff.F * 4 + W * 8))
        for i in range(n_seq):
            store.release(("k", i))
    del eng, model, store
    torch.cuda.empty_cache()

    # ---------------------------------------------------------------- Mapedra (softmax attention on every layer) at equal size
    mc = mapedra_config(W, H, G, dh, F, V, L, every=1)
    mm = random_mapedra(mc)
    eng = _throughput(mm, args, flush, V, "mapedra", out)
    store, prec = eng.store, mm.prec
    att_m = mm.blocks[0].mixer
    ffm = mm.blocks[0].ff
    for name, (n_seq, n_new, c0) in {"prefill": (B_pre, S, 0), "decode": (B_dec, 1, ctx)}.items():
        b = _entries(store, n_seq, n_new, c0)
        T = b.T
        proj = torch.randn(T, att_m.w_in.shape[0], device="cuda").to(torch.bfloat16)
        q, o = prec.empty(T, H * dh), prec.empty(T, H * dh)
        kp, vp = store.k_pages[0], store.v_pages[0]
        kp.normal_()
        vp.normal_()
        gate = proj[:, (H + G) * dh + G * dh:]
        k[f"mapedra_attn_prepare_{name}"] = dict(
            s=timed(lambda: seq_ops.attn_prepare(proj, b, att_m.freq_d, att_m.qn, att_m.kn, q, kp, vp, H, G, dh, dh, att_m.rot_dims, 1e-6, PAGE), flush=flush),
            bytes=T * (H + 2 * G) * dh * 2 * 2)
        pairs = n_seq * (n_new * c0 + n_new * (n_new + 1) // 2)
        k[f"mapedra_attention_{name}"] = dict(
            s=timed(lambda: seq_ops.attn_ragged(q, kp, vp, gate, o, b, H, G, dh, dh, att_m.scale, att_m.softcap, PAGE), flush=flush),
            flops=4 * dh * H * pairs, bytes=n_seq * (c0 + n_new) * G * 2 * dh * 2 + 3 * T * H * dh * 2)
        y, x, xa = torch.randn(T, W, device="cuda"), torch.randn(T, W, device="cuda"), prec.empty(T, W)
        w1 = torch.ones(W, device="cuda")
        k[f"mapedra_group_norm_residual_{name}"] = dict(s=timed(lambda: seq_ops.group_rmsnorm_add(y, w1, x, xa, 4, 1e-6), flush=flush), bytes=T * W * (4 + 4 + 4 + 2))
        h = torch.randn(T, W, device="cuda").to(torch.bfloat16)
        k[f"mapedra_geglu_feed_forward_{name}"] = dict(s=timed(lambda: ffm(h, b, prec), flush=flush), flops=6 * T * W * ffm.F,
                                                       bytes=3 * W * ffm.F * 2 + T * (W * 2 + ffm.F * 4 + W * 4))
        for i in range(n_seq):
            store.release(("k", i))
    for name, d in k.items():
        d["us"] = round(d.pop("s") * 1e6, 2)
        if "bytes" in d:
            d["hbm_frac"] = round(d["bytes"] / (d["us"] * 1e-6) / hbm, 4)
        if "flops" in d:
            d["tflops"] = round(d["flops"] / (d["us"] * 1e-6) / 1e12, 2)
            d["tensor_frac"] = round(d["flops"] / (d["us"] * 1e-6) / tflops, 5)
    out["kernels"] = k
    out["value"] = out["kovusun_decode_tok_s"]
    out["unit"] = "tokens/s"
    out["n_gpus"] = 1
    for key in list(out):
        if key.endswith("tok_s"):
            out[key] = round(out[key], 1)
    print(json.dumps(out), flush=True)
    return out


# ----------------------------------------------------------------------------------------------------------------------
# `bench.py --arch zigivik`: the Zigivik decoder beside the Kovusun decoder with dense feed-forwards on every layer (the closest model
# of the package: parallel layers behind one norm kernel with a per-sequence state, windowed attention over pages, a feed-forward with
# biases that ends in the residual) at equal width / heads / k/v heads / feed-forward / depth
# ----------------------------------------------------------------------------------------------------------------------
def zigivik_config(width, heads, kv_heads, dim, ff, vocab, layers, taps=4):
    """Layer types in turn: latent attention (window 1024; 64 + 32-wide keys, 64-wide values, ranks width / 2 and width / 8), two layers of
    grouped attention whose keys are the values, and a latent layer that borrows the first one's cached rows (window 512).  At width 2048 a
    cached latent row is 256 + 32 wide, a size the tensor-core decode kernel of the absorbed form is built for."""
    lat = {"heads": heads, "dim": dim, "rot_dim": dim // 2, "vdim": dim, "q_rank": width // 2, "kv_rank": width // 8, "scale": (dim + dim // 2) ** -0.5,
           "rot": {"base": 5e5, "dims": dim // 2, "scaling": {"factor": 8.0, "original": 4096, "fast": 16.0, "slow": 1.0}}}
    att = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": dim, "scale": dim ** -0.5, "rot": {"base": 1e5, "dims": dim}}
    ls = []
    for i in range(layers):
        k = i % 4
        if k == 0:
            m = {"type": "latent_attention", "mixer": dict(lat, mask={"size": 1024})}
        elif k == 3:
            m = {"type": "latent_attention", "mixer": dict(lat, mask={"size": 512}, kv_from=i - 3)}
        else:
            m = {"type": "attention", "mixer": dict(att)}
        ls.append(dict(m, mlp={"kind": "dense", "ff": ff}))
    return {"architecture": "Zigivik", "vocab": vocab, "width": width, "norm": {"eps": 1e-6}, "canon": {"taps": taps}, "residual_mult": 0.5, "layers": ls}


def random_zigivik(cfg, seed=0):
    from .modeling_zigivik import ZigivikConfig, ZigivikForCausalLM
    g = torch.Generator(device="cuda").manual_seed(seed)
    c = ZigivikConfig(cfg)
    model = ZigivikForCausalLM(c, torch.bfloat16)

    def take(name, shape):
        r = torch.randn(tuple(shape), device="cuda", generator=g)
        if name.endswith(("norm1", ".norm")):
            t = 1.0 + 0.05 * r
        elif name.endswith(".b"):
            t = 0.1 * r
        elif name.endswith("canon1"):
            t = 0.2 * r
        elif name.endswith("act"):
            t = torch.tensor([0.6, 0.3, 0.2, 0.05], device="cuda")
        else:
            t = r * shape[-1] ** -0.5
        return t.to(torch.bfloat16)

    model.embed, model.embed_norm = take("embed", (c.vocab, c.width)), take("embed.norm", ())
    for blk in model.blocks:
        blk.load(take)
    model.final_norm, model.head = take("final.norm", ()), take("head", (c.vocab, c.width))
    model.pack()
    return model


def kovusun_dense_config(width, heads, kv_heads, dim, ff, vocab, layers):
    cfg = kovusun_config(width, heads, kv_heads, dim, ff, vocab, layers)
    for l in cfg["layers"]:
        l["mlp"] = {"kind": "dense", "ff": ff, "limit": 7.0}
    return cfg


def run_zigivik(args):
    _lib.require_device()
    torch.cuda.set_device(0)
    hbm, tflops, src = peaks()
    W, H, G, dh, F, V, L = args.width, args.heads, args.kv_heads, args.head_dim, args.ff, args.vocab, args.layers
    B_pre, S, B_dec, ctx = args.prefill_batch, args.seq_len, args.decode_batch, args.context
    flush = torch.zeros(64 * 1024 * 1024, device="cuda", dtype=torch.float32)  # 256 MB > L2
    cfg = zigivik_config(W, H, G, dh, F, V, L)
    out = {"metric": "zigivik_vs_kovusun_tokens_per_s", "dtype": "bf16", "data": "synthetic", "peaks": src,
           "config": {"width": W, "heads": H, "kv_heads": G, "head_dim": dh, "ff": F, "vocab": V, "layers": L, "taps": cfg["canon"]["taps"],
                      "latent": {k: cfg["layers"][0]["mixer"][k] for k in ("dim", "rot_dim", "vdim", "q_rank", "kv_rank")},
                      "windows": [(l["mixer"].get("mask") or {}).get("size") for l in cfg["layers"][:4]],
                      "prefill": [B_pre, S], "decode": [B_dec, ctx], "l2": "256 MB buffer rewritten before every timed launch"}}
    model = random_zigivik(cfg)
    eng = _throughput(model, args, flush, V, "zigivik", out)
    prec, k, store = model.prec, {}, eng.store
    # the like kernel of the latent mixer: the same class as Pukerax uses it (no window, one gate per head, interleaved rotation), equal sizes
    from .mixers import LatentAttention
    lm = cfg["layers"][0]["mixer"]
    plain = LatentAttention(W, H, lm["dim"], lm["rot_dim"], lm["vdim"], lm["q_rank"], lm["kv_rank"], lm["scale"], lm["rot_dim"], 1e6, 1e-6)
    gen = torch.Generator(device="cuda").manual_seed(5)
    plain.load(lambda name, shape: (torch.randn(tuple(shape), device="cuda", generator=gen) * shape[-1] ** -0.5 + (1.0 if len(shape) == 1 else 0.0)).to(torch.bfloat16), "")
    plain.pack(prec)
    for name, (n_seq, n_new, c0) in {"prefill": (B_pre, S, 0), "decode": (B_dec, 1, ctx)}.items():
        b = _entries(store, n_seq, n_new, c0)
        T = b.T
        blk0 = model.blocks[0]
        x, h, hc = torch.randn(T, W, device="cuda"), prec.empty(T, W), prec.empty(T, W)
        k[f"norm_convolution_{name}"] = dict(s=timed(lambda: seq_ops.rmsnorm_conv(x, blk0.norm1_d, h, hc, 1e-6, conv_w=blk0.canon_d, state=store.state[L], b=b),
                                                     flush=flush), bytes=T * W * (4 + 2 + 2))
        z = torch.randn(T, F, device="cuda").to(torch.bfloat16)
        k[f"polynomial_of_norms_{name}"] = dict(s=timed(lambda: seq_ops.polynorm(z, blk0.ff.coef, z, 1e-6), flush=flush), bytes=T * F * (2 + 2))
        hin = torch.randn(T, W, device="cuda").to(torch.bfloat16)
        k[f"feed_forward_{name}"] = dict(s=timed(lambda: blk0.ff(hin, b, prec, resid=x, resid_scale=0.5), flush=flush), flops=4 * T * W * F,
                                         bytes=2 * W * F * 2 + T * (W * 2 + F * 6 + W * 8))
        for li, blk in enumerate(model.blocks[:4]):
            mx = blk.mixer
            if li == 2:
                continue  # the same kind as layer 1
            tag = cfg["layers"][li]["type"] + ("_borrowed" if mx.kv_from is not None else "")
            src_li = li if mx.kv_from is None else mx.kv_from
            store.k_pages[src_li].normal_()
            if store.v_pages[src_li] is not None:
                store.v_pages[src_li].normal_()
            win = mx.window or (c0 + n_new)
            pairs = n_seq * sum(min(i + 1, win) for i in range(c0, c0 + n_new))
            if tag.startswith("latent"):
                kd, R = mx.R + mx.rot, mx.R
                wts = (mx.w_in.numel() + mx.w_uq.numel() + mx.w_ukv.numel() + mx.w_o.numel()) * 2
                # explicit heads for prompt portions, absorbed heads for decoded tokens
                fl = 2 * T * W * mx.w_in.shape[0] + 2 * T * mx.Q * H * (dh + mx.rot) + 2 * T * H * dh * W
                fl += (4 * H * (dh + mx.rot // 2) * pairs + 2 * n_seq * (c0 + n_new) * R * H * 2 * dh) if n_new > 1 else (2 * H * (kd + R) * pairs + 4 * T * H * dh * R)
                by = wts + n_seq * min(c0 + n_new, win + n_new) * kd * 2 + T * W * (2 + 8)
            else:
                wts = (mx.w_in.numel() + mx.w_o.numel()) * 2
                fl = 2 * T * W * mx.w_in.shape[0] + 2 * T * H * dh * W + 4 * dh * H * pairs
                by = wts + n_seq * (c0 + n_new) * G * 2 * dh * 2 + T * W * (2 + 8)
            k[f"mixer_{tag}_{name}"] = dict(s=timed(lambda: mx(hin, b, store, li, prec, resid=x, resid_scale=0.5), flush=flush), flops=fl, bytes=by)
            if li == 0:  # the plain latent mixer over the same pages: every key is visible
                allp = n_seq * sum(i + 1 for i in range(c0, c0 + n_new))
                fl_p = fl + ((4 * H * (dh + mx.rot // 2) * (allp - pairs)) if n_new > 1 else (2 * H * (kd + R) * (allp - pairs)))
                k[f"pukerax_form_latent_mixer_{name}"] = dict(s=timed(lambda: plain(hin, b, store, 0, prec, resid=x), flush=flush), flops=fl_p,
                                                              bytes=by + n_seq * max(0, c0 + n_new - min(c0 + n_new, win + n_new)) * kd * 2)
        for i in range(n_seq):
            store.release(("k", i))
    del eng, model, store
    torch.cuda.empty_cache()

    # ---------------------------------------------------------------- Kovusun with dense feed-forwards at equal size
    kc = kovusun_dense_config(W, H, G, dh, F, V, L)
    km = random_kovusun(kc)
    eng = _throughput(km, args, flush, V, "kovusun", out)
    store, prec = eng.store, km.prec
    for name, (n_seq, n_new, c0) in {"prefill": (B_pre, S, 0), "decode": (B_dec, 1, ctx)}.items():
        b = _entries(store, n_seq, n_new, c0)
        T = b.T
        blk0 = km.blocks[0]
        x, a1, a2 = torch.randn(T, W, device="cuda"), prec.empty(T, W), prec.empty(T, W)
        k[f"kovusun_two_norms_shift_{name}"] = dict(
            s=timed(lambda: seq_ops.layernorm_shift(x, blk0.norm1_d, blk0.norm1_bd, a1, 1e-5, shift=blk0.shift_d, state=store.state[L], b=b, w2=blk0.norm2_d,
                                                    b2=blk0.norm2_bd, out2=a2), flush=flush), bytes=T * W * (4 + 2 + 2))
        hin = torch.randn(T, W, device="cuda").to(torch.bfloat16)
        k[f"kovusun_clamped_glu_feed_forward_{name}"] = dict(s=timed(lambda: blk0.ff(hin, b, prec, resid=x), flush=flush), flops=6 * T * W * F,
                                                             bytes=3 * W * F * 2 + T * (W * 2 + F * 4 + W * 8))
        gu = torch.randn(T, 2 * F, device="cuda").to(torch.bfloat16)
        mid = prec.empty(T, F)
        k[f"kovusun_gated_unit_unfused_{name}"] = dict(s=timed(lambda: seq_ops.glu(gu, mid, seq_ops.GLU_CLAMPED, 7.0, 1.702), flush=flush), bytes=T * F * (4 + 2))
        for li in (0, 1):
            mx = km.blocks[li].mixer
            store.k_pages[li].normal_()
            store.v_pages[li].normal_()
            win = mx.window or (c0 + n_new)
            pairs = n_seq * sum(min(i + 1, win) + max(0, min(mx.keep_first, i + 1 - win)) for i in range(c0, c0 + n_new))
            wts = (mx.w_in.numel() + mx.w_o.numel()) * 2
            k[f"kovusun_mixer_{kc['layers'][li]['type']}_{name}"] = dict(
                s=timed(lambda: mx(hin, b, store, li, prec, resid=x), flush=flush), flops=2 * T * W * mx.w_in.shape[0] + 2 * T * H * dh * W + 4 * dh * H * pairs,
                bytes=wts + n_seq * min(c0 + n_new, win + mx.keep_first + n_new) * G * 2 * dh * 2 + T * W * (2 + 8))
        for i in range(n_seq):
            store.release(("k", i))
    for name, d in k.items():
        d["us"] = round(d.pop("s") * 1e6, 2)
        d["hbm_frac"] = round(d["bytes"] / (d["us"] * 1e-6) / hbm, 4)
        if "flops" in d:
            d["tflops"] = round(d["flops"] / (d["us"] * 1e-6) / 1e12, 2)
            d["tensor_frac"] = round(d["flops"] / (d["us"] * 1e-6) / tflops, 5)
        # distance from the roofline: the measured time over the larger of the two bounds
        bound = max(d["bytes"] / hbm, d.get("flops", 0) / tflops)
        d["x_roofline"] = round(d["us"] * 1e-6 / bound, 2)
    out["kernels"] = k
    out["value"] = out["zigivik_decode_tok_s"]
    out["unit"] = "tokens/s"
    out["n_gpus"] = 1
    for key in list(out):
        if key.endswith("tok_s"):
            out[key] = round(out[key], 1)
    print(json.dumps(out), flush=True)
    return out
