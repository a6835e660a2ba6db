"""Plain, slow restatement of the Kovusun decoder (test infrastructure only; the product path never imports it).

One function per mechanism, one sequence at a time (positions 0 .. T-1), nothing shared with the kernels or their host
wrappers.  In my notation, for a layer with residual x [T, D]:

    a = LN1(x), b = LN2(x)                     LN(z) = (z - mean z) / sqrt(var z + eps) * w + bias
    a~_t = a_t + (a_{t-1} - a_t) * s           token shift (a_{-1} = 0); only the mixer reads it
    x <- x + mixer(a~) + ff(b)                 both branches read the SAME x

Mixers are windowed softmax attentions with grouped key/value heads; which of the optional parts a layer has is told by
its type: projection biases, weightless q/k RMS norm, a logarithmic distance penalty, a softmax sink, a per-head sigmoid
output gate, partial interleaved rotation, a per-head score temperature, kept first tokens, keys / values borrowed from an
earlier layer.  Feed-forwards: a clamped gated unit with biases, or routed silu-gated experts (+ a gated shared expert).

A "weights" argument is a dict name -> tensor (any float type) with the checkpoint's names; "cfg" is the parsed config.json.
"""
import math

import torch


def layer_norm(z, w, b, eps):
    mu = z.mean(-1, keepdim=True)
    var = ((z - mu) ** 2).mean(-1, keepdim=True)
    return (z - mu) / torch.sqrt(var + eps) * w + b


def unit_rms(z, eps):
    return z / torch.sqrt((z * z).mean(-1, keepdim=True) + eps)


def token_shift(a, s):
    """a [T, D] -> a_t + (a_{t-1} - a_t) * s, with a_{-1} = 0."""
    prev = torch.zeros_like(a)
    prev[1:] = a[:-1]
    return a + (prev - a) * s


def rotate_pairs(vec, p, base, dims):
    """vec [..., n >= dims]: the pair (2i, 2i+1), i < dims/2, is turned by the angle p * base^(-2i/dims)."""
    out = vec.clone()
    for i in range(dims // 2):
        ang = float(p) * float(base) ** (-2.0 * i / dims)
        c, s = math.cos(ang), math.sin(ang)
        u, v = vec[..., 2 * i], vec[..., 2 * i + 1]
        out[..., 2 * i] = u * c - v * s
        out[..., 2 * i + 1] = v * c + u * s
    return out


def visible(i, j, size, keep_first):
    """May query position i read key position j?"""
    if j > i:
        return False
    return (size is None or i - j < size) or j < keep_first


def keys_values(h, w, pre, kind, m, eps):
    """What a layer leaves for its own (and borrowing layers') attention: keys [T, G, dim] after norm / rotation, values."""
    T = h.shape[0]
    G, dim, vd = int(m["kv_heads"]), int(m["dim"]), int(m["vdim"])
    k = h @ w[pre + "k"].T
    v = h @ w[pre + "v"].T
    if kind == "attention":
        k = k + w[pre + "k.b"]
        v = v + w[pre + "v.b"]
    k, v = k.reshape(T, G, dim), v.reshape(T, G, vd)
    if kind in ("attention", "attention_2"):
        k = unit_rms(k, eps)
    if kind == "attention_3" and m.get("rot"):
        k = torch.stack([rotate_pairs(k[t], t, m["rot"]["base"], int(m["rot"]["dims"])) for t in range(T)])
    return k, v


def attend(q, keys, vals, scale, size=None, keep=0, sink=None, r1=None, r2=None, temp=None, first_pos=0):
    """q [T, H, dim] at positions first_pos .. first_pos + T - 1 over keys [N, G, dim] / vals [N, G, vd] at positions 0 .. N - 1
    -> [T, H, vd].  One (query, head) at a time, a plain softmax over the listed visible keys (the sink as an extra logit)."""
    T, H = q.shape[:2]
    G = keys.shape[1]
    out = torch.zeros(T, H, vals.shape[-1], dtype=q.dtype)
    for t in range(T):
        i = first_pos + t
        js = [j for j in range(min(i + 1, keys.shape[0])) if visible(i, j, size, keep)]
        jt = torch.tensor(js)
        dist = (i - jt).to(q.dtype)
        for hh in range(H):
            g = hh // (H // G)
            s = (keys[jt, g] @ q[t, hh]) * float(scale)
            if temp is not None:
                s = s * temp[hh]
            if r1 is not None:  # (no layer type has both a temperature and a penalty; here the penalty is not scaled by the temperature)
                s = s - r1[hh] * torch.log(1.0 + r2[hh] * dist)
            if sink is not None:
                p = torch.softmax(torch.cat([s, sink[hh].reshape(1).to(s.dtype)]), 0)[:-1]
            else:
                p = torch.softmax(s, 0)
            out[t, hh] = (p[:, None] * vals[jt, g]).sum(0)
    return out


def attention(h, w, pre, kind, m, eps, kv):
    """h [T, D] -> [T, D]; kv = (keys, values) of this layer or of the layer it borrows from."""
    T = h.shape[0]
    H, dim, vd = int(m["heads"]), int(m["dim"]), int(m["vdim"])
    mask = m.get("mask") or {}
    q = h @ w[pre + "q"].T
    if kind == "attention":
        q = q + w[pre + "q.b"]
    q = q.reshape(T, H, dim)
    if kind in ("attention", "attention_2"):
        q = unit_rms(q, eps)
    if kind == "attention_3" and m.get("rot"):
        q = torch.stack([rotate_pairs(q[t], t, m["rot"]["base"], int(m["rot"]["dims"])) for t in range(T)])
    out = attend(q, kv[0], kv[1], m["scale"], mask.get("size"), int(mask.get("keep_first", 0)),
                 sink=w[pre + "sink"] if kind == "attention_2" else None,
                 r1=w[pre + "r1"] if kind == "attention" else None, r2=w[pre + "r2"] if kind == "attention" else None,
                 temp=w[pre + "temp"] if kind == "attention_3" else None)
    if kind == "attention_2":
        out = out * torch.sigmoid(h @ w[pre + "g"].T)[:, :, None]
    return out.reshape(T, H * vd) @ w[pre + "o"].T


def clamped_gated_unit(h, w, pre, limit):
    g = torch.clamp(h @ w[pre + "gate"].T + w[pre + "gate.b"], max=limit)
    u = torch.clamp(h @ w[pre + "up"].T + w[pre + "up.b"], min=-limit, max=limit)
    return (g * torch.sigmoid(1.702 * g) * (u + 1.0)) @ w[pre + "down"].T + w[pre + "down.b"]


def silu_expert(h, w, pre):
    z = h @ w[pre + "gate"].T
    return (z * torch.sigmoid(z) * (h @ w[pre + "up"].T)) @ w[pre + "down"].T


def routed_experts(h, w, pre, mlp):
    n, top = int(mlp["router"]["experts"]), int(mlp["router"]["top"])
    out = torch.zeros_like(h)
    for t in range(h.shape[0]):
        z = (w[pre + "router"].float() @ h[t].float() + w[pre + "router.b"].float())
        best = sorted(range(n), key=lambda e: (-float(z[e]), e))[:top]
        wt = torch.softmax(z[best], 0)
        for e, a in zip(best, wt):
            out[t] += a.to(h.dtype) * silu_expert(h[t:t + 1], w, f"{pre}e{e}.")[0]
    if mlp.get("shared"):
        sg = torch.sigmoid(h @ w[pre + "shared.sg"].T)  # [T, 1]
        out = out + sg * silu_expert(h, w, pre + "shared.")
    return out


def feed_forward(h, w, pre, mlp):
    if not mlp:
        return torch.zeros_like(h)
    if mlp.get("kind", "dense") == "dense":
        return clamped_gated_unit(h, w, pre, float(mlp["limit"]))
    return routed_experts(h, w, pre, mlp)


def forward(cfg, w, tokens, dtype=torch.float32, return_layers=False):
    """logits [T, vocab] of one sequence (and the residual after every layer)."""
    w = {k: (v.to(dtype) if v.is_floating_point() else v) for k, v in w.items()}
    eps = float(cfg["norm"]["eps"])
    x = w["embed"][torch.tensor(list(tokens))]
    cache, layers = {}, []
    for i, layer in enumerate(cfg["layers"]):
        p, m, kind = f"l{i}.", layer["mixer"], layer["type"]
        a = layer_norm(x, w[p + "norm1"], w[p + "norm1.b"], eps)
        b = layer_norm(x, w[p + "norm2"], w[p + "norm2.b"], eps)
        if p + "shift" in w:
            a = token_shift(a, w[p + "shift"])
        if "kv_from" in m:
            kv = cache[int(m["kv_from"])]
        else:
            kv = cache[i] = keys_values(a, w, p + "mix.", kind, m, eps)
        x = x + (attention(a, w, p + "mix.", kind, m, eps, kv) + feed_forward(b, w, p + "mlp.", layer.get("mlp")))
        layers.append(x)
    logits = layer_norm(x, w["final.norm"], w["final.norm.b"], eps) @ w["head"].T
    return (logits, layers) if return_layers else logits


def tensor_shapes(cfg):
    """name -> shape of every checkpoint tensor the config implies."""
    D, V = int(cfg["width"]), int(cfg["vocab"])
    out = {"embed": (V, D), "final.norm": (D,), "final.norm.b": (D,), "head": (V, D)}
    for i, layer in enumerate(cfg["layers"]):
        p, m, kind = f"l{i}.", layer["mixer"], layer["type"]
        H, G, dim, vd = int(m["heads"]), int(m["kv_heads"]), int(m["dim"]), int(m["vdim"])
        for n in ("norm1", "norm1.b", "norm2", "norm2.b", "shift"):
            out[p + n] = (D,)
        out[p + "mix.q"] = (H * dim, D)
        if "kv_from" not in m:
            out[p + "mix.k"], out[p + "mix.v"] = (G * dim, D), (G * vd, D)
        if kind == "attention":
            out[p + "mix.q.b"] = (H * dim,)
            if "kv_from" not in m:
                out[p + "mix.k.b"], out[p + "mix.v.b"] = (G * dim,), (G * vd,)
            out[p + "mix.r1"], out[p + "mix.r2"] = (H,), (H,)
        if kind == "attention_2":
            out[p + "mix.sink"], out[p + "mix.g"] = (H,), (H, D)
        if kind == "attention_3":
            out[p + "mix.temp"] = (H,)
        out[p + "mix.o"] = (D, H * vd)
        mlp = layer.get("mlp")
        if not mlp:
            continue
        if mlp.get("kind", "dense") == "dense":
            F = int(mlp["ff"])
            out.update({p + "mlp.gate": (F, D), p + "mlp.gate.b": (F,), p + "mlp.up": (F, D), p + "mlp.up.b": (F,), p + "mlp.down": (D, F), p + "mlp.down.b": (D,)})
        else:
            F, n = int(mlp["expert"]["ff"]), int(mlp["router"]["experts"])
            for e in range(n):
                out.update({f"{p}mlp.e{e}.gate": (F, D), f"{p}mlp.e{e}.up": (F, D), f"{p}mlp.e{e}.down": (D, F)})
            out[p + "mlp.router"], out[p + "mlp.router.b"] = (n, D), (n,)
            if mlp.get("shared"):
                Fs = int(mlp["shared"]["ff"])
                out.update({p + "mlp.shared.gate": (Fs, D), p + "mlp.shared.up": (Fs, D), p + "mlp.shared.down": (D, Fs), p + "mlp.shared.sg": (1, D)})
    return out


def random_weights(cfg, seed=0):
    """bf16-representable fp32 tensors: projections ~ 1/sqrt(fan-in), norm weights around one, biases and per-head numbers of a size
    that matters (a dropped bias, sink, penalty or temperature moves the logits far beyond rounding)."""
    g = torch.Generator().manual_seed(seed)
    out = {}
    for name, shape in tensor_shapes(cfg).items():
        r = torch.randn(shape, generator=g)
        if name.endswith(("norm1", "norm2", "final.norm")):
            t = 1.0 + 0.3 * r
        elif name.endswith("shift"):
            t = torch.rand(shape, generator=g)
        elif name.endswith(".b"):
            t = 0.5 * r
        elif name.endswith(("r1", "r2")):
            t = 0.2 + torch.rand(shape, generator=g)
        elif name.endswith("temp"):
            t = 0.5 + torch.rand(shape, generator=g)
        elif name.endswith("sink"):
            t = r
        elif name == "embed":
            t = r
        elif name.endswith("router"):
            t = 3.0 * r / math.sqrt(shape[-1])
        else:
            t = r / math.sqrt(shape[-1])
        out[name] = t.to(torch.bfloat16).to(torch.float32)
    return out
