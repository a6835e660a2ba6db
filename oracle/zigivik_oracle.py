"""Plain, slow restatement of the Zigivik decoder (test infrastructure only; the product path never imports it).

One function per mechanism, one sequence at a time (positions 0 .. T-1), nothing shared with the kernels or their host
wrappers.  In my notation, for a layer with residual x [T, D] and residual multiplier m:

    h   = x / rms(x) * g                         g: ONE number per norm
    h~  = h + conv(h)                            conv(h)_t[c] = sum_j w[c, j] h_{t - taps + 1 + j}[c]   (h before the sequence = 0)
    x  <- x + m * (mixer(h~) + ff(h))            both branches come from the same norm; only the mixer sees the convolution

Mixers: latent attention (low-rank queries; keys / values as images of one cached latent row plus one rotated key part shared by
the heads; half-split rotation with rescaled frequencies; sliding window; element-wise sigmoid output gate; optionally the cached
rows of an earlier layer) and grouped-query attention whose values ARE the unrotated keys, with interleaved rotation and a softmax
denominator enlarged by one.  Feed-forward: W_down P(W_up h + b) + b with P a cubic of unit-rms powers.

A "weights" argument is a dict name -> tensor (any float type) with the checkpoint's names; "cfg" is the parsed config.json.
"""
import math

import torch


def unit_rms(z, eps):
    return z / torch.sqrt((z * z).mean(-1, keepdim=True) + eps)


def scalar_norm(x, g, eps):
    return unit_rms(x, eps) * g.reshape(())


def causal_conv(h, w):
    """h [T, D], w [D, taps] -> sum_j w[:, j] * h_{t - taps + 1 + j}."""
    T, D = h.shape
    taps = w.shape[1]
    out = torch.zeros_like(h)
    for t in range(T):
        for j in range(taps):
            s = t - taps + 1 + j
            if s >= 0:
                out[t] += w[:, j] * h[s]
    return out


def plain_frequencies(base, dims):
    return [float(base) ** (-2.0 * i / dims) for i in range(dims // 2)]


def rescaled_frequencies(base, dims, sc):
    """Long wavelengths are stretched by `factor`, short ones kept, with a linear ramp over the pair index between the indices whose
    wavelengths make `fast` and `slow` turns over `original` positions.  Returns (frequencies, multiplier of cos and sin)."""
    factor, orig, fast, slow = float(sc["factor"]), float(sc["original"]), float(sc["fast"]), float(sc["slow"])

    def index_of(turns):
        return dims * math.log(orig / (2.0 * math.pi * turns)) / (2.0 * math.log(base))

    lo = max(math.floor(index_of(fast)), 0)
    hi = min(math.ceil(index_of(slow)), dims - 1)
    out = []
    for i, f in enumerate(plain_frequencies(base, dims)):
        ramp = min(max((i - lo) / max(hi - lo, 0.001), 0.0), 1.0)
        out.append(f / factor * ramp + f * (1.0 - ramp))
    return out, 0.1 * math.log(factor) + 1.0


def turn_half(vec, p, freqs, mult):
    """vec [..., n]: element i is paired with element i + len(freqs) (half-split layout); the first 2 len(freqs) elements turn."""
    half = len(freqs)
    out = vec.clone()
    for i, f in enumerate(freqs):
        c, s = math.cos(p * f) * mult, math.sin(p * f) * mult
        u, v = vec[..., i], vec[..., i + half]
        out[..., i] = u * c - v * s
        out[..., i + half] = v * c + u * s
    return out


def turn_pairs(vec, p, freqs):
    """vec [..., n]: elements (2i, 2i+1) turn by p * freqs[i]."""
    out = vec.clone()
    for i, f in enumerate(freqs):
        c, s = math.cos(p * f), math.sin(p * f)
        u, v = vec[..., 2 * i], vec[..., 2 * i + 1]
        out[..., 2 * i] = u * c - v * s
        out[..., 2 * i + 1] = v * c + u * s
    return out


def latent_rows(hm, w, pre, m, eps):
    """What a latent layer caches: c [T, kv_rank] (normed) and r [T, rot_dim] (turned by its position)."""
    R, rot = int(m["kv_rank"]), int(m["rot_dim"])
    d = hm @ w[pre + "dkv"].T
    c = unit_rms(d[:, :R], eps) * w[pre + "dkv.norm"]
    freqs, mult = _latent_freqs(m)
    r = torch.stack([turn_half(d[t, R:], t, freqs, mult) for t in range(hm.shape[0])])
    return c, r


def _latent_freqs(m):
    rot = m["rot"]
    if rot.get("scaling"):
        return rescaled_frequencies(rot["base"], int(rot["dims"]), rot["scaling"])
    return plain_frequencies(rot["base"], int(rot["dims"])), 1.0


def latent_attention(hm, w, pre, m, eps, cached):
    """cached = (c, r) of this layer or of the layer it borrows from."""
    T = hm.shape[0]
    H, dim, rot, vdim = int(m["heads"]), int(m["dim"]), int(m["rot_dim"]), int(m["vdim"])
    c, r = cached
    cq = unit_rms(hm @ w[pre + "dq"].T, eps) * w[pre + "dq.norm"]
    q = (cq @ w[pre + "uq"].T).view(T, H, dim + rot)
    freqs, mult = _latent_freqs(m)
    kp = (c @ w[pre + "uk"].T).view(T, H, dim)
    v = (c @ w[pre + "uv"].T).view(T, H, vdim)
    size = int(m["mask"]["size"]) if m.get("mask") else None
    out = torch.zeros(T, H, vdim, dtype=hm.dtype)
    for i in range(T):
        qr = turn_half(q[i, :, dim:], i, freqs, mult)
        lo = 0 if size is None else max(0, i - size + 1)
        for h in range(H):
            s = (kp[lo:i + 1, h] @ q[i, h, :dim] + r[lo:i + 1] @ qr[h]) * float(m["scale"])
            p = torch.softmax(s, 0)
            out[i, h] = p @ v[lo:i + 1, h]
    gate = torch.sigmoid(hm @ w[pre + "g"].T)
    return (out.reshape(T, H * vdim) * gate) @ w[pre + "o"].T


def key_value_attention(hm, w, pre, m):
    T = hm.shape[0]
    H, G, dim = int(m["heads"]), int(m["kv_heads"]), int(m["dim"])
    q = (hm @ w[pre + "q"].T + w[pre + "q.b"]).view(T, H, dim)
    k = (hm @ w[pre + "k"].T + w[pre + "k.b"]).view(T, G, dim)
    v = k.clone()  # the values are the keys before they are turned
    rot = m.get("rot") or {}
    freqs = plain_frequencies(rot["base"], int(rot["dims"])) if rot.get("dims") else []
    qt = torch.stack([turn_pairs(q[t], t, freqs) for t in range(T)])
    kt = torch.stack([turn_pairs(k[t], t, freqs) for t in range(T)])
    out = torch.zeros(T, H, v.shape[-1], dtype=hm.dtype)
    for i in range(T):
        for h in range(H):
            g = h // (H // G)
            s = (kt[:i + 1, g] @ qt[i, h]) * float(m["scale"])
            mx = torch.clamp(s.max(), min=0.0)
            e = torch.exp(s - mx)
            p = e / (torch.exp(-mx) + e.sum())  # one more unit in the denominator: a key with score 0 and no value
            out[i, h] = p @ v[:i + 1, g]
    return out.reshape(T, -1) @ w[pre + "o"].T


def poly_norm(z, coef, eps):
    a, b, c, e = (coef[i] for i in range(4))
    return a * unit_rms(z, eps) + b * unit_rms(z * z, eps) + c * unit_rms(z * z * z, eps) + e


def feed_forward(h, w, pre, eps):
    z = h @ w[pre + "up"].T + w[pre + "up.b"]
    return poly_norm(z, w[pre + "act"], eps) @ w[pre + "down"].T + w[pre + "down.b"]


def forward(cfg, w, tokens, dtype=torch.float64, return_layers=False):
    """Logits [T, vocab] of one sequence (and the residual after every layer)."""
    w = {k: v.to(dtype) for k, v in w.items()}
    eps, m = float(cfg["norm"]["eps"]), float(cfg["residual_mult"])
    x = scalar_norm(w["embed"][torch.as_tensor(tokens, dtype=torch.long)], w["embed.norm"], eps)
    cached, layers = {}, []
    for i, l in enumerate(cfg["layers"]):
        pre = f"l{i}."
        h = scalar_norm(x, w[pre + "norm1"], eps)
        hm = h + causal_conv(h, w[pre + "canon1"])
        mx = l["mixer"]
        if l["type"] == "latent_attention":
            if mx.get("kv_from") is None:
                cached[i] = latent_rows(hm, w, pre + "mix.", mx, eps)
            y = latent_attention(hm, w, pre + "mix.", mx, eps, cached[i if mx.get("kv_from") is None else int(mx["kv_from"])])
        elif l["type"] == "attention":
            y = key_value_attention(hm, w, pre + "mix.", mx)
        else:
            raise ValueError(l["type"])
        if l.get("mlp"):
            y = y + feed_forward(h, w, pre + "mlp.", eps)
        x = x + m * y
        layers.append(x.clone())
    logits = scalar_norm(x, w["final.norm"], eps) @ w["head"].T
    return (logits, layers) if return_layers else logits


def tensor_shapes(cfg):
    D, V, taps = int(cfg["width"]), int(cfg["vocab"]), int(cfg["canon"]["taps"])
    s = {"embed": (V, D), "embed.norm": (), "final.norm": (), "head": (V, D)}
    for i, l in enumerate(cfg["layers"]):
        p, m = f"l{i}.", l["mixer"]
        s[p + "norm1"] = ()
        s[p + "canon1"] = (D, taps)
        H, dim = int(m["heads"]), int(m["dim"])
        if l["type"] == "latent_attention":
            rot, vdim, Q, R = int(m["rot_dim"]), int(m["vdim"]), int(m["q_rank"]), int(m["kv_rank"])
            s.update({p + "mix.dq": (Q, D), p + "mix.dq.norm": (Q,), p + "mix.uq": (H * (dim + rot), Q), p + "mix.uk": (H * dim, R),
                      p + "mix.uv": (H * vdim, R), p + "mix.g": (H * vdim, D), p + "mix.o": (D, H * vdim)})
            if m.get("kv_from") is None:
                s.update({p + "mix.dkv": (R + rot, D), p + "mix.dkv.norm": (R,)})
        else:
            G = int(m["kv_heads"])
            s.update({p + "mix.q": (H * dim, D), p + "mix.q.b": (H * dim,), p + "mix.k": (G * dim, D), p + "mix.k.b": (G * dim,),
                      p + "mix.o": (D, H * dim)})
        if l.get("mlp"):
            F = int(l["mlp"]["ff"])
            s.update({p + "mlp.up": (F, D), p + "mlp.up.b": (F,), p + "mlp.down": (D, F), p + "mlp.down.b": (D,), p + "mlp.act": (4,)})
    return s


def random_weights(cfg, seed=0):
    """bf16-representable random weights of a size that keeps activations near one."""
    g = torch.Generator().manual_seed(seed)
    w = {}
    for name, shape in tensor_shapes(cfg).items():
        if name.endswith("norm1") or name in ("embed.norm", "final.norm"):
            t = 1.0 + 0.2 * torch.randn(shape, generator=g)
        elif name.endswith(".norm"):
            t = 1.0 + 0.1 * torch.randn(shape, generator=g)
        elif name.endswith(".b"):
            t = 0.1 * torch.randn(shape, generator=g)
        elif name.endswith("mlp.act"):
            t = torch.tensor([0.6, 0.3, 0.2, 0.05]) + 0.05 * torch.randn(4, generator=g)
        elif name.endswith("canon1"):
            t = 0.3 * torch.randn(shape, generator=g)
        elif name == "embed":
            t = torch.randn(shape, generator=g)
        else:
            t = torch.randn(shape, generator=g) * (1.5 / math.sqrt(shape[-1]))
        w[name] = t.to(torch.bfloat16).float()
    return w
