"""Sub-layers of the token-sequence decoders, each a mechanism with its constants as parameters.

  GatedSoftmaxAttention   grouped-query softmax attention over the paged cache: per-head q/k RMS norm, partial interleaved
                          rotary positions with long-wavelength frequency rescaling, weightless value norm, tanh soft cap,
                          sigmoid output gate
  LightningAttention      decayed linear attention with a per-sequence fp32 state, gated RMS norm over the joined heads
  WindowedSoftmaxAttention grouped-query softmax attention over a sliding window of the paged cache; optional, each a parameter:
                          projection biases, weightless q/k RMS norm, partial interleaved rotation, a logarithmic distance penalty,
                          a per-head score multiplier, a softmax sink, kept first keys, a per-head sigmoid output gate, keys and
                          values borrowed from an earlier layer's cache
  GegluFeedForward        W_down(gelu_tanh(W_gate h) * W_up h)
  GluFeedForward          W_down(act(W_gate h) * W_up h) with act = silu, or the clamped form min(g, c) sigmoid(a min(g, c)) (clamp(u) + 1);
                          optional biases
  PolyNormFeedForward     W_down P(W_up h + b) + b, P(z) = a N(z) + b N(z^2) + c N(z^3) + e with N = division by the row's root mean square
  TokenSideInput          a per-layer, per-token low-dimensional embedding gated by a projection of the residual stream
  LatentAttention         attention over ONE cached low-rank row per token (+ one rotated key part shared by the heads); optional, each a
                          parameter: half-split rotation layout, ramped frequency rescaling with a cos / sin gain, a sliding window, a
                          per-element (instead of per-head) sigmoid output gate, cached rows borrowed from an earlier layer

Every sub-layer gets its weights from a name -> tensor dict (`take(name)` pops and checks the shape), packs them once for a
`Precision`, says what it keeps per sequence (`cache_spec`), and maps the step's rows h [T, D] (activation type) to
y [T, D] fp32; the block around it owns norms and the residual stream.  The newer sub-layers take `resid=` (the fp32 residual
rows): their last projection then adds into it in the GEMM epilogue instead of returning y.
"""
import ctypes as C
import math

import torch

from . import _lib, seq_ops
from .modeling_gemma import PAGE


def rotary_frequencies(base: float, dims: int, scaling=None):
    """f_i = base^(-2i/dims), i < dims/2 (float64).  With `scaling` = dict(factor, low, high, original): wavelengths
    2 pi / f shorter than original/high keep f, longer than original/low use f / factor, and between the two the blend
    (1 - s) f / factor + s f with s = (original / wavelength - low) / (high - low)."""
    i = torch.arange(dims // 2, dtype=torch.float64)
    f = float(base) ** (-2.0 * i / dims)
    if scaling:
        factor, low, high, orig = (float(scaling[k]) for k in ("factor", "low", "high", "original"))
        wl = 2.0 * math.pi / f
        s = (orig / wl - low) / (high - low)
        mid = (1.0 - s) * f / factor + s * f
        f = torch.where(wl < orig / high, f, torch.where(wl > orig / low, f / factor, mid))
    return f


def ramped_rotary_frequencies(base: float, dims: int, factor: float, original: float, fast: float, slow: float):
    """Frequencies f_i = base^(-2i/dims) rescaled by pair index: with idx(t) = dims ln(original / (2 pi t)) / (2 ln base), lo = max(floor(idx(fast)), 0),
    hi = min(ceil(idx(slow)), dims - 1) and ramp_i = clamp((i - lo) / max(hi - lo, 0.001), 0, 1), pair i turns with f_i / factor * ramp_i +
    f_i (1 - ramp_i).  Returns (frequencies float64 [dims / 2], gain) with gain = 0.1 ln(factor) + 1 multiplying every cosine and sine."""
    def idx(turns):
        return dims * math.log(float(original) / (2.0 * math.pi * float(turns))) / (2.0 * math.log(float(base)))

    lo, hi = max(math.floor(idx(fast)), 0), min(math.ceil(idx(slow)), dims - 1)
    i = torch.arange(dims // 2, dtype=torch.float64)
    f = float(base) ** (-2.0 * i / dims)
    ramp = ((i - lo) / max(hi - lo, 0.001)).clamp(0.0, 1.0)
    return f / float(factor) * ramp + f * (1.0 - ramp), 0.1 * math.log(float(factor)) + 1.0


def half_to_pair_order(n: int, rot_dims: int):
    """Index list that reorders a vector whose rotation pairs element i with element i + rot_dims / 2 so that the partners sit side by
    side (2i, 2i + 1): rotating the reordered vector in interleaved pairs gives the reordered result of the half-split rotation.  A
    dot product of two vectors reordered alike is unchanged, so applying this to the ROWS of the projections that make the rotated
    query and key parts lets one rotation kernel (and one cache layout) serve both conventions."""
    half = rot_dims // 2
    return [i // 2 + (i % 2) * half if i < rot_dims else i for i in range(n)]


class GatedSoftmaxAttention:
    def __init__(self, width, heads, kv_heads, dim, vdim, scale, softcap, rot_dims, rot_base, rot_scaling, eps):
        if heads % kv_heads:
            raise ValueError("query heads must be a multiple of key/value heads")
        if rot_dims % 2 or rot_dims > dim:
            raise ValueError("rotary dimensions must be even and at most the head size")
        self.D, self.H, self.G, self.dim, self.vdim = width, heads, kv_heads, dim, vdim
        self.scale, self.softcap, self.rot_dims, self.eps = float(scale), float(softcap or 0.0), int(rot_dims), float(eps)
        self.freq = rotary_frequencies(rot_base, rot_dims, rot_scaling) if rot_dims else torch.zeros(1, dtype=torch.float64)

    def cache_spec(self):
        return ("kv", self.G * self.dim, self.G * self.vdim)

    def load(self, take, pre):
        H, G, dim, vdim, D = self.H, self.G, self.dim, self.vdim, self.D
        self.w = dict(q=take(pre + "q", (H * dim, D)), k=take(pre + "k", (G * dim, D)), v=take(pre + "v", (G * vdim, D)),
                      g=take(pre + "g", (H * vdim, D)), o=take(pre + "o", (D, H * vdim)),
                      qn=take(pre + "q.norm", (dim,)), kn=take(pre + "k.norm", (dim,)))

    def pack(self, prec):
        w = self.w
        self.w_in = torch.cat([w["q"], w["k"], w["v"], w["g"]], 0).to("cuda", prec.dtype).contiguous()
        self.w_o = w["o"].to("cuda", prec.dtype).contiguous()
        self.qn, self.kn = w["qn"].to("cuda", torch.float32), w["kn"].to("cuda", torch.float32)
        self.freq_d = self.freq.to("cuda")

    def __call__(self, h, b, store, li, prec):
        H, G, dim, vdim = self.H, self.G, self.dim, self.vdim
        proj = seq_ops.linear(h, self.w_in, prec.empty(b.T, self.w_in.shape[0]))
        q = prec.empty(b.T, H * dim)
        kp, vp = store.k_pages[li], store.v_pages[li]
        seq_ops.attn_prepare(proj, b, self.freq_d, self.qn, self.kn, q, kp, vp, H, G, dim, vdim, self.rot_dims, self.eps, PAGE)
        att = prec.empty(b.T, H * vdim)
        gate = proj[:, (H + G) * dim + G * vdim:]
        seq_ops.attn_ragged(q, kp, vp, gate, att, b, H, G, dim, vdim, self.scale, self.softcap, PAGE)
        return seq_ops.linear(att, self.w_o, torch.empty(b.T, self.D, device="cuda", dtype=torch.float32))


class WindowedSoftmaxAttention:
    """q = W_q h (+ b), k, v likewise; optional weightless RMS norm of q and k per head; optional rotation of the first rot_dims
    dimensions; score(i, j) = (q_i . k_j) * scale * temp_h - r1_h * log(1 + r2_h * (i - j)); key j is visible to query i when
    j <= i and (i - j < window or j < keep_first); softmax over the visible keys, with exp(sink_h) joining the denominator when
    the layer has a sink; head output times sigmoid((W_g h)_h) when it has a gate; then W_o.

    kv_from = j: the layer has no key / value projections and attends over layer j's cached keys and values (as layer j left
    them, after its norm and rotation) with its own queries, window and score.

    value_is_key: there is no value projection; the values are the keys as projected, before norm and rotation (vdim == dim).
    unit_sink: the softmax denominator is enlarged by exactly one (a sink whose logit is 0, no tensor)."""

    def __init__(self, width, heads, kv_heads, dim, vdim, scale, eps, window=None, keep_first=0, bias=False, qk_norm=False, rot_dims=0,
                 rot_base=10000.0, distance_penalty=False, temperature=False, sink=False, head_gate=False, kv_from=None, value_is_key=False,
                 unit_sink=False):
        if heads % kv_heads:
            raise ValueError("query heads must be a multiple of key/value heads")
        if rot_dims % 2 or rot_dims > dim:
            raise ValueError("rotary dimensions must be even and at most the head size")
        if window is not None and int(window) <= 0:
            raise ValueError("a window holds at least the token itself")
        self.D, self.H, self.G, self.dim, self.vdim = int(width), int(heads), int(kv_heads), int(dim), int(vdim)
        self.scale, self.eps, self.window, self.keep_first = float(scale), float(eps), (int(window) if window is not None else None), int(keep_first)
        self.bias, self.qk_norm, self.rot_dims = bool(bias), bool(qk_norm), int(rot_dims)
        self.distance_penalty, self.temperature, self.sink, self.head_gate = bool(distance_penalty), bool(temperature), bool(sink), bool(head_gate)
        self.kv_from = None if kv_from is None else int(kv_from)
        self.value_is_key, self.unit_sink = bool(value_is_key), bool(unit_sink)
        if self.value_is_key and self.vdim != self.dim:
            raise ValueError("values that are the keys have the keys' size")
        if self.unit_sink and self.sink:
            raise ValueError("a layer has a learned sink or the unit one, not both")
        self.freq = rotary_frequencies(rot_base, rot_dims) if rot_dims else torch.zeros(1, dtype=torch.float64)

    def cache_spec(self):
        return None if self.kv_from is not None else ("kv", self.G * self.dim, self.G * self.vdim)

    def load(self, take, pre):
        H, G, dim, vdim, D = self.H, self.G, self.dim, self.vdim, self.D
        w = dict(q=take(pre + "q", (H * dim, D)))
        if self.bias:
            w["qb"] = take(pre + "q.b", (H * dim,))
        if self.kv_from is None:
            w["k"] = take(pre + "k", (G * dim, D))
            if not self.value_is_key:
                w["v"] = take(pre + "v", (G * vdim, D))
            if self.bias:
                w["kb"] = take(pre + "k.b", (G * dim,))
                if not self.value_is_key:
                    w["vb"] = take(pre + "v.b", (G * vdim,))
        if self.distance_penalty:
            w["r1"], w["r2"] = take(pre + "r1", (H,)), take(pre + "r2", (H,))
        if self.temperature:
            w["temp"] = take(pre + "temp", (H,))
        if self.sink:
            w["sink"] = take(pre + "sink", (H,))
        if self.head_gate:
            w["g"] = take(pre + "g", (H, D))
        w["o"] = take(pre + "o", (D, H * vdim))
        self.w = w

    def pack(self, prec):
        w, H = self.w, self.H
        f32 = dict(device="cuda", dtype=torch.float32)
        kv = [] if self.kv_from is not None else [w["k"]] if self.value_is_key else [w["k"], w["v"]]
        parts = [w["q"]] + kv + ([w["g"]] if self.head_gate else [])
        rows = sum(t.shape[0] for t in parts)
        pad = (-rows) % 8  # zero rows up to a multiple of 8: a shape the tensor-core product takes
        self.w_in = torch.zeros(rows + pad, self.D, device="cuda", dtype=prec.dtype)
        self.w_in[:rows] = torch.cat(parts, 0).to("cuda", prec.dtype)
        self.gate_col = rows - H if self.head_gate else None
        self.b_in = None
        if self.bias:
            self.b_in = torch.zeros(rows + pad, **f32)
            bs = torch.cat([w["qb"]] + ([] if self.kv_from is not None else [w["kb"]] if self.value_is_key else [w["kb"], w["vb"]])).to(**f32)
            self.b_in[:bs.numel()] = bs
        self.w_o = w["o"].to("cuda", prec.dtype).contiguous()
        self.freq_d = self.freq.to("cuda")

        def vec(name):
            return w[name].to(**f32).contiguous() if name in w else None

        sink = torch.zeros(H, **f32) if self.unit_sink else vec("sink")  # exp(0) = 1 joins the denominator
        self.score = seq_ops.ScoreOptions(H, self.window, self.keep_first, sink=sink, dist_a=vec("r1"), dist_b=vec("r2"), head_scale=vec("temp"))

    def __call__(self, h, b, store, li, prec, resid=None, resid_scale=1.0):
        H, G, dim, vdim = self.H, self.G, self.dim, self.vdim
        proj = seq_ops.linear(h, self.w_in, prec.empty(b.T, self.w_in.shape[0]), bias=self.b_in)
        q = prec.empty(b.T, H * dim)
        own = self.kv_from is None
        src = li if own else self.kv_from
        kp, vp = store.k_pages[src], store.v_pages[src]
        seq_ops.attn_prepare(proj, b, self.freq_d, None, None, q, kp if own else None, vp if own else None, H, G, dim, vdim, self.rot_dims, self.eps,
                             PAGE, norm_qk=self.qk_norm, norm_v=False, v_from_k=self.value_is_key)
        att = prec.empty(b.T, H * vdim)
        gate = proj[:, self.gate_col:] if self.head_gate else None
        seq_ops.attn_ragged(q, kp, vp, gate, att, b, H, G, dim, vdim, self.scale, 0.0, PAGE, gate_per_head=True, score=self.score)
        if resid is not None:
            return seq_ops.linear_add(att, self.w_o, resid, scale=resid_scale)
        return seq_ops.linear(att, self.w_o, torch.empty(b.T, self.D, device="cuda", dtype=torch.float32))


class LightningAttention:
    def __init__(self, width, heads, dim, vdim, decay, eps):
        if len(decay) != heads:
            raise ValueError("one decay per head")
        self.D, self.H, self.dim, self.vdim, self.eps = width, heads, dim, vdim, float(eps)
        self.decay = torch.tensor([float(a) for a in decay], dtype=torch.float32)

    def cache_spec(self):
        return ("state", (self.H, self.dim, self.vdim))

    def load(self, take, pre):
        H, dim, vdim, D = self.H, self.dim, self.vdim, self.D
        self.w = dict(q=take(pre + "q", (H * dim, D)), k=take(pre + "k", (H * dim, D)), v=take(pre + "v", (H * vdim, D)),
                      g=take(pre + "g", (H * vdim, D)), o=take(pre + "o", (D, H * vdim)), norm=take(pre + "norm", (H * vdim,)))

    def pack(self, prec):
        w = self.w
        self.w_in = torch.cat([w["q"], w["k"], w["v"], w["g"]], 0).to("cuda", prec.dtype).contiguous()
        self.w_o = w["o"].to("cuda", prec.dtype).contiguous()
        self.norm = w["norm"].to("cuda", torch.float32)
        self.decay_d = self.decay.to("cuda")

    def __call__(self, h, b, store, li, prec):
        H, dim, vdim = self.H, self.dim, self.vdim
        proj = seq_ops.linear(h, self.w_in, prec.empty(b.T, self.w_in.shape[0]))
        o = torch.empty(b.T, H * vdim, device="cuda", dtype=torch.float32)
        seq_ops.linear_attn(proj, store.state[li], self.decay_d, o, b, H, dim, vdim)
        att = prec.empty(b.T, H * vdim)
        seq_ops.rmsnorm_gate(o, self.norm, proj[:, 2 * H * dim + H * vdim:], att, self.eps)
        return seq_ops.linear(att, self.w_o, torch.empty(b.T, self.D, device="cuda", dtype=torch.float32))


class GegluFeedForward:
    def __init__(self, width, ff):
        self.D, self.F = width, ff

    def load(self, take, pre):
        self.w = dict(gate=take(pre + "gate", (self.F, self.D)), up=take(pre + "up", (self.F, self.D)), down=take(pre + "down", (self.D, self.F)))

    def pack(self, prec):
        w, F, D = self.w, self.F, self.D
        # bf16: the tcgen05 GEMM computes gelu(gate) * up in its epilogue from a [64 gate | 64 up] row-interleaved weight; F is
        # padded to a multiple of 64 with zero rows (gelu(0) * 0 = 0) and zero columns of the down projection
        self.fused = prec.dtype == torch.bfloat16 and D % 8 == 0
        if self.fused:
            Fp = (F + 63) // 64 * 64
            gate = torch.zeros(Fp, D, device="cuda", dtype=torch.bfloat16)
            up = torch.zeros_like(gate)
            gate[:F], up[:F] = w["gate"].to("cuda", torch.bfloat16), w["up"].to("cuda", torch.bfloat16)
            self.w_gu = torch.empty(2 * Fp, D, device="cuda", dtype=torch.bfloat16)
            _lib.check(_lib.lib().pg_pack_gate_up(gate.data_ptr(), up.data_ptr(), self.w_gu.data_ptr(), Fp, D, _lib.stream()), "pg_pack_gate_up")
            self.w_down = torch.zeros(D, Fp, device="cuda", dtype=torch.bfloat16)
            self.w_down[:, :F] = w["down"].to("cuda", torch.bfloat16)
            self.Fp = Fp
            torch.cuda.synchronize()
        else:
            self.w_gu = torch.cat([w["gate"], w["up"]], 0).to("cuda", prec.dtype).contiguous()
            self.w_down = w["down"].to("cuda", prec.dtype).contiguous()

    def __call__(self, h, b, prec):
        T = h.shape[0]
        if self.fused:
            mid = prec.empty(T, self.Fp)
            _lib.gemm(h, self.w_gu, mid, mode=_lib.EPI_GEGLU, swap=1 if T <= 128 else 0)
        else:
            gu = seq_ops.linear(h, self.w_gu, prec.empty(T, 2 * self.F))
            mid = prec.empty(T, self.F)
            seq_ops.geglu(gu, mid)
        return seq_ops.linear(mid, self.w_down, torch.empty(T, self.D, device="cuda", dtype=torch.float32))


class GluFeedForward:
    """W_down (act(W_gate h) * W_up h) (+ biases).  activation "silu": silu(g) * u; "clamped": g' = min(g, limit),
    u' = clamp(u, -limit, limit), g' * sigmoid(alpha * g') * (u' + 1)."""

    def __init__(self, width, ff, activation="silu", limit=0.0, alpha=1.0, bias=False):
        if activation not in ("silu", "clamped"):
            raise ValueError(f"unknown gated activation {activation!r}")
        self.D, self.F, self.kind = int(width), int(ff), seq_ops.GLU_CLAMPED if activation == "clamped" else seq_ops.GLU_SILU
        self.limit, self.alpha, self.bias = float(limit), float(alpha), bool(bias)

    def load(self, take, pre):
        F, D = self.F, self.D
        self.w = dict(gate=take(pre + "gate", (F, D)), up=take(pre + "up", (F, D)), down=take(pre + "down", (D, F)))
        if self.bias:
            self.w.update(gate_b=take(pre + "gate.b", (F,)), up_b=take(pre + "up.b", (F,)), down_b=take(pre + "down.b", (D,)))

    def pack(self, prec):
        w, F, D = self.w, self.F, self.D
        f32 = dict(device="cuda", dtype=torch.float32)
        self.b_down = w["down_b"].to(**f32).contiguous() if self.bias else None
        # bf16: the tcgen05 GEMM computes the gated unit (and adds the biases) in its epilogue from a [64 gate | 64 up] row-interleaved
        # weight; F is padded to a multiple of 64 with zero rows (both forms map (0, 0) to 0) and zero columns of the down projection
        self.fused = prec.dtype == torch.bfloat16 and D % 8 == 0
        if self.fused:
            Fp = (F + 63) // 64 * 64
            gate = torch.zeros(Fp, D, device="cuda", dtype=torch.bfloat16)
            up = torch.zeros_like(gate)
            gate[:F], up[:F] = w["gate"].to("cuda", torch.bfloat16), w["up"].to("cuda", torch.bfloat16)
            self.w_gu = torch.empty(2 * Fp, D, device="cuda", dtype=torch.bfloat16)
            _lib.check(_lib.lib().pg_pack_gate_up(gate.data_ptr(), up.data_ptr(), self.w_gu.data_ptr(), Fp, D, _lib.stream()), "pg_pack_gate_up")
            self.w_down = torch.zeros(D, Fp, device="cuda", dtype=torch.bfloat16)
            self.w_down[:, :F] = w["down"].to("cuda", torch.bfloat16)
            self.b_gu = None
            if self.bias:
                bg, bu = torch.zeros(Fp, **f32), torch.zeros(Fp, **f32)
                bg[:F], bu[:F] = w["gate_b"].to(**f32), w["up_b"].to(**f32)
                self.b_gu = torch.stack([bg.view(-1, 64), bu.view(-1, 64)], 1).reshape(-1).contiguous()  # the weight's packed row order
            self.Fp = Fp
            torch.cuda.synchronize()
        else:
            self.w_gu = torch.cat([w["gate"], w["up"]], 0).to("cuda", prec.dtype).contiguous()
            self.w_down = w["down"].to("cuda", prec.dtype).contiguous()
            self.b_gu = torch.cat([w["gate_b"], w["up_b"]]).to(**f32).contiguous() if self.bias else None

    def __call__(self, h, b, prec, resid=None):
        T = h.shape[0]
        if self.fused:
            mid = prec.empty(T, self.Fp)
            _lib.gemm(h, self.w_gu, mid, mode=_lib.EPI_GEGLU, act_gelu=_lib.GLU_CLAMPED if self.kind == seq_ops.GLU_CLAMPED else _lib.GLU_SILU,
                      scale=self.limit, glu_alpha=self.alpha, bias=self.b_gu, swap=1 if T <= 128 else 0)
        else:
            gu = seq_ops.linear(h, self.w_gu, prec.empty(T, 2 * self.F), bias=self.b_gu)
            mid = seq_ops.glu(gu, prec.empty(T, self.F), self.kind, self.limit, self.alpha)
        if resid is not None:
            return seq_ops.linear_add(mid, self.w_down, resid, bias=self.b_down)
        return seq_ops.linear(mid, self.w_down, torch.empty(T, self.D, device="cuda", dtype=torch.float32), bias=self.b_down)


class TokenSideInput:
    """y = P (gelu_tanh(G x) * e), e = columns [index * dim, (index + 1) * dim) of the side table's row of the token."""

    def __init__(self, width, dim, index):
        self.D, self.n, self.index = width, dim, index

    def load(self, take, pre):
        self.w = dict(gate=take(pre + "gate", (self.n, self.D)), proj=take(pre + "proj", (self.D, self.n)))

    def pack(self, prec):
        n, D = self.n, self.D
        self.n_pad = (n + 7) // 8 * 8  # TMA wants 16-byte pitches; the pad columns are zeros
        self.w_gate = torch.zeros(self.n_pad, D, device="cuda", dtype=prec.dtype)
        self.w_gate[:n] = self.w["gate"].to("cuda", prec.dtype)
        self.w_proj = torch.zeros(D, self.n_pad, device="cuda", dtype=prec.dtype)
        self.w_proj[:, :n] = self.w["proj"].to("cuda", prec.dtype)

    def __call__(self, h, b, table, prec):
        T = h.shape[0]
        z = seq_ops.linear(h, self.w_gate, torch.empty(T, self.n_pad, device="cuda", dtype=torch.float32))  # fp32: split-K when T is small
        gz = prec.empty(T, self.n_pad)
        seq_ops.side_gate(z, b.tokens, table, self.index * self.n, gz, self.n)
        return seq_ops.linear(gz, self.w_proj, torch.empty(T, self.D, device="cuda", dtype=torch.float32))


class LatentAttention:
    """Attention whose keys and values are linear images of one cached low-rank row per token.

        [c_q | c | r] = W_in h;  c_q <- rms(c_q) w_q;  c <- rms(c) w_c;  r <- rotate(r, position)       (cache row: [c | r])
        q_h = W_uq,h c_q = [q_plain | q_rot],  q_rot <- rotate(q_rot, position)
        score(i, j) = (q_plain,h(i) . W_uk,h c(j) + q_rot,h(i) . r(j)) * scale,  out_h = sigmoid(g_h) * sum_j p(i, j) W_uv,h c(j)

    The step computes it in the absorbed form -- (W_uk,h^T q_plain,h) . c(j), and W_uv,h applied after the weighted sum of the
    c(j) -- so the paged cache is read as ONE key/value head of width rank + rot (values = its first `rank` columns) shared by
    all query heads, and nothing per head is ever stored.  Prompt portions in bf16 whose head sizes the tensor-core kernel is
    built for use the explicit-head form instead: keys / values of the entry's tokens are rebuilt from the cached rows into
    scratch pages (the products are 3 .. 5 times smaller there).

    Optional parts: rot_layout "half" -- the rotation pairs element i with i + rot_dims / 2 (the rows of the projections that make the
    rotated parts are reordered once, see half_to_pair_order); rot_scaling = dict(factor, original, fast, slow) -- ramped frequency
    rescaling with its cos / sin gain (ramped_rotary_frequencies); window -- key j is visible to query i when 0 <= i - j < window;
    gate "element" -- W_g has one row per output element (H * vdim) instead of one per head; kv_from = j -- no W_dkv: the layer
    reads the rows layer j cached (same rank, rotated part and rotation) with its own up projections, queries, window and gate."""

    def __init__(self, width, heads, dim, rot_dim, vdim, q_rank, kv_rank, scale, rot_dims, rot_base, eps, rot_layout="interleaved", rot_scaling=None,
                 window=None, gate="head", kv_from=None):
        if rot_dims % 2 or rot_dims > rot_dim:
            raise ValueError("rotary dimensions must be even and at most the rotated key part")
        if rot_layout not in ("interleaved", "half") or gate not in ("head", "element"):
            raise ValueError("rot_layout is 'interleaved' or 'half', gate is 'head' or 'element'")
        if window is not None and int(window) <= 0:
            raise ValueError("a window holds at least the token itself")
        self.D, self.H, self.dim, self.rot, self.vdim, self.Q, self.R = width, heads, dim, rot_dim, vdim, q_rank, kv_rank
        self.scale, self.rot_dims, self.eps = float(scale), int(rot_dims), float(eps)
        self.rot_layout, self.gate_kind, self.window = rot_layout, gate, (int(window) if window is not None else None)
        self.kv_from = None if kv_from is None else int(kv_from)
        self.rot_gain = 1.0
        if not rot_dims:
            self.freq = torch.zeros(1, dtype=torch.float64)
        elif rot_scaling:
            self.freq, self.rot_gain = ramped_rotary_frequencies(rot_base, rot_dims, *(rot_scaling[k] for k in ("factor", "original", "fast", "slow")))
        else:
            self.freq = rotary_frequencies(rot_base, rot_dims)
        self.explicit_prefill = True

    def cache_spec(self):
        return None if self.kv_from is not None else ("latent", self.R + self.rot)

    def cache_signature(self):
        """What a layer that borrows this layer's rows must share with it."""
        return (self.R, self.rot, self.rot_dims, self.rot_layout, self.rot_gain, tuple(self.freq.tolist()))

    def load(self, take, pre):
        H, dim, rot, vdim, Q, R, D = self.H, self.dim, self.rot, self.vdim, self.Q, self.R, self.D
        self.w = dict(dq=take(pre + "dq", (Q, D)), qn=take(pre + "dq.norm", (Q,)), uq=take(pre + "uq", (H * (dim + rot), Q)))
        if self.kv_from is None:
            self.w.update(dkv=take(pre + "dkv", (R + rot, D)), cn=take(pre + "dkv.norm", (R,)))
        self.w.update(uk=take(pre + "uk", (H * dim, R)), uv=take(pre + "uv", (H * vdim, R)),
                      g=take(pre + "g", (H * vdim if self.gate_kind == "element" else H, D)), o=take(pre + "o", (D, H * vdim)))

    def pack(self, prec):
        w, H, dim, rot, vdim, R = self.w, self.H, self.dim, self.rot, self.vdim, self.R
        dev = dict(device="cuda", dtype=prec.dtype)
        uq, dkv = w["uq"], w.get("dkv")
        if self.rot_layout == "half" and self.rot_dims:
            order = torch.tensor(half_to_pair_order(rot, self.rot_dims))
            uq = uq.view(H, dim + rot, -1).clone()
            uq[:, dim:] = uq[:, dim:][:, order]
            uq = uq.reshape(H * (dim + rot), -1)
            if dkv is not None:
                dkv = torch.cat([dkv[:R], dkv[R:][order]], 0)
        parts = [w["dq"]] + ([dkv] if dkv is not None else []) + [w["g"]]
        rows = sum(t.shape[0] for t in parts)
        self.w_in = torch.zeros(rows + (-rows) % 8, self.D, **dev)  # zero rows up to a multiple of 8: a shape the tensor-core product takes
        self.w_in[:rows] = torch.cat(parts, 0).to(**dev)
        self.gate_col = rows - w["g"].shape[0]
        self.w_uq = uq.to(**dev).contiguous()
        self.w_ukT = w["uk"].to(**dev).view(H, dim, R).transpose(1, 2).contiguous()   # [H, R, dim]: q_plain -> latent space
        self.w_uv = w["uv"].to(**dev).view(H, vdim, R).contiguous()
        self.w_ukv = torch.cat([w["uk"], w["uv"]], 0).to(**dev).contiguous()            # explicit-head form
        self.w_o = w["o"].to(**dev).contiguous()
        self.qn = w["qn"].to("cuda", torch.float32)
        self.cn = w["cn"].to("cuda", torch.float32) if "cn" in w else None
        self.freq_d = self.freq.to("cuda")
        self.score = seq_ops.ScoreOptions(H, self.window) if self.window else None

    def __call__(self, h, b, store, li, prec, resid=None, resid_scale=1.0):
        H, dim, rot, vdim, Q, R = self.H, self.dim, self.rot, self.vdim, self.Q, self.R
        T, kd = b.T, R + rot
        own = self.kv_from is None
        pages = store.k_pages[li if own else self.kv_from]
        proj = seq_ops.linear(h, self.w_in, prec.empty(T, self.w_in.shape[0]))
        cq = prec.empty(T, Q)
        seq_ops.latent_prepare(proj, b, self.freq_d, self.qn, self.cn, cq, pages if own else None, Q, R, rot, self.rot_dims, self.eps, PAGE,
                               rot_gain=self.rot_gain)
        q = seq_ops.linear(cq, self.w_uq, prec.empty(T, H * (dim + rot))).view(T, H, dim + rot)
        per_head = self.gate_kind == "head"
        gate = proj[:, self.gate_col:self.gate_col + (H if per_head else H * vdim)]
        att = prec.empty(T, H, vdim)
        # rows of the lazily gathered scratch stay zero-padded to whole pages: every page a key tile touches exists
        explicit = (self.explicit_prefill and not prec.f32 and b.singles < b.E and (dim + rot, vdim) in seq_ops.MMA_HEAD_SIZES
                    and R % 8 == 0 and (H * (dim + vdim)) % 8 == 0 and b.dense_pages is not None)
        if not explicit or b.singles:
            # absorbed form; beside the explicit one it serves the single-token entries only (it still forms the absorbed query
            # of every row: a mixed step is at most a few hundred rows)
            qlat = prec.empty(T, H, kd)
            seq_ops.linear_batched(q[:, :, :dim], self.w_ukT, qlat[:, :, :R])
            seq_ops.rotate_heads(q[:, :, dim:], qlat[:, :, R:], b.pos, self.freq_d, self.rot_dims, self.rot_gain)
            olat = prec.empty(T, H, R)
            seq_ops.attn_ragged(qlat.view(T, H * kd), pages, pages, gate if per_head else None, olat.view(T, H * R), b, H, 1, kd, R, self.scale, 0.0, PAGE,
                                krow=kd, vrow=kd, gate_per_head=True, only_singles=explicit, score=self.score)
            seq_ops.linear_batched(olat, self.w_uv, att)
            if not per_head:  # the gate has the values' width: it multiplies after the value up projection
                seq_ops.sigmoid_gate_mul(att.view(T, H * vdim), gate)
        if explicit:
            # explicit heads for the multi-token entries (their rows of `att` are written last)
            kx, vx = seq_ops.latent_expand(pages, b, self.w_ukv, H, dim, rot, vdim, R, PAGE, prec)
            qr = q[:, :, dim:]
            seq_ops.rotate_heads(qr, qr, b.pos, self.freq_d, self.rot_dims, self.rot_gain)
            seq_ops.attn_ragged(q.view(T, H * (dim + rot)), kx, vx, gate, att.view(T, H * vdim), seq_ops.dense_view(b), H, H, dim + rot, vdim,
                                self.scale, 0.0, PAGE, gate_per_head=per_head, skip_singles=True, score=self.score)
        if resid is not None:
            return seq_ops.linear_add(att.view(T, H * vdim), self.w_o, resid, scale=resid_scale)
        return seq_ops.linear(att.view(T, H * vdim), self.w_o, torch.empty(T, self.D, device="cuda", dtype=torch.float32))


class PolyNormFeedForward:
    """W_down P(W_up h + b_up) + b_down with P(z) = a N(z) + b N(z^2) + c N(z^3) + e: powers element by element, N divides a row by its
    root mean square (eps inside the root), (a, b, c, e) learned.  The statistics need the whole row of the up projection, so the
    activation is a row kernel between the two products (fp32 sums over the stored activations), not a GEMM epilogue."""

    def __init__(self, width, ff, eps, bias=True):
        self.D, self.F, self.eps, self.bias = int(width), int(ff), float(eps), bool(bias)

    def load(self, take, pre):
        F, D = self.F, self.D
        self.w = dict(up=take(pre + "up", (F, D)), down=take(pre + "down", (D, F)), act=take(pre + "act", (4,)))
        if self.bias:
            self.w.update(up_b=take(pre + "up.b", (F,)), down_b=take(pre + "down.b", (D,)))

    def pack(self, prec):
        w = self.w
        f32 = dict(device="cuda", dtype=torch.float32)
        self.w_up = w["up"].to("cuda", prec.dtype).contiguous()
        self.w_down = w["down"].to("cuda", prec.dtype).contiguous()
        self.coef = w["act"].to(**f32).contiguous()
        self.b_up = w["up_b"].to(**f32).contiguous() if self.bias else None
        self.b_down = w["down_b"].to(**f32).contiguous() if self.bias else None

    def __call__(self, h, b, prec, resid=None, resid_scale=1.0):
        T = h.shape[0]
        z = seq_ops.linear(h, self.w_up, prec.empty(T, self.F), bias=self.b_up)
        mid = seq_ops.polynorm(z, self.coef, z, self.eps)
        if resid is not None:
            return seq_ops.linear_add(mid, self.w_down, resid, bias=self.b_down, scale=resid_scale)
        return seq_ops.linear(mid, self.w_down, torch.empty(T, self.D, device="cuda", dtype=torch.float32), bias=self.b_down)


class SquaredReluFeedForward:
    """W_down relu(W_up h)^2."""

    def __init__(self, width, ff):
        self.D, self.F = width, ff

    def load(self, take, pre):
        self.w = dict(up=take(pre + "up", (self.F, self.D)), down=take(pre + "down", (self.D, self.F)))

    def pack(self, prec):
        self.w_up = self.w["up"].to("cuda", prec.dtype).contiguous()
        self.w_down = self.w["down"].to("cuda", prec.dtype).contiguous()

    def __call__(self, h, b, prec):
        T = h.shape[0]
        mid = seq_ops.linear(h, self.w_up, prec.empty(T, self.F), act=seq_ops.ACT_RELU2)
        return seq_ops.linear(mid, self.w_down, torch.empty(T, self.D, device="cuda", dtype=torch.float32))


class RoutedFeedForward:
    """Mixture of experts.  Router: p = softmax(W_r h + b_r) in fp32 over `experts + identity` outputs; the choice uses
    p + correction, limited to the `group_keep` best of `group_count` runs of neighbouring outputs; the `top` chosen outputs
    weigh in with p / sum(p chosen) * scale (without a correction that is the softmax over the chosen logits alone, chosen by
    the largest logits).  The last `identity` outputs return h itself.  A shared expert (optional) is added for every token,
    times sigmoid(w_sg . h) when it is gated.  activation "relu2": experts W_down relu(W_up h)^2; "silu_glu": experts
    W_down (silu(W_gate h) * W_up h)."""

    def __init__(self, width, experts, identity, top, group_count, group_keep, scale, expert_ff, shared_ff, activation="relu2",
                 correction=True, router_bias=False, shared_gate=False):
        if activation not in ("relu2", "silu_glu"):
            raise ValueError(f"unknown expert activation {activation!r}")
        self.D, self.n_real, self.n_all, self.top = width, int(experts), int(experts) + int(identity), int(top)
        self.group_count, self.group_keep, self.scale, self.F = int(group_count), int(group_keep), float(scale), int(expert_ff)
        if self.group_count > 1 and self.n_all % self.group_count:
            raise ValueError("router outputs must divide into equal groups")
        self.glu, self.has_correction, self.router_bias = activation == "silu_glu", bool(correction), bool(router_bias)
        if not shared_ff:
            self.shared = None
        else:
            self.shared = GluFeedForward(width, int(shared_ff), "silu") if self.glu else SquaredReluFeedForward(width, int(shared_ff))
        self.shared_gate = bool(shared_gate) and self.shared is not None

    def load(self, take, pre):
        D, F = self.D, self.F
        self.w = dict(router=take(pre + "router", (self.n_all, D)), up=[take(f"{pre}e{e}.up", (F, D)) for e in range(self.n_real)],
                      down=[take(f"{pre}e{e}.down", (D, F)) for e in range(self.n_real)])
        if self.glu:
            self.w["gate"] = [take(f"{pre}e{e}.gate", (F, D)) for e in range(self.n_real)]
        if self.has_correction:
            self.w["correction"] = take(pre + "correction", (self.n_all,))
        if self.router_bias:
            self.w["router_b"] = take(pre + "router.b", (self.n_all,))
        if self.shared is not None:
            self.shared.load(take, pre + "shared.")
        if self.shared_gate:
            self.w["sg"] = take(pre + "shared.sg", (1, D))

    def pack(self, prec):
        w = self.w
        # router rows padded with zeros to a multiple of 8: a shape the tensor-core product takes (the choice only reads n_all columns)
        # (the shared expert's gate vector is one more row of the same product: column n_all of the logits)
        n_pad = (self.n_all + int(self.shared_gate) + 7) // 8 * 8
        self.w_router = torch.zeros(n_pad, self.D, device="cuda", dtype=prec.dtype)
        self.w_router[:self.n_all] = w["router"].to("cuda", prec.dtype)
        if self.shared_gate:
            self.w_router[self.n_all] = w["sg"][0].to("cuda", prec.dtype)
        self.correction = w["correction"].to("cuda", torch.float32).contiguous() if self.has_correction else None
        self.router_b = w["router_b"].to("cuda", torch.float32).contiguous() if self.router_bias else None
        if self.n_real:
            if self.glu:
                # rows alternate gate / up: an accumulator pair of the grouped product's epilogue is one output feature
                gu = torch.stack([torch.stack(w["gate"]), torch.stack(w["up"])], 2)  # [n, F, 2, D]
                self.w_up = gu.reshape(self.n_real, 2 * self.F, self.D).to("cuda", prec.dtype).contiguous()
                self.w_up_dense = None
                if prec.dtype == torch.bfloat16 and self.F % 64 == 0 and self.D % 8 == 0:
                    # second copy for the per-expert dense products of long prompt portions: [64 gate | 64 up] row blocks, the order
                    # the tcgen05 product's gated epilogue reads
                    blk = torch.stack([torch.stack(w["gate"]).view(self.n_real, -1, 64, self.D), torch.stack(w["up"]).view(self.n_real, -1, 64, self.D)], 2)
                    self.w_up_dense = blk.reshape(self.n_real, 2 * self.F, self.D).to("cuda", prec.dtype).contiguous()
            else:
                self.w_up = torch.stack(w["up"]).to("cuda", prec.dtype).contiguous()
            self.w_down = torch.stack(w["down"]).to("cuda", prec.dtype).contiguous()
        if self.shared is not None:
            self.shared.pack(prec)

    # at least this many (token, choice) pairs per real expert on average before a host round trip for the counts pays
    DENSE_SEGMENT_ROWS = 256

    def _dense_segments(self, T, prec):
        return ((not self.glu or self.w_up_dense is not None) and not prec.f32 and self.D % 8 == 0 and self.F % 8 == 0 and T * self.top >= self.DENSE_SEGMENT_ROWS * self.n_real
                and not torch.cuda.is_current_stream_capturing())

    def expert_products(self, h, plan, counts, prec):
        """fp32 rows [pairs, D] in the plan's sorted order: the expert's output for every (token, real expert) pair."""
        T = h.shape[0]
        if self._dense_segments(T, prec):
            # many rows per expert (prompt portions): the pair counts come to the host once per layer, every expert's tokens are
            # gathered into one contiguous run and each expert is two dense tcgen05 products on its run
            per = (C.c_int * self.n_real)(*counts.tolist())
            xg = seq_ops.moe_gather_rows(h, plan, prec.empty(plan.pairs, self.D))
            mid = prec.empty(plan.pairs, self.F)
            eo = torch.empty(plan.pairs, self.D, device="cuda", dtype=torch.float32)
            w_up = self.w_up_dense if self.glu else self.w_up
            _lib.check(_lib.lib().pg_moe_dense_runs(xg.data_ptr(), xg.stride(0), w_up.data_ptr(), self.w_down.data_ptr(), mid.data_ptr(), mid.stride(0),
                                                    eo.data_ptr(), eo.stride(0), C.addressof(per), self.n_real, self.D, self.F, int(self.glu), _lib.stream()),
                       "pg_moe_dense_runs")
            return eo
        mid = seq_ops.moe_gemm(h, plan, self.w_up, prec.empty(plan.pairs, self.F), gather=True, act=seq_ops.ACT_SILU_GLU if self.glu else seq_ops.ACT_RELU2)
        return seq_ops.moe_gemm(mid, plan, self.w_down, torch.empty(plan.pairs, self.D, device="cuda", dtype=torch.float32), gather=False)

    def __call__(self, h, b, prec, resid=None):
        T = h.shape[0]
        z = seq_ops.linear(h, self.w_router, torch.empty(T, self.w_router.shape[0], device="cuda", dtype=torch.float32))
        ids, wts, counts = seq_ops.moe_route(z[:, :self.n_all], self.correction, self.n_real, self.top, self.group_count, self.group_keep, self.scale,
                                             logit_bias=self.router_b)
        plan = seq_ops.MoePlan(ids, counts, max(1, self.n_real))
        eo = self.expert_products(h, plan, counts, prec) if self.n_real else None
        sh = self.shared(h, b, prec) if self.shared is not None else None
        sg = z[:, self.n_all:self.n_all + 1] if self.shared_gate else None
        if resid is not None:
            return seq_ops.moe_combine(eo, plan, ids, wts, h, sh, resid, shared_gate=sg, accumulate=True)
        return seq_ops.moe_combine(eo, plan, ids, wts, h, sh, torch.empty(T, self.D, device="cuda", dtype=torch.float32), shared_gate=sg)


class StreamCoefficients:
    """Read vector a [S], write vector b [S] and mixing matrix M [S from, S to] of one sub-layer over a multi-stream residual:
    the sub-layer reads sum_s a_s x_s and every stream becomes sum_s M[s, t] x_s + b_t y.  `plain(S)` is the ordinary residual
    sum (one stream, all ones)."""

    def __init__(self, S):
        self.S = S
        self.w = None

    def load(self, take, pre):
        S = self.S
        self.w = dict(read=take(pre + "in", (S,)), write=take(pre + "out", (S,)), mix=take(pre + "mix", (S, S)))

    def pack(self):
        f32 = dict(device="cuda", dtype=torch.float32)
        if self.w is None:
            self.read, self.write, self.mix = torch.ones(self.S, **f32), torch.ones(self.S, **f32), torch.eye(self.S, **f32)
        else:
            self.read, self.write, self.mix = (self.w[k].to(**f32).contiguous() for k in ("read", "write", "mix"))
