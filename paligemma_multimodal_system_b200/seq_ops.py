"""Host wrappers of the ragged-step kernels (csrc/seq_elementwise.cu, csrc/seq_mixers.cu) and the step's batch descriptor.

`Precision` says in which type activations and matrix operands live: bf16 (tcgen05 GEMMs with fp32 accumulation wherever
the shape allows TMA, the plain-FMA kernel otherwise) or fp32 (plain-FMA GEMMs only, no reduced-precision tensor mode).
Norm statistics, attention scores and probabilities, recurrent states and the residual stream are fp32 in both.
"""
import dataclasses
from typing import List, Optional, Sequence

import numpy as np
import torch

from . import _lib


class Precision:
    def __init__(self, dtype: torch.dtype):
        if dtype not in (torch.bfloat16, torch.float32):
            raise ValueError("activation type must be torch.bfloat16 or torch.float32")
        self.dtype = dtype
        self.f32 = int(dtype == torch.float32)

    def empty(self, *shape):
        return torch.empty(*shape, device="cuda", dtype=self.dtype)


@dataclasses.dataclass
class StepBatch:
    """One ragged step on the device.  Rows are tokens; entry e owns rows [row0[e], row0[e] + n[e])."""
    T: int
    E: int
    max_n: int
    tokens: torch.Tensor      # int32 [T]
    pos: torch.Tensor         # int32 [T] position of the row inside its sequence
    row_entry: torch.Tensor   # int32 [T]
    row0: torch.Tensor        # int32 [E]
    n: torch.Tensor           # int32 [E]
    ctx: torch.Tensor         # int32 [E] tokens of the sequence already stored before this step
    slot: torch.Tensor        # int32 [E] recurrent-state slot
    page_table: torch.Tensor  # int32 [E, max_pages]
    max_pages: int
    singles: int = 0          # entries with one new token (decode rows)
    max_single_ctx: int = 0   # the longest context among them
    # dense scratch layout of the entries with several new tokens (mixers that rebuild per-head keys / values from a compact
    # cache): entry e owns rows [dense_row0[e], + ctx + n) of a dense matrix, starting on a page boundary, so that
    # dense_pages[e] = consecutive page numbers is a page table over the scratch and the paged attention kernels read it
    dense_row0: Optional[torch.Tensor] = None   # int32 [E]
    dense_pages: Optional[torch.Tensor] = None  # int32 [E, dense_max_pages]
    dense_max_pages: int = 0
    dense_rows: int = 0       # rows of the scratch matrix (a multiple of the page size)
    dense_max_len: int = 0    # the longest ctx + n among those entries


def make_step_batch(entries: Sequence[dict]) -> StepBatch:
    """entries: dicts with tokens (list[int]), ctx (int), slot (int), pages (list[int]).  One host buffer, one copy."""
    E = len(entries)
    ns = [len(e["tokens"]) for e in entries]
    T = sum(ns)
    if E == 0 or min(ns) <= 0:
        raise ValueError("a step needs at least one entry and every entry at least one token")
    max_pages = max(1, max(len(e["pages"]) for e in entries))
    lens = [e["ctx"] + k if k > 1 else 0 for e, k in zip(entries, ns)]
    dpages = [(l + 63) // 64 for l in lens]
    dmax = max(1, max(dpages))
    buf = np.zeros(3 * T + 4 * E + E * max_pages + E + E * dmax, dtype=np.int32)
    tokens, pos, row_entry = buf[:T], buf[T:2 * T], buf[2 * T:3 * T]
    o = 3 * T
    row0, n, ctx, slot = buf[o:o + E], buf[o + E:o + 2 * E], buf[o + 2 * E:o + 3 * E], buf[o + 3 * E:o + 4 * E]
    pt = buf[o + 4 * E:o + 4 * E + E * max_pages].reshape(E, max_pages)
    o2 = o + 4 * E + E * max_pages
    drow0, dpt = buf[o2:o2 + E], buf[o2 + E:].reshape(E, dmax)
    page0 = 0
    for i in range(E):
        drow0[i] = page0 * 64
        dpt[i, :dpages[i]] = np.arange(page0, page0 + dpages[i])
        page0 += dpages[i]
    r = 0
    for i, e in enumerate(entries):
        k = ns[i]
        if (e["ctx"] + k + 63) // 64 > len(e["pages"]):
            raise ValueError("entry does not own enough pages for its new tokens")
        tokens[r:r + k] = e["tokens"]
        pos[r:r + k] = np.arange(e["ctx"], e["ctx"] + k)
        row_entry[r:r + k] = i
        row0[i], n[i], ctx[i], slot[i] = r, k, e["ctx"], e["slot"]
        pt[i, :len(e["pages"])] = e["pages"]
        r += k
    dev = torch.from_numpy(buf).pin_memory().to("cuda", non_blocking=True)
    o = 3 * T
    return StepBatch(T=T, E=E, max_n=max(ns), tokens=dev[:T], pos=dev[T:2 * T], row_entry=dev[2 * T:3 * T], row0=dev[o:o + E],
                     n=dev[o + E:o + 2 * E], ctx=dev[o + 2 * E:o + 3 * E], slot=dev[o + 3 * E:o + 4 * E],
                     page_table=dev[o + 4 * E:o2].view(E, max_pages), max_pages=max_pages, singles=sum(k == 1 for k in ns),
                     max_single_ctx=max([e["ctx"] for e, k in zip(entries, ns) if k == 1], default=0),
                     dense_row0=dev[o2:o2 + E], dense_pages=dev[o2 + E:].view(E, dmax), dense_max_pages=dmax, dense_rows=page0 * 64,
                     dense_max_len=max(lens))


class StaticDecodeBatch:
    """Fixed-address StepBatch for steps of E single-token entries (a decode step), so that the step can be captured once in a
    CUDA graph and replayed: `fill` rewrites the pinned host image and copies it over the device buffer in stream order.
    `pages_cap` is the page-table width the graph was captured with; `ctx_cap` the context bound that fixed its key split."""

    def __init__(self, E: int, pages_cap: int, ctx_cap: int):
        self.E, self.pages_cap, self.ctx_cap = E, pages_cap, ctx_cap
        n = 7 * E + E * pages_cap
        self.host = torch.zeros(n, dtype=torch.int32).pin_memory()
        self.dev = torch.zeros(n, dtype=torch.int32, device="cuda")
        d = self.dev
        self.batch = StepBatch(T=E, E=E, max_n=1, tokens=d[:E], pos=d[E:2 * E], row_entry=d[2 * E:3 * E], row0=d[3 * E:4 * E], n=d[4 * E:5 * E],
                               ctx=d[5 * E:6 * E], slot=d[6 * E:7 * E], page_table=d[7 * E:].view(E, pages_cap), max_pages=pages_cap, singles=E,
                               max_single_ctx=ctx_cap)
        self.rows = torch.arange(E, device="cuda", dtype=torch.int64)
        self._copied = None

    def fill(self, entries: Sequence[dict]):
        E, h = self.E, self.host.numpy()
        assert len(entries) == E
        if self._copied is not None:
            self._copied.synchronize()  # the previous image must have left the pinned buffer before it is rewritten
        h[7 * E:] = 0
        pt = h[7 * E:].reshape(E, self.pages_cap)
        for i, e in enumerate(entries):
            assert len(e["tokens"]) == 1 and len(e["pages"]) <= self.pages_cap and e["ctx"] <= self.ctx_cap
            h[i], h[E + i], h[2 * E + i], h[3 * E + i], h[4 * E + i], h[5 * E + i], h[6 * E + i] = e["tokens"][0], e["ctx"], i, i, 1, e["ctx"], e["slot"]
            pt[i, :len(e["pages"])] = e["pages"]
        self.dev.copy_(self.host, non_blocking=True)
        self._copied = torch.cuda.Event()
        self._copied.record()


def _aligned(t, n=16):
    return t.data_ptr() % n == 0


ACT_NONE, ACT_GELU, ACT_RELU2, ACT_SILU_GLU = 0, 1, 2, 3  # ACT_SILU_GLU: grouped products only (gate / up rows alternate)


def linear(x: torch.Tensor, w: torch.Tensor, out: torch.Tensor, act: int = ACT_NONE, bias: Optional[torch.Tensor] = None):
    """out[t, f] = act(sum_k x[t, k] w[f, k] + bias[f]) (bias fp32 or None).  x, w share a type (bf16 / fp32); out is bf16 or fp32.  bf16 operands go to the
    tcgen05 kernel when TMA can describe them (16-byte pitches and bases), everything else to the plain-FMA kernel.
    act = ACT_RELU2 (relu squared; out in the operands' type): in the tensor-core kernel's bf16 epilogue, else a pass of its own."""
    T, K = x.shape
    F = w.shape[0]
    assert x.dtype == w.dtype and w.shape[1] == K and out.shape[0] == T and out.shape[1] == F
    assert x.stride(1) == 1 and w.stride(1) == 1 and out.stride(1) == 1
    if (x.dtype == torch.bfloat16 and K % 8 == 0 and x.stride(0) % 8 == 0 and w.stride(0) % 8 == 0 and F % 8 == 0
            and out.stride(0) % 8 == 0 and _aligned(x) and _aligned(w) and _aligned(out)):
        assert act == ACT_NONE or out.dtype == torch.bfloat16
        if act != ACT_NONE:
            return _lib.gemm(x, w, out, mode=_lib.EPI_BF16, act_gelu=act, swap=1 if T <= 128 else 0, bias=bias)
        if T <= 128 and out.dtype == torch.float32 and bias is None:
            # few rows, few 128-feature tiles (output and down projections): split K over CTAs so that the whole GPU streams the
            # weights; the fp32 partials are red.add-ed into the zeroed output (as the framework's other decode GEMMs do)
            tiles, kb = (F + 127) // 128, (K + 63) // 64
            split = max(1, min(kb // 4, (2 * _lib.num_sms()) // tiles))
            if split > 1:
                out.zero_()
                return _lib.gemm(x, w, out, mode=_lib.EPI_ATOMIC_F32, swap=1, split_k=split)
        return _lib.gemm(x, w, out, mode=_lib.EPI_F32 if out.dtype == torch.float32 else _lib.EPI_BF16, swap=1 if T <= 128 else 0, bias=bias)
    if x.dtype == torch.float32 and out.dtype != torch.float32:
        raise ValueError("fp32 operands produce fp32 outputs")
    if bias is not None:
        assert bias.dtype == torch.float32 and bias.numel() == F and bias.is_contiguous()
        _lib.check(_lib.lib().pg_gemm_simt_bias(x.data_ptr(), x.stride(0), w.data_ptr(), w.stride(0), out.data_ptr(), out.stride(0), bias.data_ptr(), 0, 1.0,
                                                T, F, K, int(x.dtype == torch.float32), int(out.dtype == torch.float32), _lib.stream()), "pg_gemm_simt_bias")
    else:
        _lib.check(_lib.lib().pg_gemm_simt(x.data_ptr(), x.stride(0), w.data_ptr(), w.stride(0), out.data_ptr(), out.stride(0), T, F, K,
                                           int(x.dtype == torch.float32), int(out.dtype == torch.float32), _lib.stream()), "pg_gemm_simt")
    if act == ACT_RELU2:
        _lib.check(_lib.lib().pg_relu2(out.data_ptr(), out.stride(0), T, F, int(out.dtype == torch.float32), _lib.stream()), "pg_relu2")
    elif act != ACT_NONE:
        raise ValueError("the plain-FMA product has no fused activation but relu squared")
    return out


def linear_add(x: torch.Tensor, w: torch.Tensor, resid: torch.Tensor, bias: Optional[torch.Tensor] = None, scale: float = 1.0):
    """resid[t, f] += (sum_k x[t, k] w[f, k] + bias[f]) * scale: a projection that ends in the fp32 residual stream.  bf16 operands TMA can
    describe: the tcgen05 kernel adds the residual in its epilogue (or red.adds split-K partials into it when there are few
    tiles); everything else: the plain-FMA kernel reads and rewrites the residual element."""
    T, K = x.shape
    F = w.shape[0]
    assert x.dtype == w.dtype and w.shape[1] == K and resid.shape == (T, F) and resid.dtype == torch.float32 and resid.is_contiguous()
    assert x.stride(1) == 1 and w.stride(1) == 1
    if (x.dtype == torch.bfloat16 and K % 8 == 0 and x.stride(0) % 8 == 0 and w.stride(0) % 8 == 0 and F % 8 == 0 and _aligned(x) and _aligned(w)
            and _aligned(resid)):
        return _lib.gemm_residual(x, w, resid, bias=bias, scale=float(scale))
    assert bias is None or (bias.dtype == torch.float32 and bias.numel() == F and bias.is_contiguous())
    _lib.check(_lib.lib().pg_gemm_simt_bias(x.data_ptr(), x.stride(0), w.data_ptr(), w.stride(0), resid.data_ptr(), resid.stride(0), _lib.ptr(bias), 1, float(scale),
                                            T, F, K, int(x.dtype == torch.float32), 1, _lib.stream()), "pg_gemm_simt_bias")
    return resid


def layernorm_shift(x, w1, b1, out1, eps, shift=None, state=None, b: "StepBatch" = None, w2=None, b2=None, out2=None):
    """out1 = LN(x; w1, b1) -- blended with the previous token's when `shift` [D] is given (state: fp32 [slots, D], the batch says which
    row continues which sequence) -- and out2 = LN(x; w2, b2) from the same statistics.  x fp32 [rows, D]; outputs bf16 or fp32."""
    rows, D = x.shape
    assert x.dtype == torch.float32 and x.is_contiguous() and out1.is_contiguous() and out1.shape == x.shape
    for t in (w1, b1, shift, w2, b2):
        assert t is None or (t.dtype == torch.float32 and t.is_contiguous() and t.numel() == D)
    assert out2 is None or (out2.is_contiguous() and out2.shape == x.shape and out2.dtype == out1.dtype and w2 is not None and b2 is not None)
    if shift is not None:
        assert state is not None and state.dtype == torch.float32 and state.is_contiguous() and state.shape[-1] == D and b is not None and b.T == rows
    _lib.check(_lib.lib().pg_layernorm_shift(x.data_ptr(), w1.data_ptr(), b1.data_ptr(), _lib.ptr(shift), _lib.ptr(w2), _lib.ptr(b2), out1.data_ptr(),
                                             _lib.ptr(out2), _lib.ptr(state), *((b.pos.data_ptr(), b.row_entry.data_ptr(), b.row0.data_ptr(),
                                                                                 b.n.data_ptr(), b.slot.data_ptr()) if shift is not None else (0, 0, 0, 0, 0)),
                                             rows, D, float(eps), int(out1.dtype == torch.float32), _lib.stream()), "pg_layernorm_shift")


def rmsnorm_conv(x, w, out_h, out_conv, eps, conv_w=None, state=None, b: "StepBatch" = None):
    """h = x / rms(x) * w (w fp32: [D], or one number) -> out_h; out_conv = h + causal convolution of h over time per channel (conv_w fp32
    [taps, D], tap-major, the oldest tap first; the last taps - 1 rows h of every sequence are kept in state fp32 [slots, taps - 1, D]; the batch says which rows continue which
    sequence).  conv_w None: a bare norm.  x fp32 [rows, D]; outputs bf16 or fp32 (either may be None)."""
    rows, D = x.shape
    assert x.dtype == torch.float32 and x.is_contiguous() and w.dtype == torch.float32 and w.numel() in (1, D) and w.is_contiguous()
    outs = [o for o in (out_h, out_conv) if o is not None]
    assert outs and all(o.is_contiguous() and o.shape == x.shape and o.dtype == outs[0].dtype for o in outs)
    taps = 0
    if conv_w is not None:
        assert conv_w.dtype == torch.float32 and conv_w.is_contiguous() and conv_w.shape[1] == D and out_conv is not None
        taps = conv_w.shape[0]
        if taps > 1:
            assert state is not None and state.dtype == torch.float32 and state.is_contiguous() and tuple(state.shape[1:]) == (taps - 1, D)
            assert b is not None and b.T == rows
    ent = (b.row_entry.data_ptr(), b.row0.data_ptr(), b.n.data_ptr(), b.ctx.data_ptr(), b.slot.data_ptr()) if taps > 1 else (0, 0, 0, 0, 0)
    _lib.check(_lib.lib().pg_rmsnorm_conv(x.data_ptr(), w.data_ptr(), int(w.numel() == 1 and D != 1), _lib.ptr(conv_w), taps, _lib.ptr(state) if taps > 1 else 0,
                                          _lib.ptr(out_h), _lib.ptr(out_conv), *ent, rows, b.E if taps > 1 else 0, D, float(eps), int(outs[0].dtype == torch.float32), _lib.stream()),
               "pg_rmsnorm_conv")


def polynorm(z, coef, out, eps):
    """out = a N(z) + b N(z^2) + c N(z^3) + e per row, N(v) = v / sqrt(mean(v^2) + eps), (a, b, c, e) = coef (fp32 [4], device)."""
    rows, F = z.shape
    assert z.dtype == out.dtype and out.shape == z.shape and z.stride(1) == 1 and out.stride(1) == 1 and coef.dtype == torch.float32 and coef.numel() == 4
    _lib.check(_lib.lib().pg_polynorm(z.data_ptr(), z.stride(0), coef.data_ptr(), out.data_ptr(), out.stride(0), rows, F, float(eps),
                                      int(z.dtype == torch.float32), _lib.stream()), "pg_polynorm")
    return out


def sigmoid_gate_mul(y, gate):
    """y[t, c] *= sigmoid(gate[t, c]) in place (one type; any row pitch)."""
    rows, n = y.shape
    assert gate.shape == y.shape and gate.dtype == y.dtype and y.stride(1) == 1 and gate.stride(1) == 1
    _lib.check(_lib.lib().pg_sigmoid_gate_mul(y.data_ptr(), y.stride(0), gate.data_ptr(), gate.stride(0), rows, n, int(y.dtype == torch.float32),
                                              _lib.stream()), "pg_sigmoid_gate_mul")
    return y


GLU_SILU, GLU_CLAMPED = 1, 2


def glu(gu, out, kind, limit=0.0, alpha=1.0):
    """out[t, f] from the [gate | up] product gu [rows, 2F]: GLU_SILU silu(g) * u; GLU_CLAMPED min(g, limit) * sigmoid(alpha * .) * (clamp(u) + 1)."""
    rows, F = out.shape
    assert gu.shape[1] == 2 * F and gu.dtype == out.dtype and gu.stride(1) == 1 and out.stride(1) == 1
    _lib.check(_lib.lib().pg_glu(gu.data_ptr(), gu.stride(0), out.data_ptr(), out.stride(0), rows, F, int(kind), float(limit), float(alpha),
                                 int(out.dtype == torch.float32), _lib.stream()), "pg_glu")
    return out


def embed_rows(tokens, table, col0, D, scale):
    out = torch.empty(tokens.numel(), D, device="cuda", dtype=torch.float32)
    _lib.check(_lib.lib().pg_embed_rows(tokens.data_ptr(), table.data_ptr(), table.stride(0), int(col0), out.data_ptr(), tokens.numel(), D,
                                        float(scale), int(table.dtype == torch.float32), _lib.stream()), "pg_embed_rows")
    return out


def group_rmsnorm_add(y, w, x, out_act, groups, eps):
    """x += gnorm(y) * w (x fp32, in place; x None: bare norm); out_act (bf16 / fp32, may be None) gets a copy of the result."""
    rows, D = y.shape
    assert y.dtype == torch.float32 and y.stride(1) == 1 and w.dtype == torch.float32 and w.numel() == D
    assert x is None or (x.dtype == torch.float32 and x.is_contiguous() and x.shape == y.shape)
    assert out_act is None or (out_act.is_contiguous() and out_act.shape == y.shape)
    _lib.check(_lib.lib().pg_group_rmsnorm_add(y.data_ptr(), y.stride(0), w.data_ptr(), _lib.ptr(x), _lib.ptr(out_act), rows, D, int(groups),
                                               float(eps), int(out_act is not None and out_act.dtype == torch.float32), _lib.stream()),
               "pg_group_rmsnorm_add")


def rmsnorm_gate(o, w, gate, out, eps):
    rows, D = o.shape
    assert o.dtype == torch.float32 and o.is_contiguous() and gate.dtype == out.dtype and out.is_contiguous() and gate.stride(1) == 1
    _lib.check(_lib.lib().pg_rmsnorm_gate(o.data_ptr(), w.data_ptr(), gate.data_ptr(), gate.stride(0), out.data_ptr(), rows, D, float(eps),
                                          int(out.dtype == torch.float32), _lib.stream()), "pg_rmsnorm_gate")


def geglu(gu, out):
    rows, F = out.shape
    assert gu.shape[1] == 2 * F and gu.dtype == out.dtype
    _lib.check(_lib.lib().pg_geglu(gu.data_ptr(), gu.stride(0), out.data_ptr(), out.stride(0), rows, F, int(out.dtype == torch.float32),
                                   _lib.stream()), "pg_geglu")


def side_gate(z, tokens, table, col0, out, n):
    rows, n_pad = out.shape
    assert z.dtype == torch.float32 and out.dtype == table.dtype
    _lib.check(_lib.lib().pg_side_gate(z.data_ptr(), z.stride(0), tokens.data_ptr(), table.data_ptr(), table.stride(0), int(col0), out.data_ptr(),
                                       out.stride(0), rows, int(n), n_pad, int(out.dtype == torch.float32), _lib.stream()), "pg_side_gate")


def attn_prepare(qkv, b: StepBatch, freq, q_norm, k_norm, q_out, k_pages, v_pages, H, G, dim, vdim, rot_dims, eps, page, norm_qk=True, norm_v=True,
                 v_from_k=False):
    """q_norm / k_norm None: norms without a weight; norm_qk / norm_v False: no q/k norm / no value norm; k_pages and v_pages None: the
    rows hold queries only (the layer attends over another layer's cache); v_from_k: the rows have no value columns, the values are the
    keys as projected (before norm and rotation)."""
    assert qkv.stride(1) == 1 and freq.dtype == torch.float64 and qkv.dtype == q_out.dtype and (k_pages is None) == (v_pages is None)
    assert k_pages is None or k_pages.dtype == qkv.dtype
    _lib.check(_lib.lib().pg_attn_prepare(qkv.data_ptr(), qkv.stride(0), b.pos.data_ptr(), b.row_entry.data_ptr(), b.page_table.data_ptr(),
                                          b.max_pages, page, freq.data_ptr(), _lib.ptr(q_norm), _lib.ptr(k_norm), q_out.data_ptr(),
                                          _lib.ptr(k_pages), _lib.ptr(v_pages), b.T, H, G, dim, vdim, rot_dims, float(eps), int(bool(norm_qk)),
                                          int(bool(norm_v)), int(bool(v_from_k)), int(qkv.dtype == torch.float32), _lib.stream()), "pg_attn_prepare")


class ScoreOptions:
    """The optional parts of a softmax attention's score and mask, as the kernels read them (PgAttnScore): a sliding window of
    `window` keys (None: all) that keeps the first `keep_first` keys of the sequence visible, a per-head sink logit in the softmax
    denominator, a penalty dist_a[h] * log(1 + dist_b[h] * distance), a per-head score multiplier.  Tensors: fp32 [H] on the device."""

    def __init__(self, heads, window=None, keep_first=0, sink=None, dist_a=None, dist_b=None, head_scale=None):
        for t in (sink, dist_a, dist_b, head_scale):
            assert t is None or (t.is_cuda and t.dtype == torch.float32 and t.is_contiguous() and t.numel() == heads)
        assert (dist_a is None) == (dist_b is None)
        self.window = int(window) if window else 0
        self.keep_first = int(keep_first) if self.window else 0
        self._keep = (sink, dist_a, dist_b, head_scale)  # the struct holds raw pointers
        self.window_only = sink is None and dist_a is None and head_scale is None and not self.keep_first  # nothing but a plain sliding window
        self.c = _lib.AttnScore(self.window, self.keep_first, _lib.ptr(sink), _lib.ptr(dist_a), _lib.ptr(dist_b), _lib.ptr(head_scale))

    def visible_keys(self, context):
        """Upper bound of the keys a query at position `context` reads."""
        return context + 1 if not self.window else min(context + 1, self.window + self.keep_first)


# head sizes (dim, vdim) the tensor-core attention kernel is instantiated for
MMA_HEAD_SIZES = {(32, 32), (64, 64), (128, 128), (64, 128), (128, 64), (96, 64), (192, 128)}


# (row width, value width) of a one-row-per-token cache the tensor-core decode kernel is instantiated for
LATENT_MMA_SIZES = {(96, 64), (160, 128), (192, 128), (288, 256), (544, 512), (576, 512)}


def attn_ragged(q, k_pages, v_pages, gate, out, b: StepBatch, H, G, dim, vdim, scale, softcap, page, decode_kernel=True, tensor_cores=True,
                krow=0, vrow=0, gate_per_head=False, only_singles=False, skip_singles=False, score: Optional["ScoreOptions"] = None):
    """Entries with several new rows go to a tiled kernel -- on the tensor cores for bf16 activations and the usual head
    sizes (fp32 probabilities as three bf16 terms), plain fp32 FMAs otherwise -- and entries with ONE new row (decoded tokens)
    to the key-split kernel (`decode_kernel=False`: everything through the tiled kernel).  Same arithmetic, other summation
    order.  krow / vrow: elements per cache row when it is not G * dim / G * vdim (a latent cache: one row is key and value);
    gate_per_head: the gate holds one scalar per head instead of one per output element; only_singles / skip_singles: rows of
    entries with several new tokens / with one new token are left alone (another form computes them).  score: window, sink, distance
    penalty and per-head multiplier (ScoreOptions; None: plain causal attention)."""
    import ctypes as C
    L, f32 = _lib.lib(), int(q.dtype == torch.float32)
    sx = C.addressof(score.c) if score is not None else 0
    reach = score.visible_keys(b.max_single_ctx) if score is not None else b.max_single_ctx + 1  # keys a decoded token reads at most
    ldg = 0 if gate is None else gate.stride(0)
    gph = int(bool(gate_per_head))
    singles = b.singles if (decode_kernel or skip_singles) else 0
    dense_rows = krow in (0, G * dim) and vrow in (0, G * vdim)
    if only_singles:
        pass
    elif (singles < b.E and tensor_cores and not f32 and dense_rows and (dim, vdim) in MMA_HEAD_SIZES
            and (gate is None or gph or (ldg % 2 == 0 and gate.data_ptr() % 4 == 0))):
        _lib.check(L.pg_attn_ragged_mma(q.data_ptr(), k_pages.data_ptr(), v_pages.data_ptr(), _lib.ptr(gate), ldg, out.data_ptr(), b.row0.data_ptr(),
                                        b.n.data_ptr(), b.ctx.data_ptr(), b.page_table.data_ptr(), b.max_pages, page, b.E, b.max_n, H, G, dim, vdim,
                                        float(scale), float(softcap or 0.0), int(singles > 0), gph, sx, _lib.stream()), "pg_attn_ragged_mma")
    elif singles < b.E:
        _lib.check(L.pg_attn_ragged(q.data_ptr(), k_pages.data_ptr(), v_pages.data_ptr(), _lib.ptr(gate), ldg, out.data_ptr(), b.row0.data_ptr(),
                                    b.n.data_ptr(), b.ctx.data_ptr(), b.page_table.data_ptr(), b.max_pages, page, b.E, b.max_n, H, G, dim, vdim,
                                    float(scale), float(softcap or 0.0), int(singles > 0), f32, int(krow), int(vrow), gph, sx, _lib.stream()),
                   "pg_attn_ragged")
    latent = (k_pages.data_ptr() == v_pages.data_ptr() and G == 1 and krow == vrow == dim and k_pages.shape[-1] == dim)
    if (singles and not skip_singles and latent and tensor_cores and not f32 and (dim, vdim) in LATENT_MMA_SIZES and softcap in (0, 0.0, None)
            and (gate is None or gph) and (score is None or score.window_only)):
        # one-row-per-token cache, every head of a token against the same key tile: tensor cores
        window = score.window if score is not None else 0
        tiles = b.max_single_ctx // 64 + 1
        if window:
            tiles = min(tiles, (window + 62) // 64 + 1)  # a window of w keys touches at most this many 64-key tiles
        vs = 2 if vdim > 256 else 1  # value halves are CTAs of their own
        nsplit = max(1, min(tiles, (4 * _lib.num_sms()) // (singles * -(-H // 64) * vs), 32))  # measured: 4 CTAs per SM beat 2 despite the larger merge
        partial = torch.empty(b.E * H * nsplit * (vdim + 2), device="cuda", dtype=torch.float32) if nsplit > 1 else None
        _lib.check(L.pg_attn_latent_decode_mma(q.data_ptr(), k_pages.data_ptr(), _lib.ptr(gate), ldg, out.data_ptr(), _lib.ptr(partial), b.row0.data_ptr(),
                                               b.n.data_ptr(), b.ctx.data_ptr(), b.page_table.data_ptr(), b.max_pages, page, b.E, nsplit, H, dim, vdim,
                                               float(scale), int(window), _lib.stream()), "pg_attn_latent_decode_mma")
        if nsplit > 1:
            _lib.check(L.pg_attn_decode_merge(partial.data_ptr(), _lib.ptr(gate), ldg, out.data_ptr(), b.row0.data_ptr(), b.n.data_ptr(), b.E, nsplit, H,
                                              vdim, gph, 0, 0, _lib.stream()), "pg_attn_decode_merge")
    elif singles and not skip_singles:
        tiles = (reach - 1) // 32 + 1
        # enough CTAs for two waves, but at least two 32-key tiles for every warp of a CTA
        nsplit = max(1, min(-(-2 * _lib.num_sms() // (G * singles)), tiles // 16, 32))
        partial = torch.empty(b.E * H * nsplit * (vdim + 2), device="cuda", dtype=torch.float32) if nsplit > 1 else None
        _lib.check(L.pg_attn_decode(q.data_ptr(), k_pages.data_ptr(), v_pages.data_ptr(), _lib.ptr(gate), ldg, out.data_ptr(), _lib.ptr(partial),
                                    b.row0.data_ptr(), b.n.data_ptr(), b.ctx.data_ptr(), b.page_table.data_ptr(), b.max_pages, page, b.E, nsplit,
                                    H, G, dim, vdim, float(scale), float(softcap or 0.0), f32, int(krow), int(vrow), gph, sx, _lib.stream()),
                   "pg_attn_decode")


# ---- multi-stream residual -------------------------------------------------------------------------------------------
def embed_streams(tokens, table, S, D, scale=1.0):
    xs = torch.empty(tokens.numel(), S, D, device="cuda", dtype=torch.float32)
    _lib.check(_lib.lib().pg_embed_streams(tokens.data_ptr(), table.data_ptr(), table.stride(0), xs.data_ptr(), tokens.numel(), S, D, float(scale),
                                           int(table.dtype == torch.float32), _lib.stream()), "pg_embed_streams")
    return xs


def stream_mix_norm(xs, y=None, mix=None, write=None, read=None, norm_w=None, out_act=None, eps=1e-6):
    """One pass over the stream rows xs [T, S, D] (fp32, in place): the write-back of a finished sub-layer (y fp32 [T, D], mix
    [S, S] from x to, write [S]) and / or the normalised read of the next one (read [S], norm_w [D] -> out_act [T, D])."""
    T, S, D = xs.shape
    assert xs.dtype == torch.float32 and xs.is_contiguous()
    assert y is None or (y.dtype == torch.float32 and y.stride(1) == 1 and y.shape == (T, D))
    for t in (mix, write, read, norm_w):
        assert t is None or (t.dtype == torch.float32 and t.is_contiguous())
    assert out_act is None or (out_act.is_contiguous() and out_act.shape == (T, D))
    _lib.check(_lib.lib().pg_stream_mix_norm(xs.data_ptr(), _lib.ptr(y), 0 if y is None else y.stride(0), _lib.ptr(mix), _lib.ptr(write), _lib.ptr(read),
                                             _lib.ptr(norm_w), _lib.ptr(out_act), T, S, D, float(eps),
                                             int(out_act is not None and out_act.dtype == torch.float32), _lib.stream()), "pg_stream_mix_norm")
    return out_act


# ---- latent attention ------------------------------------------------------------------------------------------------
_BATCH_PLANS = {}


def _batch_plan(T, B):
    """Tile list (batch index, first row, rows) of a batched product over the same T rows for every index, in the layout of
    pg_moe_plan; made once per (T, B) on the host."""
    key = (T, B)
    if key not in _BATCH_PLANS:
        if torch.cuda.is_current_stream_capturing():
            return None
        tile = _lib.lib().pg_moe_tile_rows()
        rows = [(b, r0, min(tile, T - r0)) for b in range(B) for r0 in range(0, T, tile)]
        buf = np.zeros(4 + 3 * len(rows), dtype=np.int32)
        buf[0] = len(rows)
        buf[4:] = np.asarray(rows, dtype=np.int32).reshape(-1)
        _BATCH_PLANS[key] = (torch.from_numpy(buf).to("cuda"), len(rows))
        torch.cuda.current_stream().synchronize()
    return _BATCH_PLANS[key]


def linear_batched(x, w, out):
    """out[:, b, :] = x[:, b, :] @ w[b].T for every b: x [T, B, K] and out [T, B, F] are views with unit last stride, w [B, F, K].
    bf16 operands whose slices start on 16-byte boundaries run on the tensor cores (the grouped kernel of the routed experts with
    one "expert" per batch index); everything else on plain fp32 FMAs."""
    T, B, K = x.shape
    F = w.shape[1]
    assert w.shape == (B, F, K) and out.shape == (T, B, F) and x.dtype == w.dtype and w.is_contiguous()
    assert x.stride(2) == 1 and out.stride(2) == 1
    if (x.dtype == torch.bfloat16 and K % 8 == 0 and x.stride(0) % 8 == 0 and x.stride(1) % 8 == 0 and x.data_ptr() % 16 == 0
            and w.data_ptr() % 16 == 0 and len(_BATCH_PLANS) < 4096):
        plan = _batch_plan(T, B)
        if plan is not None and plan[1] <= 65535:
            _lib.check(_lib.lib().pg_moe_gemm(x.data_ptr(), x.stride(0), plan[0].data_ptr(), 0, w.data_ptr(), F * K, K, out.data_ptr(), out.stride(0),
                                              plan[0].data_ptr(), plan[1], F, K, 0, 0, int(out.dtype == torch.float32), x.stride(1), out.stride(1),
                                              _lib.stream()), "pg_moe_gemm")
            return out
    _lib.check(_lib.lib().pg_gemm_simt_batched(x.data_ptr(), x.stride(0), x.stride(1), w.data_ptr(), K, F * K, out.data_ptr(), out.stride(0),
                                               out.stride(1), T, F, K, B, int(x.dtype == torch.float32), int(out.dtype == torch.float32),
                                               _lib.stream()), "pg_gemm_simt_batched")
    return out


def latent_prepare(proj, b: StepBatch, freq, q_norm, c_norm, cq_out, pages, q_rank, rank, rot, rot_dims, eps, page, rot_gain=1.0):
    """pages None: the layer reads another layer's cached rows; only the normalised query latent is made."""
    assert proj.stride(1) == 1 and freq.dtype == torch.float64 and (pages is None or (pages.dtype == proj.dtype and pages.shape[-1] == rank + rot))
    assert cq_out is None or (cq_out.dtype == proj.dtype and cq_out.is_contiguous())
    _lib.check(_lib.lib().pg_latent_prepare(proj.data_ptr(), proj.stride(0), b.pos.data_ptr(), b.row_entry.data_ptr(), b.page_table.data_ptr(),
                                            b.max_pages, page, freq.data_ptr(), _lib.ptr(q_norm), _lib.ptr(c_norm), _lib.ptr(cq_out), _lib.ptr(pages),
                                            b.T, q_rank, rank, rot, rot_dims, float(eps), float(rot_gain), int(proj.dtype == torch.float32), _lib.stream()),
               "pg_latent_prepare")


def rotate_heads(src, dst, pos, freq, rot_dims, rot_gain=1.0):
    """src, dst: [T, H, n] views (unit last stride, any row / head pitch) of one type; the first rot_dims of every head vector are
    rotated in interleaved pairs by pos[t] * freq[i]; rot_gain multiplies cosines and sines."""
    T, H, n = src.shape
    assert dst.shape == src.shape and src.dtype == dst.dtype and src.stride(2) == 1 and dst.stride(2) == 1
    _lib.check(_lib.lib().pg_rotate_heads(src.data_ptr(), src.stride(0), src.stride(1), dst.data_ptr(), dst.stride(0), dst.stride(1), pos.data_ptr(),
                                          freq.data_ptr(), T, H, n, rot_dims, float(rot_gain), int(src.dtype == torch.float32), _lib.stream()), "pg_rotate_heads")


def latent_expand(pages, b: StepBatch, w_ukv, H, dim, rot, vdim, rank, page, prec):
    """Per-head keys [plain | rotated] and values of every multi-token entry's context + new tokens, rebuilt from the cached
    latent rows into dense scratch: k [dense_rows, H * (dim + rot)], v [dense_rows, H * vdim] (read through b.dense_pages)."""
    L, f32 = _lib.lib(), int(pages.dtype == torch.float32)
    lat = prec.empty(b.dense_rows, rank)
    _lib.check(L.pg_latent_gather(pages.data_ptr(), b.page_table.data_ptr(), b.max_pages, page, b.dense_row0.data_ptr(), b.n.data_ptr(), b.ctx.data_ptr(),
                                  lat.data_ptr(), b.E, b.dense_max_len, rank, rank + rot, f32, _lib.stream()), "pg_latent_gather")
    up = linear(lat, w_ukv, prec.empty(b.dense_rows, H * (dim + vdim)))
    k = prec.empty(b.dense_rows, H * (dim + rot))
    v = prec.empty(b.dense_rows, H * vdim)
    _lib.check(L.pg_latent_pack_kv(up.data_ptr(), up.stride(0), pages.data_ptr(), b.page_table.data_ptr(), b.max_pages, page, b.dense_row0.data_ptr(),
                                   b.n.data_ptr(), b.ctx.data_ptr(), k.data_ptr(), v.data_ptr(), b.E, b.dense_max_len, H, dim, rot, vdim, rank, f32,
                                   _lib.stream()), "pg_latent_pack_kv")
    return k, v


def dense_view(b: StepBatch) -> StepBatch:
    """The same step with the dense scratch layout in place of the cache's page table."""
    return dataclasses.replace(b, page_table=b.dense_pages, max_pages=b.dense_max_pages)


# ---- routed feed-forward ---------------------------------------------------------------------------------------------
def moe_route(logits, correction, n_real, top, group_count, group_keep, scale, logit_bias=None):
    """logits fp32 [T, n_all] (+ logit_bias fp32 [n_all]) -> ids int32 [T, top], weights fp32 [T, top], counts int32 [n_real] (device)."""
    T, n_all = logits.shape
    assert logits.dtype == torch.float32 and logits.stride(1) == 1
    ids = torch.empty(T, top, device="cuda", dtype=torch.int32)
    wts = torch.empty(T, top, device="cuda", dtype=torch.float32)
    counts = torch.empty(max(1, n_real), device="cuda", dtype=torch.int32)
    _lib.check(_lib.lib().pg_moe_route(logits.data_ptr(), logits.stride(0), _lib.ptr(correction), ids.data_ptr(), wts.data_ptr(), counts.data_ptr(), T,
                                       n_all, n_real, top, int(group_count), int(group_keep), float(scale), _lib.ptr(logit_bias), _lib.stream()), "pg_moe_route")
    return ids, wts, counts


class MoePlan:
    """Device-side order of the (token, choice) pairs by expert and the list of row tiles the grouped products walk."""

    def __init__(self, ids, counts, n_real):
        L = _lib.lib()
        T, top = ids.shape
        self.pairs, self.top = T * top, top
        self.max_tiles = -(-self.pairs // L.pg_moe_tile_rows()) + n_real
        i32 = dict(device="cuda", dtype=torch.int32)
        self.offsets = torch.empty(n_real + 1, **i32)
        self.fill = torch.empty(n_real, **i32)
        self.plan = torch.empty(4 + 3 * self.max_tiles, **i32)
        self.sorted_pair = torch.empty(self.pairs, **i32)
        self.pair_row = torch.empty(self.pairs, **i32)
        _lib.check(L.pg_moe_plan(counts.data_ptr(), ids.data_ptr(), self.offsets.data_ptr(), self.fill.data_ptr(), self.plan.data_ptr(),
                                 self.sorted_pair.data_ptr(), self.pair_row.data_ptr(), self.pairs, n_real, self.max_tiles, _lib.stream()), "pg_moe_plan")


def moe_gemm(x, plan: MoePlan, w, out, gather, act=0):
    """out[row] = act(x[src(row)] @ w[expert(row)].T) over the plan's tiles; gather: x rows are tokens (src = pair // top),
    else x rows are already in sorted order.  w [n_real, F, K] contiguous."""
    n_real, F, K = w.shape
    assert w.is_contiguous() and x.dtype == w.dtype and x.stride(1) == 1 and out.stride(1) == 1 and x.shape[1] == K
    assert out.shape[1] == (F // 2 if act == ACT_SILU_GLU else F)
    _lib.check(_lib.lib().pg_moe_gemm(x.data_ptr(), x.stride(0), plan.sorted_pair.data_ptr(), plan.top if gather else 0, w.data_ptr(), F * K, K,
                                      out.data_ptr(), out.stride(0), plan.plan.data_ptr(), plan.max_tiles, F, K, int(act),
                                      int(x.dtype == torch.float32), int(out.dtype == torch.float32), 0, 0, _lib.stream()), "pg_moe_gemm")
    return out


def moe_gather_rows(x, plan: MoePlan, out):
    """out[row] = x[token of sorted pair `row`]: every expert's tokens as one contiguous run of rows."""
    assert x.dtype == out.dtype and x.stride(1) == 1 and out.stride(1) == 1 and out.shape[0] >= plan.pairs
    _lib.check(_lib.lib().pg_moe_gather_rows(x.data_ptr(), x.stride(0), plan.sorted_pair.data_ptr(), plan.offsets[-1:].data_ptr(), plan.top, out.data_ptr(),
                                             out.stride(0), plan.pairs, x.shape[1], int(x.dtype == torch.float32), _lib.stream()), "pg_moe_gather_rows")
    return out


def moe_combine(expert_out, plan: MoePlan, ids, weights, h, shared_out, y, shared_gate=None, accumulate=False):
    """y[t] (+)= sum_k weights[t, k] * expert row (or h[t] for an identity expert) + sigmoid(shared_gate[t]) * shared_out[t]; shared_gate:
    fp32 logits, one per token (a strided column view), None: the shared term counts fully; accumulate: add into y."""
    T, D = y.shape
    assert shared_gate is None or (shared_gate.dtype == torch.float32 and shared_gate.shape[0] == T)
    assert y.dtype == torch.float32 and y.is_contiguous() and h.stride(1) == 1
    assert expert_out is None or (expert_out.dtype == torch.float32 and expert_out.stride(1) == 1)
    _lib.check(_lib.lib().pg_moe_combine(_lib.ptr(expert_out), 0 if expert_out is None else expert_out.stride(0), plan.pair_row.data_ptr(), ids.data_ptr(),
                                         weights.data_ptr(), h.data_ptr(), h.stride(0), _lib.ptr(shared_out), 0 if shared_out is None else shared_out.stride(0),
                                         y.data_ptr(), T, D, plan.top, int(h.dtype == torch.float32), _lib.ptr(shared_gate),
                                         0 if shared_gate is None else shared_gate.stride(0), int(bool(accumulate)), _lib.stream()), "pg_moe_combine")
    return y


# a portion at least this long is advanced in 32-token blocks; shorter ones (decode above all) token by token
LINEAR_ATTN_CHUNK_MIN = 8


def linear_attn(qkv, state, decay, out, b: StepBatch, H, dim, vdim, chunked=None):
    assert state.dtype == torch.float32 and out.dtype == torch.float32 and out.is_contiguous() and qkv.stride(1) == 1
    if chunked is None:
        chunked = b.max_n >= LINEAR_ATTN_CHUNK_MIN
    fn = _lib.lib().pg_linear_attn_chunked if chunked else _lib.lib().pg_linear_attn_scan
    _lib.check(fn(qkv.data_ptr(), qkv.stride(0), state.data_ptr(), decay.data_ptr(), out.data_ptr(), b.row0.data_ptr(), b.n.data_ptr(),
                  b.ctx.data_ptr(), b.slot.data_ptr(), b.E, H, dim, vdim, int(qkv.dtype == torch.float32), _lib.stream()), "pg_linear_attn")
