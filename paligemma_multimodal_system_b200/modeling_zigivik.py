"""Zigivik: a decoder-only language model of parallel layers -- ONE scalar-weight RMS norm per layer feeds a token mixer (through a
short causal convolution over time) and a feed-forward side by side -- served through the ragged-step engine (engine.py).

    x   = rms(embed[token]) g_e                                   rms(z) = z / sqrt(mean(z^2) + eps); every g is ONE number
    h   = rms(x) g;   h~_t = h_t + sum_j w[:, j] h_{t - taps + 1 + j}      (per channel; zeros before the sequence's start)
    x  <- x + m (mixer(h~) + ff(h))                               m = config `residual_mult`
    logits = head(rms(x) g_f)

Mixer types of a config:

    latent_attention  `mixers.LatentAttention` with the half-split rotation layout, ramped frequency rescaling, a sliding window, a
                      per-element sigmoid output gate; `kv_from`: j reads the latent rows layer j cached
    attention         `mixers.WindowedSoftmaxAttention` without a window: grouped key heads that also serve as values (unrotated), q / k
                      biases, partial interleaved rotation, a softmax denominator enlarged by one

Feed-forward "dense": `mixers.PolyNormFeedForward` (biases on both projections).

Every size and model-dependent constant comes from config.json (`ZigivikConfig`), tensor names from the checkpoint:

    embed, embed.norm, final.norm, head, l<i>.norm1, l<i>.canon1, l<i>.mix.{dq,dq.norm,uq,dkv,dkv.norm,uk,uv,g,o} (latent_attention),
    l<i>.mix.{q,q.b,k,k.b,o} (attention), l<i>.mlp.{up,up.b,down,down.b,act}

Per sequence a layer keeps its mixer's pages (none when it borrows) and, for the convolution, h of its last taps - 1 tokens in an fp32
state slot; `cache_layout()` lists the mixers' specs first and the convolution states after them.  The residual stream is fp32 and is
updated in place by the epilogues of the two output projections, which also apply m; one kernel per layer forms the norm, the
convolution and the state update (seq_ops.rmsnorm_conv).
"""
import json
import os
from typing import Dict, List, Optional

import torch

from . import _lib, seq_ops
from .mixers import LatentAttention, PolyNormFeedForward, WindowedSoftmaxAttention

MIXER_TYPES = ("latent_attention", "attention")
MAX_TAPS = 8  # the convolution kernel keeps a sequence's last taps - 1 rows in registers


class ZigivikConfig:
    def __init__(self, cfg: dict):
        if cfg.get("architecture") != "Zigivik":
            raise ValueError("not a Zigivik config")
        self.raw = cfg
        self.vocab = int(cfg["vocab"])
        self.width = int(cfg["width"])
        self.norm_eps = float(cfg["norm"]["eps"])
        self.residual_mult = float(cfg.get("residual_mult", 1.0))
        self.taps = int((cfg.get("canon") or {}).get("taps", 0))
        if not 0 <= self.taps <= MAX_TAPS:
            raise ValueError(f"canon.taps must be between 0 and {MAX_TAPS}")
        self.layers: List[dict] = list(cfg["layers"])
        for i, l in enumerate(self.layers):
            if l["type"] not in MIXER_TYPES:
                raise ValueError(f"layer {i}: unknown mixer type {l['type']!r}")
            if l.get("mlp") and l["mlp"].get("kind", "dense") != "dense":
                raise ValueError(f"layer {i}: unknown feed-forward kind {l['mlp'].get('kind')!r}")
            src = l["mixer"].get("kv_from")
            if src is not None:
                s = self.layers[int(src)] if 0 <= int(src) < i else None
                if l["type"] != "latent_attention" or s is None or s["type"] != "latent_attention" or s["mixer"].get("kv_from") is not None:
                    raise ValueError(f"layer {i}: kv_from must name an earlier latent-attention layer with a down projection of its own")

    @classmethod
    def from_dir(cls, path):
        with open(os.path.join(path, "config.json")) as f:
            return cls(json.load(f))


def _mixer(width: int, kind: str, m: dict, eps: float):
    mask, rot = m.get("mask") or {}, m.get("rot") or {}
    if kind == "latent_attention":
        rot_dim = int(m.get("rot_dim", 0))
        return LatentAttention(width, int(m["heads"]), int(m["dim"]), rot_dim, int(m.get("vdim", m["dim"])), int(m["q_rank"]), int(m["kv_rank"]),
                               m["scale"], int(rot.get("dims", rot_dim)), rot.get("base", 10000.0), eps, rot_layout="half",
                               rot_scaling=rot.get("scaling"), window=mask.get("size"), gate="element", kv_from=m.get("kv_from"))
    dim = int(m["dim"])
    return WindowedSoftmaxAttention(width, int(m["heads"]), int(m.get("kv_heads", m["heads"])), dim, dim, m["scale"], eps, window=mask.get("size"),
                                    bias=True, rot_dims=int(rot.get("dims", 0)), rot_base=rot.get("base", 10000.0), value_is_key=True,
                                    unit_sink=True)


class ZigivikBlock:
    def __init__(self, c: ZigivikConfig, i: int):
        l = c.layers[i]
        self.mixer = _mixer(c.width, l["type"], l["mixer"], c.norm_eps)
        self.ff = PolyNormFeedForward(c.width, int(l["mlp"]["ff"]), c.norm_eps) if l.get("mlp") else None
        self.i, self.D, self.taps = i, c.width, c.taps

    def load(self, take):
        p = f"l{self.i}."
        self.norm1 = take(p + "norm1", ())
        self.mixer.load(take, p + "mix.")
        if self.ff is not None:
            self.ff.load(take, p + "mlp.")
        self.canon = take(p + "canon1", (self.D, self.taps)) if self.taps else None

    def pack(self, prec):
        f32 = dict(device="cuda", dtype=torch.float32)
        self.norm1_d = self.norm1.to(**f32).reshape(1).contiguous()
        self.canon_d = self.canon.to(**f32).t().contiguous() if self.canon is not None else None  # tap-major: the kernels read a tap's weights as a row
        self.mixer.pack(prec)
        if self.ff is not None:
            self.ff.pack(prec)


class ZigivikForCausalLM:
    """Weights + the step function.  `step(batch, store, want_rows)` advances every entry of a ragged batch by its new tokens (cached
    rows and the convolution states are left in `store`) and returns fp32 logits of the wanted rows."""

    architecture = "Zigivik"

    def __init__(self, config: ZigivikConfig, dtype: torch.dtype = torch.bfloat16):
        self.config = config
        self.prec = seq_ops.Precision(dtype)
        self.blocks = [ZigivikBlock(config, i) for i in range(len(config.layers))]
        for i, blk in enumerate(self.blocks):
            src = getattr(blk.mixer, "kv_from", None)
            if src is not None and blk.mixer.cache_signature() != self.blocks[src].mixer.cache_signature():
                raise ValueError(f"layer {i}: rank, rotated part or rotation differ from layer {src}, whose cached rows it reads")
        self.vocab_size = config.vocab
        self._packed = False

    # -- weights -------------------------------------------------------------------------------------------------------
    def load_weights(self, tensors: Dict[str, torch.Tensor]):
        """Every tensor must be used and have the shape the config implies; anything missing or left over raises."""
        c = self.config
        left = dict(tensors)

        def take(name, shape):
            if name not in left:
                raise KeyError(f"checkpoint lacks {name}")
            t = left.pop(name)
            if tuple(t.shape) != tuple(shape):
                raise ValueError(f"{name}: shape {tuple(t.shape)}, config implies {tuple(shape)}")
            return t

        self.embed = take("embed", (c.vocab, c.width))
        self.embed_norm = take("embed.norm", ())
        for blk in self.blocks:
            blk.load(take)
        self.final_norm = take("final.norm", ())
        self.head = take("head", (c.vocab, c.width))
        if left:
            raise KeyError(f"checkpoint tensors without a place in the model: {sorted(left)[:8]}")
        self._packed = False
        return self

    def pack(self):
        _lib.require_device()
        dt = self.prec.dtype
        f32 = dict(device="cuda", dtype=torch.float32)
        self.embed_d = self.embed.to("cuda", dt).contiguous()
        self.embed_norm_d = self.embed_norm.to(**f32).reshape(1).contiguous()
        self.final_norm_d = self.final_norm.to(**f32).reshape(1).contiguous()
        self.head_d = self.head.to("cuda", dt).contiguous()
        for blk in self.blocks:
            blk.pack(self.prec)
        torch.cuda.synchronize()
        self._packed = True

    def cache_layout(self):
        """Entries 0 .. L-1: the mixers' pages (None for a layer that borrows); entries L .. 2L-1: the convolution states."""
        c = self.config
        conv = ("state", (c.taps - 1, c.width)) if c.taps > 1 else None
        return [blk.mixer.cache_spec() for blk in self.blocks] + [conv for _ in self.blocks]

    # -- compute -------------------------------------------------------------------------------------------------------
    @torch.no_grad()
    def step(self, b: seq_ops.StepBatch, store, want_rows: Optional[torch.Tensor], trace: Optional[list] = None):
        """want_rows: int64 row indices (device) whose logits are returned as fp32 [n, vocab]; None / empty: no head."""
        if not self._packed:
            self.pack()
        c, prec, eps, L, m = self.config, self.prec, self.config.norm_eps, len(self.blocks), self.config.residual_mult
        e = seq_ops.embed_rows(b.tokens, self.embed_d, 0, c.width, 1.0)
        x = torch.empty_like(e)
        seq_ops.rmsnorm_conv(e, self.embed_norm_d, x, None, eps)
        for li, blk in enumerate(self.blocks):
            h = prec.empty(b.T, c.width) if blk.ff is not None else None
            hc = prec.empty(b.T, c.width)
            seq_ops.rmsnorm_conv(x, blk.norm1_d, h, hc, eps, conv_w=blk.canon_d, state=store.state[L + li], b=b)
            # both branches were formed from x as it was; their output projections add m times their result into x one after the other
            blk.mixer(hc, b, store, li, prec, resid=x, resid_scale=m)
            if blk.ff is not None:
                blk.ff(h, b, prec, resid=x, resid_scale=m)
            if trace is not None:
                trace.append(x.clone())
        if want_rows is None or want_rows.numel() == 0:
            return None
        last = x.index_select(0, want_rows)
        hn = prec.empty(*last.shape)
        seq_ops.rmsnorm_conv(last, self.final_norm_d, hn, None, eps)
        return seq_ops.linear(hn, self.head_d, torch.empty(last.shape[0], c.vocab, device="cuda", dtype=torch.float32))


def load_zigivik(path: str, dtype: torch.dtype = torch.bfloat16) -> ZigivikForCausalLM:
    from .utils import read_safetensors
    model = ZigivikForCausalLM(ZigivikConfig.from_dir(path), dtype)
    return model.load_weights(read_safetensors(os.path.join(path, "model.safetensors")))
