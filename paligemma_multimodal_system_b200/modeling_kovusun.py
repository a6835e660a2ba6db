"""Kovusun: a decoder-only language model of parallel layers -- windowed softmax attention and a feed-forward read the SAME
residual through two layer norms and are added to it together -- served through the ragged-step engine (engine.py).

    a = LN1(x), c = LN2(x)                            LN(z) = (z - mean) / sqrt(var + eps) * w + b
    a~_t = a_t + (a_{t-1} - a_t) * shift              token shift: the mixer reads a blend with the previous token's a
    x <- x + mixer(a~) + ff(c)
    logits = head(LN_final(x))

The three mixer types of a config are one mechanism, `mixers.WindowedSoftmaxAttention`, with different optional parts:

    attention     q/k/v biases, weightless q/k RMS norm, score - r1_h log(1 + r2_h (i - j)); `kv_from`: j borrows layer j's keys / values
    attention_2   weightless q/k RMS norm, a sink in the softmax denominator, a sigmoid output gate per head
    attention_3   partial interleaved rotation, score * temp_h, a window that keeps the first tokens of the sequence

Feed-forwards: "dense" = `mixers.GluFeedForward` in its clamped form with biases; "moe" = `mixers.RoutedFeedForward` with silu-gated
experts, a router bias, weights = softmax over the chosen logits, and a shared expert gated by sigmoid(w_sg . h).

Every size and model-dependent constant comes from config.json (`KovusunConfig`), tensor names from the checkpoint:

    embed, final.norm{,.b}, head, l<i>.norm{1,2}{,.b}, l<i>.shift, l<i>.mix.{q,k,v,o}{,.b}, l<i>.mix.{r1,r2,temp,sink,g},
    l<i>.mlp.{gate,up,down}{,.b} (dense), l<i>.mlp.{router,router.b,e<k>.{gate,up,down},shared.{gate,up,down,sg}} (moe)

Per sequence a layer keeps its key / value pages (none when it borrows) and, for the token shift, a of its last token in an fp32
state slot; `cache_layout()` lists the mixers' specs first and the shift states after them.  The residual stream is fp32 and is
updated in place by the epilogues of the two output projections (or the experts' combine); one kernel per layer forms both
norms, the shift and the state update (seq_ops.layernorm_shift).
"""
import json
import os
from typing import Dict, List, Optional

import torch

from . import _lib, seq_ops
from .mixers import GluFeedForward, RoutedFeedForward, WindowedSoftmaxAttention

# constants the design fixes
SWISH_ALPHA = 1.702          # the dense feed-forward's gate is g * sigmoid(SWISH_ALPHA * g)
MIXER_TYPES = ("attention", "attention_2", "attention_3")


class KovusunConfig:
    def __init__(self, cfg: dict):
        if cfg.get("architecture") != "Kovusun":
            raise ValueError("not a Kovusun config")
        self.raw = cfg
        self.vocab = int(cfg["vocab"])
        self.width = int(cfg["width"])
        self.norm_eps = float(cfg["norm"]["eps"])
        self.layers: List[dict] = list(cfg["layers"])
        for i, l in enumerate(self.layers):
            if l["type"] not in MIXER_TYPES:
                raise ValueError(f"layer {i}: unknown mixer type {l['type']!r}")
            if l.get("mlp") and l["mlp"].get("kind", "dense") not in ("dense", "moe"):
                raise ValueError(f"layer {i}: unknown feed-forward kind {l['mlp'].get('kind')!r}")
            src = l["mixer"].get("kv_from")
            if src is not None:
                s = self.layers[int(src)] if 0 <= int(src) < i else None
                if s is None or "kv_from" in s["mixer"]:
                    raise ValueError(f"layer {i}: kv_from must name an earlier layer with key / value projections of its own")
                for k in ("kv_heads", "dim", "vdim"):
                    if int(s["mixer"][k]) != int(l["mixer"][k]):
                        raise ValueError(f"layer {i}: {k} differs from layer {src}, whose keys and values it reads")

    @classmethod
    def from_dir(cls, path):
        with open(os.path.join(path, "config.json")) as f:
            return cls(json.load(f))


def _mixer(width: int, kind: str, m: dict, eps: float):
    mask, rot = m.get("mask") or {}, m.get("rot") or {}
    return WindowedSoftmaxAttention(
        width, int(m["heads"]), int(m.get("kv_heads", m["heads"])), int(m["dim"]), int(m.get("vdim", m["dim"])), m["scale"], eps,
        window=mask.get("size"), keep_first=int(mask.get("keep_first", 0)),
        bias=kind == "attention", qk_norm=kind in ("attention", "attention_2"),
        rot_dims=int(rot.get("dims", 0)) if kind == "attention_3" else 0, rot_base=rot.get("base", 10000.0),
        distance_penalty=kind == "attention", temperature=kind == "attention_3", sink=kind == "attention_2", head_gate=kind == "attention_2",
        kv_from=m.get("kv_from"))


def _feed_forward(width: int, mlp: Optional[dict]):
    if not mlp:
        return None
    if mlp.get("kind", "dense") == "dense":
        return GluFeedForward(width, int(mlp["ff"]), "clamped", limit=float(mlp["limit"]), alpha=SWISH_ALPHA, bias=True)
    r, shared = mlp["router"], mlp.get("shared")
    return RoutedFeedForward(width, int(r["experts"]), 0, int(r["top"]), 1, 1, 1.0, int(mlp["expert"]["ff"]), int(shared["ff"]) if shared else 0,
                             activation="silu_glu", correction=False, router_bias=True, shared_gate=True)


class KovusunBlock:
    def __init__(self, c: KovusunConfig, i: int):
        l = c.layers[i]
        self.mixer = _mixer(c.width, l["type"], l["mixer"], c.norm_eps)
        self.ff = _feed_forward(c.width, l.get("mlp"))
        self.i, self.D = i, c.width
        self.shift = None

    def load(self, take, has):
        p, D = f"l{self.i}.", self.D
        self.norm1, self.norm1_b = take(p + "norm1", (D,)), take(p + "norm1.b", (D,))
        if self.ff is not None:
            self.norm2, self.norm2_b = take(p + "norm2", (D,)), take(p + "norm2.b", (D,))
        elif has(p + "norm2"):  # a layer without a feed-forward may still carry the unused second norm
            take(p + "norm2", (D,)), take(p + "norm2.b", (D,))
        self.shift = take(p + "shift", (D,)) if has(p + "shift") else None
        self.mixer.load(take, p + "mix.")
        if self.ff is not None:
            self.ff.load(take, p + "mlp.")

    def pack(self, prec):
        f32 = dict(device="cuda", dtype=torch.float32)
        self.norm1_d, self.norm1_bd = self.norm1.to(**f32).contiguous(), self.norm1_b.to(**f32).contiguous()
        self.norm2_d = self.norm2_bd = None
        if self.ff is not None:
            self.norm2_d, self.norm2_bd = self.norm2.to(**f32).contiguous(), self.norm2_b.to(**f32).contiguous()
            self.ff.pack(prec)
        self.shift_d = self.shift.to(**f32).contiguous() if self.shift is not None else None
        self.mixer.pack(prec)


class KovusunForCausalLM:
    """Weights + the step function.  `step(batch, store, want_rows)` advances every entry of a ragged batch by its new tokens
    (keys / values and the shift states are left in `store`) and returns fp32 logits of the wanted rows."""

    architecture = "Kovusun"

    def __init__(self, config: KovusunConfig, dtype: torch.dtype = torch.bfloat16):
        self.config = config
        self.prec = seq_ops.Precision(dtype)
        self.blocks = [KovusunBlock(config, i) for i in range(len(config.layers))]
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
        for blk in self.blocks:
            blk.load(take, lambda name: name in left)
        self.final_norm, self.final_norm_b = take("final.norm", (c.width,)), take("final.norm.b", (c.width,))
        self.head = take("head", (c.vocab, c.width))
        if left:
            raise KeyError(f"checkpoint tensors without a place in the model: {sorted(left)[:8]}")
        self._packed = False
        return self

    def pack(self):
        _lib.require_device()
        dt = self.prec.dtype
        self.embed_d = self.embed.to("cuda", dt).contiguous()
        self.final_norm_d = self.final_norm.to("cuda", torch.float32).contiguous()
        self.final_norm_bd = self.final_norm_b.to("cuda", torch.float32).contiguous()
        self.head_d = self.head.to("cuda", dt).contiguous()
        for blk in self.blocks:
            blk.pack(self.prec)
        torch.cuda.synchronize()
        self._packed = True

    def cache_layout(self):
        """Entries 0 .. L-1: the mixers' key / value pages (None for a layer that borrows); entries L .. 2L-1: the shift states."""
        D = self.config.width
        return [blk.mixer.cache_spec() for blk in self.blocks] + [("state", (D,)) for _ in self.blocks]

    # -- compute -------------------------------------------------------------------------------------------------------
    @torch.no_grad()
    def step(self, b: seq_ops.StepBatch, store, want_rows: Optional[torch.Tensor], trace: Optional[list] = None):
        """want_rows: int64 row indices (device) whose logits are returned as fp32 [n, vocab]; None / empty: no head."""
        if not self._packed:
            self.pack()
        c, prec, eps, L = self.config, self.prec, self.config.norm_eps, len(self.blocks)
        x = seq_ops.embed_rows(b.tokens, self.embed_d, 0, c.width, 1.0)
        for li, blk in enumerate(self.blocks):
            a = prec.empty(b.T, c.width)
            f = prec.empty(b.T, c.width) if blk.ff is not None else None
            seq_ops.layernorm_shift(x, blk.norm1_d, blk.norm1_bd, a, eps, shift=blk.shift_d, state=store.state[L + li], b=b,
                                    w2=blk.norm2_d, b2=blk.norm2_bd, out2=f)
            # both branches were formed from x as it was; their output projections add into x one after the other
            blk.mixer(a, b, store, li, prec, resid=x)
            if blk.ff is not None:
                blk.ff(f, b, prec, resid=x)
            if trace is not None:
                trace.append(x.clone())
        if want_rows is None or want_rows.numel() == 0:
            return None
        last = x.index_select(0, want_rows)
        hn = prec.empty(*last.shape)
        seq_ops.layernorm_shift(last, self.final_norm_d, self.final_norm_bd, hn, eps)
        return seq_ops.linear(hn, self.head_d, torch.empty(last.shape[0], c.vocab, device="cuda", dtype=torch.float32))


def load_kovusun(path: str, dtype: torch.dtype = torch.bfloat16) -> KovusunForCausalLM:
    from .utils import read_safetensors
    model = KovusunForCausalLM(KovusunConfig.from_dir(path), dtype)
    return model.load_weights(read_safetensors(os.path.join(path, "model.safetensors")))
