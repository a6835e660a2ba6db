"""Host-side parts of the Zigivik decoder (configuration, weight accounting, cache layout, registry, frequency tables, projection
row order) and the oracle against itself; no GPU."""
import json
import math
import os
import struct
import sys

import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)
from oracle import zigivik_oracle as O  # noqa: E402


def cfg_small():
    lat = {"heads": 2, "dim": 8, "rot_dim": 4, "vdim": 6, "q_rank": 10, "kv_rank": 12, "scale": 0.3, "mask": {"size": 7},
           "rot": {"base": 100.0, "dims": 4, "scaling": {"factor": 3.0, "original": 16, "fast": 4.0, "slow": 1.0}}}
    att = {"heads": 4, "kv_heads": 2, "dim": 8, "vdim": 8, "scale": 0.35, "rot": {"base": 50.0, "dims": 6}}
    return {"architecture": "Zigivik", "vocab": 30, "width": 24, "norm": {"eps": 1e-5}, "canon": {"taps": 4}, "residual_mult": 0.5, "layers": [
        {"type": "attention", "mixer": dict(att), "mlp": {"kind": "dense", "ff": 20}},
        {"type": "latent_attention", "mixer": dict(lat), "mlp": None},
        {"type": "latent_attention", "mixer": dict(lat, heads=3, vdim=4, kv_from=1, mask={"size": 3}), "mlp": {"kind": "dense", "ff": 9}}]}


def test_config_rejects_what_the_design_does_not_have():
    from paligemma_multimodal_system_b200.modeling_zigivik import ZigivikConfig, ZigivikForCausalLM
    c = ZigivikConfig(cfg_small())
    assert c.taps == 4 and c.residual_mult == 0.5
    bad = cfg_small()
    bad["layers"][0]["type"] = "attention_2"
    with pytest.raises(ValueError, match="unknown mixer type"):
        ZigivikConfig(bad)
    bad = cfg_small()
    bad["layers"][0]["mlp"]["kind"] = "moe"
    with pytest.raises(ValueError, match="feed-forward kind"):
        ZigivikConfig(bad)
    bad = cfg_small()
    bad["layers"][2]["mixer"]["kv_from"] = 0  # not a latent layer
    with pytest.raises(ValueError, match="earlier latent-attention layer"):
        ZigivikConfig(bad)
    bad = cfg_small()
    bad["canon"]["taps"] = 9
    with pytest.raises(ValueError, match="taps"):
        ZigivikConfig(bad)
    bad = cfg_small()
    bad["layers"][2]["mixer"]["kv_rank"] = 16  # the borrowed rows have another width
    with pytest.raises(ValueError, match="cached rows"):
        ZigivikForCausalLM(ZigivikConfig(bad))
    bad = cfg_small()
    bad["architecture"] = "Kovusun"
    with pytest.raises(ValueError):
        ZigivikConfig(bad)


def test_every_tensor_is_accounted_for_and_the_cache_layout_follows_the_layers():
    from paligemma_multimodal_system_b200.modeling_zigivik import ZigivikConfig, ZigivikForCausalLM
    cfg = cfg_small()
    w = O.random_weights(cfg, seed=0)
    m = ZigivikForCausalLM(ZigivikConfig(cfg)).load_weights(w)
    lay = m.cache_layout()
    assert lay[:3] == [("kv", 16, 16), ("latent", 16), None] and lay[3:] == [("state", (3, 24))] * 3
    assert m.blocks[2].mixer.kv_from == 1 and m.blocks[2].mixer.window == 3 and m.blocks[1].mixer.window == 7 and m.blocks[1].ff is None
    assert m.blocks[0].mixer.value_is_key and m.blocks[0].mixer.unit_sink and m.blocks[0].mixer.window is None and m.blocks[0].mixer.rot_dims == 6
    assert m.blocks[1].mixer.rot_layout == "half" and m.blocks[1].mixer.gate_kind == "element" and abs(m.blocks[1].mixer.rot_gain - (0.1 * math.log(3.0) + 1)) < 1e-12
    missing = dict(w)
    del missing["l0.mix.k.b"]
    with pytest.raises(KeyError, match="lacks l0.mix.k.b"):
        ZigivikForCausalLM(ZigivikConfig(cfg)).load_weights(missing)
    extra = dict(w, **{"l2.mix.dkv": torch.zeros(16, 24)})  # a borrowing layer has no down projection for keys
    with pytest.raises(KeyError, match="without a place"):
        ZigivikForCausalLM(ZigivikConfig(cfg)).load_weights(extra)
    wrong = dict(w, **{"l1.norm1": torch.zeros(24)})  # the norms have ONE weight
    with pytest.raises(ValueError, match="l1.norm1"):
        ZigivikForCausalLM(ZigivikConfig(cfg)).load_weights(wrong)
    one_tap = dict(cfg, canon={"taps": 1})
    assert ZigivikForCausalLM(ZigivikConfig(one_tap)).cache_layout()[3:] == [None] * 3  # nothing to remember


def test_registry_picks_the_class_by_config(tmp_path):
    from paligemma_multimodal_system_b200 import registry
    assert "zigivik" in registry.known_architectures()
    cfg = cfg_small()
    w = O.random_weights(cfg, seed=1)
    meta, blobs, off = {}, [], 0
    for name, t in w.items():
        raw = t.to(torch.bfloat16).contiguous().view(torch.int16).numpy().tobytes()
        meta[name] = {"dtype": "BF16", "shape": list(t.shape), "data_offsets": [off, off + len(raw)]}
        blobs.append(raw)
        off += len(raw)
    head = json.dumps(meta).encode()
    (tmp_path / "model.safetensors").write_bytes(struct.pack("<Q", len(head)) + head + b"".join(blobs))
    (tmp_path / "config.json").write_text(json.dumps(cfg))
    m = registry.load_model(str(tmp_path), dtype=torch.float32)
    assert type(m).__name__ == "ZigivikForCausalLM" and m.vocab_size == 30 and m.prec.f32
    assert torch.equal(m.blocks[0].canon.float(), w["l0.canon1"]) and float(m.embed_norm) == float(w["embed.norm"])


def test_frequency_table_matches_the_oracle_and_its_limits():
    from paligemma_multimodal_system_b200.mixers import ramped_rotary_frequencies
    for base, dims, sc in ((100.0, 4, dict(factor=3.0, original=16, fast=4.0, slow=1.0)), (1e6, 64, dict(factor=40.0, original=4096, fast=32.0, slow=1.0)),
                           (10.0, 2, dict(factor=2.0, original=8, fast=1.0, slow=1.0))):
        f, gain = ramped_rotary_frequencies(base, dims, sc["factor"], sc["original"], sc["fast"], sc["slow"])
        rf, rg = O.rescaled_frequencies(base, dims, sc)
        assert torch.allclose(f, torch.tensor(rf, dtype=torch.float64), rtol=1e-12, atol=0) and abs(gain - rg) < 1e-12
        plain = torch.tensor(O.plain_frequencies(base, dims), dtype=torch.float64)
        assert bool((f <= plain * (1 + 1e-12)).all()) and bool((f >= plain / sc["factor"] * (1 - 1e-12)).all())
    f, gain = ramped_rotary_frequencies(1e4, 32, 1.0, 2048, 32.0, 1.0)  # factor one: nothing changes
    assert torch.allclose(f, torch.tensor(O.plain_frequencies(1e4, 32), dtype=torch.float64), rtol=1e-12) and gain == 1.0


def test_reordered_rows_turn_in_neighbouring_pairs_like_the_half_split_layout():
    from paligemma_multimodal_system_b200.mixers import half_to_pair_order
    assert half_to_pair_order(6, 6) == [0, 3, 1, 4, 2, 5] and half_to_pair_order(7, 4) == [0, 2, 1, 3, 4, 5, 6] and half_to_pair_order(3, 0) == [0, 1, 2]
    v, u = torch.randn(3, 14, dtype=torch.float64), torch.randn(3, 14, dtype=torch.float64)
    freqs = [0.3, 0.02, 1.1, 0.5]
    order = half_to_pair_order(14, 8)
    assert torch.allclose(O.turn_pairs(v[:, order], 11, freqs), O.turn_half(v, 11, freqs, 1.0)[:, order], atol=1e-12)
    # the dot product of two vectors turned by their own positions depends on the layouts only through the pairing
    v8, u8, o8 = v[:, :8], u[:, :8], half_to_pair_order(8, 8)
    a = (O.turn_half(v8, 9, freqs, 1.3) * O.turn_half(u8, 4, freqs, 1.3)).sum()
    b = (O.turn_pairs(v8[:, o8], 9, freqs) * O.turn_pairs(u8[:, o8], 4, freqs)).sum() * 1.3 ** 2
    assert abs(float(a - b)) < 1e-10


def test_oracle_convolution_and_polynomial():
    h = torch.arange(12.0).reshape(4, 3)
    w = torch.zeros(3, 3)
    w[:, 2] = 1.0  # the last tap is the token itself
    assert torch.equal(O.causal_conv(h, w), h)
    w = torch.zeros(3, 3)
    w[:, 0] = 1.0  # the first tap is two tokens back; nothing before the start
    assert torch.equal(O.causal_conv(h, w), torch.cat([torch.zeros(2, 3), h[:2]]))
    z = torch.randn(5, 16, generator=torch.Generator().manual_seed(0))
    out = O.poly_norm(z, torch.tensor([0.0, 0.0, 0.0, 0.4]), 1e-6)
    assert torch.allclose(out, torch.full_like(out, 0.4))
    out = O.poly_norm(z, torch.tensor([1.0, 0.0, 0.0, 0.0]), 0.0)
    assert torch.allclose((out * out).mean(-1), torch.ones(5), atol=1e-5)
    sq = O.poly_norm(z, torch.tensor([0.0, 1.0, 0.0, 0.0]), 0.0)
    assert bool((sq >= 0).all()) and torch.allclose((sq * sq).mean(-1), torch.ones(5), atol=1e-5)


def test_oracle_unit_in_the_softmax_denominator_and_window():
    cfg = cfg_small()
    w = O.random_weights(cfg, seed=3)
    h = torch.randn(6, 24, generator=torch.Generator().manual_seed(2))
    m = dict(cfg["layers"][0]["mixer"], scale=0.0)  # all scores zero: every weight is 1 / (keys + 1)
    k = h @ w["l0.mix.k"].T + w["l0.mix.k.b"]
    mean = torch.stack([k[:i + 1].sum(0) / (i + 2) for i in range(6)]).view(6, 2, 8)
    want = mean[:, [0, 0, 1, 1]].reshape(6, -1) @ w["l0.mix.o"].T
    assert torch.allclose(O.key_value_attention(h, w, "l0.mix.", m), want, atol=1e-5)
    lm = cfg["layers"][1]["mixer"]
    rows = O.latent_rows(h, w, "l1.mix.", lm, 1e-5)
    wide = O.latent_attention(h, w, "l1.mix.", dict(lm, mask={"size": 6}), 1e-5, rows)
    assert torch.allclose(wide, O.latent_attention(h, w, "l1.mix.", dict(lm, mask=None), 1e-5, rows), atol=1e-6)
    narrow = O.latent_attention(h, w, "l1.mix.", dict(lm, mask={"size": 2}), 1e-5, rows)
    assert torch.allclose(narrow[:2], wide[:2], atol=1e-6) and not torch.allclose(narrow[2:], wide[2:], atol=1e-4)


def test_oracle_whole_equals_prefix():
    """Causality of the restatement itself: logits of a prefix do not change when tokens follow."""
    cfg = cfg_small()
    w = O.random_weights(cfg, seed=4)
    tk = torch.randint(0, 30, (20,), generator=torch.Generator().manual_seed(5)).tolist()
    a, b = O.forward(cfg, w, tk), O.forward(cfg, w, tk[:11])
    assert torch.allclose(a[:11], b, atol=1e-9)
