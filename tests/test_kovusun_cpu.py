"""Host-side parts of the Kovusun decoder (configuration, weight accounting, cache layout, registry) and the oracle against
itself; no GPU."""
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


def cfg_small():
    att = {"heads": 4, "kv_heads": 2, "dim": 8, "vdim": 12, "scale": 0.3, "mask": {"size": 7}}
    return {"architecture": "Kovusun", "vocab": 30, "width": 24, "norm": {"eps": 1e-5}, "layers": [
        {"type": "attention_2", "mixer": dict(att), "mlp": {"kind": "dense", "ff": 20, "limit": 1.0}},
        {"type": "attention_3", "mixer": dict(att, mask={"size": 5, "keep_first": 2}, rot={"base": 100.0, "dims": 4}),
         "mlp": {"kind": "moe", "expert": {"ff": 6}, "router": {"experts": 5, "top": 2}, "shared": {"ff": 10}}},
        {"type": "attention", "mixer": dict(att), "mlp": None},
        {"type": "attention", "mixer": dict(att, heads=2, kv_from=2, mask={"size": 3}), "mlp": {"kind": "moe", "expert": {"ff": 6}, "router": {"experts": 3, "top": 3}}}]}


def test_config_rejects_what_the_design_does_not_have():
    from paligemma_multimodal_system_b200.modeling_kovusun import KovusunConfig
    KovusunConfig(cfg_small())
    bad = cfg_small()
    bad["layers"][0]["type"] = "attention_4"
    with pytest.raises(ValueError, match="unknown mixer type"):
        KovusunConfig(bad)
    bad = cfg_small()
    bad["layers"][0]["mlp"]["kind"] = "sparse"
    with pytest.raises(ValueError, match="feed-forward kind"):
        KovusunConfig(bad)
    bad = cfg_small()
    bad["layers"][3]["mixer"]["kv_from"] = 3
    with pytest.raises(ValueError, match="earlier layer"):
        KovusunConfig(bad)
    bad = cfg_small()
    bad["layers"][3]["mixer"]["vdim"] = 16
    with pytest.raises(ValueError, match="vdim differs"):
        KovusunConfig(bad)
    bad = cfg_small()
    bad["architecture"] = "Mapedra"
    with pytest.raises(ValueError):
        KovusunConfig(bad)


def test_every_tensor_is_accounted_for_and_the_cache_layout_follows_the_layers():
    from paligemma_multimodal_system_b200.modeling_kovusun import KovusunConfig, KovusunForCausalLM
    cfg = cfg_small()
    w = O.random_weights(cfg, seed=0)
    m = KovusunForCausalLM(KovusunConfig(cfg)).load_weights(w)
    lay = m.cache_layout()
    assert lay[:4] == [("kv", 16, 24), ("kv", 16, 24), ("kv", 16, 24), None] and lay[4:] == [("state", (24,))] * 4
    assert m.blocks[3].mixer.kv_from == 2 and m.blocks[3].mixer.window == 3 and m.blocks[1].mixer.keep_first == 2
    assert m.blocks[1].mixer.rot_dims == 4 and m.blocks[0].mixer.rot_dims == 0 and m.blocks[2].ff is None
    assert m.blocks[1].ff.shared_gate and not m.blocks[3].ff.shared_gate and m.blocks[3].ff.shared is None
    missing = dict(w)
    del missing["l1.mlp.router.b"]
    with pytest.raises(KeyError, match="lacks l1.mlp.router.b"):
        KovusunForCausalLM(KovusunConfig(cfg)).load_weights(missing)
    extra = dict(w, **{"l3.mix.k": torch.zeros(16, 24)})  # a borrowing layer has no key projection
    with pytest.raises(KeyError, match="without a place"):
        KovusunForCausalLM(KovusunConfig(cfg)).load_weights(extra)
    wrong = dict(w, **{"l0.mix.sink": torch.zeros(5)})
    with pytest.raises(ValueError, match="l0.mix.sink"):
        KovusunForCausalLM(KovusunConfig(cfg)).load_weights(wrong)


def test_registry_picks_the_class_by_config(tmp_path):
    from paligemma_multimodal_system_b200 import registry
    assert "kovusun" in registry.known_architectures()
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
    assert type(m).__name__ == "KovusunForCausalLM" and m.vocab_size == 30 and m.prec.f32
    assert torch.equal(m.blocks[0].shift.float(), w["l0.shift"])


def test_oracle_window_and_kept_first_keys():
    assert O.visible(10, 10, 1, 0) and not O.visible(10, 9, 1, 0) and not O.visible(10, 11, 5, 0)
    assert O.visible(10, 6, 5, 0) and not O.visible(10, 5, 5, 0)
    assert O.visible(100, 2, 5, 3) and not O.visible(100, 3, 5, 3) and O.visible(100, 50, None, 0)
    g = torch.Generator().manual_seed(0)
    q, k, v = torch.randn(9, 2, 4, generator=g), torch.randn(9, 1, 4, generator=g), torch.randn(9, 1, 3, generator=g)
    full = O.attend(q, k, v, 0.5)
    assert torch.allclose(full, O.attend(q, k, v, 0.5, size=9), atol=1e-6)
    assert torch.allclose(full, O.attend(q, k, v, 0.5, size=2, keep=9), atol=1e-6)   # everything kept
    assert not torch.allclose(full, O.attend(q, k, v, 0.5, size=2), atol=1e-3)
    one = O.attend(q, k, v, 0.5, size=1)
    assert torch.allclose(one, v[:, 0][:, None, :].expand(9, 2, 3), atol=1e-6)          # a window of one returns the token's own value
    # portions: queries 5 .. 8 alone, told their first position
    assert torch.allclose(O.attend(q[5:], k, v, 0.5, size=3, keep=1, first_pos=5), O.attend(q, k, v, 0.5, size=3, keep=1)[5:], atol=1e-6)


def test_oracle_sink_is_a_key_with_a_zero_value_and_no_scale():
    g = torch.Generator().manual_seed(1)
    q, k, v = torch.randn(5, 2, 4, generator=g), torch.randn(5, 2, 4, generator=g), torch.randn(5, 2, 3, generator=g)
    sink = torch.tensor([0.7, -1.2])
    got = O.attend(q, k, v, 0.5, sink=sink)
    for t in range(5):
        for h in range(2):
            s = (k[:t + 1, h] @ q[t, h]) * 0.5
            den = s.exp().sum() + sink[h].exp()
            assert torch.allclose(got[t, h], (s.exp()[:, None] * v[:t + 1, h]).sum(0) / den, atol=1e-6)


def test_oracle_shift_and_router():
    a = torch.arange(12.0).reshape(4, 3)
    assert torch.equal(O.token_shift(a, torch.zeros(3)), a)
    prev = torch.cat([torch.zeros(1, 3), a[:-1]])
    assert torch.equal(O.token_shift(a, torch.ones(3)), prev)
    cfg = cfg_small()
    w = O.random_weights(cfg, seed=3)
    h = torch.randn(6, 24, generator=torch.Generator().manual_seed(2))
    mlp = cfg["layers"][3]["mlp"]  # top = all three experts, no shared expert: a full softmax over the biased logits
    z = h @ w["l3.mlp.router"].T + w["l3.mlp.router.b"]
    p = torch.softmax(z, -1)
    want = sum(p[:, e:e + 1] * O.silu_expert(h, w, f"l3.mlp.e{e}.") for e in range(3))
    assert torch.allclose(O.routed_experts(h, w, "l3.mlp.", mlp), want, atol=1e-5)


def test_oracle_whole_equals_prefix():
    """Causality of the restatement itself: logits of a prefix do not change when tokens follow."""
    cfg = cfg_small()
    w = O.random_weights(cfg, seed=4)
    tk = torch.randint(0, 30, (20,), generator=torch.Generator().manual_seed(5)).tolist()
    a, b = O.forward(cfg, w, tk), O.forward(cfg, w, tk[:11])
    assert torch.allclose(a[:11], b, atol=1e-5)


def test_score_options_bound_the_keys_a_decoded_token_reads():
    from paligemma_multimodal_system_b200.seq_ops import ScoreOptions
    assert ScoreOptions(4).visible_keys(999) == 1000
    assert ScoreOptions(4, window=64, keep_first=6).visible_keys(999) == 70
    assert ScoreOptions(4, window=64, keep_first=6).visible_keys(10) == 11
    s = ScoreOptions(4, window=None, keep_first=6)
    assert s.window == 0 and s.keep_first == 0  # without a window there is nothing to keep
