"""CPU checks of the Lurepel oracle (float64) against closed forms, and of the configuration reader: no GPU, no library calls."""
import math

import numpy as np
import pytest

from helix_b200 import weights_io
from helix_b200 import engine as E
from oracle import lurepel_ref as ref


def test_oracle_portions_equal_whole():
    cfg = ref.random_config()
    sd = ref.random_state_dict(cfg, seed=2)
    o = ref.LurepelOracle(cfg, sd)
    toks = np.random.default_rng(0).integers(0, cfg["vocab"], 70).tolist()
    whole = o.forward(toks)
    assert np.abs(whole - ref.forward(cfg, sd, toks)).max() == 0.0
    st, parts, at = o.new_state(), [], 0
    for n in (19, 2, 1, 30, 18):
        parts.append(o.forward(toks[at:at + n], st))
        at += n
    assert np.abs(np.concatenate(parts) - whole).max() < 1e-9


def test_block_mask_unit_sink_and_head_gate_by_construction():
    # zero queries: every visible key scores 0, like the extra unit, so the weights are 1 / (visible + 1); the values are the
    # key projections, planted so that token j carries j + 1; a zero gate row gives sigmoid(0) = 1/2
    H, G, D, Wd, T, size = 2, 1, 2, 3, 8, 3
    m = dict(heads=H, kv_heads=G, dim=D, vdim=D, scale=1.0, mask=dict(size=size))
    p = {"q": np.zeros((H * D, Wd)), "k": np.array([[1.0, 0, 0], [1.0, 0, 0]]), "g": np.zeros((H, Wd)), "o": np.eye(Wd, H * D)}
    p["g"][1, 1] = 1.0  # head 1's gate reads the layer input's second entry
    h = np.zeros((T, Wd))
    h[:, 0] = np.arange(1, T + 1)
    h[:, 1] = np.linspace(-2, 2, T)
    out, (kn, v, kpos) = ref.attention_mixer(h, p, m, 1e-6)
    assert np.allclose(v[:, 0, 0], np.arange(1, T + 1)) and np.allclose(kn[:, 0, :], 1.0, atol=1e-5)
    for t in range(T):
        vis = [j for j in range(T) if j <= t and j // size == t // size]
        mean = sum(j + 1 for j in vis) / (len(vis) + 1)
        assert out[t, 0] == pytest.approx(0.5 * mean)                                  # head 0, first value channel
        assert out[t, 2] == pytest.approx(mean / (1.0 + math.exp(-h[t, 1])))           # head 1, gated by its own row
    # without a mask key the attention is causal
    out2, _ = ref.attention_mixer(h, p, dict(m, mask=None), 1e-6)
    assert out2[T - 1, 0] == pytest.approx(0.5 * sum(range(1, T + 1)) / (T + 1))


def test_rotation_pairs_neighbours_and_keeps_relative_angles():
    rot = dict(base=100.0, dims=4)
    f = ref.rotary_freqs(rot)
    assert np.allclose(f, [1.0, 0.1])
    v = np.zeros((1, 1, 6))
    v[0, 0] = [1, 0, 1, 0, 7, 9]
    r = ref.rotate_interleaved(v, [5], f)
    assert np.allclose(r[0, 0], [math.cos(5), math.sin(5), math.cos(0.5), math.sin(0.5), 7, 9])  # (0,1), (2,3) turn; the rest pass
    rng = np.random.default_rng(1)
    a, b = rng.standard_normal((1, 1, 6)), rng.standard_normal((1, 1, 6))
    d1 = (ref.rotate_interleaved(a, [9], f) * ref.rotate_interleaved(b, [4], f)).sum()
    d2 = (ref.rotate_interleaved(a, [105], f) * ref.rotate_interleaved(b, [100], f)).sum()
    assert d1 == pytest.approx(d2)


def test_frequency_scaling_has_three_bands():
    rot = dict(base=10000.0, dims=32, scaling=dict(factor=8.0, low=2.0, high=6.0, original=600))
    plain = ref.rotary_freqs(dict(base=10000.0, dims=32))
    f = ref.rotary_freqs(rot)
    wl = 2 * math.pi / plain
    kept, cut, mid = wl < 100, wl > 300, (wl >= 100) & (wl <= 300)
    assert kept.any() and cut.any() and mid.any()
    assert np.array_equal(f[kept], plain[kept]) and np.allclose(f[cut], plain[cut] / 8.0)
    s = (600 / wl[mid] - 2.0) / 4.0
    assert np.allclose(f[mid], (1 - s) * plain[mid] / 8.0 + s * plain[mid])
    assert ((f[mid] > plain[mid] / 8.0) & (f[mid] < plain[mid])).all()


def test_router_weights_are_scores_and_identity_returns_the_input():
    rng = np.random.default_rng(2)
    Wd, Fn = 6, 4
    r = dict(experts=2, identity=2, top=2)
    p = {"router": rng.standard_normal((4, Wd)), "correction": np.array([0.0, 0.0, 9.0, 9.0])}
    for e in range(2):
        p[f"e{e}"] = {"gate": rng.standard_normal((Fn, Wd)), "up": rng.standard_normal((Fn, Wd)), "down": rng.standard_normal((Wd, Fn))}
    h = rng.standard_normal((5, Wd))
    idx, wt = ref.moe_route(h, p, r)
    z = h @ p["router"].T
    s = np.exp(z) / np.exp(z).sum(-1, keepdims=True)
    assert set(idx.ravel()) == {2, 3}                                    # the correction decides the choice ...
    assert np.allclose(np.sort(wt, -1), np.sort(s[:, 2:], -1))           # ... the weights are the plain scores
    assert np.allclose(ref.moe_ff(h, p, r), s[:, 2:].sum(-1, keepdims=True) * h)
    p["correction"] = np.array([9.0, 0.0, 0.0, -9.0])
    r1 = dict(r, top=1)
    y = ref.moe_ff(h, p, r1)
    q = p["e0"]
    want = s[:, :1] * ((ref.silu(h @ q["gate"].T) * (h @ q["up"].T)) @ q["down"].T)
    assert np.allclose(y, want)


def test_gelu_tanh_and_norm_on_the_sublayer_output():
    assert ref.gelu_tanh(np.array([0.0]))[0] == 0.0
    assert ref.gelu_tanh(np.array([3.0]))[0] == pytest.approx(0.5 * 3 * (1 + math.tanh(math.sqrt(2 / math.pi) * (3 + 0.044715 * 27))))
    # x <- x + norm(f(x)): scaling a sublayer's output matrix leaves the model unchanged (up to eps)
    cfg = ref.random_config(order=("dense",), eps=1e-12)
    sd = ref.random_state_dict(cfg, seed=3)
    toks = [1, 5, 9, 2]
    a = ref.forward(cfg, sd, toks)
    sd2 = dict(sd)
    sd2["l0.mix.o"] = sd["l0.mix.o"] * 4.0
    sd2["l0.mlp.down"] = sd["l0.mlp.down"] * 0.25
    assert np.abs(ref.forward(cfg, sd2, toks) - a).max() < 1e-6


def test_config_reader_maps_every_key():
    cfg = ref.random_config(order=("dense", "moe", None), per_layer={2: dict(heads=4, kv_heads=4, dim=12, mask=None, rot=None)})
    d = weights_io.desc_from_hf_config(cfg, None, compute_f32=True)
    assert (d.width, d.vocab, d.compute_f32, d.arch) == (cfg["width"], cfg["vocab"], 1, 2)
    assert (d.norm_place, d.embed_norm, d.plain_gains, d.resid_alpha, d.logit_softcap) == (E.NORM_OF_OUTPUT, 1, 1, 1.0, 0.0)
    assert d.norm_eps == cfg["norm"]["eps"]
    a, b, c = d.layers
    flags = E.ATTN_QK_UNIT_NORM | E.ATTN_V_IS_K | E.ATTN_UNIT_SINK | E.ATTN_HEAD_GATE
    assert (a.mixer, a.heads, a.kv_heads, a.dim, a.vdim, a.attn_flags) == (E.MIXER_GQA, 6, 2, 24, 24, flags)
    assert (a.mask, a.window, a.rope_dims, a.rope_base, a.rope_pairing) == (E.MASK_CHUNK, 20, 16, 5000.0, 1)
    assert (a.rope_factor, a.rope_low, a.rope_high, a.rope_original) == (4.0, 1.0, 3.0, 64)
    assert a.scale == pytest.approx(3.0 / math.sqrt(24))
    assert (a.ff_kind, a.ff) == (E.FF_GELU_TANH, 72)
    assert (b.ff_kind, b.ff, b.experts, b.identity_experts, b.top_k) == (E.FF_MOE, 40, 5, 2, 3)
    assert (c.ff, c.mask, c.rope_dims, c.rope_factor, c.heads, c.kv_heads, c.dim) == (0, E.MASK_CAUSAL, 0, 0.0, 4, 4, 12)
    del cfg["layers"][0]["mixer"]["rot"]["scaling"]
    assert weights_io.desc_from_hf_config(cfg).layers[0].rope_factor == 0.0
    cfg["layers"][1]["mlp"]["kind"] = "conv"
    with pytest.raises(ValueError):
        weights_io.desc_from_hf_config(cfg)
    cfg["layers"][1]["mlp"] = None
    cfg["layers"][0]["type"] = "gla"
    with pytest.raises(ValueError):
        weights_io.desc_from_hf_config(cfg)


def test_descriptor_mirrors_the_c_layout():
    import ctypes as C
    d = weights_io.desc_from_hf_config(ref.random_config())
    sd, arr = d.to_c()
    assert (sd.n_layers, sd.norm_place, sd.embed_norm, sd.plain_gains) == (3, 1, 1, 1)
    assert (arr[1].ff_kind, arr[1].experts, arr[1].identity_experts, arr[1].top_k, arr[1].kv_heads) == (E.FF_MOE, 5, 2, 3, 2)
    assert C.sizeof(arr) == 3 * C.sizeof(arr[0])
