"""CPU checks of the Risepel oracle (float64) and of the configuration reader: no GPU, no library calls."""
import numpy as np
import pytest

from helix_b200 import weights_io
from helix_b200.engine import MIXER_GLA, MIXER_LATENT
from oracle import risepel_ref as ref


def test_oracle_portions_equal_whole():
    cfg = ref.random_config()
    sd = ref.random_state_dict(cfg, seed=2)
    o = ref.RisepelOracle(cfg, sd)
    toks = np.random.default_rng(0).integers(0, cfg["vocab"], 70).tolist()
    whole = o.forward(toks)
    st, parts, at = o.new_state(), [], 0
    for n in (19, 2, 1, 30, 18):
        parts.append(o.forward(toks[at:at + n], st))
        at += n
    assert np.abs(np.concatenate(parts) - whole).max() < 1e-9


def test_window_and_sink_semantics_by_construction():
    # one head, identity-like weights: the score of key j is proportional to a planted value, so the softmax is known
    H, Dk, Dr, Dv, R, Q, Wd = 1, 2, 2, 2, 2, 2, 4
    m = dict(heads=H, dim=Dk, vdim=Dv, kv_rank=R, q_rank=Q, rot_dim=Dr, rot=dict(base=10000.0, dims=Dr), mask=dict(size=3),
             scale=1.0, eps=1e-6)
    p = {"dq": np.zeros((Q, Wd)), "dq.norm": np.ones(Q), "uq": np.zeros((H * (Dk + Dr), Q)), "uk": np.eye(H * Dk, R),
         "uv": np.eye(H * Dv, R), "sink": np.array([0.0]), "g": np.zeros((H * Dv, Wd)), "o": np.eye(Wd, H * Dv)}
    T = 6
    h = np.zeros((T, Wd))
    c = np.arange(1, T + 1, dtype=float)[:, None] * np.ones((T, R))  # key j carries the value j + 1
    kr = np.zeros((T, Dr))
    # q = 0 -> every visible key scores 0 = the sink: weights 1 / (visible + 1)
    out = ref.latent_attention(h, p, m, np.arange(T), c, kr, np.arange(T))
    for t in range(T):
        vis = [j for j in range(T) if 0 <= t - j < 3]
        want = sum(j + 1 for j in vis) / (len(vis) + 1) * 0.5  # sigmoid(0) gate
        assert out[t, 0] == pytest.approx(want)


def test_gla_recurrence_against_the_closed_form():
    rng = np.random.default_rng(1)
    H, Dk, Dv, Wd, r, T = 2, 3, 4, 5, 2, 7
    p = {k: rng.standard_normal(s) for k, s in (("q", (H * Dk, Wd)), ("k", (H * Dk, Wd)), ("v", (H * Dv, Wd)), ("g", (H * Dv, Wd)),
                                                 ("o", (Wd, H * Dv)), ("a1", (r, Wd)), ("a2", (H * Dk, r)), ("a2.b", (H * Dk,)))}
    p["norm"] = np.ones(Dv)
    m = dict(heads=H, dim=Dk, vdim=Dv, tau=4.0, eps=1e-6)
    h = rng.standard_normal((T, Wd))
    y, S = ref.gla_mixer(h, p, m)
    # state after T tokens = sum_t (prod_{s>t} decay_s) k_t v_t^T
    ld = ref.gla_decay_log(h, p, m["tau"]).reshape(T, H, Dk)
    k = (h @ p["k"].T).reshape(T, H, Dk)
    v = (h @ p["v"].T).reshape(T, H, Dv)
    want = np.zeros((H, Dk, Dv))
    for t in range(T):
        w = np.exp(ld[t + 1:].sum(0))
        want += (w * k[t])[:, :, None] * v[t][:, None, :]
    assert np.abs(S - want).max() < 1e-10
    y2a, S1 = ref.gla_mixer(h[:3], p, m)
    y2b, S2 = ref.gla_mixer(h[3:], p, m, S1)
    assert np.abs(np.concatenate([y2a, y2b]) - y).max() < 1e-10 and np.abs(S2 - S).max() < 1e-10


def test_config_reader_maps_every_key():
    cfg = ref.random_config(order=("gla", "latent_attention", "latent_attention"), mlp_on=("latent_attention",))
    sd = ref.random_state_dict(cfg, seed=0, decay_rank=5)
    d = weights_io.desc_from_hf_config(cfg, {k: v.shape for k, v in sd.items()}, compute_f32=True)
    assert (d.width, d.vocab, d.compute_f32, d.arch) == (cfg["width"], cfg["vocab"], 1, 2)
    assert d.resid_alpha == cfg["postln_alpha"] and d.logit_softcap == cfg["logit_softcap"] and d.norm_eps == cfg["norm"]["eps"]
    g, a, b = d.layers
    assert (g.mixer, g.heads, g.dim, g.vdim, g.tau, g.decay_rank, g.ff) == (MIXER_GLA, 3, 16, 24, 8.0, 5, 0)
    assert (a.mixer, a.q_rank, a.kv_rank, a.rot_dim, a.rope_dims, a.window, a.kv_from) == (MIXER_LATENT, 32, 48, 16, 16, 20, -1)
    assert b.kv_from == 1 and b.ff == 112 and b.ff_limit == 1.25 and a.rope_base == 10000.0
    assert a.scale == pytest.approx((24 + 16) ** -0.5)
    with pytest.raises(ValueError):
        weights_io.desc_from_hf_config(cfg)  # the decay rank lives in the checkpoint's shapes
    cfg["layers"][0]["type"] = "conv"
    with pytest.raises(ValueError):
        weights_io.desc_from_hf_config(cfg, {k: v.shape for k, v in sd.items()})


def test_safetensors_roundtrip_shapes(tmp_path):
    cfg = ref.random_config(order=("gla",), mlp_on=())
    sd = ref.random_state_dict(cfg, seed=4)
    path = tmp_path / "model.safetensors"
    weights_io.write_safetensors(path, sd)
    shapes = weights_io.safetensors_shapes(path)
    assert shapes == {k: tuple(v.shape) for k, v in sd.items()}
    got = {n: a for n, _, _, a in weights_io.read_safetensors(path)}
    from helix_b200.engine import bf16_bits
    assert all(np.array_equal(got[k], bf16_bits(v).ravel()) for k, v in sd.items())
