"""Plain, slow float64 restatement of the Risepel decoder (numpy only; one function per mechanism).

The design: a post-norm residual stream (x <- norm(a*x + sublayer(x)), norm gain stored around zero), layers whose
mixer is either a gated linear-attention recurrence with a per-key-channel decay or a sliding-window attention over a
low-rank latent with a learned softmax sink and a sigmoid output gate, optional clamped gated feed-forward, and a
soft-capped LM head.  Notation below: T tokens, W width, H heads, Dk / Dv per-head key / value sizes, R latent rank,
Dr rotated dims.  Nothing here is shared with the CUDA path; the GPU tests compare the engine against these functions.
"""
import math

import numpy as np

F = np.float64


def rms_unit(x, eps):
    """x / sqrt(mean(x^2) + eps) over the last axis."""
    x = np.asarray(x, F)
    return x / np.sqrt((x * x).mean(-1, keepdims=True) + eps)


def norm_offset_gain(x, w, eps):
    """RMS norm whose stored gain is an offset from one."""
    return rms_unit(x, eps) * (1.0 + np.asarray(w, F))


def norm_plain_gain(x, w, eps):
    return rms_unit(x, eps) * np.asarray(w, F)


def sigmoid(z):
    return 1.0 / (1.0 + np.exp(-z))


def silu(z):
    return z * sigmoid(z)


def rotate_half_pairs(v, pos, base, dims):
    """Rotate the first `dims` entries of the last axis: entry i pairs with i + dims/2, angle pos * base^(-2i/dims)."""
    v = np.array(v, F)
    half = dims // 2
    f = base ** (-2.0 * np.arange(half, dtype=F) / dims)
    a = np.asarray(pos, F)[..., None] * f
    c, s = np.cos(a), np.sin(a)
    while c.ndim < v.ndim:  # broadcast over head axes between the token axis and the last axis
        c, s = c[..., None, :], s[..., None, :]
    u, w = v[..., :half].copy(), v[..., half:dims].copy()
    v[..., :half] = u * c - w * s
    v[..., half:dims] = w * c + u * s
    return v


# ------------------------------------------------------------------ gated linear attention
def gla_decay_log(h, p, tau):
    """log of the per-key-channel decay in (0, 1): sigmoid(z)^(1/tau), z from a low-rank projection with bias."""
    z = (h @ p["a1"].T) @ p["a2"].T + p["a2.b"]
    return -np.logaddexp(0.0, -z) / tau


def gla_mixer(h, p, m, state=None):
    """h [T, W] -> ([T, W], final state [H, Dk, Dv]).  state: the recurrence matrix left by earlier tokens (or None)."""
    T = h.shape[0]
    H, Dk, Dv = m["heads"], m["dim"], m["vdim"]
    q = (h @ p["q"].T).reshape(T, H, Dk) * Dk ** -0.5
    k = (h @ p["k"].T).reshape(T, H, Dk)
    v = (h @ p["v"].T).reshape(T, H, Dv)
    decay = np.exp(gla_decay_log(h, p, m["tau"])).reshape(T, H, Dk)
    S = np.zeros((H, Dk, Dv), F) if state is None else np.array(state, F)
    o = np.empty((T, H, Dv), F)
    for t in range(T):
        S = decay[t][:, :, None] * S + k[t][:, :, None] * v[t][:, None, :]
        o[t] = np.einsum("hkv,hk->hv", S, q[t])
    o = norm_plain_gain(o, p["norm"], m["eps"]).reshape(T, H * Dv)
    return (o * silu(h @ p["g"].T)) @ p["o"].T, S


# ------------------------------------------------------------------ latent attention
def latent_kv(h, p, m, pos):
    """What the cache keeps per token: the normed latent [T, R] and the rotated shared key part [T, Dr]."""
    R, Dr = m["kv_rank"], m["rot_dim"]
    d = h @ p["dkv"].T
    c = norm_plain_gain(d[:, :R], p["dkv.norm"], m["eps"])
    kr = rotate_half_pairs(d[:, R:R + Dr], pos, m["rot"]["base"], m["rot"]["dims"])
    return c, kr


def latent_attention(h, p, m, pos, c, kr, kpos):
    """h [T, W] at positions pos; c / kr / kpos: latent, rotated key part and positions of EVERY key the sequence has so
    far (this call's tokens included).  Returns [T, W]."""
    T = h.shape[0]
    H, Dk, Dr, Dv = m["heads"], m["dim"], m["rot_dim"], m["vdim"]
    cq = norm_plain_gain(h @ p["dq"].T, p["dq.norm"], m["eps"])
    q = (cq @ p["uq"].T).reshape(T, H, Dk + Dr)
    qn = q[:, :, :Dk]
    qr = rotate_half_pairs(q[:, :, Dk:], pos, m["rot"]["base"], m["rot"]["dims"])
    kn = (c @ p["uk"].T).reshape(-1, H, Dk)
    val = (c @ p["uv"].T).reshape(-1, H, Dv)
    s = (np.einsum("thd,jhd->thj", qn, kn) + np.einsum("thd,jd->thj", qr, kr)) * m["scale"]
    dist = np.asarray(pos)[:, None] - np.asarray(kpos)[None, :]
    seen = (dist >= 0) & (dist < m["mask"]["size"])
    s = np.where(seen[:, None, :], s, -np.inf)
    sink = np.asarray(p["sink"], F)[None, :, None]
    mx = np.maximum(s.max(-1, keepdims=True), sink)
    e = np.exp(s - mx)
    w = e / (e.sum(-1, keepdims=True) + np.exp(sink - mx))
    o = np.einsum("thj,jhv->thv", w, val).reshape(T, H * Dv)
    return (o * sigmoid(h @ p["g"].T)) @ p["o"].T


# ------------------------------------------------------------------ feed-forward
def dense_ff(h, p, limit):
    g = np.minimum(h @ p["gate"].T + p["gate.b"], limit)
    u = np.clip(h @ p["up"].T + p["up.b"], -limit, limit)
    return (g * sigmoid(1.702 * g) * (u + 1.0)) @ p["down"].T + p["down.b"]


def softcap(z, cap):
    return cap * np.tanh(z / cap) if cap else z  # no cap configured: plain logits


# ------------------------------------------------------------------ the model
class RisepelOracle:
    """cfg: the checkpoint's config dict; sd: {tensor name: ndarray}.  `forward` runs a portion of one sequence from the
    state an earlier call left (sequence state is a plain dict), so prefill, portions and token-by-token decoding are the
    same function called differently."""

    def __init__(self, cfg, sd):
        self.cfg = cfg
        self.sd = {k: np.asarray(v, F) for k, v in sd.items()}
        self.eps = cfg["norm"]["eps"]

    def sub(self, prefix):
        n = len(prefix)
        return {k[n:]: v for k, v in self.sd.items() if k.startswith(prefix)}

    def new_state(self):
        return {"pos": 0, "gla": {}, "lat": {}}

    def forward(self, tokens, st=None, taps=None):
        """tokens -> logits [T, vocab]; st is updated in place.  taps (a list) receives the stream after every layer."""
        cfg, eps = self.cfg, self.eps
        st = self.new_state() if st is None else st
        T = len(tokens)
        pos = np.arange(st["pos"], st["pos"] + T)
        alpha = cfg["postln_alpha"]
        x = self.sd["embed"][np.asarray(tokens)]
        for i, ly in enumerate(cfg["layers"]):
            m = dict(ly["mixer"], eps=eps)
            p = self.sub(f"l{i}.mix.")
            if ly["type"] == "gla":
                y, st["gla"][i] = gla_mixer(x, p, m, st["gla"].get(i))
            elif ly["type"] == "latent_attention":
                src = m.get("kv_from")
                if src is None:
                    c, kr = latent_kv(x, p, m, pos)
                    old = st["lat"].get(i)
                    st["lat"][i] = (c, kr) if old is None else (np.concatenate([old[0], c]), np.concatenate([old[1], kr]))
                    src = i
                c, kr = st["lat"][src]
                y = latent_attention(x, p, m, pos, c, kr, np.arange(c.shape[0]))
            else:
                raise ValueError(ly["type"])
            x = norm_offset_gain(alpha * x + y, self.sd[f"l{i}.norm1"], eps)
            if ly.get("mlp"):
                if ly["mlp"]["kind"] != "dense":
                    raise ValueError(ly["mlp"]["kind"])
                x = norm_offset_gain(alpha * x + dense_ff(x, self.sub(f"l{i}.mlp."), ly["mlp"]["limit"]), self.sd[f"l{i}.norm2"], eps)
            if taps is not None:
                taps.append(x.copy())
        st["pos"] += T
        z = norm_offset_gain(x, self.sd["final.norm"], eps) @ self.sd["head"].T
        return softcap(z, cfg.get("logit_softcap"))

    def greedy(self, prompt, n):
        st = self.new_state()
        z = self.forward(prompt, st)[-1]
        out, rows = [], []
        for _ in range(n):
            rows.append(z)
            out.append(int(np.argmax(z)))
            z = self.forward([out[-1]], st)[-1]
        return out, np.stack(rows)


# ------------------------------------------------------------------ random checkpoints for tests
def random_config(seed=0, width=96, vocab=160, order=("gla", "latent_attention", "gla", "latent_attention"), share=True,
                  gla=None, lat=None, ff=112, limit=1.25, alpha=1.5, cap=12.0, eps=1e-5, mlp_on=("latent_attention",)):
    """A small configuration with sizes that are pairwise different wherever the design allows it."""
    gla = dict(dict(heads=3, dim=16, vdim=24, tau=8.0), **(gla or {}))
    lat = dict(dict(heads=3, dim=24, vdim=40, kv_rank=48, q_rank=32, rot_dim=16, window=20, base=10000.0), **(lat or {}))
    layers, first_lat = [], None
    for i, t in enumerate(order):
        if t == "gla":
            mixer = dict(heads=gla["heads"], dim=gla["dim"], vdim=gla["vdim"], tau=gla["tau"])
        else:
            mixer = dict(heads=lat["heads"], dim=lat["dim"], vdim=lat["vdim"], kv_rank=lat["kv_rank"], q_rank=lat["q_rank"],
                         rot_dim=lat["rot_dim"], rot=dict(base=lat["base"], dims=lat["rot_dim"]), mask=dict(size=lat["window"]),
                         scale=float((lat["dim"] + lat["rot_dim"]) ** -0.5))
            if first_lat is None:
                first_lat = i
            elif share:
                mixer["kv_from"] = first_lat
        layers.append(dict(type=t, mixer=mixer, mlp=dict(kind="dense", ff=ff, limit=limit) if t in mlp_on else None))
    return dict(architecture="Risepel", width=width, vocab=vocab, layers=layers, postln_alpha=alpha, logit_softcap=cap,
                norm=dict(eps=eps))


def random_state_dict(cfg, seed=0, decay_rank=8, std=None):
    from .weights import _t
    W, V = cfg["width"], cfg["vocab"]
    s = lambda n: (std if std is not None else 1.0 / math.sqrt(n))
    sd = {"embed": _t(seed, "embed", (V, W), 1.0), "final.norm": _t(seed, "fn", (W,), 0.1), "head": _t(seed, "head", (V, W), s(W))}
    for i, ly in enumerate(cfg["layers"]):
        m, p = ly["mixer"], f"l{i}."
        sd[p + "norm1"] = _t(seed, p + "n1", (W,), 0.1)
        H, Dk, Dv = m["heads"], m["dim"], m["vdim"]
        if ly["type"] == "gla":
            for n, rows in (("q", H * Dk), ("k", H * Dk), ("v", H * Dv), ("g", H * Dv)):
                sd[p + "mix." + n] = _t(seed, p + n, (rows, W), s(W))
            sd[p + "mix.o"] = _t(seed, p + "o", (W, H * Dv), s(H * Dv))
            sd[p + "mix.norm"] = _t(seed, p + "hn", (Dv,), 0.1, 1.0)
            sd[p + "mix.a1"] = _t(seed, p + "a1", (decay_rank, W), s(W))
            sd[p + "mix.a2"] = _t(seed, p + "a2", (H * Dk, decay_rank), 1.0)
            sd[p + "mix.a2.b"] = _t(seed, p + "a2b", (H * Dk,), 1.0, 2.0)
        else:
            R, Dr, Q = m["kv_rank"], m["rot_dim"], m["q_rank"]
            sd[p + "mix.dq"] = _t(seed, p + "dq", (Q, W), s(W))
            sd[p + "mix.dq.norm"] = _t(seed, p + "dqn", (Q,), 0.1, 1.0)
            sd[p + "mix.uq"] = _t(seed, p + "uq", (H * (Dk + Dr), Q), 2.0 * s(Q))
            if "kv_from" not in m:
                sd[p + "mix.dkv"] = _t(seed, p + "dkv", (R + Dr, W), s(W))
                sd[p + "mix.dkv.norm"] = _t(seed, p + "dkvn", (R,), 0.1, 1.0)
            sd[p + "mix.uk"] = _t(seed, p + "uk", (H * Dk, R), 2.0 * s(R))
            sd[p + "mix.uv"] = _t(seed, p + "uv", (H * Dv, R), s(R))
            sd[p + "mix.sink"] = _t(seed, p + "sink", (H,), 1.0)
            sd[p + "mix.g"] = _t(seed, p + "g", (H * Dv, W), s(W))
            sd[p + "mix.o"] = _t(seed, p + "o", (W, H * Dv), s(H * Dv))
        if ly.get("mlp"):
            Fn = ly["mlp"]["ff"]
            sd[p + "norm2"] = _t(seed, p + "n2", (W,), 0.1)
            sd[p + "mlp.gate"] = _t(seed, p + "gate", (Fn, W), 2.0 * s(W))
            sd[p + "mlp.gate.b"] = _t(seed, p + "gateb", (Fn,), 0.3)
            sd[p + "mlp.up"] = _t(seed, p + "up", (Fn, W), 2.0 * s(W))
            sd[p + "mlp.up.b"] = _t(seed, p + "upb", (Fn,), 0.3)
            sd[p + "mlp.down"] = _t(seed, p + "down", (W, Fn), s(Fn))
            sd[p + "mlp.down.b"] = _t(seed, p + "downb", (W,), 0.1)
    return sd
