"""Plain, slow float64 restatement of the Lurepel decoder (numpy only; one function per mechanism).

The design: the embedding is normed; every sublayer reads the residual stream itself and its OUTPUT is normed before it is
added (x <- x + norm(f(x))).  The mixer is grouped-query attention whose values are the key projections themselves (taken
before rotation and normalisation), with a partial interleaved rotary embedding (Llama-3 style frequency scaling), unit
RMS normalisation of rotated queries and keys, a block-diagonal ("chunked") causal mask, one extra unit in the softmax
denominator, and a per-head sigmoid output gate.  The feed-forward is a gated unit (tanh-GELU) or a mixture of small
SiLU-gated experts with a corrected top-k choice, un-renormalised softmax weights and identity experts.
Notation: T tokens, W width, H / G query / key-value heads, D per-head size.  Nothing here is shared with the CUDA path.
"""
import math

import numpy as np

F = np.float64


def rms_unit(x, eps):
    """x / sqrt(mean(x^2) + eps) over the last axis."""
    x = np.asarray(x, F)
    return x / np.sqrt((x * x).mean(-1, keepdims=True) + eps)


def norm_gain(x, w, eps):
    return rms_unit(x, eps) * np.asarray(w, F)


def sigmoid(z):
    return 1.0 / (1.0 + np.exp(-np.asarray(z, F)))


def silu(z):
    return z * sigmoid(z)


def gelu_tanh(z):
    z = np.asarray(z, F)
    return 0.5 * z * (1.0 + np.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


# ------------------------------------------------------------------ rotary embedding
def rotary_freqs(rot):
    """Per-pair frequencies f_i = base^(-2i/dims), i < dims/2, with the wavelength-dependent rescaling when rot["scaling"]
    is given: long wavelengths (> original/low) are divided by `factor`, short ones (< original/high) kept, and the band
    between is blended linearly in original/wavelength."""
    dims = int(rot["dims"])
    f = float(rot["base"]) ** (-2.0 * np.arange(dims // 2, dtype=F) / dims)
    sc = rot.get("scaling")
    if not sc:
        return f
    factor, low, high, orig = float(sc["factor"]), float(sc["low"]), float(sc["high"]), float(sc["original"])
    out = f.copy()
    for i, fi in enumerate(f):
        wl = 2.0 * math.pi / fi
        if wl < orig / high:
            continue
        if wl > orig / low:
            out[i] = fi / factor
        else:
            s = (orig / wl - low) / (high - low)
            out[i] = (1.0 - s) * fi / factor + s * fi
    return out


def rotate_interleaved(v, pos, freqs):
    """v [T, heads, D]: entries (2i, 2i+1), i < len(freqs), turn by the angle pos * freqs[i]; the rest pass."""
    v = np.array(v, F)
    n = len(freqs)
    a = np.asarray(pos, F)[:, None] * freqs[None, :]
    c, s = np.cos(a)[:, None, :], np.sin(a)[:, None, :]
    u, w = v[..., 0:2 * n:2].copy(), v[..., 1:2 * n:2].copy()
    v[..., 0:2 * n:2] = u * c - w * s
    v[..., 1:2 * n:2] = w * c + u * s
    return v


# ------------------------------------------------------------------ attention
def chunk_visible(i, j, size):
    """Position i sees position j: causal, and both in the same block of `size` positions counted from 0 (size None or
    <= 0: plain causal)."""
    if j > i:
        return False
    return True if not size or size <= 0 else (i // size) == (j // size)


def attention_kv(h, p, m, pos, eps):
    """What a token leaves behind: its rotated unit-RMS key [T, G, D] and its value = the raw key projection [T, G, D]."""
    T = h.shape[0]
    G, D = m["kv_heads"], m["dim"]
    k = (h @ p["k"].T).reshape(T, G, D)
    rot = m.get("rot")
    kr = rotate_interleaved(k, pos, rotary_freqs(rot)) if rot and rot.get("dims") else k
    return rms_unit(kr, eps), k


def attention_mixer(h, p, m, eps, pos=None, past=None):
    """h [T, W] at positions pos (default 0..T-1) -> ([T, W], (keys, values, positions) including the past).
    past: (keys, values, positions) of earlier tokens of the sequence."""
    T = h.shape[0]
    H, G, D = m["heads"], m["kv_heads"], m["dim"]
    pos = np.arange(T) if pos is None else np.asarray(pos)
    q = (h @ p["q"].T).reshape(T, H, D)
    rot = m.get("rot")
    if rot and rot.get("dims"):
        q = rotate_interleaved(q, pos, rotary_freqs(rot))
    q = rms_unit(q, eps)
    kn, v = attention_kv(h, p, m, pos, eps)
    if past is not None:
        kn, v, kpos = np.concatenate([past[0], kn]), np.concatenate([past[1], v]), np.concatenate([past[2], pos])
    else:
        kpos = pos
    size = (m.get("mask") or {}).get("size")
    unit = 1.0 if m.get("sink", True) else 0.0  # the design always has it; tests switch it off to show that it matters
    gate = sigmoid(h @ p["g"].T)  # [T, H]
    out = np.zeros((T, H, v.shape[-1]), F)
    for t in range(T):
        see = np.array([chunk_visible(int(pos[t]), int(j), size) for j in kpos])
        for hh in range(H):
            g = hh // (H // G)
            s = (kn[see, g] @ q[t, hh]) * m["scale"]
            mx = max(0.0, s.max())
            e = np.exp(s - mx)
            pr = e / (unit * np.exp(-mx) + e.sum())  # one unit of weight (score 0) belongs to nothing
            out[t, hh] = pr @ v[see, g]
    out = out * gate[:, :, None]
    return out.reshape(T, -1) @ p["o"].T, (kn, v, kpos)


# ------------------------------------------------------------------ feed-forward
def dense_ff(h, p):
    return (gelu_tanh(h @ p["gate"].T) * (h @ p["up"].T)) @ p["down"].T


def moe_route(h, p, r):
    """-> (chosen expert ids [T, top], their weights [T, top]).  The choice adds the correction to the softmax scores;
    the weights are the uncorrected scores of the chosen, not renormalised."""
    z = np.asarray(h, F) @ p["router"].T
    z = z - z.max(-1, keepdims=True)
    s = np.exp(z)
    s = s / s.sum(-1, keepdims=True)
    pick = s + np.asarray(p["correction"], F)
    idx = np.argsort(-pick, axis=-1, kind="stable")[:, :r["top"]]
    return idx, np.take_along_axis(s, idx, -1)


def route_margin(h, p, r):
    """Per token: how far the last chosen output's choice score lies above the best one left out (inf when all are chosen)."""
    z = np.asarray(h, F) @ p["router"].T
    s = np.exp(z - z.max(-1, keepdims=True))
    pick = -np.sort(-(s / s.sum(-1, keepdims=True) + np.asarray(p["correction"], F)), axis=-1)
    return pick[:, r["top"] - 1] - pick[:, r["top"]] if pick.shape[1] > r["top"] else np.full(len(pick), np.inf)


def moe_ff(h, p, r):
    """Experts 0..experts-1 have weights; the `identity` outputs after them return their input."""
    idx, wt = moe_route(h, p, r)
    out = np.zeros_like(np.asarray(h, F))
    for t in range(h.shape[0]):
        for e, w in zip(idx[t], wt[t]):
            if e >= r["experts"]:
                out[t] += w * h[t]
            else:
                q = p[f"e{e}"]
                out[t] += w * ((silu(h[t] @ q["gate"].T) * (h[t] @ q["up"].T)) @ q["down"].T)
    return out


# ------------------------------------------------------------------ the model
def split_params(sd, n_layers):
    """Flat {name: array} of a checkpoint -> nested per-layer dictionaries of float64 arrays."""
    g = lambda k: np.asarray(sd[k], F)
    layers = []
    for i in range(n_layers):
        pre = f"l{i}."
        mix, mlp, norms = {}, {}, {}
        for k in sd:
            if not k.startswith(pre):
                continue
            rest = k[len(pre):]
            if rest.startswith("mix."):
                mix[rest[4:]] = g(k)
            elif rest.startswith("mlp."):
                parts = rest[4:].split(".")
                if len(parts) == 2:
                    mlp.setdefault(parts[0], {})[parts[1]] = g(k)
                else:
                    mlp[parts[0]] = g(k)
            else:
                norms[rest] = g(k)
        layers.append(dict(mix=mix, mlp=mlp, **norms))
    return dict(embed=g("embed"), embed_norm=g("embed.norm"), final_norm=g("final.norm"), head=g("head"), layers=layers)


def forward(cfg, sd, tokens, trace=None):
    """Whole sequence from position 0 -> logits [T, vocab].  trace (a list) receives the stream after every layer."""
    P = split_params(sd, len(cfg["layers"]))
    eps = float(cfg["norm"]["eps"])
    x = norm_gain(P["embed"][np.asarray(tokens)], P["embed_norm"], eps)
    for ly, p in zip(cfg["layers"], P["layers"]):
        if ly["type"] != "attention":
            raise ValueError(ly["type"])
        y, _ = attention_mixer(x, p["mix"], ly["mixer"], eps)
        x = x + norm_gain(y, p["norm1"], eps)
        mlp = ly.get("mlp")
        if mlp:
            y = dense_ff(x, p["mlp"]) if mlp["kind"] == "dense" else moe_ff(x, p["mlp"], mlp["router"])
            x = x + norm_gain(y, p["norm2"], eps)
        if trace is not None:
            trace.append(x.copy())
    return norm_gain(x, P["final_norm"], eps) @ P["head"].T


class LurepelOracle:
    """The decoder over a checkpoint, fed in portions: `state` keeps every layer's keys and values of the tokens seen."""

    def __init__(self, cfg, sd):
        self.cfg = cfg
        self.P = split_params(sd, len(cfg["layers"]))
        self.eps = float(cfg["norm"]["eps"])

    def new_state(self):
        return dict(pos=0, kv={})

    def forward(self, tokens, state=None, taps=None, margins=None):
        """The next tokens of one sequence -> logits [T, vocab].  taps / margins (lists) receive the stream after every
        layer / every router's choice margins per token."""
        P, eps = self.P, self.eps
        st = state if state is not None else self.new_state()
        T = len(tokens)
        pos = st["pos"] + np.arange(T)
        x = norm_gain(P["embed"][np.asarray(tokens)], P["embed_norm"], eps)
        for i, (ly, p) in enumerate(zip(self.cfg["layers"], P["layers"])):
            if ly["type"] != "attention":
                raise ValueError(ly["type"])
            y, st["kv"][i] = attention_mixer(x, p["mix"], ly["mixer"], eps, pos, st["kv"].get(i))
            x = x + norm_gain(y, p["norm1"], eps)
            mlp = ly.get("mlp")
            if mlp:
                if margins is not None and mlp["kind"] == "moe":
                    margins.append(route_margin(x, p["mlp"], mlp["router"]))
                y = dense_ff(x, p["mlp"]) if mlp["kind"] == "dense" else moe_ff(x, p["mlp"], mlp["router"])
                x = x + norm_gain(y, p["norm2"], eps)
            if taps is not None:
                taps.append(x.copy())
        st["pos"] += T
        return norm_gain(x, P["final_norm"], eps) @ P["head"].T

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
def random_config(width=80, vocab=150, order=("dense", "moe", None), heads=6, kv_heads=2, dim=24, chunk=20, rot_dims=16,
                  base=5000.0, scaling=dict(factor=4.0, low=1.0, high=3.0, original=64), scale=None, ff=72, expert_ff=40,
                  experts=5, identity=2, top=3, eps=1e-5, per_layer=None):
    """A small configuration; `order` lists each layer's feed-forward ("dense", "moe" or None), per_layer[i] overrides
    mixer keys of layer i.  The default scaling band (wavelengths 64/3 .. 64) has rotary pairs below, inside and above it."""
    layers = []
    for i, kind in enumerate(order):
        mixer = dict(heads=heads, kv_heads=kv_heads, dim=dim, vdim=dim, scale=float(scale if scale is not None else 3.0 / math.sqrt(dim)))
        if chunk:
            mixer["mask"] = dict(size=chunk)
        if rot_dims:
            mixer["rot"] = dict(base=base, dims=rot_dims)
            if scaling:
                mixer["rot"]["scaling"] = dict(scaling)
        mixer.update((per_layer or {}).get(i, {}))
        mixer["vdim"] = mixer["dim"]
        if kind == "dense":
            mlp = dict(kind="dense", ff=ff)
        elif kind == "moe":
            mlp = dict(kind="moe", expert=dict(ff=expert_ff), router=dict(experts=experts, identity=identity, top=top))
        else:
            mlp = None
        layers.append(dict(type="attention", mixer=mixer, mlp=mlp))
    return dict(architecture="Lurepel", width=width, vocab=vocab, layers=layers, norm=dict(eps=eps))


def random_state_dict(cfg, seed=0):
    from .weights import _t
    W, V = cfg["width"], cfg["vocab"]
    s = lambda n: 1.0 / math.sqrt(n)
    sd = {"embed": _t(seed, "embed", (V, W), 1.0), "embed.norm": _t(seed, "en", (W,), 0.1, 1.0),
          "final.norm": _t(seed, "fn", (W,), 0.1, 1.0), "head": _t(seed, "head", (V, W), s(W))}
    for i, ly in enumerate(cfg["layers"]):
        m, p = ly["mixer"], f"l{i}."
        H, G, D = m["heads"], m["kv_heads"], m["dim"]
        sd[p + "norm1"] = _t(seed, p + "n1", (W,), 0.1, 1.0)
        sd[p + "mix.q"] = _t(seed, p + "q", (H * D, W), s(W))
        sd[p + "mix.k"] = _t(seed, p + "k", (G * D, W), s(W))
        sd[p + "mix.g"] = _t(seed, p + "g", (H, W), 2.0 * s(W))
        sd[p + "mix.o"] = _t(seed, p + "o", (W, H * D), s(H * D))
        mlp = ly.get("mlp")
        if not mlp:
            continue
        sd[p + "norm2"] = _t(seed, p + "n2", (W,), 0.1, 1.0)
        if mlp["kind"] == "dense":
            Fn = mlp["ff"]
            sd[p + "mlp.gate"] = _t(seed, p + "gate", (Fn, W), 2.0 * s(W))
            sd[p + "mlp.up"] = _t(seed, p + "up", (Fn, W), 2.0 * s(W))
            sd[p + "mlp.down"] = _t(seed, p + "down", (W, Fn), s(Fn))
        else:
            r, Fn = mlp["router"], mlp["expert"]["ff"]
            R = r["experts"] + r.get("identity", 0)
            sd[p + "mlp.router"] = _t(seed, p + "router", (R, W), 3.0 * s(W))
            # choice corrections on a grid of 0.08, shuffled: no two outputs tie by their corrections alone, so a choice is
            # a close call only where two scores happen to differ by a grid step
            from .weights import _rng, to_bf16_f32
            sd[p + "mlp.correction"] = to_bf16_f32((_rng(seed, p + "corr").permutation(R) - (R - 1) / 2.0) * 0.08)
            for e in range(r["experts"]):
                sd[p + f"mlp.e{e}.gate"] = _t(seed, p + f"e{e}g", (Fn, W), 2.0 * s(W))
                sd[p + f"mlp.e{e}.up"] = _t(seed, p + f"e{e}u", (Fn, W), 2.0 * s(W))
                sd[p + f"mlp.e{e}.down"] = _t(seed, p + f"e{e}d", (W, Fn), s(Fn))
    return sd
