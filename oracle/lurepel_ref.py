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
    gate = sigmoid(h @ p["g"].T)  # [T, H]
    out = np.zeros((T, H, v.shape[-1]), F)
    for t in range(T):
        see = np.array([chunk_visible(int(pos[t]), int(j), size) for j in kpos])
        for hh in range(H):
            g = hh // (H // G)
            s = (kn[see, g] @ q[t, hh]) * m["scale"]
            mx = max(0.0, s.max()) if s.size else 0.0
            e = np.exp(s - mx)
            pr = e / (np.exp(-mx) + e.sum())  # one unit of weight (score 0) belongs to nothing
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
