"""A plain, slow statement of the Pikalorn decoder: one function per mechanism, float64 NumPy on the CPU, one
masked matrix per head and one token at a time in the recurrence.  It shares no code with the library: it has its
own file reader, reads ``config.json`` itself and knows nothing of pages, slots or steps.  The tests hold the
library to it.

Notation: x is the residual stream [T, W], h a sublayer's input, p a position (from 0), H heads, G key/value
heads, d the query/key size of a head, e its value size, r the size of a latent, R the rotated lanes of a head.

The design in short.  x0 = embed[token] * s.  The layers are listed one by one; every layer is parallel with ONE
norm: h = n1(x), x <- x + mixer(h) + ff(h).  Mixers:

* ``attention``: grouped-query softmax attention with biases on q, k and the output, a per-head RMS norm of q and
  k, a half-split rotation of a head's first R lanes, values that ARE the keys as projected (before norm and
  rotation), a learned sink logit per head in the softmax's denominator, and an elementwise sigmoid gate on the
  concatenated heads;
* ``latent_attention``: queries through a normed latent; one normed latent c per position from which every head's
  unrotated key part and value are made, plus one rotated key part that all heads share (pairs of neighbouring
  lanes, frequencies rescaled per pair between two wavelengths, cos and sin stretched); a sink; a layer may read
  an earlier layer's c and rotated key part instead of making its own;
* ``delta``: the gated delta rule: short causal convolutions and SiLU on q, k, v, unit q and k, a decay and a
  write strength per head and token, S <- g S; u = b (v - S^T k); S <- S + k u^T; o = S^T q; per-head RMS norm,
  a SiLU gate.

Feed-forward: down(silu(gate h) * up h).  Output: final norm, then the vocabulary matrix.
"""
from __future__ import annotations

import json
import math
import struct
from pathlib import Path

import numpy as np

UNIT_EPS = 1e-6         # inside the root that makes q and k of the delta rule unit vectors
STRETCH_SLOPE = 0.1     # cos and sin of a rescaled rotation are multiplied by STRETCH_SLOPE * ln(factor) + 1
RAMP_FLOOR = 0.001      # the least width of the ramp between the two wavelengths


# -- files ----------------------------------------------------------------------------

def read_safetensors(path) -> dict:
    raw = Path(path).read_bytes()
    (n,) = struct.unpack("<Q", raw[:8])
    header = json.loads(raw[8:8 + n])
    data = raw[8 + n:]
    out = {}
    for name, info in header.items():
        if name == "__metadata__":
            continue
        lo, hi = info["data_offsets"]
        buf, dt = data[lo:hi], info["dtype"]
        if dt == "BF16":
            a = (np.frombuffer(buf, dtype="<u2").astype(np.uint32) << 16).view(np.float32).astype(np.float64)
        elif dt == "F32":
            a = np.frombuffer(buf, dtype="<f4").astype(np.float64)
        elif dt == "I32":
            a = np.frombuffer(buf, dtype="<i4").astype(np.int64)
        else:
            raise ValueError(f"{name}: element type {dt}")
        out[name] = a.reshape(info["shape"])
    return out


def load(folder):
    folder = Path(folder)
    return json.loads((folder / "config.json").read_text()), read_safetensors(folder / "model.safetensors")


# -- small functions --------------------------------------------------------------------

def sigmoid(z):
    return 1.0 / (1.0 + np.exp(-z))


def silu(z):
    return z * sigmoid(z)


def softplus(z):
    return np.maximum(z, 0.0) + np.log1p(np.exp(-np.abs(z)))


def rms_norm(x, w, eps):
    return x / np.sqrt(np.mean(x * x, axis=-1, keepdims=True) + eps) * w


def sink_softmax(s, visible, sink):
    """Rows of s [T, T] over the visible keys, with exp(sink) as one more term of the denominator (it has no value)."""
    s = np.where(visible, s, -np.inf)
    m = np.maximum(s.max(axis=-1, keepdims=True), sink)
    w = np.exp(s - m)
    return w / (w.sum(axis=-1, keepdims=True) + np.exp(sink - m))


def causal(T):
    i = np.arange(T)
    return i[None, :] <= i[:, None]


# -- positions ----------------------------------------------------------------------------

def rotary_frequencies(rot: dict):
    """(f [dims / 2], stretch): pair i turns by p * f_i; with ``scaling`` the frequencies between two wavelengths are
    blended towards f_i / factor and cos and sin are multiplied by ``stretch``."""
    dims, base = int(rot["dims"]), float(rot["base"])
    i = np.arange(dims // 2, dtype=np.float64)
    f = base ** (-2.0 * i / dims)
    sc = rot.get("scaling")
    if sc is None:
        return f, 1.0
    factor, original = float(sc["factor"]), float(sc["original"])

    def lane_of(turns):          # the (fractional) pair whose wavelength makes ``turns`` turns over the original range
        return dims * math.log(original / (2.0 * math.pi * turns)) / (2.0 * math.log(base))
    lo = max(math.floor(lane_of(float(sc["fast"]))), 0)
    hi = min(math.ceil(lane_of(float(sc["slow"]))), dims - 1)
    ramp = np.clip((i - lo) / max(hi - lo, RAMP_FLOOR), 0.0, 1.0)
    return f / factor * ramp + f * (1.0 - ramp), STRETCH_SLOPE * math.log(factor) + 1.0


def rotate(x, positions, rot: dict, layout: str):
    """x [T, heads, lanes]: the first ``dims`` lanes of every head are turned, the rest pass.  ``layout`` "half": lane i
    pairs with lane i + dims/2; "pairs": lane 2i with lane 2i + 1."""
    dims = int(rot["dims"])
    f, stretch = rotary_frequencies(rot)
    a = np.asarray(positions, dtype=np.float64)[:, None] * f[None, :]
    c, s = (np.cos(a) * stretch)[:, None, :], (np.sin(a) * stretch)[:, None, :]
    out = x.copy()
    if layout == "half":
        u, v = x[..., :dims // 2], x[..., dims // 2:dims]
        out[..., :dims // 2], out[..., dims // 2:dims] = u * c - v * s, v * c + u * s
    else:
        u, v = x[..., 0:dims:2], x[..., 1:dims:2]
        out[..., 0:dims:2], out[..., 1:dims:2] = u * c - v * s, v * c + u * s
    return out


# -- mixers ---------------------------------------------------------------------------------

def attention(h, positions, m: dict, w: dict, p: str, eps: float):
    T = h.shape[0]
    H, G, d = m["heads"], m["kv_heads"], m["dim"]
    q = (h @ w[p + "q"].T + w[p + "q.b"]).reshape(T, H, d)
    k = (h @ w[p + "k"].T + w[p + "k.b"]).reshape(T, G, d)
    v = k                                           # the values are the keys as projected
    q, k = rms_norm(q, w[p + "q.norm"], eps), rms_norm(k, w[p + "k.norm"], eps)
    if m.get("rot") is not None:
        q, k = rotate(q, positions, m["rot"], "half"), rotate(k, positions, m["rot"], "half")
    see = causal(T)
    heads = np.zeros((T, H, d))
    for a in range(H):
        g = a // (H // G)
        pr = sink_softmax(q[:, a] @ k[:, g].T * m["scale"], see, w[p + "sink"][a])
        heads[:, a] = pr @ v[:, g]
    gated = heads.reshape(T, H * d) * sigmoid(h @ w[p + "g"].T)
    return gated @ w[p + "o"].T + w[p + "o.b"]


def latent_kv(h, positions, m: dict, w: dict, p: str, eps: float):
    """What a latent layer keeps per position: (c [T, r], the shared rotated key part [T, R])."""
    r, R = m["kv_rank"], m["rot_dim"]
    z = h @ w[p + "dkv"].T
    c = rms_norm(z[:, :r], w[p + "dkv.norm"], eps)
    kr = rotate(z[:, None, r:r + R], positions, m["rot"], "pairs")[:, 0]
    return c, kr


def latent_attention(h, positions, m: dict, w: dict, p: str, eps: float, kept):
    """``kept``: (c, rotated key part) of this layer or of the layer it reads."""
    T = h.shape[0]
    H, d, R, e = m["heads"], m["dim"], m["rot_dim"], m["vdim"]
    c, kr = kept
    cq = rms_norm(h @ w[p + "dq"].T, w[p + "dq.norm"], eps)
    q = (cq @ w[p + "uq"].T).reshape(T, H, d + R)
    qn, qr = q[..., :d], rotate(q[..., d:], positions, m["rot"], "pairs")
    kn = (c @ w[p + "uk"].T).reshape(T, H, d)
    v = (c @ w[p + "uv"].T).reshape(T, H, e)
    see = causal(T)
    heads = np.zeros((T, H, e))
    for a in range(H):
        s = (qn[:, a] @ kn[:, a].T + qr[:, a] @ kr.T) * m["scale"]
        heads[:, a] = sink_softmax(s, see, w[p + "sink"][a]) @ v[:, a]
    return heads.reshape(T, H * e) @ w[p + "o"].T


def short_conv(x, taps_w):
    """x [T, C], taps_w [C, taps]: y[t] = sum_j taps_w[:, j] x[t - (taps - 1) + j], zeros before the start."""
    T, C = x.shape
    taps = taps_w.shape[1]
    pad = np.concatenate([np.zeros((taps - 1, C)), x], axis=0)
    y = np.zeros((T, C))
    for j in range(taps):
        y += pad[j:j + T] * taps_w[:, j][None, :]
    return y


def delta_rule(q, k, v, g, b):
    """q, k [T, H, d] (unit k; q scaled), v [T, H, e], g, b [T, H].  One token at a time, the state from zero."""
    T, H, d = q.shape
    e = v.shape[2]
    S = np.zeros((H, d, e))
    o = np.zeros((T, H, e))
    for t in range(T):
        for a in range(H):
            S[a] *= g[t, a]
            u = b[t, a] * (v[t, a] - S[a].T @ k[t, a])
            S[a] += np.outer(k[t, a], u)
            o[t, a] = S[a].T @ q[t, a]
    return o


def delta(h, m: dict, w: dict, p: str, eps: float):
    T = h.shape[0]
    H, G, d, e = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = silu(short_conv(h @ w[p + "q"].T, w[p + "q.conv"])).reshape(T, G, d)
    k = silu(short_conv(h @ w[p + "k"].T, w[p + "k.conv"])).reshape(T, G, d)
    v = silu(short_conv(h @ w[p + "v"].T, w[p + "v.conv"])).reshape(T, H, e)
    q = q / np.sqrt((q * q).sum(-1, keepdims=True) + UNIT_EPS) * d ** -0.5
    k = k / np.sqrt((k * k).sum(-1, keepdims=True) + UNIT_EPS)
    group = np.arange(H) // (H // G)
    b = sigmoid(h @ w[p + "b"].T)
    g = np.exp(-np.exp(w[p + "A_log"])[None, :] * softplus(h @ w[p + "a"].T + w[p + "dt_bias"][None, :]))
    o = delta_rule(q[:, group], k[:, group], v, g, b)
    o = rms_norm(o, w[p + "norm"], eps) * silu(h @ w[p + "g"].T).reshape(T, H, e)
    return o.reshape(T, H * e) @ w[p + "o"].T


def feed_forward(h, w: dict, p: str):
    return (silu(h @ w[p + "gate"].T) * (h @ w[p + "up"].T)) @ w[p + "down"].T


# -- the model --------------------------------------------------------------------------------

def forward(config: dict, w: dict, tokens, return_streams: bool = False):
    """Logits [T, vocab] of one sequence from position 0; with ``return_streams`` also the stream after every layer."""
    eps = float(config["norm"]["eps"])
    tokens = np.asarray(tokens, dtype=np.int64)
    positions = np.arange(len(tokens))
    x = w["embed"][tokens] * float((config.get("embedding") or {}).get("scale", 1.0))
    kept, streams = {}, []
    for i, layer in enumerate(config["layers"]):
        m, p = layer["mixer"], f"l{i}.mix."
        h = rms_norm(x, w[f"l{i}.norm1"], eps)
        if layer["type"] == "attention":
            y = attention(h, positions, m, w, p, eps)
        elif layer["type"] == "latent_attention":
            src = m.get("kv_from")
            if src is None:
                kept[i] = latent_kv(h, positions, m, w, p, eps)
                src = i
            y = latent_attention(h, positions, m, w, p, eps, kept[src])
        elif layer["type"] == "delta":
            y = delta(h, m, w, p, eps)
        else:
            raise ValueError(f"layer {i}: type {layer['type']!r}")
        if layer.get("mlp") is not None:
            y = y + feed_forward(h, w, f"l{i}.mlp.")
        x = x + y
        streams.append(x.copy())
    logits = rms_norm(x, w["final.norm"], eps) @ w["head"].T
    return (logits, np.stack(streams)) if return_streams else logits


def greedy(config: dict, w: dict, prompt, n: int):
    """n tokens chosen greedily (the first largest logit), the whole sequence recomputed for every token."""
    seq, out = list(prompt), []
    for _ in range(n):
        out.append(int(np.argmax(forward(config, w, seq)[-1])))
        seq.append(out[-1])
    return out
