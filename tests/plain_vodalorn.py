"""A plain, slow statement of the Vodalorn decoder: one function per mechanism, float64 NumPy on the CPU, one masked
matrix per head for the softmax side and one token at a time in the recurrences.  It shares no code with the library:
it has its own file reader, reads ``config.json`` itself and knows nothing of pages, slots, steps or state rows.  The
tests hold the library to it.

Notation: x is the residual stream [T, W], h a sublayer's input, p a position (from 0), H heads, G key/value (or
query/key) heads, d the query/key size of a head, e its value size, m the residual weight.

The design in short.  x0 = embed[token] + pair[hash(previous token, token)].  The layers are listed one by one; a
range of them may run several times with the same weights, and before every such pass x <- W_in [x; x0] + step[t].
A layer: x <- x + m mixer(LN1(x)); x <- x + m ff(LN2(x)); x <- x + m rms(W_p (gelu(W_s x) * lanes[token])) w.
Mixers: ``parallel`` (half the sum of the RMS-normed outputs of windowed softmax attention and of retention) and
``channel_delta`` (the gated delta rule with a decay per key channel).  Feed-forwards: the square of relu between two
matrices, or routed experts.  Output: LN, then the vocabulary matrix.
"""
from __future__ import annotations

import json
import math
import struct
from pathlib import Path

import numpy as np

UNIT_EPS = 1e-6          # inside the root that makes q and k of the delta rule unit vectors
WEIGHT_EPS = 1e-20       # added to the sum of the chosen experts' scores
SWISH = 1.702            # the experts' gate is g * sigmoid(SWISH * g)


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


def gelu_tanh(z):
    return 0.5 * z * (1.0 + np.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def rms(x, eps):
    """x over the root of its mean square along the last axis, eps inside the root; no weight."""
    return x / np.sqrt(np.mean(x * x, axis=-1, keepdims=True) + eps)


def layer_norm(x, w, b, eps):
    mean = np.mean(x, axis=-1, keepdims=True)
    var = np.mean((x - mean) ** 2, axis=-1, keepdims=True)
    return (x - mean) / np.sqrt(var + eps) * w + b


def rotate(x, positions, rot):
    """x [T, heads, d]: lane i < dims/2 of every head is paired with lane i + dims/2 and the pair is turned by
    p * base^(-2i/dims); lanes from dims on pass.  ``rot`` None: nothing turns."""
    if not rot:
        return x
    dims, half = rot["dims"], rot["dims"] // 2
    angle = np.asarray(positions, dtype=np.float64)[:, None] * (float(rot["base"]) ** (-2.0 * np.arange(half) / dims))[None, :]
    c, s = np.cos(angle)[:, None, :], np.sin(angle)[:, None, :]
    lo, hi = x[..., :half], x[..., half:dims]
    return np.concatenate([lo * c - hi * s, hi * c + lo * s, x[..., dims:]], axis=-1)


# -- the embedding ----------------------------------------------------------------------

def pair_rows(tokens, pair):
    """The row of the pair table for every token: a hash of (previous token, token), the table's last row for the
    first token."""
    rows = [pair["buckets"]]
    for prev, cur in zip(tokens[:-1], tokens[1:]):
        rows.append((prev * pair["mul_prev"] + cur * pair["mul_cur"]) % pair["buckets"])
    return rows[:len(tokens)]


def embedding(config, w, tokens):
    x = w["embed"][tokens]
    pair = (config.get("embedding") or {}).get("bigram")
    if pair:
        x = x + w["bigram"][pair_rows(list(tokens), pair)]
    return x


# -- mixers -------------------------------------------------------------------------------

def window_attention(h, positions, m, w, p):
    """Grouped-query softmax attention with biases on q, k, v; query i sees key j when 0 <= i - j < window (all
    earlier keys without a window)."""
    T, H, G, d, e = h.shape[0], m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = (h @ w[p + ".q"].T + w[p + ".q.b"]).reshape(T, H, d)
    k = (h @ w[p + ".k"].T + w[p + ".k.b"]).reshape(T, G, d)
    v = (h @ w[p + ".v"].T + w[p + ".v.b"]).reshape(T, G, e)
    q, k = rotate(q, positions, m.get("rot")), rotate(k, positions, m.get("rot"))
    dist = np.arange(T)[:, None] - np.arange(T)[None, :]
    seen = dist >= 0
    if m.get("mask"):
        seen &= dist < m["mask"]["size"]
    out = np.zeros((T, H, e))
    for a in range(H):
        g = a // (H // G)
        s = np.where(seen, (q[:, a] @ k[:, g].T) * m["scale"], -np.inf)
        pr = np.exp(s - s.max(axis=-1, keepdims=True))
        out[:, a] = (pr / pr.sum(axis=-1, keepdims=True)) @ v[:, g]
    return out.reshape(T, H * e) @ w[p + ".o"].T


def retention_rule(q, k, v, decay):
    """One head: S <- decay S + k v^T; o = S^T q, token by token, from S = 0.  q, k [T, d]; v [T, e]."""
    S = np.zeros((q.shape[1], v.shape[1]))
    o = np.zeros_like(v)
    for t in range(q.shape[0]):
        S = decay * S + np.outer(k[t], v[t])
        o[t] = S.T @ q[t]
    return o


def retention(h, positions, m, w, p, eps):
    T, H, d, e = h.shape[0], m["heads"], m["dim"], m["vdim"]
    q = rotate((h @ w[p + ".q"].T).reshape(T, H, d), positions, m.get("rot"))
    k = rotate((h @ w[p + ".k"].T).reshape(T, H, d), positions, m.get("rot")) * d ** -0.5
    v = (h @ w[p + ".v"].T).reshape(T, H, e)
    o = np.stack([retention_rule(q[:, a], k[:, a], v[:, a], m["decay"][a]) for a in range(H)], axis=1)
    return (rms(o, eps).reshape(T, H * e) * silu(h @ w[p + ".g"].T)) @ w[p + ".o"].T


def mixer_pair(h, positions, m, w, p, eps):
    left = window_attention(h, positions, m["left"], w, p + ".left")
    right = retention(h, positions, m["right"], w, p + ".right", eps)
    return 0.5 * (rms(left, eps) * w[p + ".left.out"] + rms(right, eps) * w[p + ".right.out"])


def short_conv(x, taps_w):
    """x [T, C], taps_w [C, taps]: a causal convolution over time per channel; the last tap is the current token's,
    and what lies before the sequence is zero."""
    T, taps = x.shape[0], taps_w.shape[1]
    padded = np.concatenate([np.zeros((taps - 1, x.shape[1])), x], axis=0)
    return sum(padded[j:j + T] * taps_w[:, j] for j in range(taps))


def channel_delta_rule(q, k, v, g, beta):
    """One head: S <- diag(g) S; u = beta (v - S^T k); S <- S + k u^T; o = S^T q (the read-out sees the write).
    q, k, g [T, d]; v [T, e]; beta [T]."""
    S = np.zeros((q.shape[1], v.shape[1]))
    o = np.zeros_like(v)
    for t in range(q.shape[0]):
        S = g[t][:, None] * S
        u = beta[t] * (v[t] - S.T @ k[t])
        S = S + np.outer(k[t], u)
        o[t] = S.T @ q[t]
    return o


def channel_delta(h, m, w, p, eps):
    T, H, G, d, e = h.shape[0], m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = silu(short_conv(h @ w[p + ".q"].T, w[p + ".q.conv"])).reshape(T, G, d)
    k = silu(short_conv(h @ w[p + ".k"].T, w[p + ".k.conv"])).reshape(T, G, d)
    v = silu(short_conv(h @ w[p + ".v"].T, w[p + ".v.conv"])).reshape(T, H, e)
    q = q / np.sqrt(np.sum(q * q, axis=-1, keepdims=True) + UNIT_EPS) * d ** -0.5
    k = k / np.sqrt(np.sum(k * k, axis=-1, keepdims=True) + UNIT_EPS)
    beta = sigmoid(h @ w[p + ".b"].T)
    z = (h @ w[p + ".a1"].T) @ w[p + ".a2"].T + w[p + ".dt_bias"]
    g = np.exp(-np.exp(w[p + ".A_log"])[None, :, None] * softplus(z).reshape(T, H, d))
    o = np.stack([channel_delta_rule(q[:, a // (H // G)], k[:, a // (H // G)], v[:, a], g[:, a], beta[:, a])
                  for a in range(H)], axis=1)
    gate = sigmoid((h @ w[p + ".g1"].T) @ w[p + ".g2"].T)
    return ((rms(o, eps) * w[p + ".norm"]).reshape(T, H * e) * gate) @ w[p + ".o"].T


# -- feed-forwards ---------------------------------------------------------------------------

def dense_ff(h, w, p):
    return (np.maximum(h @ w[p + ".up"].T, 0.0) ** 2) @ w[p + ".down"].T


def route(z, router):
    """One token's logits z [E] -> (chosen experts, their weights).  Scores are the softmax over all experts; with
    groups only the experts of the best groups (by their largest score) can be chosen."""
    E, top = router["experts"], router["top"]
    s = np.exp(z - z.max())
    s = s / s.sum()
    allowed = np.ones(E, dtype=bool)
    groups = router.get("groups")
    if groups:
        per = E // groups["count"]
        best = np.argsort(-s.reshape(groups["count"], per).max(axis=-1), kind="stable")[:groups["keep"]]
        allowed[:] = False
        for b in best:
            allowed[b * per:(b + 1) * per] = True
    chosen = np.argsort(-np.where(allowed, s, -1.0), kind="stable")[:top]
    return chosen, s[chosen] / (s[chosen].sum() + WEIGHT_EPS) * router.get("scale", 1.0)


def expert(h, w, p, limit):
    g = np.minimum(w[p + ".gate"] @ h, limit)
    u = np.clip(w[p + ".up"] @ h, -limit, limit)
    return w[p + ".down"] @ (g * sigmoid(SWISH * g) * (u + 1.0))


def routed_ff(h, mlp, w, p):
    out = np.zeros_like(h)
    for t in range(h.shape[0]):
        chosen, weights = route(w[p + ".router"] @ h[t], mlp["router"])
        for a, c in zip(chosen, weights):
            out[t] += c * expert(h[t], w, f"{p}.e{a}", mlp["expert"]["limit"])
    return out


def token_side(x, tokens, w, p, lanes, eps):
    """What a token adds to its own stream at the end of a layer, before the residual weight: lanes [T, D] are the
    layer's part of the token's row of the shared table."""
    y = (gelu_tanh(x @ w[p + ".gate"].T) * lanes) @ w[p + ".proj"].T
    return rms(y, eps) * w[p + ".norm"]


# -- the model ---------------------------------------------------------------------------------

def layer_runs(config):
    """[(layer, pass or None)]: the layers in running order; the first layer of a pass of the loop carries the pass."""
    n, loop = len(config["layers"]), config.get("loop")
    if not loop:
        return [(i, None) for i in range(n)]
    a, b = loop["start"], loop["stop"]
    runs = [(i, None) for i in range(a)]
    for t in range(loop["times"]):
        runs += [(i, t if i == a else None) for i in range(a, b)]
    return runs + [(i, None) for i in range(b, n)]


def forward(config, w, tokens, return_streams: bool = False):
    """Logits [T, V] of one sequence from its first token; with ``return_streams`` also x after every layer run."""
    tokens = [int(t) for t in tokens]
    T, eps, m = len(tokens), config["norm"]["eps"], config.get("residual_mult", 1.0)
    positions = np.arange(T)
    x = embedding(config, w, tokens)
    x0 = x.copy()
    streams = []
    side = config.get("token_side")
    for i, t in layer_runs(config):
        layer, p = config["layers"][i], f"l{i}"
        if t is not None:
            x = np.concatenate([x, x0], axis=-1) @ w["loop.in"].T + w["loop.step"][t]
        h = layer_norm(x, w[p + ".norm1"], w[p + ".norm1.b"], eps)
        if layer["type"] == "parallel":
            x = x + m * mixer_pair(h, positions, layer["mixer"], w, p + ".mix", eps)
        else:
            x = x + m * channel_delta(h, layer["mixer"], w, p + ".mix", eps)
        if layer.get("mlp"):
            h = layer_norm(x, w[p + ".norm2"], w[p + ".norm2.b"], eps)
            x = x + m * (dense_ff(h, w, p + ".mlp") if layer["mlp"]["kind"] == "dense" else routed_ff(h, layer["mlp"], w, p + ".mlp"))
        if side:
            D = side["dim"]
            x = x + m * token_side(x, tokens, w, p + ".side", w["side.embed"][tokens][:, i * D:(i + 1) * D], eps)
        streams.append(x.copy())
    logits = layer_norm(x, w["final.norm"], w["final.norm.b"], eps) @ w["head"].T
    return (logits, streams) if return_streams else logits


def greedy(config, w, prompt, n: int):
    """n tokens chosen one by one as the largest logit (the lower index wins a tie), each from a full forward pass."""
    tokens = [int(t) for t in prompt]
    out = []
    for _ in range(n):
        nxt = int(np.argmax(forward(config, w, tokens)[-1]))
        out.append(nxt)
        tokens.append(nxt)
    return out
