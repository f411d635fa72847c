"""The Vodalorn design against its plain statement (``plain_vodalorn``): every mechanism alone, then the model through
``Engine.step`` cut in every way (whole prompts, token by token, portions down to two tokens, unequal batches, slots,
pages and state rows used again, windows and pages crossed while decoding), and greedy generation through
``Session.generate``, the command line and the trace replay.  Configurations and weights are made here; where random
weights would hide a fault (a window's edge, a key far back, a write the recurrence must remember) the weights or
inputs are made so that it shows."""
import json

import numpy as np
import pytest
import torch

import plain_vodalorn as P
from gpu_util import DEV, TOL, check
from nncpu_b200 import Engine, GenerateParams, Model, SamplerParams, Session, SessionParams
from nncpu_b200.cache import PAGE
from nncpu_b200.config import config_from_dict
from nncpu_b200.engine.model import parameter_list
from nncpu_b200.kernels import ops
from nncpu_b200.parts import Runtime
from nncpu_b200.weights import random_tensors, write_safetensors

pytestmark = pytest.mark.gpu
DTYPES = ["float32", "bfloat16"]
STORE = {"float32": torch.float32, "bfloat16": torch.bfloat16}


def dense(ff):
    return {"kind": "dense", "ff": ff}


def moe(experts, top, ff, limit, scale=None, groups=None):
    r = {"experts": experts, "top": top}
    if scale is not None:
        r["scale"] = scale
    if groups:
        r["groups"] = {"count": groups[0], "keep": groups[1]}
    return {"kind": "moe", "expert": {"ff": ff, "limit": limit}, "router": r}


def rot(base, dims):
    return {"base": base, "dims": dims}


def left(heads, kv, dim, vdim, scale, window=None, r=None):
    m = {"heads": heads, "kv_heads": kv, "dim": dim, "vdim": vdim, "scale": scale}
    if window:
        m["mask"] = {"size": window}
    if r:
        m["rot"] = r
    return m


def right(heads, dim, vdim, decay, r=None):
    m = {"heads": heads, "dim": dim, "vdim": vdim, "decay": list(decay)}
    if r:
        m["rot"] = r
    return m


def par(l, r, mlp=None):
    return {"type": "parallel", "mixer": {"left": l, "right": r}, "mlp": mlp}


def dlt(heads, kv, dim, vdim, conv, rank, gate_rank, mlp=None):
    return {"type": "channel_delta", "mlp": mlp,
            "mixer": {"heads": heads, "kv_heads": kv, "dim": dim, "vdim": vdim, "conv": conv, "rank": rank, "gate_rank": gate_rank}}


CONFIGS = {
    # odd sizes everywhere and a width that is no multiple of 8 (no tensor-core product takes it); the recurrent layer
    # first; the loop starts at the first layer and runs three times; windows of 5 and 70; a layer without a feed-forward;
    # query/key heads shared by three value heads; decays of 1 and 1/2
    "A": {"architecture": "Vodalorn", "vocab": 211, "width": 76, "norm": {"eps": 3e-6}, "residual_mult": 0.6,
          "embedding": {"bigram": {"buckets": 97, "mul_prev": 31, "mul_cur": 7}}, "token_side": {"dim": 5},
          "loop": {"start": 0, "stop": 2, "times": 3},
          "layers": [dlt(6, 2, 20, 12, 3, 7, 5, mlp=moe(6, 2, 20, 1.2, scale=1.5, groups=(3, 2))),
                     par(left(6, 2, 24, 10, 0.3, 5, rot(1e4, 16)), right(3, 10, 14, (0.9, 0.95, 0.99), rot(300.0, 6)), mlp=dense(100)),
                     par(left(4, 4, 16, 16, 0.25, 70), right(2, 8, 8, (0.5, 1.0))),
                     dlt(3, 3, 10, 36, 2, 4, 9, mlp=dense(40))]},
    # sizes the tensor-core paths take: heads of 64 and 128 lanes with values of the same size (and one layer with
    # values of another size), whole and partly rotated heads, states of 64 x 64 and 128 x 128, experts of 64 and 128
    "B": {"architecture": "Vodalorn", "vocab": 640, "width": 256, "norm": {"eps": 1e-5}, "residual_mult": 0.75,
          "embedding": {"bigram": {"buckets": 509, "mul_prev": 1009, "mul_cur": 13}}, "token_side": {"dim": 32},
          "loop": {"start": 1, "stop": 3, "times": 2},
          "layers": [par(left(8, 2, 64, 64, 0.125, 100, rot(1e6, 64)), right(4, 64, 64, (0.9, 0.97, 0.99, 0.999), rot(1e4, 32)), mlp=dense(512)),
                     dlt(4, 4, 64, 64, 4, 16, 16, mlp=moe(8, 2, 64, 1.25, scale=1.75, groups=(4, 2))),
                     par(left(4, 1, 128, 128, 0.09, 77, rot(4e5, 64)), right(2, 128, 128, (0.98, 0.995), rot(1e4, 128)), mlp=moe(16, 4, 128, 2.0)),
                     dlt(2, 1, 128, 128, 2, 20, 8, mlp=dense(256)),
                     par(left(4, 4, 64, 128, 0.125, 64, rot(1e4, 32)), right(8, 32, 32, (0.9,) * 8, rot(1e6, 32)), mlp=dense(256))]},
    # values at the edges: a window of one key, 32 query heads on one key/value head, values of one lane, a decay of
    # zero, states of one row and of one column, a convolution of one tap, one expert, every expert chosen, every group
    # kept, a residual weight of 1, no pair embedding, no per-layer token input, attention without a window and
    # without a rotation, a loop of one pass around the last layer
    "C": {"architecture": "Vodalorn", "vocab": 97, "width": 100, "norm": {"eps": 1e-5},
          "loop": {"start": 3, "stop": 4, "times": 1},
          "layers": [par(left(32, 1, 8, 1, 0.5, 1, rot(100.0, 2)), right(1, 1, 9, (0.0,))),
                     dlt(1, 1, 1, 9, 1, 1, 1, mlp=moe(1, 1, 8, 0.7)),
                     dlt(4, 2, 5, 1, 7, 3, 2, mlp=moe(4, 4, 12, 1.0, scale=1.0, groups=(4, 4))),
                     par(left(3, 3, 10, 10, 0.3), right(2, 130, 3, (0.999, 0.9), rot(50.0, 10)), mlp=dense(36))]},
}


def write_folder(path, cfg_dict, seed, store, sharpen=4.0, change=None):
    """A model folder with random weights; the softmax side's query and key matrices are scaled up so that attention
    is not close to uniform and a key that is wrongly seen or missed changes the logits."""
    config = config_from_dict(cfg_dict)
    tensors = random_tensors(parameter_list(config.model_spec()), seed, store)
    for name in list(tensors):
        if name.endswith((".left.q", ".left.k")):
            tensors[name] = (tensors[name].float() * sharpen).to(store)
        elif name.endswith((".q", ".k", ".v", ".o", ".g", ".up", ".gate", ".down", ".proj", ".b", ".a1", ".g1", "embed", "head",
                            "bigram", "loop.step")) and tensors[name].dim() == 2:
            tensors[name] = (tensors[name].float() * 3.0).to(store)
    if change:
        change(tensors)
    path.mkdir(parents=True, exist_ok=True)
    (path / "config.json").write_text(json.dumps(config.to_dict()))
    write_safetensors(path / "model.safetensors", tensors, {"format": "pt"})
    return path


@pytest.fixture(scope="module")
def folders(tmp_path_factory):
    root = tmp_path_factory.mktemp("vodalorn")
    return {(name, dtype): write_folder(root / f"{name}_{dtype}", cfg, 31 + i, STORE[dtype])
            for i, (name, cfg) in enumerate(CONFIGS.items()) for dtype in DTYPES}


def toks(cfg, n, seed):
    return np.random.RandomState(seed).randint(0, cfg["vocab"], size=n).tolist()


def i32(x):
    return torch.tensor(x, dtype=torch.int32, device=DEV)


def f32(x):
    return torch.tensor(np.asarray(x), dtype=torch.float32, device=DEV)


# -- mechanisms alone -----------------------------------------------------------------------------

@pytest.mark.parametrize("dim", [1, 76, 256, 1000, 2048, 4100, 8192, 9001])
def test_layer_norm(dim):
    g = np.random.RandomState(dim)
    x, w, b = g.randn(9, dim) * 3 + 1.5, g.randn(dim), g.randn(dim)
    out = torch.empty(9, dim, dtype=torch.float32, device=DEV)
    ops.layernorm(f32(x), f32(w), f32(b), 1e-5, out)
    check(out, P.layer_norm(x, w, b, 1e-5), 1e-5, "layer norm")
    rows = [7, 0, 7, 3]
    out = torch.empty(4, dim, dtype=torch.bfloat16, device=DEV)
    ops.layernorm(f32(x), f32(w).bfloat16(), f32(b).bfloat16(), 1e-5, out, i32(rows))
    wb, bb = f32(w).bfloat16().double().cpu().numpy(), f32(b).bfloat16().double().cpu().numpy()
    check(out, P.layer_norm(x[rows], wb, bb, 1e-5), 1e-2, "layer norm of picked rows, 16-bit out")


def test_pair_embedding_keeps_the_last_token_per_slot():
    """Steps of unequal sequences: the first token of a sequence takes the table's last row, the first token of a later
    step pairs with what the slot kept, a slot used again starts afresh, a padding row changes nothing."""
    g = np.random.RandomState(0)
    hidden, buckets, a, b = 12, 11, 1000003, 77
    table = g.randn(buckets + 1, hidden)
    last = torch.full((5, 1), 123, dtype=torch.int32, device=DEV)
    seqs = {0: [5, 9, 2, 7, 7, 3], 3: [8, 1, 4]}
    pair = {"buckets": buckets, "mul_prev": a, "mul_cur": b}
    want = {s: table[P.pair_rows(t, pair)] for s, t in seqs.items()}

    def step(parts):      # parts: [(slot, start, tokens)]
        ids = [t for _, _, ts in parts for t in ts]
        seq = [i for i, (_, _, ts) in enumerate(parts) for _ in ts]
        pos = [st + j for _, st, ts in parts for j in range(len(ts))]
        cu = np.cumsum([0] + [len(ts) for _, _, ts in parts]).tolist()
        out = torch.zeros(len(ids) + 1, hidden, dtype=torch.float32, device=DEV)
        ops.pair_embed(f32(table), i32(ids + [0]), i32(seq + [-1]), i32(pos + [0]), i32(cu), i32([s for s, _, _ in parts]),
                       last, out, buckets, a, b)
        assert float(out[-1].abs().max()) == 0.0, "a padding row was written"
        return out[:-1].cpu().numpy()

    got = step([(0, 0, seqs[0][:1]), (3, 0, seqs[3][:2])])
    np.testing.assert_allclose(got, np.concatenate([want[0][:1], want[3][:2]]), rtol=1e-6)
    got = step([(3, 2, seqs[3][2:]), (0, 1, seqs[0][1:4])])
    np.testing.assert_allclose(got, np.concatenate([want[3][2:], want[0][1:4]]), rtol=1e-6)
    got = step([(0, 4, seqs[0][4:5])])
    np.testing.assert_allclose(got, want[0][4:5], rtol=1e-6)
    got = step([(0, 5, seqs[0][5:])])
    np.testing.assert_allclose(got, want[0][5:], rtol=1e-6)
    assert last.view(-1).tolist() == [3, 123, 123, 4, 123]
    got = step([(3, 0, [6])])             # the slot is used again: position 0 does not look at what it kept
    np.testing.assert_allclose(got, table[[buckets]], rtol=1e-6)


def plain_retention(proj, H, d, e, decays, positions, r, eps):
    T = proj.shape[0]
    q = P.rotate(proj[:, :H * d].reshape(T, H, d), positions, r)
    k = P.rotate(proj[:, H * d:2 * H * d].reshape(T, H, d), positions, r) * d ** -0.5
    v = proj[:, 2 * H * d:2 * H * d + H * e].reshape(T, H, e)
    o = np.stack([P.retention_rule(q[:, a], k[:, a], v[:, a], decays[a]) for a in range(H)], axis=1)
    return P.rms(o, eps).reshape(T, H * e) * P.silu(proj[:, 2 * H * d + H * e:])


def rope_table(positions, r):
    half = r["dims"] // 2
    inv = torch.tensor(float(r["base"]) ** (-2.0 * np.arange(half) / r["dims"]), dtype=torch.float32, device=DEV)
    t = torch.empty(len(positions), half, 2, dtype=torch.float32, device=DEV)
    ops.rope_table(i32(positions), inv, t)
    return t


@pytest.mark.parametrize("H,d,e,r", [(3, 10, 14, rot(300.0, 6)), (2, 64, 64, rot(1e4, 64)), (1, 1, 9, None), (2, 130, 3, rot(50.0, 10)),
                                     (4, 32, 200, rot(1e6, 32))])
def test_retention_alone_in_portions_batches_and_steps(H, d, e, r):
    """Rotation, the recurrence with fixed decays, the heads' norm and the gate against the plain rule: one sequence
    whole; the same in portions beside another sequence and a padding sequence (same bits); then token by token with
    the decode-step kernel."""
    g = np.random.RandomState(H * 100 + d)
    T, eps = 75, 1e-5
    decays = [0.0, 1.0, 0.97, 0.5][:H]
    row = 2 * H * (d + e)
    seqs = [g.randn(T, row), g.randn(40, row)]
    want = [plain_retention(s, H, d, e, decays, np.arange(len(s)), r, eps) for s in seqs]
    state = torch.full((4, H, d, e), 7.0, dtype=torch.float32, device=DEV)
    hd = f32(decays)

    def run(parts):           # [(slot, start, rows)] -> gated output per part
        proj = f32(np.concatenate([rows for _, _, rows in parts]))
        pos = [st + j for _, st, rows in parts for j in range(len(rows))]
        cu = i32(np.cumsum([0] + [len(rows) for _, _, rows in parts]).tolist())
        slots = i32([s for s, _, _ in parts])
        n = proj.shape[0]
        out = torch.empty(n, H * e, dtype=torch.float32, device=DEV)
        table = None if r is None else rope_table(pos, r)
        if all(len(rows) == 1 for _, _, rows in parts) and e <= 1024:      # the step kernel rotates on the way in
            ops.gla_step(proj, None, state, slots, None, eps, out, H, d, e, 1.0, 1.0, head_decay=hd, cos_sin=table,
                         k_scale=d ** -0.5)
        else:
            ops.retention_prepare(proj, table, H, d, d ** -0.5)
            o = torch.empty(n, H * e, dtype=torch.float32, device=DEV)
            ops.gla_scan(proj, None, state, slots, cu, o, len(parts), H, d, e, 1.0, 1.0, head_decay=hd)
            ops.gla_output(o, proj, None, eps, out, H, d, e)
        return out

    state[0].zero_()
    whole = run([(0, 0, seqs[0])]).clone()
    check(whole, want[0], 2e-5, "whole")
    state[1].zero_(); state[2].zero_()
    rows, at = [], 0
    for n in (2, 3, 33, 1, 36):
        other = seqs[1][at:at + n] if at + n <= 40 else seqs[1][:0]
        parts = [(1, at, seqs[0][at:at + n])] + ([(2, at, other)] if len(other) else []) + [(-1, 0, seqs[1][:2])]
        out = run(parts)
        rows.append(out[:n].clone())
        assert float(out[-2:].abs().max()) == 0.0, "a padding sequence gets zeros"
        at += n
    assert torch.equal(torch.cat(rows), whole), "portions and batches change the bits"
    state[3].zero_()
    steps = torch.cat([run([(3, t, seqs[0][t:t + 1])]).clone() for t in range(T)])
    check(steps, want[0], 2e-5, "token by token")
    check(state[3], state[0], 1e-5, "the state after the steps against the state after the prompt")


def plain_channel_delta(proj, z, conv_w, a_log, H, G, d, e):
    """proj rows: q (G d), k (G d), v (H e), beta's logits (H); z [T, H d] the decays' logits."""
    T, C = proj.shape[0], 2 * G * d + H * e
    xc = P.silu(P.short_conv(proj[:, :C], conv_w))
    q, k, v = xc[:, :G * d].reshape(T, G, d), xc[:, G * d:2 * G * d].reshape(T, G, d), xc[:, 2 * G * d:].reshape(T, H, e)
    q = q / np.sqrt((q * q).sum(-1, keepdims=True) + P.UNIT_EPS) * d ** -0.5
    k = k / np.sqrt((k * k).sum(-1, keepdims=True) + P.UNIT_EPS)
    beta = P.sigmoid(proj[:, C:C + H])
    g = np.exp(-np.exp(a_log)[None, :, None] * P.softplus(z).reshape(T, H, d))
    return np.stack([P.channel_delta_rule(q[:, a // (H // G)], k[:, a // (H // G)], v[:, a], g[:, a], beta[:, a])
                     for a in range(H)], axis=1).reshape(T, H * e)


def run_channel_delta(parts, state, conv_w, a_log, H, G, d, e, taps, decode=False):
    """parts: [(slot, proj rows, z rows)] of one step; returns o [n, H e]."""
    C = 2 * G * d + H * e
    proj = f32(np.concatenate([p for _, p, _ in parts]))
    z = f32(np.concatenate([zz for _, _, zz in parts]))
    n = proj.shape[0]
    seq = i32([i if s >= 0 else -1 for i, (s, p, _) in enumerate(parts) for _ in range(len(p))])
    cu = i32(np.cumsum([0] + [len(p) for _, p, _ in parts]).tolist())
    slots = i32([s for s, _, _ in parts])
    xc = torch.empty(n, C, dtype=torch.float32, device=DEV)
    gb = torch.empty(n, 2 * H, dtype=torch.float32, device=DEV)
    o = torch.empty(n, H * e, dtype=torch.float32, device=DEV)
    ops.delta_prepare(proj, f32(conv_w), state, H * d * e, seq, slots, cu, f32(a_log), None, xc, gb, len(parts), H, G, d, e, taps,
                      one_token_each=decode, beta_col=C, chan_z=z)
    ops.delta_scan(xc, gb, state, slots, cu, o, len(parts), H, G, d, e, chan_g=z)
    return o


@pytest.mark.parametrize("H,G,d,e,taps", [(6, 2, 20, 12, 3), (1, 1, 64, 128, 4), (2, 2, 130, 33, 2), (4, 1, 128, 64, 4),
                                          (1, 1, 1, 9, 1), (4, 2, 5, 1, 7), (2, 1, 300, 40, 2), (1, 1, 600, 8, 3)])
def test_channel_delta_rule_alone_in_portions_and_batches(H, G, d, e, taps):
    g = np.random.RandomState(H * 1000 + d)
    C, T = 2 * G * d + H * e, 70
    conv_w, a_log = g.randn(C, taps) * 0.5, g.randn(H) * 0.5
    seqs = [(g.randn(n, C + H) * 2, g.randn(n, H * d) * 2) for n in (T, 37)]
    want = [plain_channel_delta(p, z, conv_w, a_log, H, G, d, e) for p, z in seqs]
    row = H * d * e + (taps - 1) * C
    state = torch.full((4, row), 3.0, dtype=torch.float32, device=DEV)
    state[0].zero_()
    whole = run_channel_delta([(0, *seqs[0])], state, conv_w, a_log, H, G, d, e, taps).clone()
    check(whole, want[0], 3e-5, "whole")
    state[1].zero_(); state[2].zero_()
    rows, rows2, at = [], [], 0
    for n in (2, 3, 30, 1, 34):
        parts = [(1, seqs[0][0][at:at + n], seqs[0][1][at:at + n])]
        if at + n <= 37 or at < 37:
            m = min(n, 37 - at)
            parts.append((2, seqs[1][0][at:at + m], seqs[1][1][at:at + m]))
        parts.append((-1, seqs[1][0][:2], seqs[1][1][:2]))
        out = run_channel_delta(parts, state, conv_w, a_log, H, G, d, e, taps)
        rows.append(out[:n].clone())
        if len(parts) == 3:
            rows2.append(out[n:n + len(parts[1][1])].clone())
        assert float(out[-2:].abs().max()) == 0.0, "a padding sequence gets zeros"
        at += n
    assert torch.equal(torch.cat(rows), whole), "portions and batches change the bits"
    check(torch.cat(rows2), want[1], 3e-5, "the second sequence of the batch")
    state[3].zero_()
    steps = torch.cat([run_channel_delta([(3, seqs[0][0][t:t + 1], seqs[0][1][t:t + 1])], state, conv_w, a_log, H, G, d, e, taps,
                                         decode=True).clone() for t in range(T)])
    assert torch.equal(steps, whole), "token by token changes the bits"


def test_channel_delta_remembers_a_write_far_back():
    """600 tokens: decays close to one for most channels, so that what the first tokens wrote is still read at the end;
    the result must follow the plain rule, and must change when the first token's value changes."""
    H, G, d, e, taps = 2, 1, 16, 8, 2
    g = np.random.RandomState(5)
    C, T = 2 * G * d + H * e, 600
    conv_w, a_log = g.randn(C, taps) * 0.5, np.array([-6.0, -2.0])
    proj, z = g.randn(T, C + H) * 2, g.randn(T, H * d) - 3.0
    proj[:, C:] = -4.0                       # weak writes after the first tokens,
    proj[:3, C:] = 6.0                       # strong ones at the start
    state = torch.zeros(2, H * d * e + (taps - 1) * C, dtype=torch.float32, device=DEV)
    got = run_channel_delta([(0, proj, z)], state, conv_w, a_log, H, G, d, e, taps)
    want = plain_channel_delta(proj, z, conv_w, a_log, H, G, d, e)
    check(got[-5:], want[-5:], 1e-4, "the last tokens")
    other = proj.copy()
    other[0, 2 * G * d:C] += 3.0
    assert np.abs(plain_channel_delta(other, z, conv_w, a_log, H, G, d, e)[-1] - want[-1]).max() > 1e-3 * np.abs(want[-1]).max()


@pytest.mark.parametrize("E,top,groups,scale", [(8, 3, (4, 3), 2.5), (6, 2, (3, 2), 1.5), (16, 4, None, 1.0), (1, 1, None, 0.5),
                                                 (4, 4, (4, 4), 1.0), (12, 2, (6, 1), 3.0), (64, 8, (8, 2), 1.0)])
def test_router_scores_over_all_experts_groups_and_scale(E, top, groups, scale):
    g = np.random.RandomState(E * 10 + top)
    z = g.randn(50, E) * 3
    z[7] = 0.0                                   # all equal: the lower index wins everywhere
    z[8, :] = np.round(z[8, :])                  # ties between some
    router = {"experts": E, "top": top, "scale": scale}
    if groups:
        router["groups"] = {"count": groups[0], "keep": groups[1]}
    ids = torch.empty(50, top, dtype=torch.int32, device=DEV)
    w = torch.empty(50, top, dtype=torch.float32, device=DEV)
    scoring = ("all", groups[0] if groups else 1, groups[1] if groups else 1, scale)
    ops.moe_route(f32(z), top, ids, w, scoring)
    for t in range(50):
        chosen, weights = P.route(z[t].astype(np.float32).astype(np.float64), router)
        assert ids[t].tolist() == chosen.tolist(), f"token {t}"
        np.testing.assert_allclose(w[t].cpu().numpy(), weights, rtol=2e-5)
    # the same through the kernel that makes the logits itself
    x, wr = g.randn(50, 40), g.randn(E, 40)
    ids2 = torch.empty(50, top, dtype=torch.int32, device=DEV)
    w2 = torch.empty(50, top, dtype=torch.float32, device=DEV)
    ops.moe_router(f32(x), f32(wr), None, top, ids2, w2, scoring)
    zz = (f32(x).double() @ f32(wr).double().T).cpu().numpy()
    for t in range(50):
        chosen, weights = P.route(zz[t], router)
        if np.sort(zz[t])[::-1][:top + 1].std() > 1e-3:
            assert sorted(ids2[t].tolist()) == sorted(chosen.tolist())


@pytest.mark.parametrize("m", [3, 40, 130, 600])
def test_square_of_relu_in_the_products_and_alone(m):
    g = torch.Generator(device=DEV).manual_seed(m)
    x = torch.randn(m, 256, generator=g, device=DEV).bfloat16()
    w = (torch.randn(512, 256, generator=g, device=DEV) * 0.1).bfloat16()
    want = 0.6 * torch.relu(x.double() @ w.double().T) ** 2
    rt = Runtime(DEV, torch.bfloat16)
    out = torch.empty(m, 512, dtype=torch.bfloat16, device=DEV)
    rt.linear(x, w, None, out, activation=("relu2", 0.6, 0.0))
    check(out, want, 1e-2, "in the product's epilogue")
    up = torch.empty(m, 512, dtype=torch.float32, device=DEV)
    rt.linear(x, w, None, up)
    alone = torch.empty(m, 512, dtype=torch.float32, device=DEV)
    ops.relu2(up, alone, 0.6)
    check(alone, want, 1e-5, "as a kernel")
    rt.check_status()


@pytest.mark.parametrize("W,D,store", [(76, 5, torch.float32), (256, 32, torch.bfloat16), (2048, 128, torch.bfloat16),
                                       (1000, 12, torch.bfloat16), (4096, 256, torch.float32)])
def test_the_gate_of_a_tokens_own_input_for_a_few_tokens(W, D, store):
    g = np.random.RandomState(W)
    for n in (1, 9, 16):
        V = 50
        x, table, ids = g.randn(n, W) * 2, g.randn(V, 3 * D), g.randint(0, V, size=n).tolist()
        w = torch.tensor(g.randn(D, W) * 0.1).to(store)
        want = P.gelu_tanh(x @ w.double().numpy().T) * table[ids][:, D:2 * D]
        out = torch.empty(n, D, dtype=torch.float32, device=DEV)
        ops.token_gate_rows(f32(x), w.to(DEV), f32(table), i32(ids), D, out)
        check(out, want, 2e-5, f"{n} tokens")


@pytest.mark.parametrize("W", [76, 2048, 4100, 9000])
def test_what_joins_the_stream(W):
    """Two normed branches with a weight, one normed branch (the token's own input), a plain weighted sum, the lanes of
    a token's row that gate a projection, and the pair of streams side by side."""
    g = np.random.RandomState(3)
    n = 7
    x, a, b, wa, wb = g.randn(n, W), g.randn(n, W) * 4, g.randn(n, W) * 0.1, g.randn(W), g.randn(W)
    xs = f32(x)
    ops.branch_norm_add(xs, f32(a), f32(wa), f32(b), f32(wb), 1e-5, 0.35)
    check(xs, x + 0.35 * (P.rms(a, 1e-5) * wa + P.rms(b, 1e-5) * wb), 1e-5, "two branches")
    xs = f32(x)
    ops.branch_norm_add(xs, f32(a), f32(wa), None, None, 1e-5, 0.7)
    check(xs, x + 0.7 * P.rms(a, 1e-5) * wa, 1e-5, "one branch")
    xs = f32(x)
    ops.stream_axpy(xs, f32(a), 0.6)
    check(xs, x + 0.6 * a, 1e-6, "a weighted sum")
    table, ids, z = g.randn(30, 20), [3, 29, 0, 3, 11, 5, 7], g.randn(n, 5) * 2
    out = torch.empty(n, 5, dtype=torch.float32, device=DEV)
    ops.token_gate(f32(z), f32(table), i32(ids), 10, out)
    check(out, P.gelu_tanh(z) * table[ids][:, 10:15], 1e-5, "a token's lanes gate a projection")
    both = torch.empty(n, 2 * W, dtype=torch.bfloat16, device=DEV)
    ops.concat_rows(f32(x), f32(a), both)
    assert torch.equal(both, torch.cat([f32(x), f32(a)], dim=1).bfloat16())


# -- the model ------------------------------------------------------------------------------------

def close(got, want, dtype, what):
    """Logits against the plain model's.  float32: the largest difference within 1e-4 of the largest logit.
    bfloat16: rounding of the activations to 8 bits of mantissa is the design's own noise (and where two router scores
    are closer than that noise a token may go to another expert), so the measure is the root mean square of the
    differences over all the rows given, held to 5 % of the logits' own; a fault of the cache, the state or a window
    moves far more than that with these weights, and the float32 runs hold the same code to 1e-4."""
    if dtype == "float32":
        return check(got, want, TOL[dtype], what)
    g = got.detach().double().cpu().numpy()
    w = np.asarray(want, dtype=np.float64).reshape(g.shape)
    assert np.isfinite(g).all(), f"{what}: NaN or infinity"
    rms = float(np.sqrt(np.mean((g - w) ** 2)) / np.sqrt(np.mean(w ** 2)))
    assert rms <= 5e-2, f"{what}: root mean square of the differences {rms:.3e} of the logits' own"


class Rows:
    """Rows of logits that arrive one step at a time: float32 rows are judged as they come, bfloat16 rows together
    at the end (see ``close``)."""

    def __init__(self, dtype, what):
        self.dtype, self.what, self.got, self.want = dtype, what, [], []

    def add(self, got, want, where=""):
        if self.dtype == "float32":
            return close(got, want, self.dtype, f"{self.what} {where}")
        self.got.append(got.detach().float().reshape(-1).clone())
        self.want.append(np.asarray(want, dtype=np.float64).reshape(-1))

    def done(self):
        if self.got:
            close(torch.stack(self.got), np.stack(self.want), self.dtype, self.what)


def plain_logits(folder, tokens):
    cfg, w = P.load(folder)
    return P.forward(cfg, w, tokens)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", list(CONFIGS))
def test_whole_prompt_every_position(folders, name, dtype):
    cfg = CONFIGS[name]
    t = toks(cfg, 150, 1)
    want = plain_logits(folders[name, dtype], t)
    model = Model.load(folders[name, dtype], dtype=dtype)
    engine = Engine(model, max_tokens=256)
    got = engine.step([engine.alloc_slot()], [t], [list(range(150))])
    close(got, want, dtype, f"{name} whole prompt")
    if dtype == "float32":         # the first tokens of a sequence (the pair table's last row, zeros before the
        for i in range(4):         # convolutions, empty states, a softmax of one key), one by one
            close(got[i], want[i], dtype, f"{name} token {i}")


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", list(CONFIGS))
def test_every_layer_run_against_the_plain_model(folders, name, dtype):
    """The stream after every layer run (a layer of the loop counts each time)."""
    t = toks(CONFIGS[name], 40, 4)
    cfg, w = P.load(folders[name, dtype])
    _, streams = P.forward(cfg, w, t, True)
    model = Model.load(folders[name, dtype], dtype=dtype)
    engine = Engine(model, max_tokens=64, use_graphs=False)
    caught = []
    for b in set(model.blocks):
        def wrapped(ctx, residual, caches, _o=b.forward):
            _o(ctx, residual, caches)
            caught.append(residual.detach().clone())
        b.forward = wrapped
    engine.step([engine.alloc_slot()], [t], [[39]])
    assert len(caught) == len(streams) == len(P.layer_runs(cfg))
    for r, (got, want) in enumerate(zip(caught, streams)):
        assert got.dtype == torch.float32, "the residual sum is 32-bit in both run types"
        if dtype == "float32":
            check(got, want, 1e-5, f"stream after layer run {r}")
        else:
            rms = float(np.sqrt(np.mean((got.double().cpu().numpy() - want) ** 2)) / np.sqrt(np.mean(want ** 2)))
            assert rms <= 3e-2, f"stream after layer run {r}: {rms:.3e}"


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", list(CONFIGS))
def test_portions_and_token_by_token_against_the_whole(folders, name, dtype):
    """The same 200 tokens: whole; in portions of 2, 3, 64, 1, 65, ... tokens; a prompt of 40 and then one token a
    step for 160 steps (across page borders and windows, the states, the convolutions' inputs and the last token handed
    from step to step).  All against the plain model; in float32 the three runs agree with one another far below
    the tolerance."""
    cfg = CONFIGS[name]
    t = toks(cfg, 200, 2)
    want = plain_logits(folders[name, dtype], t)
    model = Model.load(folders[name, dtype], dtype=dtype)
    engine = Engine(model, max_tokens=64 * 12)
    s = engine.alloc_slot()
    whole = engine.step([s], [t], [list(range(200))]).clone()
    close(whole, want, dtype, "whole")
    s2 = engine.alloc_slot()
    rows, at, sizes, i = [], 0, [2, 3, 64, 1, 65, 2, 7], 0
    while at < 200:
        n = min(sizes[i % len(sizes)], 200 - at)
        rows.append(engine.step([s2], [t[at:at + n]], [list(range(n))]).clone())
        at += n
        i += 1
    portions = torch.cat(rows)
    close(portions, want, dtype, "portions")
    engine.free_slot(s)
    s3 = engine.alloc_slot()                 # the slot, pages and state rows that the whole run used
    engine.step([s3], [t[:40]], [[]])
    decoded = torch.cat([engine.step([s3], [[t[i]]]).clone() for i in range(40, 200)])
    close(decoded, want[40:], dtype, "token by token")
    s4 = engine.alloc_slot()                 # portions that want their last place only
    at, last = 0, []
    for n in (5, 2, 33, 2, 100, 58):
        last.append(engine.step([s4], [t[at:at + n]]).clone())
        at += n
    close(torch.cat(last), want[[4, 6, 39, 41, 141, 199]], dtype, "portions that want their last place")
    if dtype == "float32":
        check(portions, whole, 2e-5, "portions against the whole")
        check(decoded, whole[40:], 2e-5, "token by token against the whole")
    engine.cache.check()


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", list(CONFIGS))
def test_unequal_batch_then_decoding_together_on_reused_slots(folders, name, dtype):
    """Four prompts of 1, 33, 130 and 64 tokens in one step, then one token each per step; the short ones end
    early and give their slots, pages and state rows back; a newcomer takes them while the others go on (its states
    must start at zero and its first token must take the pair table's last row although the rows were used)."""
    cfg = CONFIGS[name]
    lens, tails = [1, 33, 130, 64], [3, 10, 24, 24]
    seqs = [toks(cfg, n + k, 10 + i) for i, (n, k) in enumerate(zip(lens, tails))]
    want = [plain_logits(folders[name, dtype], t) for t in seqs]
    model = Model.load(folders[name, dtype], dtype=dtype)
    engine = Engine(model, max_tokens=64 * 8)
    slots = [engine.alloc_slot() for _ in seqs]
    out = engine.step(slots, [t[:n] for t, n in zip(seqs, lens)], [[n - 1] for n in lens])
    rows = [Rows(dtype, f"sequence {b}") for b in range(4)]
    for b in range(4):
        rows[b].add(out[b], want[b][lens[b] - 1], "prompt")
    live = list(range(4))
    newcomer = toks(cfg, 90, 99)
    want_new = plain_logits(folders[name, dtype], newcomer)
    for step in range(24):
        live = [b for b in live if step < tails[b]]
        out = engine.step([slots[b] for b in live], [[seqs[b][lens[b] + step]] for b in live])
        for i, b in enumerate(live):
            rows[b].add(out[i], want[b][lens[b] + step], f"decoded token {step}")
        for b in list(range(4)):
            if step + 1 == tails[b] and b in live and tails[b] < 24:
                engine.free_slot(slots[b])
        if step == 11:                      # both short sequences are gone: their slots and pages are used again
            s = engine.alloc_slot()
            got = engine.step([s], [newcomer], [[0, 1, 63, 64, 89]])
            close(got, want_new[[0, 1, 63, 64, 89]], dtype, "a newcomer on used slots")
            engine.free_slot(s)
    for r in rows:
        r.done()
    engine.cache.check()


@pytest.mark.parametrize("dtype", DTYPES)
def test_long_decoding_across_pages_and_windows(folders, dtype):
    """420 decoded tokens after a prompt of 150: pages pass by and are given back, the windows (64, 77 and 100 keys) move
    over decoded tokens only, and the recurrent states have been rewritten 570 times."""
    cfg = CONFIGS["B"]
    n = 570
    t = toks(cfg, n, 5)
    want = plain_logits(folders["B", dtype], t)
    model = Model.load(folders["B", dtype], dtype=dtype)
    engine = Engine(model, max_tokens=640)
    s = engine.alloc_slot()
    engine.step([s], [t[:150]], [[]])
    rows = Rows(dtype, "long decoding")
    for i in range(150, n):
        out = engine.step([s], [[t[i]]])
        if i % 7 == 0 or i % PAGE in (PAGE - 1, 0, 1) or i > n - 10:
            rows.add(out[0], want[i], f"decoded position {i}")
    rows.done()
    engine.cache.check()


def test_long_prompt_on_the_tensor_core_paths(folders):
    """600 tokens in one step through sizes that the tensor-core kernels take, then ten tokens one by one: bfloat16 and
    float32 against the plain model."""
    cfg = CONFIGS["B"]
    t = toks(cfg, 610, 3)
    rows = list(range(0, 600, 7)) + [63, 64, 76, 77, 78, 99, 100, 101, 127, 128, 129, 255, 256, 511, 512, 599]
    for dtype in ("bfloat16", "float32"):
        want = plain_logits(folders["B", dtype], t)
        model = Model.load(folders["B", dtype], dtype=dtype)
        engine = Engine(model, max_tokens=64 * 11)
        s = engine.alloc_slot()
        close(engine.step([s], [t[:600]], [rows]), want[rows], dtype, f"{dtype}: a prompt of 600 tokens")
        out = torch.cat([engine.step([s], [[t[i]]]).clone() for i in range(600, 610)])
        close(out, want[600:], dtype, f"{dtype}: ten tokens after it")
        model.rt.check_status()


@pytest.mark.parametrize("dim,vdim", [(16, 24), (64, 64)])
@pytest.mark.parametrize("window", [1, 5, 64, 65, 77])
def test_keys_just_inside_and_just_outside_a_window(tmp_path, window, dim, vdim):
    """One layer whose softmax side is so sharp that single keys take most of a row's weight: a key that is wrongly seen
    or missed at the window's edge changes the logits.  As a prompt across page borders, and token by token; with
    head sizes that the 32-bit kernel and that the tensor-core kernels take."""
    cfg = {"architecture": "Vodalorn", "vocab": 64, "width": 48, "norm": {"eps": 1e-5}, "residual_mult": 0.9,
           "layers": [par(left(2, 1, dim, vdim, 1.0, window, rot(1e4, 8)), right(1, 4, 4, (0.9,)), mlp=dense(64))]}
    t = toks(cfg, 210, 8)
    for dtype in DTYPES:
        folder = write_folder(tmp_path / dtype, cfg, 3, STORE[dtype], sharpen=12.0)
        want = plain_logits(folder, t)
        pcfg, w = P.load(folder)
        if window > 1:
            for off in (-1, 1):                  # the same model with a window one key off answers otherwise
                pcfg["layers"][0]["mixer"]["left"]["mask"]["size"] = window + off
                assert np.abs(P.forward(pcfg, w, t)[window:] - want[window:]).max() > 0.02 * np.abs(want).max(), "the edge does not show"
        model = Model.load(folder, dtype=dtype)
        engine = Engine(model, max_tokens=512)
        s = engine.alloc_slot()
        picks = sorted(p for p in {0, 1, window - 1, window, window + 1, 63, 64, 65, 127, 128, 128 + window, 199} if 0 <= p < 200)
        close(engine.step([s], [t[:200]], [picks]), want[picks], dtype, f"window {window}: a prompt")
        out = torch.cat([engine.step([s], [[t[i]]]).clone() for i in range(200, 210)])
        close(out, want[200:], dtype, f"window {window}: decoded after it")
        s2 = engine.alloc_slot()
        engine.step([s2], [t[:3]], [[]])
        out = torch.cat([engine.step([s2], [[t[i]]]).clone() for i in range(3, 140)])
        close(out, want[3:140], dtype, f"window {window}: decoded from the start")


@pytest.mark.parametrize("dtype", DTYPES)
def test_twenty_requests_decode_together(folders, dtype):
    """More sequences than the few-token products take (20 prompts of 1 to 150 tokens in one step, then 6 decode steps of 20
    tokens through the captured step of 32 rows, 12 of them padding) against each request alone in the plain model."""
    cfg = CONFIGS["B"]
    lens = [1 + (37 * i) % 150 for i in range(20)]
    seqs = [toks(cfg, n + 6, 200 + i) for i, n in enumerate(lens)]
    want = [plain_logits(folders["B", dtype], t) for t in seqs]
    model = Model.load(folders["B", dtype], dtype=dtype)
    engine = Engine(model, max_tokens=64 * 64)
    slots = [engine.alloc_slot() for _ in seqs]
    rows = Rows(dtype, "twenty requests")
    out = engine.step(slots, [t[:n] for t, n in zip(seqs, lens)], [[n - 1] for n in lens])
    for b in range(20):
        rows.add(out[b], want[b][lens[b] - 1], f"prompt {b}")
    for step in range(6):
        out = engine.step(slots, [[seqs[b][lens[b] + step]] for b in range(20)])
        for b in range(20):
            rows.add(out[b], want[b][lens[b] + step], f"request {b} decoded token {step}")
    rows.done()
    engine.cache.check()
    model.rt.check_status()


@pytest.mark.parametrize("dim", [64, 128])
def test_many_query_heads_on_one_key_value_head_at_tensor_core_sizes(tmp_path, dim):
    """32 query heads on one key/value head with heads of 64 and 128 lanes, a partly rotated head, a window that ends inside
    a page: a prompt across pages and token by token, in both run types."""
    cfg = {"architecture": "Vodalorn", "vocab": 120, "width": 128, "norm": {"eps": 1e-5}, "residual_mult": 0.8,
           "layers": [par(left(32, 1, dim, dim, dim ** -0.5, 50, rot(1e4, dim // 2)), right(2, 16, 16, (0.9, 0.99), rot(1e4, 16)), mlp=dense(64)),
                      par(left(20, 1, dim, dim, dim ** -0.5, None, rot(1e4, dim)), right(1, 32, 8, (0.95,)), mlp=None)]}
    t = toks(cfg, 150, 6)
    for dtype in DTYPES:
        folder = write_folder(tmp_path / dtype, cfg, 9, STORE[dtype], sharpen=3.0)
        want = plain_logits(folder, t)
        model = Model.load(folder, dtype=dtype)
        engine = Engine(model, max_tokens=512)
        s = engine.alloc_slot()
        close(engine.step([s], [t[:130]], [list(range(130))]), want[:130], dtype, f"{dtype}: a prompt")
        out = torch.cat([engine.step([s], [[t[i]]]).clone() for i in range(130, 150)])
        close(out, want[130:], dtype, f"{dtype}: decoded after it")
        s2 = engine.alloc_slot()
        out = torch.cat([engine.step([s2], [t[i:i + 3]], [[0, 1, 2]]).clone() for i in range(0, 150, 3)])
        close(out, want, dtype, f"{dtype}: portions of three tokens")
        model.rt.check_status()


def test_a_key_far_back(tmp_path):
    """Attention without a window, sharp queries and keys, 560 positions: most rows look far back and across pages."""
    cfg = {"architecture": "Vodalorn", "vocab": 64, "width": 48, "norm": {"eps": 1e-5},
           "layers": [par(left(2, 1, 16, 16, 1.0, None, rot(1e4, 8)), right(2, 8, 8, (0.999, 0.99), rot(1e4, 8)), mlp=dense(64))]}
    folder = write_folder(tmp_path / "m", cfg, 3, torch.float32, sharpen=12.0)
    t = toks(cfg, 560, 8)
    want = plain_logits(folder, t)
    model = Model.load(folder, dtype="float32")
    engine = Engine(model, max_tokens=1280)
    s = engine.alloc_slot()
    got = engine.step([s], [t], [[0, 1, 20, 529, 530, 559]])
    check(got, want[[0, 1, 20, 529, 530, 559]], 1e-4, "a prompt with far keys")
    s2 = engine.alloc_slot()
    engine.step([s2], [t[:500]], [[]])
    for i in range(500, 535):
        out = engine.step([s2], [[t[i]]])
    check(out[0], want[534], 1e-4, "decoded past far keys")


@pytest.mark.parametrize("name", list(CONFIGS))
def test_greedy_generation_through_the_session(folders, name):
    """``Session.generate`` (scheduler, batches, captured decode steps) against greedy decoding of the plain model."""
    cfg = CONFIGS[name]
    folder = folders[name, "float32"]
    pcfg, w = P.load(folder)
    prompts = [toks(cfg, 70, 21), toks(cfg, 3, 22), toks(cfg, 129, 23)]
    want = [P.greedy(pcfg, w, p, 8) for p in prompts]
    model = Model.load(folder, dtype="float32")
    session = Session(model, SessionParams(n_ctx=256, seed=1, max_batch=2))
    res = session.generate(prompts, GenerateParams(8, SamplerParams.greedy()), stop_token_ids=())
    assert [r.tokens for r in res] == want
    # the same in bfloat16: the length of every reply (tokens may part ways by rounding)
    model = Model.load(folders[name, "bfloat16"], dtype="bfloat16")
    session = Session(model, SessionParams(n_ctx=256, seed=1, max_batch=3))
    res = session.generate(prompts, GenerateParams(4, SamplerParams.greedy()), stop_token_ids=())
    assert all(len(r.tokens) == 4 for r in res)


def test_command_line_random_weights_info_and_generation(tmp_path):
    """The command line's modes on this design: a folder with random weights from a configuration file, its --info,
    the greedy token harness against the plain model, and a sampled continuation."""
    import io
    from nncpu_b200.cli import parse_options, run_gen, run_generate, run_info, run_random_weights

    def run(fn, argv):
        out = io.StringIO()
        assert fn(parse_options(argv), out) == 0
        return out.getvalue()

    cfg = tmp_path / "cfg.json"
    cfg.write_text(json.dumps(CONFIGS["A"]))
    run(run_random_weights, ["--random-weights", str(cfg), "5", str(tmp_path / "m"), "--fp32"])
    info = json.loads(run(run_info, ["--info", str(tmp_path / "m")]))
    assert info["config"]["architecture"] == "Vodalorn" and info["parameters"] > 0
    prompt = toks(CONFIGS["A"], 40, 3)
    got = [int(t) for t in run(run_gen, ["--gen", str(tmp_path / "m"), " ".join(map(str, prompt)), "6", "--fp32"]).splitlines()[0].split()]
    pcfg, w = P.load(tmp_path / "m")
    assert got == P.greedy(pcfg, w, prompt, 6)
    out = run(run_generate, ["-m", str(tmp_path / "m"), "--tokens", " ".join(map(str, prompt)), "-n", "6", "--temp", "0.8",
                             "--top-k", "20", "-s", "4", "-b", "3"]).split()
    assert len(out) >= 6 and all(0 <= int(t) < CONFIGS["A"]["vocab"] for t in out[:6])


def test_trace_replay_of_many_short_requests(folders, tmp_path):
    """``bin/trace_run`` as a subprocess on this design: eight requests of unequal lengths in one batch, decoded
    together while the shorter ones end; then a second batch on the slots, pages and state rows that were given back."""
    import subprocess
    import sys
    from conftest import ROOT
    cfg = CONFIGS["A"]
    folder = folders["A", "float32"]
    V = cfg["vocab"]
    lens, tails = [3, 5, 70, 1, 9, 64, 2, 31], [2, 6, 6, 1, 4, 6, 3, 6]
    seqs = {f"r{i}": toks(cfg, n + k, 50 + i) for i, (n, k) in enumerate(zip(lens, tails))}
    seqs.update({f"s{i}": toks(cfg, n, 70 + i) for i, n in enumerate((66, 4, 17))})
    want = {k: plain_logits(folder, t) for k, t in seqs.items()}
    steps, expect = [], {}

    def add(entries, end=()):
        n = len(steps)
        steps.append({"step": n, "entries": [{"id": k, "tokens": seqs[k][a:b], "want": w} for k, a, b, w in entries], "end": list(end)})
        if any(w for *_, w in entries):
            expect[n] = [(k, [a + i for i in w]) for k, a, b, w in entries if w]

    add([(f"r{i}", 0, n, [0, n - 1] if n > 1 else [0]) for i, n in enumerate(lens)])
    for step in range(max(tails)):
        live = [i for i in range(len(lens)) if step < tails[i]]
        add([(f"r{i}", lens[i] + step, lens[i] + step + 1, [0]) for i in live],
            end=[f"r{i}" for i in live if step + 1 == tails[i]])
    add([(f"s{i}", 0, len(seqs[f"s{i}"]), [0, len(seqs[f"s{i}"]) - 1]) for i in range(3)], end=[f"s{i}" for i in range(3)])
    out = tmp_path / "out"
    text = "".join(json.dumps(s) + "\n" for s in steps)
    p = subprocess.run([sys.executable, str(ROOT / "bin" / "trace_run"), "--model", str(folder), "--dtype", "float32",
                        "--out", str(out), "--max-tokens", str(sum(lens) + sum(tails))], input=text, capture_output=True,
                       text=True, timeout=600)
    assert p.returncode == 0, p.stderr[-2000:]
    assert [l for l in p.stdout.splitlines() if l.startswith("done")] == [f"done {s['step']}" for s in steps]
    for n, rows in expect.items():
        got = np.fromfile(out / f"{n}.f32", dtype="<f4").reshape(-1, V)
        ref = np.concatenate([want[k][pos] for k, pos in rows])
        check(got, ref, 1e-4, f"step {n}")


def random_vodalorn(rs):
    """A random configuration: any order of the two kinds of layer, head sizes in and out of what the tensor-core
    kernels take, any grouping of heads, windows short and long, with and without a loop, a pair embedding, a per-layer
    token input, groups of experts."""
    width = int(rs.choice([72, 100, 136, 200, 256]))
    layers = []
    for i in range(int(rs.randint(2, 6))):
        roll = rs.rand()
        if roll < 0.35:
            mlp = dense(int(rs.choice([40, 88, 136, 264])))
        elif roll < 0.85:
            E = int(rs.choice([2, 4, 6, 8, 12]))
            count = int(rs.choice([c for c in (1, 2, 3, 4, 6) if E % c == 0]))
            keep = int(rs.randint(1, count + 1))
            top = int(rs.randint(1, keep * (E // count) + 1))
            mlp = moe(E, top, int(rs.choice([16, 20, 64, 80])), float(rs.choice([0.8, 1.25, 7.0])),
                      scale=float(rs.choice([1.0, 2.0, 2.5])), groups=(count, keep) if count > 1 or rs.rand() < 0.3 else None)
        else:
            mlp = None
        if rs.rand() < 0.6:
            kv, group, dim = int(rs.choice([1, 2, 3])), int(rs.choice([1, 2, 4, 8])), int(rs.choice([16, 24, 64, 128]))
            vdim = int(rs.choice([dim, dim, 8, 40, 128]))
            dims = int(rs.choice([dim, dim // 2, 2]))
            window = None if rs.rand() < 0.15 else int(rs.choice([1, 3, 17, 64, 77, 100, 130]))
            H, rd = int(rs.choice([1, 2, 3, 6])), int(rs.choice([8, 16, 32, 64]))
            rdims = int(rs.choice([rd, rd // 2]))
            layers.append(par(left(kv * group, kv, dim, vdim, float(rs.choice([dim ** -0.5, 0.2])), window,
                                   rot(float(rs.choice([1e4, 4e5, 300.0])), dims) if rs.rand() < 0.9 else None),
                              right(H, rd, int(rs.choice([8, 32, 64])), [float(1 - 2.0 ** -(3 + j)) for j in range(H)],
                                    rot(float(rs.choice([1e4, 1e6])), rdims) if rs.rand() < 0.9 else None), mlp=mlp))
        else:
            kv, group = int(rs.choice([1, 2, 3])), int(rs.choice([1, 2, 3]))
            layers.append(dlt(kv * group, kv, int(rs.choice([8, 20, 64, 128])), int(rs.choice([8, 20, 64, 128])),
                              int(rs.choice([1, 2, 4, 5])), int(rs.choice([3, 8, 20])), int(rs.choice([5, 8, 28])), mlp=mlp))
    cfg = {"architecture": "Vodalorn", "vocab": int(rs.randint(100, 600)), "width": width,
           "norm": {"eps": float(rs.choice([1e-6, 1e-5]))}, "residual_mult": float(rs.choice([1.0, 0.7, 0.5])), "layers": layers}
    if rs.rand() < 0.8:
        cfg["embedding"] = {"bigram": {"buckets": int(rs.choice([17, 1013, 4093])), "mul_prev": int(rs.choice([1, 131, 99991])),
                                       "mul_cur": int(rs.choice([1, 23, 31337]))}}
    if rs.rand() < 0.8:
        cfg["token_side"] = {"dim": int(rs.choice([1, 8, 16, 40]))}
    if rs.rand() < 0.75:
        a = int(rs.randint(0, len(layers)))
        cfg["loop"] = {"start": a, "stop": int(rs.randint(a + 1, len(layers) + 1)), "times": int(rs.choice([1, 2, 3]))}
    return cfg


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("seed", range(10))
def test_random_configuration_and_trace(tmp_path, seed, dtype):
    """Random configurations, each with a batch of unequal prompts (the first one cut in two steps the second time
    round), decoding with early leavers, then the same again on the slots, pages and state rows given back."""
    rs = np.random.RandomState(7000 + seed)
    cfg = random_vodalorn(rs)
    folder = write_folder(tmp_path / "m", cfg, seed, STORE[dtype], sharpen=3.0)
    model = Model.load(folder, dtype=dtype)
    lens = [int(rs.choice([1, 2, 17, 40, 65, 130, 260])) for _ in range(int(rs.choice([1, 2, 3, 4])))]
    if rs.rand() < 0.4:
        lens[0] = int(rs.choice([300, 520]))
    n_decode = [int(rs.randint(0, 10)) for _ in lens]
    reqs = [rs.randint(0, cfg["vocab"], size=n + d).tolist() for n, d in zip(lens, n_decode)]
    want = [plain_logits(folder, r) for r in reqs]
    engine = Engine(model, max_tokens=64 * (sum((len(r) + 63) // 64 for r in reqs) + 2))
    for round_ in range(2):
        slots = [engine.alloc_slot() for _ in reqs]
        # float32 rows are judged one by one; bfloat16 rows of a round together (a request may have one row only, and a
        # token that goes to another expert by rounding must not stand for the whole)
        shared = Rows(dtype, f"seed {seed} round {round_}")
        rows = [shared for _ in reqs]
        cut = lens[0] // 2 if lens[0] > 40 and round_ == 1 else 0
        if cut:
            engine.step(slots[:1], [reqs[0][:cut]], [[]])
        out = engine.step(slots, [r[(cut if b == 0 else 0):n] for b, (r, n) in enumerate(zip(reqs, lens))],
                          [[n - 1 - (cut if b == 0 else 0)] for b, n in enumerate(lens)])
        for b in range(len(reqs)):
            rows[b].add(out[b], want[b][lens[b] - 1], "prompt")
        for step in range(max(n_decode)):
            live = [b for b in range(len(reqs)) if step < n_decode[b]]
            out = engine.step([slots[b] for b in live], [[reqs[b][lens[b] + step]] for b in live])
            for i, b in enumerate(live):
                rows[b].add(out[i], want[b][lens[b] + step], f"decoded token {step}")
            for b in live:
                if step + 1 == n_decode[b]:
                    engine.free_slot(slots[b])
        for b in range(len(reqs)):
            if n_decode[b] == 0:
                engine.free_slot(slots[b])
        shared.done()
    engine.cache.check()
    model.rt.check_status()
