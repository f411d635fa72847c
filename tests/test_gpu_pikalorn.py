"""The Pikalorn design against its plain statement (``plain_pikalorn``): every mechanism alone, then the model
through ``Engine.step`` cut in every way (whole prompts, token by token, portions down to two tokens, unequal
batches, slots, pages and state rows used again, pages crossed while decoding), and greedy generation through
``Session.generate`` and the command line.  Configurations and weights are made here; where random weights would
hide a fault (a sink, a key far back, a write the recurrence must remember) the inputs are made so that it shows."""
import json
import math

import numpy as np
import pytest
import torch

import plain_pikalorn as P
from gpu_util import DEV, TOL, check, scatter_pages
from nncpu_b200 import Engine, GenerateParams, Model, SamplerParams, Session, SessionParams
from nncpu_b200.cache import PAGE
from nncpu_b200.config import PositionSpec, config_from_dict
from nncpu_b200.engine.model import parameter_list
from nncpu_b200.kernels import ops
from nncpu_b200.parts import Runtime, build
from nncpu_b200.weights import random_tensors, write_safetensors

pytestmark = pytest.mark.gpu
DTYPES = ["float32", "bfloat16"]
STORE = {"float32": torch.float32, "bfloat16": torch.bfloat16}


def dense(ff):
    return {"kind": "dense", "ff": ff}


def rot(base, dims, scaling=None):
    d = {"base": base, "dims": dims}
    if scaling:
        d["scaling"] = dict(zip(("factor", "original", "fast", "slow"), scaling))
    return d


def att(heads, kv, dim, scale, r, mlp=None):
    return {"type": "attention", "mixer": {"heads": heads, "kv_heads": kv, "dim": dim, "vdim": dim, "scale": scale, "rot": r},
            "mlp": mlp}


def lat(heads, dim, rot_dim, vdim, rank, q_rank, scale, r, kv_from=None, mlp=None):
    m = {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "kv_rank": rank, "q_rank": q_rank, "scale": scale,
         "rot": r}
    if kv_from is not None:
        m["kv_from"] = kv_from
    return {"type": "latent_attention", "mixer": m, "mlp": mlp}


def dlt(heads, kv, dim, vdim, conv, mlp=None):
    return {"type": "delta", "mixer": {"heads": heads, "kv_heads": kv, "dim": dim, "vdim": vdim, "conv": conv}, "mlp": mlp}


YARN_P = (6.0, 48.0, 8.0, 0.5)
YARN_Q = (3.0, 128.0, 16.0, 2.0)
CONFIGS = {
    # odd sizes everywhere, nothing a power of two; the recurrent layer first; a rotation of a part of the head; two
    # layers that read the first latent layer's cache, with heads and sizes of their own; layers without a
    # feed-forward; query/key heads shared by three value heads and not shared at all; two and three taps
    "P": {"architecture": "Pikalorn", "vocab": 301, "width": 88, "norm": {"eps": 3e-6}, "embedding": {"scale": 7.0},
          "layers": [dlt(6, 2, 20, 12, 3, mlp=dense(136)),
                     lat(3, 20, 6, 28, 36, 30, 0.25, rot(3000.0, 6, YARN_P), mlp=dense(40)),
                     att(6, 2, 24, 0.3, rot(10000.0, 16)),
                     lat(2, 12, 6, 20, 36, 44, 0.4, rot(3000.0, 6, YARN_P), kv_from=1, mlp=dense(72)),
                     dlt(3, 3, 10, 36, 2),
                     lat(5, 8, 6, 4, 36, 9, 0.5, rot(3000.0, 6, YARN_P), kv_from=1)]},
    # sizes the tensor-core paths take: heads of 64 and 128 lanes, kept rows of 64 and 128 lanes, states of 64 x 64
    # and 128 x 128
    "Q": {"architecture": "Pikalorn", "vocab": 640, "width": 256, "norm": {"eps": 1e-5}, "embedding": {"scale": 3.0},
          "layers": [att(8, 2, 64, 0.125, rot(1000000.0, 64), mlp=dense(512)),
                     lat(8, 32, 64, 32, 64, 96, 0.1, rot(10000.0, 64, YARN_Q), mlp=dense(256)),
                     dlt(4, 4, 64, 64, 4, mlp=dense(384)),
                     lat(4, 64, 64, 64, 64, 64, 0.09, rot(10000.0, 64, YARN_Q), kv_from=1, mlp=dense(256)),
                     att(2, 1, 128, 0.09, rot(500.0, 64), mlp=dense(256)),
                     dlt(2, 1, 128, 128, 2),
                     lat(2, 16, 32, 128, 32, 256, 0.15, rot(777.0, 32), mlp=dense(128))]},
    # values at the edges and what keeps every fast path out: a width that is no multiple of 8, 32 query heads on one
    # key/value head, a rotation of two lanes, one latent head with one value lane and a kept row of 1 000 lanes, a
    # rescaled rotation whose ramp has no width and one with a factor of 1, a convolution of one tap (no inputs to
    # keep), a state of one row and one of one column, no embedding scale, no feed-forward anywhere but once
    "W": {"architecture": "Pikalorn", "vocab": 97, "width": 100, "norm": {"eps": 1e-5},
          "layers": [att(32, 1, 8, 0.5, rot(100.0, 2)),
                     lat(1, 10, 2, 1, 998, 3, 0.3, rot(50.0, 2, (2.0, 40.0, 3.0, 3.0))),
                     dlt(1, 1, 1, 9, 1),
                     dlt(4, 2, 5, 1, 7, mlp=dense(36)),
                     att(3, 3, 10, 0.3, rot(50.0, 10)),
                     lat(4, 6, 8, 5, 12, 20, 0.3, rot(9.0, 8, (1.0, 16.0, 4.0, 1.0)))]},
}


def write_folder(path, cfg_dict, seed, store, sharpen=3.0, change=None):
    """A model folder with random weights; the query and key matrices are scaled up so that attention is not close
    to uniform and a key that is wrongly seen or missed changes the logits; the sinks are drawn around 1 with a
    spread of 1, so that they take a share of every row that leaving them out would show."""
    config = config_from_dict(cfg_dict)
    tensors = random_tensors(parameter_list(config.model_spec()), seed, store)
    for name in list(tensors):
        if name.endswith((".mix.q", ".mix.k", ".mix.uk", ".mix.uq")) and not name.endswith(".conv"):
            tensors[name] = (tensors[name].float() * sharpen).to(store)
        if name.endswith((".mix.v", ".mix.o", ".mix.dkv", ".mix.dq", ".up", ".gate", ".down", "embed", "head", ".mix.b", ".mix.a")):
            tensors[name] = (tensors[name].float() * 3.0).to(store)
    if change:
        change(tensors)
    path.mkdir(parents=True, exist_ok=True)
    (path / "config.json").write_text(json.dumps(config.to_dict()))
    write_safetensors(path / "model.safetensors", tensors, {"format": "pt"})
    return path


@pytest.fixture(scope="module")
def folders(tmp_path_factory):
    root = tmp_path_factory.mktemp("pikalorn")
    return {(name, dtype): write_folder(root / f"{name}_{dtype}", cfg, 21 + i, STORE[dtype])
            for i, (name, cfg) in enumerate(CONFIGS.items()) for dtype in DTYPES}


def toks(cfg, n, seed):
    return np.random.RandomState(seed).randint(0, cfg["vocab"], size=n).tolist()


def i32(x):
    return torch.tensor(x, dtype=torch.int32, device=DEV)


# -- mechanisms alone -----------------------------------------------------------------------------

@pytest.mark.parametrize("r", [rot(3000.0, 6, YARN_P), rot(10000.0, 64, YARN_Q), rot(50.0, 2, (2.0, 40.0, 3.0, 3.0)),
                               rot(9.0, 8, (1.0, 16.0, 4.0, 1.0)), rot(250000.0, 48, (40.0, 4096.0, 24.0, 1.5)), rot(123.0, 10)])
def test_rescaled_frequencies_and_stretched_tables(r):
    """The rotation's frequencies (plain, rescaled between two wavelengths, a ramp without width, a factor of one)
    and the table of cosines and sines at near and far positions."""
    sc = r.get("scaling") or {}
    spec = PositionSpec("rope_pairs", r["base"], r["dims"], scaling_factor=sc.get("factor", 0.0),
                        scaling_original=sc.get("original", 0.0), scaling_fast=sc.get("fast", 0.0), scaling_slow=sc.get("slow", 0.0))
    part = build("position", spec)
    part.bind({}, Runtime(DEV, torch.float32))
    f, stretch = P.rotary_frequencies(r)
    check(part.inv_freq, f, 1e-6, "frequencies")
    assert abs(part.stretch - stretch) < 1e-12
    pos = [0, 1, 2, 63, 64, 65, 1000, 4097]
    out = torch.empty(len(pos), r["dims"] // 2, 2, device=DEV)
    ops.rope_table(i32(pos), part.inv_freq, out, 1.0, False, part.stretch)
    # the angle is a 32-bit product of the position and the frequency
    a = (np.asarray(pos, dtype=np.float32)[:, None] * part.inv_freq.cpu().numpy()[None, :]).astype(np.float64)
    assert np.abs(out[..., 0].cpu().numpy() - np.cos(a) * stretch).max() < 3e-6 * stretch
    assert np.abs(out[..., 1].cpu().numpy() - np.sin(a) * stretch).max() < 3e-6 * stretch


def plain_sink_attention(q, k, v, positions, scale, sinks):
    """q [n, H, d] at ``positions`` over keys k, v [T, G, d]: every key up to the query's position."""
    n, H, d = q.shape
    G = k.shape[1]
    see = np.arange(k.shape[0])[None, :] <= np.asarray(positions)[:, None]
    out = np.zeros((n, H, v.shape[2]))
    for a in range(H):
        g = a // (H // G)
        out[:, a] = P.sink_softmax(q[:, a] @ k[:, g].T * scale, see, sinks[a]) @ v[:, g]
    return out


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("nh,nkv,hd", [(6, 2, 24), (4, 4, 16), (5, 1, 32), (4, 2, 64), (32, 1, 8)])
def test_softmax_with_a_sink_alone(dtype, nh, nkv, hd):
    """The 32-bit attention kernel with sinks: one that takes almost all of a row (the output shrinks towards zero), one
    so low that it changes nothing, ordinary ones; three sequences, one of them with a single key."""
    lens, new = [150, 1, 300], [9, 1, 130]
    dt = STORE[dtype]
    g = torch.Generator().manual_seed(nh * hd)
    kp, vp, table, ks, vs = scatter_pages(12, nkv, hd, lens, dt, seed=4)
    sinks = torch.randn(nh, generator=g)
    sinks[0], sinks[-1] = 20.0, -40.0
    q = [torch.randn(n, nh, hd, generator=g).to(dt) for n in new]
    n = sum(new)
    tok_seq = i32([b for b in range(3) for _ in range(new[b])])
    tok_pos = i32([p for b in range(3) for p in range(lens[b] - new[b], lens[b])])
    out = torch.empty(n, nh * hd, dtype=dt, device=DEV)
    ops.attention(torch.cat(q).view(n, -1).to(DEV), kp, vp, table, tok_seq, tok_pos, out, nh, nkv, hd, 0.3, sinks=sinks.to(DEV))
    want = np.concatenate([plain_sink_attention(q[b].double().numpy(), ks[b].double().numpy(), vs[b].double().numpy(),
                                                range(lens[b] - new[b], lens[b]), 0.3, sinks.double().numpy())
                           for b in range(3)]).reshape(n, -1)
    check(out, want, 1e-5 if dtype == "float32" else 2e-2, "attention with sinks")
    none = torch.empty_like(out)
    ops.attention(torch.cat(q).view(n, -1).to(DEV), kp, vp, table, tok_seq, tok_pos, none, nh, nkv, hd, 0.3)
    last = slice((nh - 1) * hd, nh * hd)
    check(out[:, last], none[:, last], 1e-6, "a sink far below the scores")
    assert float(out[:, :hd].float().abs().max()) < 0.2 * float(none[:, :hd].float().abs().max()), "a sink far above them"


@pytest.mark.parametrize("nh,nkv,hd", [(4, 2, 64), (2, 1, 128), (16, 1, 64), (12, 4, 128), (5, 5, 64), (1, 1, 64), (9, 1, 128),
                                       (32, 1, 128), (40, 2, 64), (17, 1, 64)])
def test_softmax_with_a_sink_on_the_tensor_core_kernels(nh, nkv, hd):
    """The bfloat16 kernels for prompts (mma.sync tiles, tcgen05 tiles) and for decode steps (one split; several merged
    inside a cluster; several merged through scratch) with sinks: one far above the scores, one far below, ordinary ones.
    Three sequences: a portion of 9 tokens, a whole prompt of 67, a portion of 130 that crosses pages."""
    lens, new = [150, 67, 300], [9, 67, 130]
    g = torch.Generator().manual_seed(nh + hd)
    kp, vp, table, ks, vs = scatter_pages(12, nkv, hd, lens, torch.bfloat16, seed=3)
    sinks = torch.randn(nh, generator=g) + 1.0
    sinks[0] = 20.0
    if nh > 2:
        sinks[-1] = -40.0
    dsinks = sinks.to(DEV)
    q = [torch.randn(n, nh, hd, generator=g).bfloat16() for n in new]
    n = sum(new)
    cu = i32(np.cumsum([0] + new).tolist())
    tok_pos = i32([p for b in range(3) for p in range(lens[b] - new[b], lens[b])])
    want = np.concatenate([plain_sink_attention(q[b].double().numpy(), ks[b].double().numpy(), vs[b].double().numpy(),
                                                range(lens[b] - new[b], lens[b]), 0.2, sinks.double().numpy())
                           for b in range(3)]).reshape(n, -1)
    qs = torch.cat(q).view(n, -1).to(DEV)
    out = torch.empty(n, nh * hd, dtype=torch.bfloat16, device=DEV)
    ops.attention_prefill_mma(qs, kp, vp, table, cu, tok_pos, out, 3, nh, nkv, hd, 0.2, 0, 0.0, dsinks)
    check(out, want, 2e-2, "prompt kernel")
    plain = torch.empty_like(out)
    ops.attention_prefill_mma(qs, kp, vp, table, cu, tok_pos, plain, 3, nh, nkv, hd, 0.2, 0)
    assert float((out.float() - plain.float()).abs().max()) > 0.05, "the sinks do not show"
    if ops.attention_prefill_tc_supported(nh, nkv, hd):
        status = torch.zeros(1, dtype=torch.int32, device=DEV)
        out_tc = torch.empty_like(out)
        ops.attention_prefill_tc(qs, kp, vp, table, cu, tok_pos, out_tc, status, 3, nh, nkv, hd, 0.2, 0, 0.0, dsinks)
        assert int(status.item()) == 0
        check(out_tc, want, 2e-2, "tcgen05 prompt kernel")
    last = torch.stack([q[b][-1] for b in range(3)]).view(3, -1).to(DEV)
    seq, pos = i32([0, 1, 2]), i32([l - 1 for l in lens])
    want_last = np.stack([want[int(cu[b + 1]) - 1] for b in range(3)])
    for n_splits, with_scratch in ((1, False), (2, False), (3, False), (2, True), (5, True)):
        scratch = None
        if with_scratch:
            scratch = torch.empty(ops.attention_decode_scratch_floats(3, nh, nkv, hd, n_splits), device=DEV)
        got = torch.empty(3, nh * hd, dtype=torch.bfloat16, device=DEV)
        ops.attention_decode_mma(last, kp, vp, table, seq, pos, got, scratch, nh, nkv, hd, 0.2, 0, n_splits, 0.0, dsinks)
        check(got, want_last, 2e-2, f"decode kernel, {n_splits} splits" + (" through scratch" if with_scratch else ""))


def test_values_that_are_the_keys_and_the_gate_on_the_heads():
    """The append of an attention layer whose values are its keys as projected: the key pages get the normed, rotated
    keys, the value pages the keys as they left the projection; then the sigmoid gate on the heads."""
    nh, nkv, hd, half, n = 6, 3, 10, 3, 70
    g = torch.Generator().manual_seed(2)
    qkv = torch.randn(n, (nh + nkv) * hd + nh * hd + 5, generator=g)          # q, k, the gate's logits, spare lanes
    qg, kg = torch.randn(hd, generator=g) + 1, torch.randn(hd, generator=g) + 1
    r = rot(77.0, 2 * half)
    pos = list(range(30, 30 + n))
    f, _ = P.rotary_frequencies(r)
    cs = torch.tensor(np.stack([np.cos(np.outer(pos, f)), np.sin(np.outer(pos, f))], axis=-1), dtype=torch.float32, device=DEV)
    table = i32([[3, 0]])
    kp, vp = torch.zeros(4, nkv, PAGE, hd, device=DEV), torch.zeros(4, nkv, PAGE, hd, device=DEV)
    q_out = torch.empty(n, nh * hd, device=DEV)
    ops.qk_norm_rope_append(qkv.to(DEV), qg.to(DEV), kg.to(DEV), 1e-5, cs, i32([0] * n), i32(pos), table, kp, vp, q_out, nh, nkv, hd,
                            values_are_keys=True)
    x = qkv.double().numpy()
    q = P.rotate(P.rms_norm(x[:, :nh * hd].reshape(n, nh, hd), qg.double().numpy(), 1e-5), pos, r, "half")
    k_raw = x[:, nh * hd:(nh + nkv) * hd].reshape(n, nkv, hd)
    k = P.rotate(P.rms_norm(k_raw, kg.double().numpy(), 1e-5), pos, r, "half")
    check(q_out, q.reshape(n, -1), 1e-5, "queries")
    for t in (0, 33, 34, 69):
        page, row = (3, pos[t]) if pos[t] < PAGE else (0, pos[t] - PAGE)
        check(kp[page, :, row], k[t], 1e-5, f"key of token {t}")
        check(vp[page, :, row], k_raw[t], 1e-6, f"value of token {t}")
    heads = torch.randn(n, nh * hd, generator=g)
    got = heads.to(DEV)
    ops.sigmoid_gate(got, qkv.to(DEV), (nh + nkv) * hd)
    check(got, heads.double().numpy() * P.sigmoid(x[:, (nh + nkv) * hd:(nh + nkv + nh) * hd]), 1e-6, "gated heads")


@pytest.mark.parametrize("nh,nkv,hd,n_splits,with_scratch", [(4, 2, 64, 1, False), (8, 2, 128, 3, False), (16, 1, 64, 2, True),
                                                             (6, 6, 128, 5, True), (3, 1, 64, 2, False)])
def test_decode_step_from_the_projections_with_sinks_own_values_and_the_gate(nh, nkv, hd, n_splits, with_scratch):
    """One token each of three sequences (at positions 0, 64 and 299: the first key of a sequence, the first of a page,
    far into a sequence) through the decode kernel that starts from the 32-bit projections: per-head norms, rotation,
    the append of the key and of the key as projected as the value, softmax with sinks, and the sigmoid gate, against
    the plain statement of every one of them; then the pages must hold what the separate append kernel writes."""
    lens = [1, 65, 300]
    g = torch.Generator().manual_seed(nh * hd + n_splits)
    kp, vp, table, ks, vs = scatter_pages(12, nkv, hd, lens, torch.bfloat16, seed=6)
    sinks = torch.randn(nh, generator=g) + 1.0
    qg, kg = torch.randn(hd, generator=g) + 1, torch.randn(hd, generator=g) + 1
    r = rot(10000.0, hd)
    pos = [l - 1 for l in lens]
    qkv = torch.randn(3, (nh + nkv + nh) * hd, generator=g)
    x = qkv.double().numpy()
    f, _ = P.rotary_frequencies(r)
    cs = torch.tensor(np.stack([np.cos(np.outer(pos, f)), np.sin(np.outer(pos, f))], axis=-1), dtype=torch.float32, device=DEV)
    q = P.rotate(P.rms_norm(x[:, :nh * hd].reshape(3, nh, hd), qg.double().numpy(), 1e-5), pos, r, "half")
    k_raw = x[:, nh * hd:(nh + nkv) * hd].reshape(3, nkv, hd)
    k_new = P.rotate(P.rms_norm(k_raw, kg.double().numpy(), 1e-5), pos, r, "half")
    gate = P.sigmoid(x[:, (nh + nkv) * hd:])
    want = []
    for b in range(3):
        kb, vb = ks[b].double().numpy().copy(), vs[b].double().numpy().copy()
        kb[-1], vb[-1] = k_new[b], k_raw[b]                 # the token's own key and value replace the last stored ones
        want.append(plain_sink_attention(q[b:b + 1], kb, vb, [pos[b]], 0.2, sinks.double().numpy()).reshape(-1) * gate[b])
    seq, dpos = i32([0, 1, 2]), i32(pos)
    scratch = torch.empty(ops.attention_decode_scratch_floats(3, nh, nkv, hd, n_splits), device=DEV) if with_scratch else None
    got = torch.empty(3, nh * hd, dtype=torch.bfloat16, device=DEV)
    kp2, vp2 = kp.clone(), vp.clone()
    ops.attention_decode_mma_from_qkv(qkv.to(DEV), qg.to(DEV), kg.to(DEV), 1e-5, cs, kp, vp, True, table, seq, dpos, got, scratch,
                                      nh, nkv, hd, 0.2, 0, n_splits, sinks=sinks.to(DEV), values_are_keys=True, gated=True)
    check(got, np.stack(want), 2e-2, "decode from the projections")
    q_out = torch.empty(3, nh * hd, dtype=torch.bfloat16, device=DEV)
    ops.qk_norm_rope_append(qkv.to(DEV), qg.to(DEV), kg.to(DEV), 1e-5, cs, seq, dpos, table, kp2, vp2, q_out, nh, nkv, hd,
                            values_are_keys=True)
    assert torch.equal(kp, kp2) and torch.equal(vp, vp2), "the pages differ from the separate append kernel's"


@pytest.mark.parametrize("r,R,qr", [(36, 6, 30), (64, 64, 96), (998, 2, 3), (12, 8, 20)])
def test_what_a_latent_layer_keeps_and_its_queries_in_latent_space(r, R, qr):
    """The kept row [normed latent, rotated shared key part] in its page, the queries' own normed latent, and the
    rotated query lanes where the attention kernels read them."""
    n, H, d = 70, 3, 10
    g = torch.Generator().manual_seed(r)
    rt = rot(300.0, R, (4.0, 64.0, 8.0, 1.0))
    pos = list(range(40, 40 + n))
    f, stretch = P.rotary_frequencies(rt)
    cs = torch.tensor(np.stack([np.cos(np.outer(pos, f)), np.sin(np.outer(pos, f))], axis=-1) * stretch, dtype=torch.float32, device=DEV)
    proj = torch.randn(n, qr + r + R, generator=g) * 2             # the queries' latent, the latent, the shared key part
    gamma, qgamma = torch.randn(r, generator=g) + 1, torch.randn(qr, generator=g) + 1
    pages = torch.zeros(3, 1, PAGE, r + R, device=DEV)
    cq = torch.empty(n, qr, device=DEV)
    ops.latent_append(proj.to(DEV), qr, gamma.to(DEV), 2e-5, i32([0] * n), i32(pos), i32([[2, 1]]), pages, None, rot_dim=R, cos_sin=cs,
                      q_norm=(qgamma.to(DEV), 0, qr, cq))
    x = proj.double().numpy()
    c = P.rms_norm(x[:, qr:qr + r], gamma.double().numpy(), 2e-5)
    kr = P.rotate(x[:, None, qr + r:], pos, rt, "pairs")[:, 0]
    check(cq, P.rms_norm(x[:, :qr], qgamma.double().numpy(), 2e-5), 1e-5, "the queries' latent")
    for t in (0, 23, 24, 69):
        page, row = (2, pos[t]) if pos[t] < PAGE else (1, pos[t] - PAGE)
        check(pages[page, 0, row, :r], c[t], 1e-5, f"latent of token {t}")
        check(pages[page, 0, row, r:], kr[t], 1e-5, f"shared key part of token {t}")
    q = torch.randn(n, H * (d + R), generator=g)
    q_lat = torch.zeros(n, H * (r + R), device=DEV)
    ops.latent_query(q.to(DEV), cs, q_lat, H, d, R, r)
    want = P.rotate(q.double().numpy().reshape(n, H, d + R)[..., d:], pos, rt, "pairs")
    check(q_lat.view(n, H, r + R)[..., r:], want, 1e-5, "rotated query lanes")


def delta_inputs(g, T, H, G, d, e, taps):
    """Random projections of T tokens [T, C + H e + 2 H] and what the plain functions make of them."""
    C = 2 * G * d + H * e
    proj = torch.randn(T, C + H * e + 2 * H, generator=g)
    proj[:, C + H * e:] *= 2
    return proj


def plain_delta(proj, conv_w, a_log, dt_bias, H, G, d, e):
    x = proj.double().numpy()
    T, C = x.shape[0], 2 * G * d + H * e
    y = P.silu(P.short_conv(x[:, :C], conv_w.double().numpy()))
    q, k, v = y[:, :G * d].reshape(T, G, d), y[:, G * d:2 * G * d].reshape(T, G, d), y[:, 2 * G * d:].reshape(T, H, e)
    q = q / np.sqrt((q * q).sum(-1, keepdims=True) + P.UNIT_EPS) * d ** -0.5
    k = k / np.sqrt((k * k).sum(-1, keepdims=True) + P.UNIT_EPS)
    b = P.sigmoid(x[:, C + H * e:C + H * e + H])
    gd = np.exp(-np.exp(a_log.double().numpy())[None] * P.softplus(x[:, C + H * e + H:] + dt_bias.double().numpy()[None]))
    group = np.arange(H) // (H // G)
    return P.delta_rule(q[:, group], k[:, group], v, gd, b)


@pytest.mark.parametrize("H,G,d,e,taps", [(6, 2, 20, 12, 3), (1, 1, 64, 128, 4), (2, 2, 130, 33, 2), (4, 1, 128, 64, 4),
                                          (1, 1, 300, 40, 1), (3, 3, 1, 9, 5), (4, 2, 5, 1, 7), (2, 1, 600, 20, 2)])
def test_delta_rule_alone_in_portions_and_batches(H, G, d, e, taps):
    """Convolutions, unit vectors, decays and the recurrence: three sequences of unequal lengths in one step against
    the plain functions, then the same tokens cut into portions (2, 1, 5, ... tokens, shorter than the convolution)
    with the state and the convolutions' inputs carried in the state area: the same bits."""
    g = torch.Generator().manual_seed(d + taps)
    lens, slots, n_slots = [37, 5, 70], [4, 0, 2], 6
    C = 2 * G * d + H * e
    conv_w = torch.randn(C, taps, generator=g) * 0.5
    a_log, dt_bias = torch.randn(H, generator=g) * 0.5, torch.randn(H, generator=g) * 0.5
    data = []
    for T in lens:
        proj = delta_inputs(g, T, H, G, d, e, taps)
        data.append((proj, plain_delta(proj, conv_w, a_log, dt_bias, H, G, d, e)))
    S = H * d * e
    state = torch.zeros(n_slots + 1, S + (taps - 1) * C, device=DEV)

    def run(pieces):          # pieces: list of (sequence index, first, last) run as one step
        proj = torch.cat([data[b][0][lo:hi] for b, lo, hi in pieces]).to(DEV)
        n = proj.shape[0]
        cu = i32(np.cumsum([0] + [hi - lo for _, lo, hi in pieces]).tolist())
        sl = i32([slots[b] for b, _, _ in pieces])
        ts = i32([i for i, (_, lo, hi) in enumerate(pieces) for _ in range(hi - lo)])
        xc, gb, o = torch.empty(n, C, device=DEV), torch.empty(n, 2 * H, device=DEV), torch.empty(n, H * e, device=DEV)
        ops.delta_prepare(proj, conv_w.to(DEV), state, S, ts, sl, cu, a_log.to(DEV), dt_bias.to(DEV), xc, gb, len(pieces), H, G, d, e, taps)
        ops.delta_scan(xc, gb, state, sl, cu, o, len(pieces), H, G, d, e)
        return o.cpu()

    whole = run([(b, 0, lens[b]) for b in range(3)])
    at = 0
    for b in range(3):
        check(whole[at:at + lens[b]].view(lens[b], H, e), data[b][1], 3e-5, f"sequence {b} in a batch")
        at += lens[b]
    kept = state.clone()
    state.zero_()
    done, outs = [0, 0, 0], [[], [], []]
    sizes = [2, 1, 5, 3, 2, 64, 2]
    i = 0
    while any(done[b] < lens[b] for b in range(3)):
        pieces = []
        for b in range(3):
            if done[b] < lens[b]:
                n = min(sizes[(i + b) % len(sizes)], lens[b] - done[b])
                pieces.append((b, done[b], done[b] + n))
        o = run(pieces)
        at = 0
        for b, lo, hi in pieces:
            outs[b].append(o[at:at + hi - lo])
            at += hi - lo
            done[b] = hi
        i += 1
    at = 0
    for b in range(3):
        assert torch.equal(torch.cat(outs[b]), whole[at:at + lens[b]]), "portions give other bits than the whole"
        at += lens[b]
    assert torch.equal(state, kept), "the state after portions differs from the state after the whole"
    assert float(state[n_slots].abs().max()) == 0 and float(state[1].abs().max()) == 0, "a foreign state row was written"
    if taps > 1:                # the last inputs of the longest sequence, oldest first
        tail = data[2][0][lens[2] - (taps - 1):, :C]
        assert torch.equal(state[2, S:].view(taps - 1, C).cpu(), tail)


def test_delta_rule_remembers_a_write_far_back_and_padding_leaves_the_state_alone():
    """One write of full strength at position 3 with decays near one ever after, 600 weak tokens, and a query at the
    end that asks for that key: it must get most of the value back; a padding sequence (slot -1) gets zeros and no
    state row is touched for it."""
    H, G, d, e, taps, T = 2, 1, 24, 40, 2, 604
    g = torch.Generator().manual_seed(5)
    C = 2 * G * d + H * e
    proj = delta_inputs(g, T, H, G, d, e, taps) * 0.05
    conv_w = torch.zeros(C, taps)
    conv_w[:, -1] = 1.0                                   # the convolution passes the current token
    a_log, dt_bias = torch.full((H,), -3.0), torch.zeros(H)
    proj[:, C + H * e + H:] = -12.0                       # decays near one
    proj[:, C + H * e:C + H * e + H] = -9.0               # weak writes ...
    proj[3, C + H * e:C + H * e + H] = 9.0                # ... but for one
    proj[3, G * d + 7] = 30.0                             # its key: channel 7
    proj[3, 2 * G * d:2 * G * d + e] = torch.arange(e).float() / 4
    proj[T - 1, 7] = 30.0                                 # the last query asks for it
    want = plain_delta(proj, conv_w, a_log, dt_bias, H, G, d, e)
    assert abs(want[T - 1, 0, e - 1]) > 10 * np.abs(want[T - 2, 0]).max(), "the test's far token does not stand out"
    S = H * d * e
    state = torch.zeros(3, S + (taps - 1) * C, device=DEV)
    o = torch.empty(T, H * e, device=DEV)

    def step(lo, hi, slots):
        n = hi - lo + (len(slots) - 1)
        pj = torch.cat([proj[lo:hi]] + [proj[:1]] * (len(slots) - 1)).to(DEV)
        cu = i32([0, hi - lo] + [hi - lo + i + 1 for i in range(len(slots) - 1)])
        ts = i32([0] * (hi - lo) + list(range(1, len(slots))))
        xc, gb, out = torch.empty(n, C, device=DEV), torch.empty(n, 2 * H, device=DEV), torch.empty(n, H * e, device=DEV)
        ops.delta_prepare(pj, conv_w.to(DEV), state, S, ts, i32(slots), cu, a_log.to(DEV), dt_bias.to(DEV), xc, gb, len(slots), H, G, d, e, taps,
                          one_token_each=hi - lo == 1)      # a decode step advances the kept inputs inside the one kernel
        ops.delta_scan(xc, gb, state, i32(slots), cu, out, len(slots), H, G, d, e)
        o[lo:hi] = out[:hi - lo]
        return out[hi - lo:]

    pad = step(0, 500, [1, -1])
    assert float(pad.abs().max()) == 0 and float(state[2].abs().max()) == 0 and float(state[0].abs().max()) == 0
    for t in range(500, T):                               # the rest token by token, as decoding does
        step(t, t + 1, [1])
    got = o.cpu().view(T, H, e)
    check(got[T - 1], want[T - 1], 1e-4, "the far write's value")
    check(got, want, 1e-4, "all rows")


def test_delta_output_stage():
    H, d, e, T = 3, 20, 44, 11
    g = torch.Generator().manual_seed(6)
    o = torch.randn(T, H * e, generator=g) * 3
    proj = torch.randn(T, 100 + H * e + 7, generator=g)
    w = torch.randn(e, generator=g) + 1
    want = (P.rms_norm(o.double().numpy().reshape(T, H, e), w.double().numpy(), 1e-5)
            * P.silu(proj[:, 100:100 + H * e].double().numpy().reshape(T, H, e))).reshape(T, -1)
    for dt, tol in ((torch.float32, 1e-5), (torch.bfloat16, 1e-2)):
        out = torch.empty(T, H * e, dtype=dt, device=DEV)
        ops.gla_output(o.to(DEV), proj.to(DEV), w.to(DEV), 1e-5, out, H, d, e, gate_col=100)
        check(out, want, tol, "norm, weight and gate of the heads")


# -- the model ------------------------------------------------------------------------------------

def close(got, want, dtype, what):
    """Logits against the plain model's.  float32: the largest difference within 1e-4 of the largest logit.
    bfloat16: rounding of the activations to 8 bits of mantissa is the design's own noise, so the measure is the
    root mean square of the differences over all the rows given, held to 4 % of the logits' own; a fault of the cache,
    the state or a sink moves far more than that with these weights, and the float32 runs hold the same code to 1e-4."""
    if dtype == "float32":
        return check(got, want, TOL[dtype], what)
    g = got.detach().double().cpu().numpy()
    w = np.asarray(want, dtype=np.float64).reshape(g.shape)
    assert np.isfinite(g).all(), f"{what}: NaN or infinity"
    rms = float(np.sqrt(np.mean((g - w) ** 2)) / np.sqrt(np.mean(w ** 2)))
    assert rms <= 4e-2, f"{what}: root mean square of the differences {rms:.3e} of the logits' own"
    check(got, want, 0.25, what)


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
    if dtype == "float32":         # the first tokens of a sequence (zeros before the convolutions, an empty state, a
        for i in range(4):         # softmax of one key and the sink), one by one in the sharper arithmetic
            close(got[i], want[i], dtype, f"{name} token {i}")


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["P", "Q"])
def test_every_layer_against_the_plain_model(folders, name, dtype):
    """The stream after every layer, float32 and bfloat16."""
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
    assert len(caught) == len(streams) == len(CONFIGS[name]["layers"])
    for r, (got, want) in enumerate(zip(caught, streams)):
        assert got.dtype == torch.float32, "the residual sum is 32-bit in both run types"
        check(got, want, 1e-5 if dtype == "float32" else 3e-2, f"stream after layer {r}")


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", list(CONFIGS))
def test_portions_and_token_by_token_against_the_whole(folders, name, dtype):
    """The same 200 tokens: whole; in portions of 2, 3, 64, 1, 65, ... tokens; a prompt of 40 and then one token a
    step for 160 steps (across page borders, the state and the convolutions' inputs handed from step to step).  All
    against the plain model; in float32 the three runs agree with one another far below the tolerance."""
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
    s3 = engine.alloc_slot()                 # the slot, pages and state row that the whole run used
    engine.step([s3], [t[:40]], [[]])
    rows = [engine.step([s3], [[t[i]]]).clone() for i in range(40, 200)]
    decoded = torch.cat(rows)
    close(decoded, want[40:], dtype, "token by token")
    s4 = engine.alloc_slot()                 # portions that want their last place only: the captured prompt steps
    at, last = 0, []
    for n in (5, 2, 33, 2, 100, 58):
        last.append(engine.step([s4], [t[at:at + n]]).clone())
        at += n
    close(torch.cat(last), want[[4, 6, 39, 41, 141, 199]], dtype, "portions through captured steps")
    if dtype == "float32":
        check(portions, whole, 2e-5, "portions against the whole")
        check(decoded, whole[40:], 2e-5, "token by token against the whole")
    engine.cache.check()


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", list(CONFIGS))
def test_unequal_batch_then_decoding_together_on_reused_slots(folders, name, dtype):
    """Four prompts of 1, 33, 130 and 64 tokens in one step, then one token each per step; the short ones end
    early and give their slots, pages and state rows back; a newcomer takes them while the others go on (its state
    must start at zero although the row was used)."""
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
def test_long_decoding_across_pages(folders, dtype):
    """420 decoded tokens after a prompt of 150: pages pass by, every attention layer's keys go back 570 positions
    (the layer that reads another's cache too), and the recurrent state has been rewritten 570 times."""
    cfg = CONFIGS["Q"]
    n = 570
    t = toks(cfg, n, 5)
    want = plain_logits(folders["Q", dtype], t)
    model = Model.load(folders["Q", dtype], dtype=dtype)
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


def test_long_prompt_on_the_tensor_core_paths(tmp_path):
    """600 tokens in one step through sizes that the tensor-core kernels take (heads of 128 and 64 lanes, a kept row of
    128 lanes, a state of 128 x 128), then ten tokens one by one: bfloat16 against the plain model, and the same
    folder run in float32."""
    cfg = {"architecture": "Pikalorn", "vocab": 300, "width": 256, "norm": {"eps": 1e-5}, "embedding": {"scale": 2.0},
           "layers": [att(4, 2, 128, 0.09, rot(1000000.0, 128), mlp=dense(256)),
                      lat(4, 64, 64, 64, 64, 96, 0.09, rot(10000.0, 64, YARN_Q), mlp=dense(256)),
                      dlt(2, 1, 128, 128, 4, mlp=dense(128)),
                      lat(8, 32, 64, 32, 64, 64, 0.1, rot(10000.0, 64, YARN_Q), kv_from=1),
                      att(8, 8, 64, 0.125, rot(10000.0, 32), mlp=dense(256))]}
    folder = write_folder(tmp_path / "m", cfg, 5, torch.bfloat16, sharpen=2.0)
    t = toks(cfg, 610, 3)
    want = plain_logits(folder, t)
    rows = list(range(0, 600, 7)) + [63, 64, 127, 128, 129, 255, 256, 511, 512, 599]
    for dtype in ("bfloat16", "float32"):
        model = Model.load(folder, dtype=dtype)
        engine = Engine(model, max_tokens=64 * 11)
        s = engine.alloc_slot()
        close(engine.step([s], [t[:600]], [rows]), want[rows], dtype, f"{dtype}: a prompt of 600 tokens")
        out = torch.cat([engine.step([s], [[t[i]]]).clone() for i in range(600, 610)])
        close(out, want[600:], dtype, f"{dtype}: ten tokens after it")
        model.rt.check_status()


def sharpened(names, factor):
    def change(tensors):
        for n in list(tensors):
            if n.endswith(names):
                tensors[n] = (tensors[n].float() * factor).to(tensors[n].dtype)
    return change


@pytest.mark.parametrize("kind", ["attention", "latent_attention"])
def test_a_key_far_back_and_large_sinks(tmp_path, kind):
    """One attention layer with queries and keys so sharp that single keys take most of a row's weight, most of them
    far back and across pages (560 positions), and sinks drawn so large that where no key stands out the sink takes the
    row: the logits must follow the plain model as a prompt and token by token."""
    layer = (att(2, 1, 16, 1.0, rot(10000.0, 8), mlp=dense(64)) if kind == "attention" else
             lat(2, 16, 8, 24, 40, 20, 1.0, rot(10000.0, 8, YARN_P), mlp=dense(64)))
    cfg = {"architecture": "Pikalorn", "vocab": 64, "width": 48, "norm": {"eps": 1e-5}, "embedding": {"scale": 2.0},
           "layers": [layer]}

    def change(tensors):
        tensors["l0.mix.sink"] = tensors["l0.mix.sink"] * 0 + torch.tensor([6.0, 2.5])

    folder = write_folder(tmp_path / "m", cfg, 3, torch.float32, sharpen=10.0, change=change)
    t = toks(cfg, 560, 8)
    want = plain_logits(folder, t)
    pcfg, w = P.load(folder)
    w["l0.mix.sink"] = w["l0.mix.sink"] - 30.0              # the same model without sinks answers otherwise
    assert np.abs(P.forward(pcfg, w, t[:100]) - want[:100]).max() > 0.05 * np.abs(want).max(), "the sinks do not show"
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
    the greedy token harness against the plain model, and a sampled continuation (device-side sampling chain)."""
    import io
    from nncpu_b200.cli import parse_options, run_gen, run_generate, run_info, run_random_weights

    def run(fn, argv):
        out = io.StringIO()
        assert fn(parse_options(argv), out) == 0
        return out.getvalue()

    cfg = tmp_path / "cfg.json"
    cfg.write_text(json.dumps(CONFIGS["P"]))
    run(run_random_weights, ["--random-weights", str(cfg), "5", str(tmp_path / "m"), "--fp32"])
    info = json.loads(run(run_info, ["--info", str(tmp_path / "m")]))
    assert info["config"]["architecture"] == "Pikalorn" and info["parameters"] > 0
    prompt = toks(CONFIGS["P"], 40, 3)
    got = [int(t) for t in run(run_gen, ["--gen", str(tmp_path / "m"), " ".join(map(str, prompt)), "6", "--fp32"]).splitlines()[0].split()]
    pcfg, w = P.load(tmp_path / "m")
    assert got == P.greedy(pcfg, w, prompt, 6)
    out = run(run_generate, ["-m", str(tmp_path / "m"), "--tokens", " ".join(map(str, prompt)), "-n", "6", "--temp", "0.8",
                             "--top-k", "20", "-s", "4", "-b", "3"]).split()
    assert len(out) >= 6 and all(0 <= int(t) < CONFIGS["P"]["vocab"] for t in out[:6])


def test_trace_replay_of_many_short_requests(folders, tmp_path):
    """``bin/trace_run`` as a subprocess on this design: eight requests of unequal lengths in one batch with
    ``--max-tokens`` set to exactly the tokens they hold (most of them end inside a page), decoded together while
    the shorter ones end; then a second batch on the slots, pages and state rows that were given back."""
    import subprocess
    import sys
    from conftest import ROOT
    cfg = CONFIGS["P"]
    folder = folders["P", "float32"]
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

    first = [(f"r{i}", 0, n, [0, n - 1] if n > 1 else [0]) for i, n in enumerate(lens)]
    add(first, end=[])
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


def random_pikalorn(rs):
    """A random configuration: any order of the three kinds of layer, head sizes in and out of what the tensor-core
    kernels take, any grouping of heads, layers that read an earlier latent layer's cache, some without a feed-forward."""
    width = int(rs.choice([72, 100, 136, 200, 256]))
    layers, owners = [], []
    for i in range(int(rs.randint(2, 7))):
        kind = rs.choice(["attention", "latent_attention", "delta"])
        mlp = dense(int(rs.choice([40, 88, 136, 264]))) if rs.rand() < 0.8 else None
        if kind == "attention":
            kv, group, dim = int(rs.choice([1, 2, 3])), int(rs.choice([1, 2, 4, 5])), int(rs.choice([16, 24, 48, 64, 128]))
            dims = int(rs.choice([dim, dim // 2, 2]))
            layers.append(att(kv * group, kv, dim, float(rs.choice([dim ** -0.5, 0.2])), rot(float(rs.choice([1e4, 1e6, 300.0])), dims - dims % 2 or 2), mlp=mlp))
        elif kind == "latent_attention":
            if owners and rs.rand() < 0.5:
                j = int(rs.choice(owners))
                m = layers[j]["mixer"]
                layers.append(lat(int(rs.choice([1, 2, 3, 8])), int(rs.choice([8, 16, 32, 64])), m["rot_dim"], int(rs.choice([8, 20, 64])),
                                  m["kv_rank"], int(rs.choice([12, 64, 100])), float(rs.choice([0.1, 0.25])), m["rot"], kv_from=j, mlp=mlp))
            else:
                R = int(rs.choice([2, 8, 32, 64]))
                rank = int(rs.choice([24, 32, 64, 96, 128 - R]))
                sc = None if rs.rand() < 0.3 else (float(rs.choice([2.0, 4.0, 16.0])), float(rs.choice([32, 256, 1024])),
                                                   float(rs.choice([8.0, 32.0])), float(rs.choice([0.5, 1.0, 2.0])))
                owners.append(i)
                layers.append(lat(int(rs.choice([1, 2, 4, 6])), int(rs.choice([8, 16, 32, 64])), R, int(rs.choice([8, 20, 64])), rank,
                                  int(rs.choice([12, 64, 100])), float(rs.choice([0.1, 0.25])), rot(float(rs.choice([1e4, 500.0])), R, sc), mlp=mlp))
        else:
            kv, group = int(rs.choice([1, 2, 3])), int(rs.choice([1, 2, 3]))
            layers.append(dlt(kv * group, kv, int(rs.choice([8, 20, 64, 128, 136])), int(rs.choice([8, 20, 64, 128])), int(rs.choice([1, 2, 4, 5])), mlp=mlp))
    cfg = {"architecture": "Pikalorn", "vocab": int(rs.randint(100, 600)), "width": width,
           "norm": {"eps": float(rs.choice([1e-6, 1e-5]))}, "layers": layers}
    if rs.rand() < 0.7:
        cfg["embedding"] = {"scale": float(rs.choice([1.0, 3.0, width ** 0.5]))}
    return cfg


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("seed", range(8))
def test_random_configuration_and_trace(tmp_path, seed, dtype):
    """Random configurations, each with a batch of unequal prompts (the first one cut in two steps the second time
    round), decoding with early leavers, then the same again on the slots, pages and state rows given back."""
    rs = np.random.RandomState(4000 + seed)
    cfg = random_pikalorn(rs)
    folder = write_folder(tmp_path / "m", cfg, seed, STORE[dtype], sharpen=2.0)
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
        rows = [Rows(dtype, f"seed {seed} round {round_} request {b}") for b in range(len(reqs))]
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
            rows[b].done()
    engine.cache.check()
    model.rt.check_status()
