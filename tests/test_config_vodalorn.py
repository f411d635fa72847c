"""Vodalorn's configuration on the CPU: the keys of its ``config.json``, the registry's choice by the ``architecture``
key, the schedule of a looped range of layers, the tensors its parts ask for, what the cache keeps (pages for the
softmax side, state rows for the recurrences and for the embedding's last token), and the plain model's own
consistency."""
import json

import numpy as np
import pytest
import torch

import plain_vodalorn as P
from nncpu_b200.cache import Cache
from nncpu_b200.config import VodalornConfig, config_from_dict
from nncpu_b200.engine.model import parameter_list
from nncpu_b200.errors import BadFormat, UnsupportedModel
from nncpu_b200.parts import base
from nncpu_b200.weights import check_tensors, write_model_folder

CFG = {"architecture": "Vodalorn", "vocab": 97, "width": 40, "norm": {"eps": 2e-6}, "residual_mult": 0.8,
       "embedding": {"bigram": {"buckets": 53, "mul_prev": 19, "mul_cur": 3}}, "token_side": {"dim": 6},
       "loop": {"start": 1, "stop": 3, "times": 2},
       "layers": [{"type": "parallel", "mlp": {"kind": "dense", "ff": 72},
                   "mixer": {"left": {"heads": 6, "kv_heads": 3, "dim": 8, "vdim": 12, "scale": 0.25, "mask": {"size": 9},
                                      "rot": {"base": 1234.0, "dims": 6}},
                             "right": {"heads": 2, "dim": 10, "vdim": 14, "decay": [0.9, 0.99], "rot": {"base": 50.0, "dims": 10}}}},
                  {"type": "channel_delta", "mlp": {"kind": "moe", "expert": {"ff": 16, "limit": 1.5},
                                                    "router": {"experts": 6, "top": 2, "scale": 2.0, "groups": {"count": 3, "keep": 2}}},
                   "mixer": {"heads": 6, "kv_heads": 2, "dim": 10, "vdim": 14, "conv": 3, "rank": 4, "gate_rank": 5}},
                  {"type": "parallel", "mlp": None,
                   "mixer": {"left": {"heads": 2, "kv_heads": 2, "dim": 4, "vdim": 4, "scale": 0.5},
                             "right": {"heads": 1, "dim": 4, "vdim": 4, "decay": [1.0]}}},
                  {"type": "channel_delta", "mlp": {"kind": "dense", "ff": 24},
                   "mixer": {"heads": 1, "kv_heads": 1, "dim": 8, "vdim": 8, "conv": 2, "rank": 3, "gate_rank": 3}}]}


def test_keys_round_trip_and_specs():
    cfg = config_from_dict(CFG)
    assert isinstance(cfg, VodalornConfig)
    assert config_from_dict(cfg.to_dict()) == cfg and cfg.to_dict() == CFG
    spec = cfg.model_spec()
    a, d, b, z = spec.layers
    assert {x.kind for x in spec.layers} == {"prenorm"} and all(x.residual_mult == 0.8 for x in spec.layers)
    assert all(x.norm1.kind == "layernorm" for x in spec.layers) and spec.output.norm.kind == "layernorm"
    assert a.feed_forward.activation == "relu2" and not a.feed_forward.bias and b.feed_forward is None
    m = a.mixer
    assert (m.kind, m.weight, m.eps) == ("mixer_pair", 0.5, 2e-6)
    l, r = m.left, m.right
    assert (l.n_heads, l.n_kv_heads, l.head_dim, l.v_head_dim, l.scale, l.window, l.qkv_bias) == (6, 3, 8, 12, 0.25, 9, True)
    assert (l.position.kind, l.position.theta, l.position.rotary_dim) == ("rope_neox", 1234.0, 6)
    assert (r.kind, r.n_heads, r.key_dim, r.value_dim, r.decays, r.position.rotary_dim) == ("retention", 2, 10, 14, (0.9, 0.99), 10)
    assert b.mixer.left.window == 0 and b.mixer.left.position is None and b.mixer.right.position is None
    m = d.mixer
    assert (m.kind, m.n_heads, m.n_kv_heads, m.key_dim, m.value_dim, m.conv, m.channel_decay) == ("gated_delta", 6, 2, 10, 14, 3, True)
    f = d.feed_forward
    assert (f.n_experts, f.top, f.scores, f.n_groups, f.keep_groups, f.weight_scale, f.router_bias) == (6, 2, "all", 3, 2, 2.0, False)
    assert (a.side.col, b.side.col, a.side.dim, a.side.table_width) == (0, 12, 6, 24)
    e = spec.embedding
    assert (e.pair_table, e.pair_buckets, e.pair_mul_prev, e.pair_mul_cur) == ("bigram", 53, 19, 3)


def test_the_loop_is_in_the_schedule():
    spec = config_from_dict(CFG).model_spec()
    assert [e.layer for e in spec.schedule] == [0, 1, 2, 1, 2, 3]
    marks = [(i, e.inject.row, e.inject.mix, e.inject.table) for i, e in enumerate(spec.schedule) if e.inject is not None]
    assert marks == [(1, 0, "loop.in", "loop.step"), (3, 1, "loop.in", "loop.step")]
    d = json.loads(json.dumps(CFG))
    del d["loop"]
    assert [e.layer for e in config_from_dict(d).model_spec().schedule] == [0, 1, 2, 3]
    assert P.layer_runs(CFG) == [(0, None), (1, 0), (2, None), (1, 1), (2, None), (3, None)]


def test_tensor_names_and_shapes():
    params = parameter_list(config_from_dict(CFG).model_spec())
    names = {p.name: p.shape for p in params}
    for n in ("embed", "bigram", "loop.in", "loop.step", "side.embed", "head", "final.norm", "final.norm.b", "l0.norm1", "l0.norm1.b",
              "l0.norm2.b", "l0.mix.left.q", "l0.mix.left.q.b", "l0.mix.left.k.b", "l0.mix.left.v.b", "l0.mix.left.o", "l0.mix.left.out",
              "l0.mix.right.q", "l0.mix.right.k", "l0.mix.right.v", "l0.mix.right.g", "l0.mix.right.o", "l0.mix.right.out", "l0.mlp.up",
              "l0.mlp.down", "l0.side.gate", "l0.side.proj", "l0.side.norm", "l1.mix.q.conv", "l1.mix.b", "l1.mix.A_log", "l1.mix.a1",
              "l1.mix.a2", "l1.mix.dt_bias", "l1.mix.g1", "l1.mix.g2", "l1.mix.norm", "l1.mlp.router", "l1.mlp.e5.down", "l2.norm2"):
        assert n in names, n
    for n in ("l0.mlp.gate", "l0.mlp.up.b", "l1.mlp.router.b", "l0.mix.left.o.b", "l1.mix.g", "l1.mix.a", "l2.mlp.up", "l0.mix.right.norm"):
        assert n not in names, n
    assert names["bigram"] == (54, 40) and names["loop.in"] == (40, 80) and names["loop.step"] == (2, 40)
    assert names["side.embed"] == (97, 24) and names["l0.side.gate"] == (6, 40) and names["l0.side.proj"] == (40, 6)
    assert names["l0.mix.left.q"] == (48, 40) and names["l0.mix.left.k"] == (24, 40) and names["l0.mix.left.v"] == (36, 40)
    assert names["l0.mix.left.o"] == (40, 72) and names["l0.mix.right.o"] == (40, 28)
    assert names["l1.mix.q"] == (20, 40) and names["l1.mix.v.conv"] == (84, 3) and names["l1.mix.a2"] == (60, 4)
    assert names["l1.mix.dt_bias"] == (60,) and names["l1.mix.g2"] == (84, 5) and names["l1.mix.A_log"] == (6,)
    assert not next(p for p in params if p.name == "l2.norm2").required
    check_tensors({k: v for k, v in names.items() if not k.startswith("l2.norm2")}, params, "file")
    # the ranks are the file's to give when the configuration does not name them
    d = json.loads(json.dumps(CFG))
    del d["layers"][1]["mixer"]["rank"], d["layers"][1]["mixer"]["gate_rank"]
    free = parameter_list(config_from_dict(d).model_spec())
    check_tensors(dict(names, **{"l1.mix.a1": (11, 40), "l1.mix.a2": (60, 11)}), free, "file")
    wrong = dict(names)
    wrong["l1.mix.k.conv"] = (20, 4)
    with pytest.raises(BadFormat, match="l1.mix.k.conv"):
        check_tensors(wrong, params, "file")


def test_random_weights_folder_and_the_plain_model_reads_it(tmp_path):
    folder = write_model_folder(tmp_path / "m", config_from_dict(CFG), 1, torch.float32)
    d = json.loads((folder / "config.json").read_text())
    assert d["layers"][2]["mlp"] is None and d["loop"] == CFG["loop"]
    cfg, w = P.load(folder)
    t = np.random.RandomState(0).randint(0, 97, size=24)
    logits, streams = P.forward(cfg, w, t, return_streams=True)
    assert logits.shape == (24, 97) and len(streams) == 6 and np.isfinite(logits).all()
    # causal: what comes later changes nothing earlier; the token after the changed one sees it through the pair table
    t2 = t.copy()
    t2[17] = (t2[17] + 1) % 97
    again = P.forward(cfg, w, t2)
    assert np.array_equal(again[:17], logits[:17]) and not np.allclose(again[17:], logits[17:])


def test_plain_router_keeps_to_the_best_groups():
    router = {"experts": 6, "top": 2, "scale": 2.0, "groups": {"count": 3, "keep": 1}}
    chosen, weights = P.route(np.array([0.0, 5.0, 4.9, 4.8, 1.0, 3.0]), router)
    assert chosen.tolist() == [1, 0] and abs(weights.sum() - 2.0) < 1e-12      # the best group is experts 0 and 1 (its best score is 5)
    chosen, weights = P.route(np.array([0.0, 5.0, 4.9, 4.8, 1.0, 3.0]), {"experts": 6, "top": 2})
    assert chosen.tolist() == [1, 2] and abs(weights.sum() - 1.0) < 1e-12


@pytest.mark.parametrize("change,error", [
    (lambda d: d["layers"][0].update(type="conv"), UnsupportedModel),
    (lambda d: d["layers"][0]["mlp"].update(kind="gated"), UnsupportedModel),
    (lambda d: d["layers"][0]["mixer"]["left"].update(kv_heads=4), BadFormat),
    (lambda d: d["layers"][0]["mixer"]["left"]["rot"].update(dims=5), BadFormat),
    (lambda d: d["layers"][0]["mixer"]["left"]["rot"].update(dims=10), BadFormat),
    (lambda d: d["layers"][0]["mixer"]["right"].update(decay=[0.9]), BadFormat),
    (lambda d: d["layers"][0]["mixer"]["right"].update(decay=[0.9, 1.5]), BadFormat),
    (lambda d: d["layers"][0]["mixer"].pop("right"), BadFormat),
    (lambda d: d["layers"][1]["mixer"].update(kv_heads=4), BadFormat),
    (lambda d: d["layers"][1]["mixer"].pop("conv"), BadFormat),
    (lambda d: d["layers"][1]["mlp"]["router"].update(top=7), BadFormat),
    (lambda d: d["layers"][1]["mlp"]["router"]["groups"].update(count=4), BadFormat),
    (lambda d: d["layers"][1]["mlp"]["router"]["groups"].update(keep=1, count=6), BadFormat),
    (lambda d: d["loop"].update(stop=5), BadFormat),
    (lambda d: d["loop"].update(start=3, stop=3), BadFormat),
    (lambda d: d["embedding"]["bigram"].pop("buckets"), BadFormat),
    (lambda d: d.pop("norm"), BadFormat),
    (lambda d: d.update(layers=[]), BadFormat),
])
def test_refusals(change, error):
    d = json.loads(json.dumps(CFG))
    change(d)
    with pytest.raises(error):
        config_from_dict(d).model_spec()


def test_cache_keeps_pages_for_the_softmax_side_and_state_rows_for_the_recurrences():
    """A pair of mixers is one cache user with both: key and value pages of the windowed softmax side (given back as the
    window moves on) and the retention state; a channel-delta layer keeps one row of 32-bit state (every head's S, then the
    convolutions' last inputs)."""
    spec = config_from_dict(CFG).model_spec()
    blocks = [base.build("block", b) for b in spec.layers]
    reqs = [blocks[e.layer].cache_requests()[0] for e in spec.schedule]
    assert len(reqs) == 6
    kv0, st0 = reqs[0]
    assert (kv0.n_kv_heads, kv0.head_dim, kv0.v_head_dim, kv0.window) == (3, 8, 12, 9) and st0.shape == (2, 10, 14)
    kv1, st1 = reqs[1]
    C = 2 * 2 * 10 + 6 * 14
    assert kv1 is None and st1.shape == (6 * 10 * 14 + 2 * C,) and st1.dtype == torch.float32
    assert reqs[3] == reqs[1] and reqs[2] == reqs[4] and reqs[2][0].window == 0
    cache = Cache(reqs + [(None, base.StateRequest((1,), torch.int32))], [None] * 7, 64 * 4, torch.float32, "cpu")
    s = cache.alloc_slot()
    cache.prepare([s], [80])
    cache.commit([s], [80])
    windowed = [g for g in cache.groups if g.request.window]
    assert len(windowed) == 1 and windowed[0].pool.n_held == 1          # the first page is out of every later query's sight
    assert cache.states[-1].dtype == torch.int32 and cache.states[-1].shape == (cache.n_slots + 1, 1)
    cache.check()
    cache.free_slot(s)
    assert all(g.pool.n_held == 0 for g in cache.groups)
