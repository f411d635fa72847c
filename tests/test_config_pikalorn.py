"""Pikalorn's configuration on the CPU: the keys of its ``config.json``, the registry's choice by the
``architecture`` key, the schedule of layers that read another layer's cache, the tensors its parts ask for, what
the cache keeps for latent layers and for the recurrent mixer, and the plain model's own consistency (a prompt cut
in two gives what the whole gives)."""
import json

import numpy as np
import pytest
import torch

import plain_pikalorn as P
from nncpu_b200.cache import Cache
from nncpu_b200.config import PikalornConfig, config_from_dict
from nncpu_b200.engine.model import parameter_list
from nncpu_b200.errors import BadFormat, UnsupportedModel
from nncpu_b200.parts import base
from nncpu_b200.weights import check_tensors, write_model_folder

ROT = {"base": 777.0, "dims": 6, "scaling": {"factor": 8.0, "original": 64.0, "fast": 16.0, "slow": 2.0}}
CFG = {"architecture": "Pikalorn", "vocab": 97, "width": 40, "norm": {"eps": 2e-6}, "embedding": {"scale": 5.0},
       "layers": [{"type": "latent_attention", "mlp": {"kind": "dense", "ff": 72},
                   "mixer": {"heads": 2, "dim": 12, "rot_dim": 6, "vdim": 20, "kv_rank": 28, "q_rank": 18, "scale": 0.3,
                             "rot": ROT}},
                  {"type": "delta", "mlp": None, "mixer": {"heads": 6, "kv_heads": 2, "dim": 10, "vdim": 14, "conv": 3}},
                  {"type": "attention", "mlp": {"kind": "dense", "ff": 24},
                   "mixer": {"heads": 6, "kv_heads": 3, "dim": 8, "vdim": 8, "scale": 0.25, "rot": {"base": 1234.0, "dims": 6}}},
                  {"type": "latent_attention", "mlp": None,
                   "mixer": {"heads": 3, "dim": 4, "rot_dim": 6, "vdim": 10, "kv_rank": 28, "q_rank": 7, "scale": 0.4,
                             "rot": ROT, "kv_from": 0}}]}


def test_keys_round_trip_and_specs():
    cfg = config_from_dict(CFG)
    assert isinstance(cfg, PikalornConfig)
    assert config_from_dict(cfg.to_dict()) == cfg and cfg.to_dict() == CFG
    spec = cfg.model_spec()
    l, d, a, z = spec.layers
    assert {x.kind for x in spec.layers} == {"parallel"} and all(x.norm2 is None for x in spec.layers)
    assert d.feed_forward is None and z.feed_forward is None and a.feed_forward.activation == "silu"
    m = l.mixer
    assert (m.n_heads, m.head_dim, m.rot_dim, m.v_head_dim, m.latent_dim, m.q_rank, m.sink) == (2, 12, 6, 20, 28, 18, True)
    assert (m.position.kind, m.position.theta, m.position.rotary_dim) == ("rope_pairs", 777.0, 6)
    assert (m.position.scaling_factor, m.position.scaling_original, m.position.scaling_fast, m.position.scaling_slow) == (8.0, 64.0, 16.0, 2.0)
    m = d.mixer
    assert (m.kind, m.n_heads, m.n_kv_heads, m.key_dim, m.value_dim, m.conv, m.eps) == ("gated_delta", 6, 2, 10, 14, 3, 2e-6)
    m = a.mixer
    assert (m.n_heads, m.n_kv_heads, m.head_dim, m.scale) == (6, 3, 8, 0.25)
    assert m.values_are_keys and m.sink and m.out_gate and m.out_bias and m.qkv_bias and m.qk_norm.eps == 2e-6
    assert (m.position.kind, m.position.rotary_dim, m.position.scaling_factor) == ("rope_neox", 6, 0.0)
    assert spec.embedding.scale == 5.0 and not spec.output.tied


def test_a_layer_that_reads_another_layers_cache_is_in_the_schedule():
    spec = config_from_dict(CFG).model_spec()
    assert [(e.layer, e.cache_of) for e in spec.schedule] == [(0, None), (1, None), (2, None), (3, 0)]


def test_tensor_names_and_shapes():
    params = parameter_list(config_from_dict(CFG).model_spec())
    names = {p.name: p.shape for p in params}
    for n in ("embed", "head", "final.norm", "l0.norm1", "l0.mix.dq", "l0.mix.dq.norm", "l0.mix.uq", "l0.mix.dkv",
              "l0.mix.dkv.norm", "l0.mix.uk", "l0.mix.uv", "l0.mix.sink", "l0.mix.o", "l0.mlp.gate", "l0.mlp.up", "l0.mlp.down",
              "l1.mix.q", "l1.mix.q.conv", "l1.mix.k", "l1.mix.k.conv", "l1.mix.v", "l1.mix.v.conv", "l1.mix.b", "l1.mix.a",
              "l1.mix.A_log", "l1.mix.dt_bias", "l1.mix.g", "l1.mix.norm", "l1.mix.o", "l2.mix.q", "l2.mix.q.b", "l2.mix.k",
              "l2.mix.k.b", "l2.mix.q.norm", "l2.mix.k.norm", "l2.mix.sink", "l2.mix.g", "l2.mix.o", "l2.mix.o.b", "l3.mix.dq",
              "l3.mix.uk", "l3.mix.uv", "l3.mix.sink"):
        assert n in names, n
    for n in ("l0.norm2", "l1.mlp.gate", "l2.mix.v", "l2.mix.v.b", "l3.mix.dkv", "l3.mix.dkv.norm", "l2.mix.g.b"):
        assert n not in names, n
    assert names["l0.mix.dkv"] == (34, 40) and names["l0.mix.dkv.norm"] == (28,) and names["l0.mix.uq"] == (36, 18)
    assert names["l0.mix.uk"] == (24, 28) and names["l0.mix.uv"] == (40, 28) and names["l3.mix.uq"] == (30, 7)
    assert names["l1.mix.q"] == (20, 40) and names["l1.mix.v.conv"] == (84, 3) and names["l1.mix.b"] == (6, 40)
    assert names["l1.mix.norm"] == (14,) and names["l2.mix.k"] == (24, 40) and names["l2.mix.g"] == (48, 40)
    assert names["l2.mix.sink"] == (6,) and names["l2.mix.q.norm"] == (8,)
    check_tensors(dict(names), params, "file")
    wrong = dict(names)
    wrong["l1.mix.k.conv"] = (20, 4)
    with pytest.raises(BadFormat, match="l1.mix.k.conv"):
        check_tensors(wrong, params, "file")


def test_random_weights_folder_and_the_plain_model_reads_it(tmp_path):
    folder = write_model_folder(tmp_path / "m", config_from_dict(CFG), 1, torch.float32)
    d = json.loads((folder / "config.json").read_text())
    assert d["layers"][3]["mixer"]["kv_from"] == 0 and d["layers"][1]["mlp"] is None
    cfg, w = P.load(folder)
    t = np.random.RandomState(0).randint(0, 97, size=24)
    logits, streams = P.forward(cfg, w, t, return_streams=True)
    assert logits.shape == (24, 97) and streams.shape == (4, 24, 40) and np.isfinite(logits).all()
    # causal: what comes later changes nothing earlier
    t2 = t.copy()
    t2[17] = (t2[17] + 1) % 97
    again = P.forward(cfg, w, t2)
    assert np.array_equal(again[:17], logits[:17]) and not np.allclose(again[17:], logits[17:])


@pytest.mark.parametrize("change,error", [
    (lambda d: d["layers"][0].update(type="conv"), UnsupportedModel),
    (lambda d: d["layers"][0]["mlp"].update(kind="moe"), UnsupportedModel),
    (lambda d: d["layers"][2]["mixer"].update(kv_heads=4), BadFormat),
    (lambda d: d["layers"][2]["mixer"].update(vdim=12), BadFormat),
    (lambda d: d["layers"][2]["mixer"]["rot"].update(dims=5), BadFormat),
    (lambda d: d["layers"][2]["mixer"]["rot"].update(dims=10), BadFormat),
    (lambda d: d["layers"][1]["mixer"].update(kv_heads=4), BadFormat),
    (lambda d: d["layers"][1]["mixer"].pop("conv"), BadFormat),
    (lambda d: d["layers"][0]["mixer"].pop("kv_rank"), BadFormat),
    (lambda d: d["layers"][0]["mixer"]["rot"]["scaling"].pop("slow"), BadFormat),
    (lambda d: d["layers"][3]["mixer"].update(kv_from=3), BadFormat),
    (lambda d: d["layers"][3]["mixer"].update(kv_from=2), BadFormat),
    (lambda d: d["layers"][3]["mixer"].update(kv_rank=20), BadFormat),
    (lambda d: d.pop("norm"), BadFormat),
    (lambda d: d.update(layers=[]), BadFormat),
])
def test_refusals(change, error):
    d = json.loads(json.dumps(CFG))
    change(d)
    with pytest.raises(error):
        config_from_dict(d).model_spec()


def test_cache_keeps_one_row_for_latent_layers_and_a_state_row_for_the_recurrence():
    """What the blocks ask of the cache: the first latent layer one key head of latent + rotated lanes with no value
    pages of its own, the recurrent layer no pages and one row of 32-bit state per slot (every head's S, then the
    convolutions' last inputs), the attention layer key and value pages (a value is the key before its norm and rotation, so
    both are kept), and the layer that reads another's cache nothing."""
    spec = config_from_dict(CFG).model_spec()
    blocks = [base.build("block", b, **({"reads_other_cache": True} if e.cache_of is not None else {}))
              for b, e in zip(spec.layers, spec.schedule)]
    reqs = [b.cache_requests()[0] for b in blocks]
    (kv0, st0), (kv1, st1), (kv2, st2), (kv3, st3) = reqs
    assert (kv0.n_kv_heads, kv0.head_dim, kv0.keys_only) == (1, 34, True) and st0 is None
    C = 2 * 2 * 10 + 6 * 14
    assert kv1 is None and st1.shape == (6 * 10 * 14 + 2 * C,) and st1.dtype == torch.float32
    assert (kv2.n_kv_heads, kv2.head_dim, kv2.keys_only) == (3, 8, False) and st2 is None
    assert kv3 is None and st3 is None
    cache = Cache(reqs, [None, None, None, 0], 64 * 4, torch.float32, "cpu")
    s = cache.alloc_slot()
    cache.prepare([s], [70])
    cache.commit([s], [70])
    assert sum(g.v is g.k for g in cache.groups) == 1 and sum(g.pool.n_held for g in cache.groups) == 2 * len(cache.groups)
    cache.check()
    cache.free_slot(s)
    assert all(g.pool.n_held == 0 for g in cache.groups)
