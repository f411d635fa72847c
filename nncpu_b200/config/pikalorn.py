"""Pikalorn: a decoder whose ``config.json`` lists its layers one by one.

Every layer is a "parallel" block with ONE norm: h = norm1(x), x += mixer(h) + feed_forward(h).  The mixer is one of

* ``attention``: grouped-query softmax attention with biases on q, k and the output, a per-head RMS norm of q and k,
  a (possibly partial) half-split rotation, values that are the keys as projected, a learned sink logit per head in
  the softmax's denominator, and a sigmoid gate on the concatenated heads;
* ``latent_attention``: queries through a normed latent; one normed latent per position from which every head's
  unrotated key part and value are made, plus one rotated key part shared by all heads (rotation of neighbouring
  lanes, optionally with frequencies rescaled between two wavelengths); a sink; with ``kv_from`` the layer reads an
  earlier latent layer's cache instead of keeping one;
* ``delta``: the gated delta rule with short convolutions (a state per sequence instead of keys and values).

The feed-forward is gated with SiLU, or absent.  The embedding rows are scaled.

``config.json``::

    {"architecture": "Pikalorn", "vocab": V, "width": W, "norm": {"eps": e}, "embedding": {"scale": s},
     "layers": [{"type": "attention",
                 "mixer": {"heads", "kv_heads", "dim", "vdim", "scale", "rot": {"base", "dims"}},
                 "mlp": {"kind": "dense", "ff": F}},
                {"type": "latent_attention",
                 "mixer": {"heads", "dim", "rot_dim", "vdim", "kv_rank", "q_rank", "scale", "kv_from": j,
                           "rot": {"base", "dims", "scaling": {"factor", "original", "fast", "slow"}}}, "mlp": ...},
                {"type": "delta", "mixer": {"heads", "kv_heads", "dim", "vdim", "conv"}, "mlp": null}, ...]}

Tensor names: ``embed``, ``final.norm``, ``head`` and per layer i ``l<i>.norm1``, ``l<i>.mix.*``, ``l<i>.mlp.*``.
"""
from __future__ import annotations

import math
from dataclasses import dataclass, field
from typing import List, Optional, Tuple

from ..errors import BadFormat, UnsupportedModel
from .registry import register_architecture
from .specs import (AttentionSpec, BlockSpec, EmbeddingSpec, GatedDeltaSpec, GatedMlpSpec, LatentAttentionSpec,
                    ModelSpec, NormSpec, OutputSpec, PositionSpec, ScheduleEntry)


def _int(d: dict, key: str, where: str, minimum: int = 1) -> int:
    v = d.get(key)
    if isinstance(v, bool) or not isinstance(v, int):
        raise BadFormat(f'config.json: {where} needs an integer "{key}", not {v!r}')
    if v < minimum:
        raise BadFormat(f'config.json: {where}: "{key}" is {v}, expected at least {minimum}')
    return v


def _num(d: dict, key: str, where: str) -> float:
    v = d.get(key)
    if isinstance(v, bool) or not isinstance(v, (int, float)) or not math.isfinite(v) or v <= 0:
        raise BadFormat(f'config.json: {where} needs a positive number "{key}", not {v!r}')
    return float(v)


def _obj(d: dict, key: str, where: str) -> dict:
    v = d.get(key)
    if not isinstance(v, dict):
        raise BadFormat(f'config.json: {where} needs an object "{key}", not {v!r}')
    return v


@dataclass(frozen=True)
class PikalornRotation:
    """A mixer's ``rot``: ``dims`` lanes of a head turn, pair i by position * base^(-2i/dims); ``factor`` > 0: the
    frequencies are rescaled between the wavelengths that make ``fast`` and ``slow`` turns over ``original`` positions."""
    base: float
    dims: int
    factor: float = 0.0
    original: float = 0.0
    fast: float = 0.0
    slow: float = 0.0

    @classmethod
    def from_dict(cls, d: dict, where: str, lanes: int) -> "PikalornRotation":
        base, dims = _num(d, "base", where), _int(d, "dims", where, minimum=2)
        if dims % 2 or dims > lanes:
            raise BadFormat(f"config.json: {where} turns {dims} of {lanes} lanes: an even number of at most all of them "
                            "is needed")
        if base == 1.0:
            raise BadFormat(f"config.json: {where}: a base of 1 has no frequencies")
        if d.get("scaling") is None:
            return cls(base, dims)
        sc = _obj(d, "scaling", where)
        w = f"{where}.scaling"
        return cls(base, dims, _num(sc, "factor", w), _num(sc, "original", w), _num(sc, "fast", w), _num(sc, "slow", w))

    def to_dict(self) -> dict:
        d = {"base": self.base, "dims": self.dims}
        if self.factor:
            d["scaling"] = {"factor": self.factor, "original": self.original, "fast": self.fast, "slow": self.slow}
        return d

    def spec(self, kind: str) -> PositionSpec:
        return PositionSpec(kind, self.base, self.dims, scaling_factor=self.factor, scaling_original=self.original,
                            scaling_fast=self.fast, scaling_slow=self.slow)


@dataclass(frozen=True)
class PikalornLayer:
    """One entry of ``layers``, checked.  ``ff`` 0: no feed-forward.  ``kv_from`` -1: a cache of its own."""
    type: str
    heads: int
    dim: int
    vdim: int
    kv_heads: int = 0
    scale: float = 0.0
    rot: Optional[PikalornRotation] = None
    rot_dim: int = 0
    kv_rank: int = 0
    q_rank: int = 0
    kv_from: int = -1
    conv: int = 0
    ff: int = 0

    @classmethod
    def from_dict(cls, i: int, d: dict) -> "PikalornLayer":
        where = f"layers[{i}]"
        if not isinstance(d, dict):
            raise BadFormat(f"config.json: {where} is not an object")
        kind = d.get("type")
        m = _obj(d, "mixer", where)
        mw = f"{where}.mixer"
        heads, dim, vdim = _int(m, "heads", mw), _int(m, "dim", mw), _int(m, "vdim", mw)
        ff = 0
        if d.get("mlp") is not None:
            mlp = _obj(d, "mlp", where)
            if mlp.get("kind") != "dense":
                raise UnsupportedModel(f'config.json: {where}.mlp has "kind": {mlp.get("kind")!r} (supported: "dense")')
            ff = _int(mlp, "ff", f"{where}.mlp")
        if kind == "attention":
            kv = _int(m, "kv_heads", mw)
            if heads % kv:
                raise BadFormat(f"config.json: {mw}: {heads} heads are no multiple of {kv} key/value heads")
            if vdim != dim:
                raise BadFormat(f"config.json: {mw}: the values are the keys, so a value head has {dim} lanes, not {vdim}")
            rot = None if m.get("rot") is None else PikalornRotation.from_dict(_obj(m, "rot", mw), f"{mw}.rot", dim)
            return cls("attention", heads, dim, vdim, kv_heads=kv, scale=_num(m, "scale", mw), rot=rot, ff=ff)
        if kind == "latent_attention":
            rot_dim = _int(m, "rot_dim", mw, minimum=0) if m.get("rot_dim") is not None else 0
            rot = None
            if rot_dim:
                rot = PikalornRotation.from_dict(_obj(m, "rot", mw), f"{mw}.rot", rot_dim)
            kv_from = -1
            if m.get("kv_from") is not None:
                kv_from = _int(m, "kv_from", mw, minimum=0)
                if kv_from >= i:
                    raise BadFormat(f"config.json: {mw} reads the cache of layer {kv_from}, which is not an earlier layer")
            return cls("latent_attention", heads, dim, vdim, scale=_num(m, "scale", mw), rot=rot, rot_dim=rot_dim,
                       kv_rank=_int(m, "kv_rank", mw), q_rank=_int(m, "q_rank", mw), kv_from=kv_from, ff=ff)
        if kind == "delta":
            kv = _int(m, "kv_heads", mw)
            if heads % kv:
                raise BadFormat(f"config.json: {mw}: {heads} heads are no multiple of {kv} query/key heads")
            return cls("delta", heads, dim, vdim, kv_heads=kv, conv=_int(m, "conv", mw), ff=ff)
        raise UnsupportedModel(f'config.json: {where} has "type": {kind!r} (supported: "attention", '
                               '"latent_attention", "delta")')

    def to_dict(self) -> dict:
        if self.type == "attention":
            m = {"heads": self.heads, "kv_heads": self.kv_heads, "dim": self.dim, "vdim": self.vdim, "scale": self.scale}
            if self.rot is not None:
                m["rot"] = self.rot.to_dict()
        elif self.type == "latent_attention":
            m = {"heads": self.heads, "dim": self.dim, "rot_dim": self.rot_dim, "vdim": self.vdim,
                 "kv_rank": self.kv_rank, "q_rank": self.q_rank, "scale": self.scale}
            if self.rot is not None:
                m["rot"] = self.rot.to_dict()
            if self.kv_from >= 0:
                m["kv_from"] = self.kv_from
        else:
            m = {"heads": self.heads, "kv_heads": self.kv_heads, "dim": self.dim, "vdim": self.vdim, "conv": self.conv}
        return {"type": self.type, "mixer": m, "mlp": {"kind": "dense", "ff": self.ff} if self.ff else None}


@register_architecture("Pikalorn")
@dataclass
class PikalornConfig:
    vocab: int
    width: int
    norm_eps: float
    layers: Tuple[PikalornLayer, ...]
    embedding_scale: float = 1.0
    max_positions: int = 1 << 20  # rotary angles are computed, the recurrent state has no length: nothing runs out
    eos_token_id: Tuple[int, ...] = field(default_factory=tuple)

    @classmethod
    def from_dict(cls, d: dict) -> "PikalornConfig":
        layers = d.get("layers")
        if not isinstance(layers, list) or not layers:
            raise BadFormat('config.json needs a non-empty list "layers"')
        scale = 1.0
        if d.get("embedding") is not None:
            scale = _num(_obj(d, "embedding", "the model"), "scale", "embedding")
        eos = d.get("eos_token_id")
        eos = tuple(eos) if isinstance(eos, list) else (() if eos is None else (eos,))
        cfg = cls(vocab=_int(d, "vocab", "the model"), width=_int(d, "width", "the model"),
                  norm_eps=_num(_obj(d, "norm", "the model"), "eps", "norm"),
                  layers=tuple(PikalornLayer.from_dict(i, l) for i, l in enumerate(layers)), embedding_scale=scale,
                  max_positions=_int(d, "max_positions", "the model") if d.get("max_positions") is not None else 1 << 20,
                  eos_token_id=eos)
        for i, l in enumerate(cfg.layers):
            if l.kv_from >= 0:
                src = cfg.layers[l.kv_from]
                if src.type != "latent_attention" or src.kv_from >= 0:
                    raise BadFormat(f"config.json: layers[{i}] reads the cache of layer {l.kv_from}, which is not a "
                                    "latent-attention layer with a cache of its own")
                if (src.kv_rank, src.rot_dim, src.rot) != (l.kv_rank, l.rot_dim, l.rot):
                    raise BadFormat(f"config.json: layers[{i}] reads the cache of layer {l.kv_from}, whose latent size, "
                                    "rotated lanes or rotation differ from its own")
        for e in cfg.eos_token_id:
            if isinstance(e, bool) or not isinstance(e, int) or not 0 <= e < cfg.vocab:
                raise BadFormat(f'config.json: "eos_token_id" holds {e!r}')
        return cfg

    def to_dict(self) -> dict:
        d = {"architecture": self.architecture, "vocab": self.vocab, "width": self.width,
             "norm": {"eps": self.norm_eps}, "embedding": {"scale": self.embedding_scale},
             "layers": [l.to_dict() for l in self.layers]}
        if self.max_positions != 1 << 20:
            d["max_positions"] = self.max_positions
        if self.eos_token_id:
            d["eos_token_id"] = list(self.eos_token_id)
        return d

    def schedule(self) -> Tuple[ScheduleEntry, ...]:
        """Every layer once, in order; a layer with ``kv_from`` reads that layer's run."""
        return tuple(ScheduleEntry(i, cache_of=l.kv_from if l.kv_from >= 0 else None) for i, l in enumerate(self.layers))

    def model_spec(self) -> ModelSpec:
        w, eps = self.width, self.norm_eps

        def norm(name: str) -> NormSpec:
            return NormSpec("rmsnorm", w, eps, name, suffix="")

        blocks: List[BlockSpec] = []
        for i, l in enumerate(self.layers):
            p = f"l{i}"
            if l.type == "attention":
                mixer = AttentionSpec(kind="attention", name=f"{p}.mix", hidden_size=w, n_heads=l.heads,
                                      n_kv_heads=l.kv_heads, head_dim=l.dim, v_head_dim=l.vdim, scale=l.scale,
                                      qkv_bias=True, out_bias=True, values_are_keys=True, sink=True, out_gate=True,
                                      qk_norm=NormSpec("rmsnorm", l.dim, eps, f"{p}.mix", suffix=""),
                                      position=None if l.rot is None else l.rot.spec("rope_neox"),
                                      tensor_names="short")
            elif l.type == "latent_attention":
                mixer = LatentAttentionSpec(kind="latent_attention", name=f"{p}.mix", hidden_size=w, n_heads=l.heads,
                                            head_dim=l.dim, v_head_dim=l.vdim, latent_dim=l.kv_rank, scale=l.scale,
                                            eps=eps, rot_dim=l.rot_dim, q_rank=l.q_rank, sink=True,
                                            position=None if l.rot is None else l.rot.spec("rope_pairs"))
            else:
                mixer = GatedDeltaSpec(kind="gated_delta", name=f"{p}.mix", hidden_size=w, n_heads=l.heads,
                                       n_kv_heads=l.kv_heads, key_dim=l.dim, value_dim=l.vdim, conv=l.conv, eps=eps)
            ff = None
            if l.ff:
                ff = GatedMlpSpec(kind="gated_mlp", name=f"{p}.mlp", hidden_size=w, intermediate_size=l.ff,
                                  activation="silu", tensor_names="short")
            # one norm a layer: both sublayers read its output
            blocks.append(BlockSpec(kind="parallel", norm1=norm(f"{p}.norm1"), mixer=mixer, norm2=None, feed_forward=ff))
        return ModelSpec(
            architecture=self.architecture, hidden_size=w, vocab_size=self.vocab, max_positions=self.max_positions,
            embedding=EmbeddingSpec("embed", self.vocab, w, scale=self.embedding_scale, suffix=""),
            layers=tuple(blocks), schedule=self.schedule(),
            output=OutputSpec(norm=norm("final.norm"), name="head", tied=False, vocab_size=self.vocab, hidden_size=w,
                              suffix=""),
            stop_token_ids=tuple(self.eos_token_id))
