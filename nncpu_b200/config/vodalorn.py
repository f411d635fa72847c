"""Vodalorn: a decoder whose ``config.json`` lists its layers one by one and may run a range of them several times.

Every layer is a pre-norm block with a residual weight m: x += m * mixer(norm1(x)); x += m * feed_forward(norm2(x));
then a per-layer token input (``token_side``).  The norms are layer norms with weight and bias.  The mixer is one of

* ``parallel``: two mixers side by side on the same input, half the sum of their outputs, each RMS-normed over the
  width with a plain weight: sliding-window grouped-query softmax attention with biases on q, k, v, value heads of their
  own size and a half-split rotation of a head's first ``rot.dims`` lanes; and retention (linear attention with a fixed
  decay per head, rotated q and k, per-head RMS norm, a SiLU gate);
* ``channel_delta``: the gated delta rule with short convolutions, a decay per head and key channel through a low
  rank, and a sigmoid output gate through a low rank.

The feed-forward is dense with the square of relu, or routed experts (softmax over all experts, the choice limited to
the best groups, weights renormalised and scaled; clamped gated experts), or absent.  The embedding adds a hashed
embedding of the pair (previous token, token).  ``loop`` names a range of layers that runs ``times`` times in a row with
the same weights and a cache per pass; before every pass the stream becomes ``loop.in`` [x; x0] (x0 the embedding
output) plus row t of ``loop.step``.  The output is the model's norm and the matrix ``head``.

``config.json``::

    {"architecture": "Vodalorn", "vocab": V, "width": W, "norm": {"eps": e}, "residual_mult": m,
     "embedding": {"bigram": {"buckets": B, "mul_prev": a, "mul_cur": b}}, "token_side": {"dim": D},
     "loop": {"start": a, "stop": b, "times": n},
     "layers": [{"type": "parallel",
                 "mixer": {"left": {"heads", "kv_heads", "dim", "vdim", "scale", "mask": {"size"}, "rot": {"base", "dims"}},
                           "right": {"heads", "dim", "vdim", "decay": [..], "rot": {"base", "dims"}}},
                 "mlp": {"kind": "dense", "ff": F}},
                {"type": "channel_delta", "mixer": {"heads", "kv_heads", "dim", "vdim", "conv"},
                 "mlp": {"kind": "moe", "expert": {"ff", "limit"},
                         "router": {"experts", "top", "scale", "groups": {"count", "keep"}}}}, ...]}

``embedding``, ``token_side``, ``loop``, ``mask``, ``rot``, ``groups`` and a layer's ``mlp`` may be absent (or null).
The ranks of a ``channel_delta`` layer are what the file's tensors have (``mix.a1`` is [rank, width], ``mix.g1``
[gate rank, width]); a configuration that is to be filled with random weights names them as ``mixer.rank`` and
``mixer.gate_rank``.

Tensor names: ``embed``, ``bigram``, ``loop.in``, ``loop.step``, ``side.embed``, ``final.norm`` (+ ``.b``), ``head`` and
per layer i ``l<i>.norm1`` / ``norm2`` (+ ``.b``), ``l<i>.mix.*``, ``l<i>.mlp.*`` (experts ``.e<j>.gate / .up / .down``,
``.router``) and ``l<i>.side.gate / .proj / .norm``.
"""
from __future__ import annotations

import math
from dataclasses import dataclass, field
from typing import List, Optional, Tuple

from ..errors import BadFormat, UnsupportedModel
from .registry import register_architecture
from .specs import (AttentionSpec, BlockSpec, DenseMlpSpec, EmbeddingSpec, GatedDeltaSpec, MixerPairSpec, ModelSpec,
                    NormSpec, OutputSpec, PositionSpec, RetentionSpec, RoutedExpertsSpec, ScheduleEntry,
                    StreamInjection, TokenSideSpec)

LOOP_TABLE = "loop.step"
LOOP_MIX = "loop.in"
PAIR_TABLE = "bigram"
SIDE_TABLE = "side.embed"
PAIR_WEIGHT = 0.5       # the two mixers of a "parallel" layer: half the sum of their normed outputs


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


def _rot(m: dict, dim: int, where: str) -> Tuple[float, int]:
    """(base, dims) of a mixer's ``rot`` entry; (0, 0) without one."""
    if m.get("rot") is None:
        return 0.0, 0
    rot = _obj(m, "rot", where)
    base, dims = _num(rot, "base", f"{where}.rot"), _int(rot, "dims", f"{where}.rot", minimum=2)
    if dims % 2 or dims > dim:
        raise BadFormat(f"config.json: {where}.rot turns {dims} of a head's {dim} lanes: an even number of at most all "
                        "of them is needed")
    return base, dims


@dataclass(frozen=True)
class VodalornMlp:
    """A layer's feed-forward, checked.  ``kind`` "dense": ``ff``.  ``kind`` "moe": ``ff`` and ``limit`` of an expert;
    ``experts``, ``top`` and ``scale`` of the router, and its groups (``groups`` 0: none)."""
    kind: str
    ff: int
    limit: float = 0.0
    experts: int = 0
    top: int = 0
    scale: float = 1.0
    groups: int = 0
    keep: int = 0

    @classmethod
    def from_dict(cls, d, where: str) -> Optional["VodalornMlp"]:
        if d is None:
            return None
        if not isinstance(d, dict):
            raise BadFormat(f"config.json: {where} is neither null nor an object")
        kind = d.get("kind")
        if kind == "dense":
            return cls("dense", _int(d, "ff", where))
        if kind == "moe":
            ex, ro = _obj(d, "expert", where), _obj(d, "router", where)
            experts, top = _int(ro, "experts", f"{where}.router"), _int(ro, "top", f"{where}.router")
            if top > experts:
                raise BadFormat(f"config.json: {where}.router takes the top {top} of {experts} experts")
            scale = 1.0 if ro.get("scale") is None else _num(ro, "scale", f"{where}.router")
            groups = keep = 0
            if ro.get("groups") is not None:
                g = _obj(ro, "groups", f"{where}.router")
                groups, keep = _int(g, "count", f"{where}.router.groups"), _int(g, "keep", f"{where}.router.groups")
                if experts % groups or keep > groups or keep * (experts // groups) < top:
                    raise BadFormat(f"config.json: {where}.router: the {keep} best of {groups} groups of {experts} "
                                    f"experts cannot give the top {top}")
            return cls("moe", _int(ex, "ff", f"{where}.expert"), _num(ex, "limit", f"{where}.expert"), experts, top,
                       scale, groups, keep)
        raise UnsupportedModel(f'config.json: {where} has "kind": {kind!r} (supported: "dense", "moe")')

    def to_dict(self) -> dict:
        if self.kind == "dense":
            return {"kind": "dense", "ff": self.ff}
        ro = {"experts": self.experts, "top": self.top, "scale": self.scale}
        if self.groups:
            ro["groups"] = {"count": self.groups, "keep": self.keep}
        return {"kind": "moe", "expert": {"ff": self.ff, "limit": self.limit}, "router": ro}


@dataclass(frozen=True)
class VodalornAttention:
    """The softmax side of a "parallel" layer.  ``window`` 0: every earlier key; ``rot_dims`` 0: no rotation."""
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    window: int = 0
    rot_base: float = 0.0
    rot_dims: int = 0

    @classmethod
    def from_dict(cls, m: dict, where: str) -> "VodalornAttention":
        heads, kv = _int(m, "heads", where), _int(m, "kv_heads", where)
        if heads % kv:
            raise BadFormat(f"config.json: {where}: {heads} heads are no multiple of {kv} key/value heads")
        dim = _int(m, "dim", where)
        window = 0 if m.get("mask") is None else _int(_obj(m, "mask", where), "size", f"{where}.mask")
        base, dims = _rot(m, dim, where)
        return cls(heads, kv, dim, _int(m, "vdim", where), _num(m, "scale", where), window, base, dims)

    def to_dict(self) -> dict:
        m = {"heads": self.heads, "kv_heads": self.kv_heads, "dim": self.dim, "vdim": self.vdim, "scale": self.scale}
        if self.window:
            m["mask"] = {"size": self.window}
        if self.rot_dims:
            m["rot"] = {"base": self.rot_base, "dims": self.rot_dims}
        return m


@dataclass(frozen=True)
class VodalornRetention:
    """The recurrent side of a "parallel" layer: one decay per head."""
    heads: int
    dim: int
    vdim: int
    decay: Tuple[float, ...]
    rot_base: float = 0.0
    rot_dims: int = 0

    @classmethod
    def from_dict(cls, m: dict, where: str) -> "VodalornRetention":
        heads, dim = _int(m, "heads", where), _int(m, "dim", where)
        decay = m.get("decay")
        if (not isinstance(decay, list) or len(decay) != heads
                or any(isinstance(a, bool) or not isinstance(a, (int, float)) or not 0.0 <= a <= 1.0 for a in decay)):
            raise BadFormat(f'config.json: {where} needs "decay": a list of {heads} numbers from 0 to 1, not {decay!r}')
        base, dims = _rot(m, dim, where)
        return cls(heads, dim, _int(m, "vdim", where), tuple(float(a) for a in decay), base, dims)

    def to_dict(self) -> dict:
        m = {"heads": self.heads, "dim": self.dim, "vdim": self.vdim, "decay": list(self.decay)}
        if self.rot_dims:
            m["rot"] = {"base": self.rot_base, "dims": self.rot_dims}
        return m


@dataclass(frozen=True)
class VodalornDelta:
    """A "channel_delta" mixer.  ``rank`` / ``gate_rank`` 0: taken from the file's tensors."""
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    conv: int
    rank: int = 0
    gate_rank: int = 0

    @classmethod
    def from_dict(cls, m: dict, where: str) -> "VodalornDelta":
        heads, kv = _int(m, "heads", where), _int(m, "kv_heads", where)
        if heads % kv:
            raise BadFormat(f"config.json: {where}: {heads} heads are no multiple of {kv} query/key heads")
        return cls(heads, kv, _int(m, "dim", where), _int(m, "vdim", where), _int(m, "conv", where),
                   0 if m.get("rank") is None else _int(m, "rank", where),
                   0 if m.get("gate_rank") is None else _int(m, "gate_rank", where))

    def to_dict(self) -> dict:
        m = {"heads": self.heads, "kv_heads": self.kv_heads, "dim": self.dim, "vdim": self.vdim, "conv": self.conv}
        if self.rank:
            m["rank"] = self.rank
        if self.gate_rank:
            m["gate_rank"] = self.gate_rank
        return m


@dataclass(frozen=True)
class VodalornLayer:
    """One entry of ``layers``, checked: ``type`` "parallel" (``left`` and ``right``) or "channel_delta" (``delta``)."""
    type: str
    left: Optional[VodalornAttention] = None
    right: Optional[VodalornRetention] = None
    delta: Optional[VodalornDelta] = None
    mlp: Optional[VodalornMlp] = None

    @classmethod
    def from_dict(cls, i: int, d: dict) -> "VodalornLayer":
        where = f"layers[{i}]"
        if not isinstance(d, dict):
            raise BadFormat(f"config.json: {where} is not an object")
        kind = d.get("type")
        m = _obj(d, "mixer", where)
        mlp = VodalornMlp.from_dict(d.get("mlp"), f"{where}.mlp")
        if kind == "parallel":
            return cls("parallel", left=VodalornAttention.from_dict(_obj(m, "left", f"{where}.mixer"), f"{where}.mixer.left"),
                       right=VodalornRetention.from_dict(_obj(m, "right", f"{where}.mixer"), f"{where}.mixer.right"), mlp=mlp)
        if kind == "channel_delta":
            return cls("channel_delta", delta=VodalornDelta.from_dict(m, f"{where}.mixer"), mlp=mlp)
        raise UnsupportedModel(f'config.json: {where} has "type": {kind!r} (supported: "parallel", "channel_delta")')

    def to_dict(self) -> dict:
        if self.type == "parallel":
            m = {"left": self.left.to_dict(), "right": self.right.to_dict()}
        else:
            m = self.delta.to_dict()
        return {"type": self.type, "mixer": m, "mlp": None if self.mlp is None else self.mlp.to_dict()}


@register_architecture("Vodalorn")
@dataclass
class VodalornConfig:
    vocab: int
    width: int
    norm_eps: float
    layers: Tuple[VodalornLayer, ...]
    residual_mult: float = 1.0
    pair_buckets: int = 0        # 0: no embedding of token pairs
    pair_mul_prev: int = 0
    pair_mul_cur: int = 0
    side_dim: int = 0            # 0: no per-layer token input
    loop_start: int = 0
    loop_stop: int = 0
    loop_times: int = 1
    has_loop: bool = False
    max_positions: int = 1 << 20  # the design has no table of positions: rotary angles are computed, nothing runs out
    eos_token_id: Tuple[int, ...] = field(default_factory=tuple)

    @classmethod
    def from_dict(cls, d: dict) -> "VodalornConfig":
        layers = d.get("layers")
        if not isinstance(layers, list) or not layers:
            raise BadFormat('config.json needs a non-empty list "layers"')
        buckets = mul_prev = mul_cur = 0
        if d.get("embedding") is not None and _obj(d, "embedding", "the model").get("bigram") is not None:
            bg = _obj(d["embedding"], "bigram", "embedding")
            buckets = _int(bg, "buckets", "embedding.bigram")
            mul_prev = _int(bg, "mul_prev", "embedding.bigram", minimum=0)
            mul_cur = _int(bg, "mul_cur", "embedding.bigram", minimum=0)
        side_dim = 0
        if d.get("token_side") is not None:
            side_dim = _int(_obj(d, "token_side", "the model"), "dim", "token_side")
        start = stop = 0
        times, has_loop = 1, False
        if d.get("loop") is not None:
            lp = _obj(d, "loop", "the model")
            start, stop = _int(lp, "start", "loop", minimum=0), _int(lp, "stop", "loop", minimum=0)
            times, has_loop = _int(lp, "times", "loop"), True
            if not start < stop <= len(layers):
                raise BadFormat(f"config.json: loop runs layers {start} to {stop - 1} of {len(layers)}")
        mult = 1.0 if d.get("residual_mult") is None else _num(d, "residual_mult", "the model")
        eos = d.get("eos_token_id")
        eos = tuple(eos) if isinstance(eos, list) else (() if eos is None else (eos,))
        cfg = cls(vocab=_int(d, "vocab", "the model"), width=_int(d, "width", "the model"),
                  norm_eps=_num(_obj(d, "norm", "the model"), "eps", "norm"),
                  layers=tuple(VodalornLayer.from_dict(i, l) for i, l in enumerate(layers)), residual_mult=mult,
                  pair_buckets=buckets, pair_mul_prev=mul_prev, pair_mul_cur=mul_cur, side_dim=side_dim,
                  loop_start=start, loop_stop=stop, loop_times=times, has_loop=has_loop,
                  max_positions=_int(d, "max_positions", "the model") if d.get("max_positions") is not None else 1 << 20,
                  eos_token_id=eos)
        for e in cfg.eos_token_id:
            if isinstance(e, bool) or not isinstance(e, int) or not 0 <= e < cfg.vocab:
                raise BadFormat(f'config.json: "eos_token_id" holds {e!r}')
        return cfg

    def to_dict(self) -> dict:
        d = {"architecture": self.architecture, "vocab": self.vocab, "width": self.width,
             "norm": {"eps": self.norm_eps}, "residual_mult": self.residual_mult,
             "layers": [l.to_dict() for l in self.layers]}
        if self.pair_buckets:
            d["embedding"] = {"bigram": {"buckets": self.pair_buckets, "mul_prev": self.pair_mul_prev,
                                         "mul_cur": self.pair_mul_cur}}
        if self.side_dim:
            d["token_side"] = {"dim": self.side_dim}
        if self.has_loop:
            d["loop"] = {"start": self.loop_start, "stop": self.loop_stop, "times": self.loop_times}
        if self.max_positions != 1 << 20:
            d["max_positions"] = self.max_positions
        if self.eos_token_id:
            d["eos_token_id"] = list(self.eos_token_id)
        return d

    def schedule(self) -> Tuple[ScheduleEntry, ...]:
        """The layers in running order.  The first layer of pass t of the loop carries what happens to the stream
        before that pass (the first too): it is mixed with the embedding output, and row t of ``loop.step`` is added."""
        n = len(self.layers)
        if not self.has_loop:
            return tuple(ScheduleEntry(i) for i in range(n))
        a, b, times = self.loop_start, self.loop_stop, self.loop_times
        runs: List[ScheduleEntry] = [ScheduleEntry(i) for i in range(a)]
        for t in range(times):
            for i in range(a, b):
                inject = StreamInjection(table=LOOP_TABLE, n_rows=times, row=t, mix=LOOP_MIX) if i == a else None
                runs.append(ScheduleEntry(i, inject=inject))
        return tuple(runs + [ScheduleEntry(i) for i in range(b, n)])

    def model_spec(self) -> ModelSpec:
        w, eps = self.width, self.norm_eps

        def norm(name: str) -> NormSpec:
            return NormSpec("layernorm", w, eps, name, suffix="")

        def rope(base: float, dims: int) -> Optional[PositionSpec]:
            return PositionSpec("rope_neox", base, dims) if dims else None

        blocks: List[BlockSpec] = []
        for i, l in enumerate(self.layers):
            p = f"l{i}"
            if l.type == "parallel":
                a, r = l.left, l.right
                left = AttentionSpec(kind="attention", name=f"{p}.mix.left", hidden_size=w, n_heads=a.heads,
                                     n_kv_heads=a.kv_heads, head_dim=a.dim, v_head_dim=a.vdim, qkv_bias=True,
                                     scale=a.scale, window=a.window, position=rope(a.rot_base, a.rot_dims),
                                     tensor_names="short")
                right = RetentionSpec(kind="retention", name=f"{p}.mix.right", hidden_size=w, n_heads=r.heads,
                                      key_dim=r.dim, value_dim=r.vdim, decays=r.decay,
                                      position=rope(r.rot_base, r.rot_dims), eps=eps)
                mixer = MixerPairSpec(kind="mixer_pair", name=f"{p}.mix", hidden_size=w, left=left, right=right, eps=eps,
                                      weight=PAIR_WEIGHT)
            else:
                m = l.delta
                mixer = GatedDeltaSpec(kind="gated_delta", name=f"{p}.mix", hidden_size=w, n_heads=m.heads,
                                       n_kv_heads=m.kv_heads, key_dim=m.dim, value_dim=m.vdim, conv=m.conv, eps=eps,
                                       channel_decay=True, decay_rank=m.rank, gate_rank=m.gate_rank)
            ff = None
            if l.mlp is not None and l.mlp.kind == "dense":
                ff = DenseMlpSpec(kind="dense_mlp", name=f"{p}.mlp", hidden_size=w, intermediate_size=l.mlp.ff,
                                  activation="relu2", bias=False)
            elif l.mlp is not None:
                f = l.mlp
                ff = RoutedExpertsSpec(kind="routed_experts", name=f"{p}.mlp", hidden_size=w, intermediate_size=f.ff,
                                       n_experts=f.experts, top=f.top, activation="swish_clamp", limit=f.limit,
                                       scores="all", n_groups=max(1, f.groups), keep_groups=max(1, f.keep),
                                       weight_scale=f.scale, router_bias=False)
            side = None
            if self.side_dim:
                side = TokenSideSpec(name=f"{p}.side", table=SIDE_TABLE, table_width=self.side_dim * len(self.layers),
                                     col=i * self.side_dim, dim=self.side_dim, hidden_size=w, vocab_size=self.vocab, eps=eps)
            blocks.append(BlockSpec(kind="prenorm", norm1=norm(f"{p}.norm1"), mixer=mixer,
                                    norm2=norm(f"{p}.norm2"), feed_forward=ff,
                                    residual_mult=self.residual_mult, side=side))
        emb = EmbeddingSpec("embed", self.vocab, w, suffix="")
        if self.pair_buckets:
            emb = EmbeddingSpec("embed", self.vocab, w, suffix="", pair_table=PAIR_TABLE, pair_buckets=self.pair_buckets,
                                pair_mul_prev=self.pair_mul_prev, pair_mul_cur=self.pair_mul_cur)
        return ModelSpec(
            architecture=self.architecture, hidden_size=w, vocab_size=self.vocab, max_positions=self.max_positions,
            embedding=emb, layers=tuple(blocks), schedule=self.schedule(),
            output=OutputSpec(norm=norm("final.norm"), name="head", tied=False, vocab_size=self.vocab, hidden_size=w,
                              suffix=""),
            stop_token_ids=tuple(self.eos_token_id))
