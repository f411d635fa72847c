"""Feed-forwards.  Gated: down(act(gate(x)) * up(x)) with act = SiLU
(crates/nncpu/src/model/forward.rs:763-782,
crates/nncpu/src/kernels/scalar.rs:146-150) or one of the other gated activations.  gate and up are stored as one
matrix so the input is read once; the result is added to the residual stream.
Routed experts: a router picks a few small gated feed-forwards per token.
Dense: down(act(up(x) + b_up)) + b_down with act = xIELU, an activation with two learned numbers.
"""
from __future__ import annotations

import math

import torch

from ..errors import UnsupportedModel
from ..kernels import ops
from ..weights.params import ParamSpec
from .base import DeferredNorm, FeedForward, register_feed_forward


GATED_ACTIVATIONS = ("silu", "gelu_tanh", "swish_clamp")
# From this many token slots (token, choice) in a step, the experts run as one grouped product on the tensor cores;
# below it every slot reads its expert's rows itself.  Measured at 16 experts of 3 x 1536 x 2048 and 3 x 3072 x 4096 with
# the top 2: one token 56 / 112 us per slot against 103 / 161 us grouped, eight tokens 136 / 419 us against 120 / 265 us.
GROUPED_FROM_SLOTS = 8
# From this many tokens the router's logits are a product of their own instead of part of the router's one kernel,
# in which every token's block reads all of the router's rows.
ROUTER_PRODUCT_FROM_TOKENS = 256

@register_feed_forward("gated_mlp")
class GatedMlp(FeedForward):
    """down(act(gate(x), up(x))) with act one of ``GATED_ACTIVATIONS`` (see ``ops.gated_act``), computed in 32-bit on
    the two products' 32-bit results: in the gate/up product's epilogue on the tensor cores, in a kernel of its own
    elsewhere."""
    accepts_deferred_norm = True    # x goes to Runtime.linear, which finishes a norm's unfinished output

    def __init__(self, spec):
        if spec.activation not in GATED_ACTIVATIONS:
            raise UnsupportedModel(f"{spec.name}: activation {spec.activation!r} is not supported "
                                   f"(supported: {', '.join(GATED_ACTIVATIONS)})")
        if spec.tensor_names not in ("proj", "short"):
            raise UnsupportedModel(f"{spec.name}: tensor names of style {spec.tensor_names!r}")
        self.spec = spec
        self.activation = None if spec.activation == "silu" else (spec.activation, float(spec.limit), 0.0)

    def _tensor(self, which: str) -> str:
        s = self.spec
        return f"{s.name}.{which}" if s.tensor_names == "short" else f"{s.name}.{which}_proj.weight"

    def params(self):
        s = self.spec
        return [ParamSpec(self._tensor("gate"), (s.intermediate_size, s.hidden_size)),
                ParamSpec(self._tensor("up"), (s.intermediate_size, s.hidden_size)),
                ParamSpec(self._tensor("down"), (s.hidden_size, s.intermediate_size))]

    def bind(self, tensors, rt):
        s, self.rt = self.spec, rt
        gate, up = tensors.pop(self._tensor("gate")), tensors.pop(self._tensor("up"))
        # On the tensor-core path the activation runs in the product's epilogue, on the 32-bit
        # accumulators; for that, gate and up rows are interleaved in blocks of 8.
        self.fused = (gate.dtype == up.dtype and s.intermediate_size % 8 == 0
                      and rt.tensor_cores_take(rt.dtype, gate, s.hidden_size))
        if self.fused:
            h = s.hidden_size
            self.w_gate_up = torch.stack([gate.view(-1, 8, h), up.view(-1, 8, h)], dim=1).reshape(-1, h).contiguous()
        else:
            self.w_gate_up = torch.cat([gate, up], dim=0).contiguous()
        del gate, up
        self.w_down = tensors[self._tensor("down")]

    def weight_bytes(self):
        return sum(t.numel() * t.element_size() for t in (self.w_gate_up, self.w_down))

    def forward(self, ctx, x, residual):
        s, rt = self.spec, self.rt
        n = x.shape[0]
        act = rt.empty(n, s.intermediate_size)
        if self.fused:
            with rt.phase("ffn_gate_up", self.w_gate_up, n):
                rt.linear(x, self.w_gate_up, None, act, epilogue="swiglu", activation=self.activation)
        else:
            gate_up = rt.empty(n, 2 * s.intermediate_size, dtype=torch.float32)
            with rt.phase("ffn_gate_up", self.w_gate_up, n):
                rt.linear(x, self.w_gate_up, None, gate_up)
            with rt.phase("ffn_act"):
                ops.gated_act(gate_up, act, s.activation, s.limit)
        with rt.phase("ffn_down", self.w_down, n):
            # the last write into the residual stream: it may leave the next norm its input
            rt.linear(act, self.w_down, None, residual, accumulate=not getattr(ctx, "branch_is_fresh", False),
                      then_norm=getattr(ctx, "next_norm", None))


@register_feed_forward("routed_experts")
class RoutedExperts(FeedForward):
    """Every token runs the ``top`` of ``n_experts`` gated feed-forwards with the largest router logits, weighted by
    the softmax over those logits alone, and (optionally) a shared gated feed-forward.

    The router is a 32-bit product (its input may be the run's rounding of the norm's output) with a bias; the choice
    and the weights are made on the device by one kernel, so a step never waits for the host.  Experts' matrices are
    stacked [n_experts, rows, cols] when the weights are bound.

    ``scores`` "all" (see ``RoutedExpertsSpec``): the softmax runs over all experts, the choice may be limited to the
    best groups of experts, and the chosen scores are divided by their sum and multiplied by ``weight_scale``.
    ``out_scale`` (and the step's ``ctx.out_scale``) multiply what the part adds to the stream: they enter the
    tokens' weights, so the sum over a token's experts is scaled at no cost."""
    scales_output = True

    def __init__(self, spec):
        if spec.activation not in GATED_ACTIVATIONS:
            raise UnsupportedModel(f"{spec.name}: activation {spec.activation!r} is not supported")
        if not 0 < spec.top <= spec.n_experts:
            raise UnsupportedModel(f"{spec.name}: the top {spec.top} of {spec.n_experts} experts")
        if spec.scores not in ("chosen", "all"):
            raise UnsupportedModel(f"{spec.name}: router scores of kind {spec.scores!r}")
        if spec.scores == "chosen" and (spec.n_groups > 1 or spec.weight_scale != 1.0 or spec.out_scale != 1.0):
            raise UnsupportedModel(f"{spec.name}: groups and scales go with scores over all experts")
        if spec.n_groups > 1 and (spec.n_experts % spec.n_groups or not 1 <= spec.keep_groups <= spec.n_groups
                                  or spec.keep_groups * (spec.n_experts // spec.n_groups) < spec.top):
            raise UnsupportedModel(f"{spec.name}: the {spec.keep_groups} best of {spec.n_groups} groups of "
                                   f"{spec.n_experts} experts cannot give the top {spec.top}")
        self.spec = spec
        self.shared = None if spec.shared is None else GatedMlp(spec.shared)

    def params(self):
        s, p = self.spec, []
        for e in range(s.n_experts):
            p += [ParamSpec(f"{s.name}.e{e}.gate", (s.intermediate_size, s.hidden_size)),
                  ParamSpec(f"{s.name}.e{e}.up", (s.intermediate_size, s.hidden_size)),
                  ParamSpec(f"{s.name}.e{e}.down", (s.hidden_size, s.intermediate_size))]
        p.append(ParamSpec(f"{s.name}.router", (s.n_experts, s.hidden_size), init=("normal", 0.5)))
        if s.router_bias:
            p.append(ParamSpec(f"{s.name}.router.b", (s.n_experts,), init=("normal", 0.5)))
        return p + (self.shared.params() if self.shared is not None else [])

    def bind(self, tensors, rt):
        s, self.rt = self.spec, rt
        def stack(which):
            parts = [tensors.pop(f"{s.name}.e{e}.{which}") for e in range(s.n_experts)]
            return torch.stack(parts, dim=0).contiguous()
        gate, up, self.w_down = stack("gate"), stack("up"), stack("down")
        # Where the tensor cores take the sizes, an expert's gate and up rows are interleaved in blocks of 8, so that
        # the grouped product applies the activation in its epilogue; the kernel for few tokens reads the same layout.
        h, f = s.hidden_size, s.intermediate_size
        self.grouped = (gate.dtype == up.dtype == self.w_down.dtype and f % 8 == 0
                        and rt.tensor_cores_take(rt.dtype, gate[0], h) and rt.tensor_cores_take(rt.dtype, self.w_down[0], f))
        if self.grouped:
            self.w_gate = torch.stack([gate.view(s.n_experts, -1, 8, h), up.view(s.n_experts, -1, 8, h)],
                                      dim=2).reshape(s.n_experts, 2 * f, h).contiguous()
            self.w_up = None
        else:
            self.w_gate, self.w_up = gate, up
        del gate, up
        self.w_router, self.b_router = tensors[f"{s.name}.router"], tensors.get(f"{s.name}.router.b")
        if self.shared is not None:
            self.shared.bind(tensors, rt)

    def weight_bytes(self):
        """Bytes a decode step of one token reads: the router, the chosen experts, the shared expert."""
        s = self.spec
        per_expert = 3 * s.intermediate_size * s.hidden_size * self.w_gate.element_size()
        return (self.w_router.numel() * self.w_router.element_size() + s.top * per_expert
                + (self.shared.weight_bytes() if self.shared is not None else 0))

    def forward(self, ctx, x, residual):
        s, rt = self.spec, self.rt
        if isinstance(x, DeferredNorm):
            x = x.finish(ctx)
        n = x.shape[0]
        if getattr(ctx, "branch_is_fresh", False):
            raise UnsupportedModel(f"{s.name}: routed experts add into the stream they are given")
        ids = rt.empty(n, s.top, dtype=torch.int32)
        weights = rt.empty(n, s.top, dtype=torch.float32)
        out_scale = float(getattr(ctx, "out_scale", 1.0)) * s.out_scale
        scoring = None
        if s.scores == "all":
            scoring = ("all", s.n_groups, s.keep_groups, s.weight_scale * out_scale)
        elif out_scale != 1.0:
            raise UnsupportedModel(f"{s.name}: a scaled output goes with scores over all experts")
        with rt.phase("moe_route", self.w_router, n):
            many = n >= ROUTER_PRODUCT_FROM_TOKENS and rt.tensor_cores_take(x.dtype, self.w_router, s.hidden_size)
            if not many and ops.moe_router_fits(s.n_experts, s.hidden_size):
                ops.moe_router(x, self.w_router, self.b_router, s.top, ids, weights, scoring)
            else:
                # many tokens: the logits as a product of their own (bfloat16 operands are multiplied exactly and
                # added in 32-bit on the tensor cores; a float32 run, and sizes those refuse, use the CUDA cores)
                logits = rt.empty(n, s.n_experts, dtype=torch.float32)
                if many:
                    rt.linear(x, self.w_router, self.b_router, logits)
                else:
                    ops.linear_simt(x, self.w_router, self.b_router, logits)
                ops.moe_route(logits, s.top, ids, weights, scoring)
        S, f, h = n * s.top, s.intermediate_size, s.hidden_size
        esize = self.w_gate.element_size()
        experts_read = min(S, s.n_experts)
        if self.grouped and S >= GROUPED_FROM_SLOTS:
            # many tokens: sorted by expert, one grouped product each for gate/up (activation in its epilogue) and
            # down on the tensor cores, then the choices of a token added up in their order
            act = (s.activation, float(s.limit), 0.0) if s.activation != "silu" else None
            with rt.phase("moe_sort", nbytes=4.0 * S * h):
                rows, slots = rt.empty(S, dtype=torch.int32), rt.empty(S, dtype=torch.int32)
                plan = rt.empty(1 + 3 * ops.moe_plan_tiles(S, s.n_experts), dtype=torch.int32)
                ops.moe_plan(ids, s.n_experts, rows, slots, plan)
                xs = rt.empty(S, h, dtype=torch.bfloat16)
                ops.moe_gather(x, slots, s.top, xs)
            mid = rt.empty(S, f, dtype=torch.bfloat16)
            with rt.phase("moe_gate_up", nbytes=experts_read * 2.0 * f * h * esize, flops=4.0 * S * f * h):
                ops.linear_tc_grouped(xs, self.w_gate, mid, plan, s.n_experts, rt.workspace, "swiglu", act)
            y = rt.empty(S, h, dtype=torch.float32)
            with rt.phase("moe_down", nbytes=experts_read * 1.0 * f * h * esize + 4.0 * S * h, flops=2.0 * S * f * h):
                ops.linear_tc_grouped(mid, self.w_down, y, plan, s.n_experts, rt.workspace)
            with rt.phase("moe_combine", nbytes=4.0 * S * h + 8.0 * n * h):
                ops.moe_combine(y, rows, weights, residual)
        else:
            mid = rt.empty(S, f)
            with rt.phase("moe_experts", nbytes=experts_read * 3.0 * f * h * esize, flops=6.0 * S * f * h):
                ops.moe_experts(x, self.w_gate, self.w_up, self.w_down, ids, weights, mid, residual, s.activation, s.limit)
        if self.shared is not None:
            if out_scale != 1.0:
                raise UnsupportedModel(f"{s.name}: a shared expert under a scaled output")
            self.shared.forward(ctx, x, residual)


@register_feed_forward("dense_mlp")
class DenseMlp(FeedForward):
    """down(act(up(x) + b_up)) + b_down with act xIELU or the square of relu; ``bias`` False: no biases.  The activation (softplus of xIELU's two numbers included) is computed in
    32-bit on the up product's 32-bit result, in the product's epilogue where it runs on the tensor cores and in a
    kernel of its own elsewhere; its output is rounded to the run's element type for the down product.  Tensors: ``<name>.up``, ``.up.b``, ``.down``, ``.down.b``, ``.act`` (p, q)."""

    def __init__(self, spec):
        if spec.activation not in ("xielu", "relu2"):
            raise UnsupportedModel(f"{spec.name}: activation {spec.activation!r} is not supported (supported: xielu, relu2)")
        self.spec = spec
        # without biases a factor on the part's output can ride on the square of relu: down(a relu(z)^2) = a down(relu(z)^2)
        self.scales_output = spec.activation == "relu2" and not spec.bias

    def params(self):
        s = self.spec
        p = [ParamSpec(f"{s.name}.up", (s.intermediate_size, s.hidden_size)),
             ParamSpec(f"{s.name}.down", (s.hidden_size, s.intermediate_size))]
        if s.bias:
            p += [ParamSpec(f"{s.name}.up.b", (s.intermediate_size,)), ParamSpec(f"{s.name}.down.b", (s.hidden_size,))]
        if s.activation == "xielu":
            p.append(ParamSpec(f"{s.name}.act", (2,), init=("normal", 0.5)))
        return p

    def bind(self, tensors, rt):
        s, self.rt = self.spec, rt
        self.w_up, self.b_up = tensors[f"{s.name}.up"], tensors.get(f"{s.name}.up.b")
        self.w_down, self.b_down = tensors[f"{s.name}.down"], tensors.get(f"{s.name}.down.b")
        self.act = tensors.get(f"{s.name}.act")
        # On the tensor-core path the activation runs in the up product's epilogue, on its 32-bit accumulators; xIELU's
        # two numbers enter as softplus(p) and 1/2 + softplus(q), worked out once here in 32-bit.
        self.fused = rt.tensor_cores_take(rt.dtype, self.w_up, s.hidden_size) and (self.act is None or not self.act.is_meta)
        if self.fused and s.activation == "relu2":
            self.activation = ("relu2", 1.0, 0.0)
        elif self.fused:
            p, q = (math.log1p(math.exp(-abs(v))) + max(v, 0.0) for v in self.act.detach().float().tolist())   # softplus
            self.activation = ("xielu", p, 0.5 + q)

    def weight_bytes(self):
        return sum(t.numel() * t.element_size() for t in (self.w_up, self.w_down))

    def forward(self, ctx, x, residual):
        s, rt = self.spec, self.rt
        n = x.shape[0]
        act = rt.empty(n, s.intermediate_size)
        scale = float(getattr(ctx, "out_scale", 1.0)) if self.scales_output else 1.0
        if self.fused:
            with rt.phase("ffn_up", self.w_up, n):
                rt.linear(x, self.w_up, self.b_up, act,
                          activation=("relu2", scale, 0.0) if s.activation == "relu2" else self.activation)
        else:
            up = rt.empty(n, s.intermediate_size, dtype=torch.float32)
            with rt.phase("ffn_up", self.w_up, n):
                rt.linear(x, self.w_up, self.b_up, up)
            with rt.phase("ffn_act"):
                if s.activation == "relu2":
                    ops.relu2(up, act, scale)
                else:
                    ops.xielu(up, self.act, act)
        with rt.phase("ffn_down", self.w_down, n):
            rt.linear(act, self.w_down, self.b_down, residual, accumulate=not getattr(ctx, "branch_is_fresh", False))
