"""Feed-forwards beyond the gated MLP: a dense one with a PolyNorm activation, and a mixture of gated experts whose
choice is a table lookup by token id.

`polynorm_mlp`   down( P(up(x)) ),  P(z) = a n(z) + b n(z^2) + c n(z^3) + e  with powers taken element by element and
                 n(v) = v / sqrt(mean(v^2) + eps) over the token's whole vector; the four numbers are a tensor.
`table_moe`      every token runs `top` of `experts` gated MLPs  down_e( silu(gate_e x) * up_e x ), each weighted 1 / top;
                 which ones is read from an integer table [vocab, top] at the token's id (no router product, no
                 softmax); optionally a shared expert of the same form runs for every token and is added.
                 The experts' matrices are kept stacked ([experts, 2 ff, width] gate rows then up rows, and
                 [experts, width, ff]) so that one kernel serves all of them.
`routed_moe`     every token runs `top` of `experts` plain MLPs  down_e( act(up_e x) ), act = relu squared, chosen by a router:
                 s = sigmoid(Wr x) in float32; the choice is made among s + correction (a number per expert), only within
                 the `keep_groups` best of `groups` equal groups of neighbouring experts (a group counts by the sum of its
                 two largest corrected scores); the weights are the chosen experts' s divided by their sum (+ 1e-20).
                 Optionally a shared expert of the same form runs for every token and is added times
                 sigmoid(w_sg . x), one number per token.
"""
from __future__ import annotations

from typing import Optional

import torch

from .base import FEED_FORWARDS, Part, TensorSpec
from .linear import Linear
from .mlp import GatedMLP


class PolyNormMLP(Part):
    def __init__(self, hidden_size: int, intermediate_size: int, eps: float, names=("up", "down", "act"), suffix: str = ""):
        self.hidden_size, self.intermediate_size, self.eps = hidden_size, intermediate_size, eps
        self.up = Linear(hidden_size, [intermediate_size], [names[0]], suffix=suffix)
        self.down = Linear(intermediate_size, [hidden_size], [names[1]], suffix=suffix)
        self.coef_name = names[2]
        self.coef = None

    def tensor_specs(self):
        return {**self.up.tensor_specs(), **self.down.tensor_specs(), self.coef_name: TensorSpec((4,), "coef")}

    def bind(self, get):
        self.up.bind(get)
        self.down.bind(get)
        self.coef = get(self.coef_name).float().contiguous()        # norms are float32

    def __call__(self, x, ctx, residual=None, out_dtype=None):
        z = self.up(x, ctx, out_dtype=torch.float32)
        h = ctx.kernels.polynorm(z, self.coef, self.eps, x.dtype)
        return self.down(h, ctx, residual=residual, out_dtype=out_dtype)


class TableMoE(Part):
    def __init__(self, hidden_size: int, intermediate_size: int, experts: int, top: int, vocab_size: int,
                 shared_intermediate_size: Optional[int] = None, names=("gate", "up", "down"), table: str = "table",
                 expert_prefix: str = "e", shared_prefix: str = "shared.", suffix: str = ""):
        from ..errors import ConfigError
        if not 1 <= top <= experts:
            raise ConfigError(f"a token uses {top} of {experts} experts")
        self.hidden_size, self.intermediate_size, self.experts, self.top = hidden_size, intermediate_size, experts, top
        self.vocab_size, self.names, self.table_name, self.expert_prefix = vocab_size, tuple(names), table, expert_prefix
        self.suffix = suffix
        self.shared_prefix = shared_prefix
        self.shared = None
        if shared_intermediate_size is not None:
            self.shared = GatedMLP(hidden_size, shared_intermediate_size, "silu", names=names, suffix=suffix)
        self.table = self.gate_up = self.down = None

    def tensor_specs(self):
        g, u, d = self.names
        specs = {self.table_name: TensorSpec((self.vocab_size, self.top), f"choice:{self.experts}")}
        for e in range(self.experts):
            p = f"{self.expert_prefix}{e}."
            specs[f"{p}{g}{self.suffix}"] = TensorSpec((self.intermediate_size, self.hidden_size), "matrix")
            specs[f"{p}{u}{self.suffix}"] = TensorSpec((self.intermediate_size, self.hidden_size), "matrix")
            specs[f"{p}{d}{self.suffix}"] = TensorSpec((self.hidden_size, self.intermediate_size), "matrix")
        if self.shared is not None:
            specs.update({self.shared_prefix + n: ts for n, ts in self.shared.tensor_specs().items()})
        return specs

    def bind(self, get):
        g, u, d = self.names
        self.table = get(self.table_name).to(torch.int32).contiguous()
        rows = []
        for e in range(self.experts):
            p = f"{self.expert_prefix}{e}."
            rows.append(torch.cat([get(f"{p}{g}{self.suffix}"), get(f"{p}{u}{self.suffix}")], dim=0))
        self.gate_up = torch.stack(rows).contiguous()                                   # [E, 2 ff, width]
        self.down = torch.stack([get(f"{self.expert_prefix}{e}.{d}{self.suffix}") for e in range(self.experts)]).contiguous()
        if self.shared is not None:
            self.shared.bind(lambda name: get(self.shared_prefix + name))

    def __call__(self, x, ctx, residual=None, out_dtype=None):
        k = ctx.kernels
        y = self.shared(x, ctx, residual=residual, out_dtype=torch.float32) if self.shared is not None else residual
        chosen = k.gather_rows(self.table, ctx.token_ids)                 # [tokens, top] expert numbers
        return k.moe_experts(x, chosen, self.gate_up, self.down, 1.0 / self.top, add=y, out_dtype=out_dtype or x.dtype)


class RoutedMoE(Part):
    ACTIVATIONS = ("relu2",)

    def __init__(self, hidden_size: int, intermediate_size: int, experts: int, top: int, groups: int = 1, keep_groups: int = 1,
                 shared_intermediate_size: Optional[int] = None, activation: str = "relu2", names=("up", "down"),
                 router: str = "router", correction: str = "correction", expert_prefix: str = "e",
                 shared_prefix: str = "shared.", shared_gate: str = "sg", suffix: str = "", weight_eps: float = 1e-20):
        from ..errors import ConfigError
        problems = []
        if not 1 <= top <= experts:
            problems.append(f"a token uses {top} of {experts} experts")
        if groups < 1 or experts % max(groups, 1) or not 1 <= keep_groups <= groups:
            problems.append(f"{experts} experts in {groups} equal groups of which {keep_groups} are kept")
        elif top > keep_groups * (experts // groups):
            problems.append(f"{top} experts per token out of {keep_groups} groups of {experts // groups}")
        if experts > 1024:
            problems.append(f"the router serves at most 1,024 experts, got {experts}")
        if activation not in self.ACTIVATIONS:
            problems.append(f"expert activation {activation!r} is not known ({', '.join(self.ACTIVATIONS)})")
        if problems:
            raise ConfigError(problems, "routed mixture of experts")
        self.hidden_size, self.intermediate_size, self.experts, self.top = hidden_size, intermediate_size, experts, top
        self.groups, self.keep_groups, self.activation, self.weight_eps = groups, keep_groups, activation, weight_eps
        self.names, self.router_name, self.correction_name, self.expert_prefix = tuple(names), router, correction, expert_prefix
        self.shared_prefix, self.shared_gate, self.suffix = shared_prefix, shared_gate, suffix
        self.shared_ff = shared_intermediate_size
        self.shared_up = self.shared_down = None
        if shared_intermediate_size is not None:
            self.shared_up = Linear(hidden_size, [shared_intermediate_size], [names[0]], suffix=suffix)
            self.shared_down = Linear(shared_intermediate_size, [hidden_size], [names[1]], suffix=suffix)
        self.router = self.correction = self.up = self.down = None

    def tensor_specs(self):
        u, d = self.names
        specs = {self.router_name + self.suffix: TensorSpec((self.experts, self.hidden_size), "matrix"),
                 self.correction_name: TensorSpec((self.experts,), "bias")}
        for e in range(self.experts):
            p = f"{self.expert_prefix}{e}."
            specs[f"{p}{u}{self.suffix}"] = TensorSpec((self.intermediate_size, self.hidden_size), "matrix")
            specs[f"{p}{d}{self.suffix}"] = TensorSpec((self.hidden_size, self.intermediate_size), "matrix")
        if self.shared_up is not None:
            for lin in (self.shared_up, self.shared_down):
                specs.update({self.shared_prefix + n: ts for n, ts in lin.tensor_specs().items()})
            specs[self.shared_prefix + self.shared_gate + self.suffix] = TensorSpec((1, self.hidden_size), "matrix")
        return specs

    def bind(self, get):
        u, d = self.names
        rows = [get(self.router_name + self.suffix)]
        if self.shared_up is not None:                       # the shared expert's gate is one more row of the router's product
            rows.append(get(self.shared_prefix + self.shared_gate + self.suffix))
            self.shared_up.bind(lambda name: get(self.shared_prefix + name))
            self.shared_down.bind(lambda name: get(self.shared_prefix + name))
        self.router = torch.cat(rows, dim=0).contiguous()
        self.correction = get(self.correction_name).float().contiguous()       # the router is float32
        self.up = torch.stack([get(f"{self.expert_prefix}{e}.{u}{self.suffix}") for e in range(self.experts)]).contiguous()
        self.down = torch.stack([get(f"{self.expert_prefix}{e}.{d}{self.suffix}") for e in range(self.experts)]).contiguous()

    def __call__(self, x, ctx, residual=None, out_dtype=None):
        k = ctx.kernels
        scores = k.linear(x, self.router, None, None, torch.float32)
        chosen, weights, shared_gate = k.moe_route_top(scores, self.correction, self.experts, self.top, self.groups,
                                                       self.keep_groups, self.weight_eps, shared_gate=self.shared_up is not None)
        add = residual
        if self.shared_up is not None:
            u = self.shared_up(x, ctx, out_dtype=torch.float32)
            a = k.act_rows(u, self.activation, x.dtype, row_scale=shared_gate)      # W (g a) = g (W a): the gate rides on the activation
            add = self.shared_down(a, ctx, residual=residual, out_dtype=torch.float32)
        return k.moe_experts(x, chosen, self.up, self.down, 1.0, add=add, out_dtype=out_dtype or x.dtype, weights=weights,
                             activation=self.activation)


FEED_FORWARDS.register("polynorm_mlp", PolyNormMLP)
FEED_FORWARDS.register("routed_moe", RoutedMoE)
FEED_FORWARDS.register("table_moe", TableMoE)
