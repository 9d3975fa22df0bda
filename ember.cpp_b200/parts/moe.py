"""Experts chosen by a table: every token id names its `top` experts in a stored integer table
[vocab, top] (the entries of a row differ), each weighing 1/top; there is no router product.

An expert is a small gated feed-forward without biases, `down(silu(gate h) * (up h))`.  An
optional shared expert of the same form (a size of its own) runs for every token and is added.
The experts' matrices are stacked at load ([experts, gate | up, width] and [experts, width, inner]),
the step's (token, choice) pairs are sorted by expert on the device, and two grouped products run
each expert over its own pairs; nothing comes back to the host, so the step replays as a graph.
"""
from __future__ import annotations

from .base import FeedForward, WeightSpec, build_part, register_part
from .spec import PartSpec


class TableExperts(FeedForward):
    needs_tokens = True

    def __init__(self, prefix: str, width: int, vocab: int, experts: int, top: int, inner: int,
                 shared_inner: int = 0, table: str = "table", expert: str = "e{}.", shared: str = "shared.",
                 gate: str = "gate", up: str = "up", down: str = "down", suffix: str = ".weight",
                 init_std: float = 0.02, down_init_std: float = 0.02):
        super().__init__(prefix)
        self.width, self.vocab, self.experts, self.top, self.inner = int(width), int(vocab), int(experts), int(top), int(inner)
        if not 1 <= self.top <= self.experts:
            raise ValueError(f"experts {prefix!r}: top = {self.top} of {self.experts} experts")
        if self.top > 15:
            raise ValueError(f"experts {prefix!r}: top = {self.top}; at most 15 experts a token")
        self.table_name = prefix + table
        self.expert_names = [tuple(prefix + expert.format(e) + n + suffix for n in (gate, up, down)) for e in range(self.experts)]
        self.init_std, self.down_init_std = init_std, down_init_std
        self.shared = None
        if shared_inner:
            self.shared = build_part("ffn", PartSpec("gated", prefix + shared, dict(
                width=width, inner=int(shared_inner), activation="silu", gate=gate, up=up, down=down, suffix=suffix,
                init_std=init_std, down_init_std=down_init_std)))
        self.w_gate_up = self.w_down = self.table = None

    def weight_specs(self):
        specs = [WeightSpec(self.table_name, (self.vocab, self.top), integer=True, below=self.experts)]
        for g, u, d in self.expert_names:
            specs += [WeightSpec(g, (self.inner, self.width), std=self.init_std),
                      WeightSpec(u, (self.inner, self.width), std=self.init_std),
                      WeightSpec(d, (self.width, self.inner), std=self.down_init_std)]
        return specs + (self.shared.weight_specs() if self.shared is not None else [])

    def load(self, get, runtime):
        import torch
        table = get(self.table_name).to(torch.int64)
        if int(table.min()) < 0 or int(table.max()) >= self.experts:
            raise ValueError(f"experts {self.prefix!r}: the table names an expert outside [0, {self.experts})")
        self.table = runtime.index_table(table)
        self.w_gate_up = torch.stack([torch.cat([runtime.matrix(get(g)), runtime.matrix(get(u))]) for g, u, _ in self.expert_names]).contiguous()
        self.w_down = torch.stack([runtime.matrix(get(d)) for _, _, d in self.expert_names]).contiguous()
        if self.shared is not None:
            self.shared.load(get, runtime)

    def stream_weights(self):
        return self.shared.stream_weights() if self.shared is not None else []

    def _chosen(self, ctx, h):
        ops = ctx.ops
        routing = ops.moe_route(ctx.plan.tokens, ctx.plan.T, self.table, self.experts, self.top)
        inner = ops.moe_gate_up(h, self.w_gate_up, routing, out_dtype=ctx.dtype)     # [T * top, inner], silu(g) * u
        y = ops.moe_down(inner, self.w_down, routing)                                 # float32 [T, top, width]
        return [(y[:, k, :], 1.0 / self.top) for k in range(self.top)]

    def branches(self, ctx, h):
        if self.shared is None:
            return self._chosen(ctx, h)
        runs = [lambda: self._chosen(ctx, h), lambda: self.shared.branches(ctx, h)]
        together = getattr(ctx.ops, "side_by_side", None)     # (one-token steps: the shared expert beside the chosen ones)
        chosen, shared = together(runs) if together is not None and ctx.plan.all_single else [run() for run in runs]
        return chosen + shared

    def forward(self, ctx, h, residual):
        x = residual
        for rows, f in self.branches(ctx, h):
            x = x + f * rows
        return x


register_part("ffn", "table_experts", TableExperts)


class RoutedExperts(FeedForward):
    """Experts chosen by a router: z = W_router h in float32, scores s = sigmoid(z); the choice is made on
    s + correction (a stored vector, one value an expert), the weights use s alone.  The experts form
    `groups` equal groups of neighbours; a group's score is the sum of its two largest choice scores, and only
    experts of the `keep_groups` best groups can be chosen (DeepSeek-V3's routing: DeepSeek-AI, "DeepSeek-V3
    Technical Report").  The `top` chosen experts' scores, divided by their sum (+ 1e-20) and multiplied by
    `route_scale`, weigh the experts' outputs.  An expert is a gated feed-forward without biases: silu(g) * u, or
    with `limit` > 0 the clamped form (g capped at limit, u within +-limit, g * sigmoid(alpha g) * (u + shift)).
    An optional shared expert of the same form (sizes and limit of its own) runs for every token and is added,
    multiplied by sigmoid(w_sg . h), one number a token, where `shared_gate` names w_sg.

    The router's rows and the shared expert's gate row are one product with float32 sums; scores, choice,
    weights and the weighted sum are float32.  Nothing returns to the host."""

    def __init__(self, prefix: str, width: int, experts: int, top: int, inner: int, route_scale: float = 1.0,
                 groups: int = 1, keep_groups: int = 1, limit: float = 0.0, alpha: float = 1.0, shift: float = 0.0,
                 shared_inner: int = 0, shared_limit: float = 0.0, shared_gate: str | None = None,
                 router: str = "router", correction: str | None = "correction", expert: str = "e{}.", shared: str = "shared.",
                 gate: str = "gate", up: str = "up", down: str = "down", suffix: str = "", init_std: float = 0.02,
                 down_init_std: float = 0.02):
        super().__init__(prefix)
        self.width, self.experts, self.top, self.inner = int(width), int(experts), int(top), int(inner)
        self.groups, self.keep_groups, self.route_scale = int(groups), int(keep_groups), float(route_scale)
        self.limit, self.alpha, self.shift = float(limit), float(alpha), float(shift)
        if not 1 <= self.top <= self.experts or self.top > 32 or self.experts > 1024:
            raise ValueError(f"experts {prefix!r}: top = {self.top} of {self.experts} experts (at most 32 of 1024)")
        if self.groups < 1 or self.experts % self.groups or not 1 <= self.keep_groups <= self.groups:
            raise ValueError(f"experts {prefix!r}: {self.experts} experts in {self.groups} groups, {self.keep_groups} kept")
        if self.keep_groups * (self.experts // self.groups) < self.top:
            raise ValueError(f"experts {prefix!r}: {self.keep_groups} groups of {self.experts // self.groups} hold fewer "
                             f"than top = {self.top} experts")
        self.router_name = prefix + router
        self.correction_name = None if correction is None else prefix + correction
        self.expert_names = [tuple(prefix + expert.format(e) + n + suffix for n in (gate, up, down)) for e in range(self.experts)]
        self.init_std, self.down_init_std = init_std, down_init_std
        self.shared = self.shared_gate_name = None
        if shared_inner:
            act = dict(activation="clamped_sigmoid", limit=float(shared_limit), alpha=alpha, shift=shift) if shared_limit > 0 \
                else dict(activation="silu")
            self.shared = build_part("ffn", PartSpec("gated", prefix + shared, dict(
                width=width, inner=int(shared_inner), gate=gate, up=up, down=down, suffix=suffix, init_std=init_std,
                down_init_std=down_init_std, **act)))
            self.shared_gate_name = None if shared_gate is None else prefix + shared + shared_gate
        self.w_gate_up = self.w_down = self.w_router = self.correction = None

    def weight_specs(self):
        specs = [WeightSpec(self.router_name, (self.experts, self.width), std=0.3)]
        if self.correction_name is not None:
            specs.append(WeightSpec(self.correction_name, (self.experts,), std=0.1))
        for g, u, d in self.expert_names:
            specs += [WeightSpec(g, (self.inner, self.width), std=self.init_std),
                      WeightSpec(u, (self.inner, self.width), std=self.init_std),
                      WeightSpec(d, (self.width, self.inner), std=self.down_init_std)]
        if self.shared is not None:
            specs += self.shared.weight_specs()
            if self.shared_gate_name is not None:
                specs.append(WeightSpec(self.shared_gate_name, (1, self.width), std=0.1))
        return specs

    def load(self, get, runtime):
        import torch
        rows = [runtime.matrix(get(self.router_name))]
        if self.shared_gate_name is not None:
            rows.append(runtime.matrix(get(self.shared_gate_name)))
        w = torch.cat(rows)
        pad = -w.shape[0] % 8       # (rows of zeros: the product's output rows are whole 16-byte pieces)
        if pad:
            w = torch.cat([w, torch.zeros((pad, self.width), dtype=w.dtype, device=w.device)])
        self.w_router = w.contiguous()
        self.correction = (torch.zeros(self.experts, dtype=torch.float32, device=w.device) if self.correction_name is None
                           else runtime.vector(get(self.correction_name)))
        self.w_gate_up = torch.stack([torch.cat([runtime.matrix(get(g)), runtime.matrix(get(u))]) for g, u, _ in self.expert_names]).contiguous()
        self.w_down = torch.stack([runtime.matrix(get(d)) for _, _, d in self.expert_names]).contiguous()
        if self.shared is not None:
            self.shared.load(get, runtime)

    def stream_weights(self):
        return self.shared.stream_weights() if self.shared is not None else []

    def _chosen(self, ctx, h, logits):
        ops = ctx.ops
        chosen, weights = ops.moe_pick(logits, self.correction, self.experts, self.top, self.groups, self.keep_groups,
                                       self.route_scale)
        routing = ops.moe_route(None, ctx.plan.T, chosen, self.experts, self.top)
        inner = ops.moe_gate_up(h, self.w_gate_up, routing, out_dtype=ctx.dtype, limit=self.limit, alpha=self.alpha,
                                shift=self.shift)                                     # [T * top, inner]
        return ops.moe_down(inner, self.w_down, routing), weights                     # float32 [T, top, width], [T, top]

    def forward(self, ctx, h, residual):
        import torch
        logits = ctx.ops.linear(h, self.w_router, None, out_dtype=torch.float32)      # float32 [T, experts (| sg) (| 0)]
        if self.shared is None:
            y, weights = self._chosen(ctx, h, logits)
            return ctx.ops.moe_combine(residual, y, weights, None, None, 0)
        runs = [lambda: self._chosen(ctx, h, logits), lambda: self.shared.branches(ctx, h)[0][0]]
        together = getattr(ctx.ops, "side_by_side", None)     # (one-token steps: the shared expert beside the chosen ones)
        (y, weights), shared = together(runs) if together is not None and ctx.plan.all_single else [run() for run in runs]
        gated = self.shared_gate_name is not None
        return ctx.ops.moe_combine(residual, y, weights, shared, logits if gated else None, self.experts)

    def branches(self, ctx, h):
        import torch
        zero = torch.zeros((h.shape[0], self.width), dtype=torch.float32, device=h.device)
        return [(self.forward(ctx, h, zero), 1.0)]


register_part("ffn", "routed_experts", RoutedExperts)
