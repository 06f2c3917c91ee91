"""Routed experts: a router picks ``top`` of ``experts`` small gated feed-forwards per token; a shared expert may run
for every token beside them.

Router: logits ``W_r x`` in float32, scores ``sigmoid(logits)``, the ``top`` largest chosen; the chosen scores are the
weights (divided by their sum only with ``renormalize``).  ``weight_on_input`` (the form built here): an expert is fed
``score * x`` and its output added as it is, so for ``out = sum_k expert_k(score_k x) + shared(x)`` the score passes
through the expert's activation.  Expert: ``W_down (silu(W_gate a) * (W_up a))``, no biases.

The experts' weights are stacked at load ([experts, 2 ff, hidden] and [experts, hidden, ff]); a step sorts its
(token, choice) pairs by expert on the device and runs two grouped products over them, with the same launches
whatever the routing, so the part can be captured in a CUDA graph.
"""

from __future__ import annotations

import torch

from slipstream_b200 import ops

from .base import FEED_FORWARDS, FeedForward, Part, Runtime, WeightSpec


@FEED_FORWARDS.register("routed_experts")
class RoutedExperts(FeedForward):
    cuda_graph_safe = True
    can_return_terms = True  # ``forward(..., as_terms=True)`` leaves the sum over the choices to the caller's kernel

    def __init__(self, name: str, hidden_size: int, expert_size: int, experts: int, top: int,
                 shared: FeedForward | None = None, renormalize: bool = False, weight_on_input: bool = True,
                 router_tensor: str | None = None, expert_names: str | None = None) -> None:
        """``expert_names``: a pattern with ``{e}`` and ``{role}`` (gate, up, down) for the experts' tensors
        (default ``<name>.experts.{e}.{role}_proj.weight``); ``router_tensor``: the router's (``<name>.gate.weight``)."""
        if not 1 <= top <= experts or experts > 1024:
            raise ValueError(f"top ({top}) must be between 1 and experts ({experts}), experts at most 1024")
        if not weight_on_input:
            raise ValueError("only experts that take their weight on the input are built")
        self.name = name
        self.hidden_size, self.expert_size, self.experts, self.top = hidden_size, expert_size, experts, top
        self.shared = shared
        self.renormalize = bool(renormalize)
        self.router_tensor = router_tensor or f"{name}.gate.weight"
        self.expert_names = expert_names or f"{name}.experts.{{e}}.{{role}}_proj.weight"

    def children(self) -> list[Part]:
        return [self.shared] if self.shared is not None else []

    def weight_specs(self) -> list[WeightSpec]:
        h, f = self.hidden_size, self.expert_size
        specs = [WeightSpec(self.router_tensor, (self.experts, h), init=("normal", 0.2))]
        for e in range(self.experts):
            specs += [WeightSpec(self.expert_names.format(e=e, role="gate"), (f, h)),
                      WeightSpec(self.expert_names.format(e=e, role="up"), (f, h)),
                      WeightSpec(self.expert_names.format(e=e, role="down"), (h, f))]
        return specs

    def bind(self, weights: dict[str, torch.Tensor], runtime: Runtime) -> None:
        super().bind(weights, runtime)
        name = self.expert_names.format
        self.router_weight = weights[self.router_tensor]
        # gate and up rows alternate in runs of `run`, so that a tile of the stacked product holds 64 gate features and
        # the 64 matching up features (the tcgen05 kernel's fused activation needs both in one block)
        f = self.expert_size
        self.run = 64 if f % 64 == 0 else f

        def stacked(e: int) -> torch.Tensor:
            g, u = weights[name(e=e, role="gate")], weights[name(e=e, role="up")]
            return torch.stack([g.reshape(f // self.run, self.run, -1), u.reshape(f // self.run, self.run, -1)], dim=1).reshape(2 * f, -1)

        self.gate_up = torch.stack([stacked(e) for e in range(self.experts)]).contiguous()
        self.down = torch.stack([weights[name(e=e, role="down")] for e in range(self.experts)]).contiguous()

    def weight_bytes(self) -> int:
        """What a step reads at most: the router and the chosen experts of one token (a lower bound for a batch)."""
        per_expert = (self.gate_up[0].numel() + self.down[0].numel()) * self.down.element_size()
        return self.router_weight.numel() * self.router_weight.element_size() + self.top * per_expert

    def forward(self, x: torch.Tensor, ctx, as_terms: bool = False):
        ids, scores = ops.router(x, self.router_weight, self.top, self.renormalize)
        y, term_rows = ops.moe_experts(x, ids, scores, self.gate_up, self.down, self.run)
        shared = self.shared.forward(x, ctx) if self.shared is not None else None
        if as_terms:
            return {"terms": y, "extra": shared, "term_rows": term_rows, "count": self.top}
        return ops.moe_combine(y, shared, self.runtime.dtype, term_rows, self.top)
