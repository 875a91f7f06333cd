"""Routed experts: a router picks ``top`` of ``experts`` small feed-forwards per token; a shared expert may run
for every token beside them.

Router: logits ``W_r x`` in float32, scores ``sigmoid(logits)`` (or, ``scores="softmax"``, their softmax over all
experts), the ``top`` largest chosen; the chosen scores are the weights (divided by their sum only with
``renormalize``).  ``correction``: a tensor [experts] added to the scores for the CHOICE only.  ``groups`` = (count,
keep): the experts form ``count`` equal groups of neighbours, a group's score is its largest choice score, and only
experts of the ``keep`` best groups can be chosen.  ``identity`` n: the router has n more outputs behind the
experts', which take part in scores, groups and choice like experts; such an expert has no tensors and its output is
its input.

Two forms of expert.  ``gated`` (the default): ``W_down (silu(W_gate a) * (W_up a))`` fed ``a = score * x``
(``weight_on_input``), its output added as it is.  Not ``gated``: ``W_down relu(W_up x)^2`` fed ``x``, its output
times the score.  No biases.  ``shared_gate``: a tensor [1, hidden]; the shared expert's output is multiplied by
``sigmoid(shared_gate . x)``, one number per token (its logit rides along in the router's product, in float32).

The experts' weights are stacked at load ([experts, 2 ff, hidden] or [experts, ff, hidden], and [experts, hidden, ff]);
a step sorts its (token, choice) pairs by expert on the device and runs two grouped products over them, with the same
launches whatever the routing, so the part can be captured in a CUDA graph.
"""

from __future__ import annotations

import torch

from slipstream_b200 import ops

from .base import FEED_FORWARDS, FeedForward, Part, Runtime, WeightSpec


@FEED_FORWARDS.register("routed_experts")
class RoutedExperts(FeedForward):
    cuda_graph_safe = True
    can_return_terms = True  # ``forward(..., as_terms=True)`` leaves the sum over the choices to the caller's kernel
    # (the gated form; the un-gated form always forms its weighted sum itself)

    def __init__(self, name: str, hidden_size: int, expert_size: int, experts: int, top: int,
                 shared: FeedForward | None = None, renormalize: bool = False, weight_on_input: bool = True,
                 router_tensor: str | None = None, expert_names: str | None = None, *, gated: bool = True,
                 scores: str = "sigmoid", correction: str | None = None, groups: tuple[int, int] | None = None,
                 identity: int = 0, shared_gate: str | None = None) -> None:
        """``expert_names``: a pattern with ``{e}`` and ``{role}`` (gate, up, down) for the experts' tensors
        (default ``<name>.experts.{e}.{role}_proj.weight``); ``router_tensor``: the router's (``<name>.gate.weight``);
        ``correction`` and ``shared_gate``: tensor names."""
        slots = experts + int(identity)
        if not 1 <= top <= slots or slots > 1024 or identity < 0:
            raise ValueError(f"top ({top}) must be between 1 and experts + identity ({slots}), that at most 1024")
        if gated != bool(weight_on_input):
            raise ValueError("built: gated experts with their weight on the input, un-gated ones with it on the output")
        if gated and identity:
            raise ValueError("experts that hand their input on come with the un-gated form")
        if scores not in ("sigmoid", "softmax"):
            raise ValueError(f"unknown router scores {scores!r} (known: sigmoid, softmax)")
        if groups is not None and (groups[0] < 1 or slots % groups[0] or not 1 <= groups[1] <= groups[0]
                                   or top > groups[1] * (slots // groups[0])):
            raise ValueError("experts + identity must split into groups[0] groups of which groups[1] are kept, with room for top")
        if shared_gate is not None and shared is None:
            raise ValueError("a gate on the shared expert comes with a shared expert")
        self.gated, self.scores, self.correction, self.groups = bool(gated), scores, correction, groups
        self.identity, self.slots, self.shared_gate = int(identity), slots, shared_gate
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
        specs = [WeightSpec(self.router_tensor, (self.slots, h), init=("normal", 0.2))]
        if self.correction is not None:
            specs.append(WeightSpec(self.correction, (self.slots,), kind="vector", init=("normal", 0.02)))
        if self.shared_gate is not None:
            specs.append(WeightSpec(self.shared_gate, (1, h), init=("normal", 0.2)))
        for e in range(self.experts):
            if self.gated:
                specs.append(WeightSpec(self.expert_names.format(e=e, role="gate"), (f, h)))
            specs += [WeightSpec(self.expert_names.format(e=e, role="up"), (f, h)),
                      WeightSpec(self.expert_names.format(e=e, role="down"), (h, f))]
        return specs

    def bind(self, weights: dict[str, torch.Tensor], runtime: Runtime) -> None:
        super().bind(weights, runtime)
        name = self.expert_names.format
        self.router_weight = weights[self.router_tensor]
        if self.shared_gate is not None:  # one product for the router's logits and the shared expert's gate
            self.router_weight = torch.cat([self.router_weight, weights[self.shared_gate].reshape(1, -1)]).contiguous()
        self.correction_weight = (weights[self.correction].to(torch.float32).contiguous()
                                  if self.correction is not None else None)
        self.down = torch.stack([weights[name(e=e, role="down")] for e in range(self.experts)]).contiguous()
        if not self.gated:
            self.up = torch.stack([weights[name(e=e, role="up")] for e in range(self.experts)]).contiguous()
            return
        # gate and up rows alternate in runs of `run`, so that a tile of the stacked product holds 64 gate features and
        # the 64 matching up features (the tcgen05 kernel's fused activation needs both in one block)
        f = self.expert_size
        self.run = 64 if f % 64 == 0 else f

        def stacked(e: int) -> torch.Tensor:
            g, u = weights[name(e=e, role="gate")], weights[name(e=e, role="up")]
            return torch.stack([g.reshape(f // self.run, self.run, -1), u.reshape(f // self.run, self.run, -1)], dim=1).reshape(2 * f, -1)

        self.gate_up = torch.stack([stacked(e) for e in range(self.experts)]).contiguous()

    def weight_bytes(self) -> int:
        """What a step reads at most: the router and the chosen experts of one token (a lower bound for a batch)."""
        first = self.gate_up if self.gated else self.up
        per_expert = (first[0].numel() + self.down[0].numel()) * self.down.element_size()
        return self.router_weight.numel() * self.router_weight.element_size() + self.top * per_expert

    def forward(self, x: torch.Tensor, ctx, as_terms: bool = False):
        count, keep = self.groups or (1, 1)
        routed = ops.router(x, self.router_weight, self.top, self.renormalize, softmax=self.scores == "softmax",
                            correction=self.correction_weight, groups=count, keep=keep,
                            extra=1 if self.shared_gate is not None else 0)
        ids, scores = routed[0], routed[1]
        shared = self.shared.forward(x, ctx) if self.shared is not None else None
        if not self.gated:  # the weights, the experts that hand their input on and the shared expert's gate meet in one sum
            y, term_rows = ops.moe_experts_single(x, ids, self.up, self.down, self.slots)
            return ops.moe_mix(y, term_rows, ids, scores, self.experts, x, shared,
                               routed[2] if self.shared_gate is not None else None)
        y, term_rows = ops.moe_experts(x, ids, scores, self.gate_up, self.down, self.run)
        if as_terms:
            return {"terms": y, "extra": shared, "term_rows": term_rows, "count": self.top}
        return ops.moe_combine(y, shared, self.runtime.dtype, term_rows, self.top)
