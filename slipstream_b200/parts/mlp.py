"""Dense SwiGLU feed-forward: ``down(silu(gate(x)) * up(x))``
(slipstream/models/layers/mlp.py:33-40).  The gate and up matrices are stacked at
load so that one product feeds the activation kernel.

The activation has three constants, so that relatives of SwiGLU are the same part: with ``g = min(gate, limit)``
and ``u = clamp(up, -limit, limit)`` (no ``limit``: unclamped) the hidden vector is
``g * sigmoid(alpha * g) * (u + up_shift)``; alpha = 1, no limit and up_shift = 0 is SwiGLU."""

from __future__ import annotations

import torch

from slipstream_b200 import ops

from .base import FEED_FORWARDS, FeedForward, IntoNorm, Runtime, WeightSpec


@FEED_FORWARDS.register("swiglu")
class SwiGLUFeedForward(FeedForward):
    cuda_graph_safe = True
    takes_into = True
    takes_pending_norm = True

    def __init__(self, name: str, hidden_size: int, intermediate_size: int, bias: bool = False, *,
                 alpha: float = 1.0, limit: float | None = None, up_shift: float = 0.0,
                 names: dict[str, str] | None = None) -> None:
        """``names``: the checkpoint's tensor names by role (gate, up, down, gate_bias, up_bias, down_bias)."""
        self.name = name
        self.hidden_size = hidden_size
        self.intermediate_size = intermediate_size
        self.bias = bias
        self.alpha = float(alpha)
        self.limit = None if limit is None else float(limit)
        self.up_shift = float(up_shift)
        if self.limit is not None and not self.limit > 0.0:
            raise ValueError("limit must be positive")
        n = name
        self.names = {"gate": f"{n}.gate_proj.weight", "up": f"{n}.up_proj.weight", "down": f"{n}.down_proj.weight",
                      "gate_bias": f"{n}.gate_proj.bias", "up_bias": f"{n}.up_proj.bias",
                      "down_bias": f"{n}.down_proj.bias"}
        self.names.update(names or {})

    @property
    def is_swiglu(self) -> bool:
        return self.alpha == 1.0 and self.limit is None and self.up_shift == 0.0

    def weight_specs(self) -> list[WeightSpec]:
        h, i, names = self.hidden_size, self.intermediate_size, self.names
        specs = [WeightSpec(names["gate"], (i, h)), WeightSpec(names["up"], (i, h)), WeightSpec(names["down"], (h, i))]
        if self.bias:
            specs += [WeightSpec(names["gate_bias"], (i,), kind="vector"),
                      WeightSpec(names["up_bias"], (i,), kind="vector"),
                      WeightSpec(names["down_bias"], (h,), kind="vector")]
        return specs

    def bind(self, weights: dict[str, torch.Tensor], runtime: Runtime) -> None:
        super().bind(weights, runtime)
        n = self.name
        weights = {**weights, **{f"{n}.{role}_proj.weight": weights[self.names[role]] for role in ("gate", "up", "down")}}
        if self.bias:
            weights.update({f"{n}.{role}_proj.bias": weights[self.names[f"{role}_bias"]] for role in ("gate", "up", "down")})
        # gate and up rows alternate in runs of `block`, so that one 128-row tile of the stacked product holds
        # 64 gate features and the 64 matching up features (the fused epilogue needs both in one block)
        i = self.intermediate_size
        self.block = 64 if i % 64 == 0 else i

        def interleave(gate: torch.Tensor, up: torch.Tensor) -> torch.Tensor:
            g = gate.reshape(i // self.block, self.block, *gate.shape[1:])
            u = up.reshape(i // self.block, self.block, *up.shape[1:])
            return torch.stack([g, u], dim=1).reshape(2 * i, *gate.shape[1:]).contiguous()

        self.gate_up = interleave(weights[f"{n}.gate_proj.weight"], weights[f"{n}.up_proj.weight"])
        self.down = weights[f"{n}.down_proj.weight"]
        self.gate_up_bias = self.down_bias = None
        if self.bias:
            self.gate_up_bias = interleave(weights[f"{n}.gate_proj.bias"], weights[f"{n}.up_proj.bias"]).to(runtime.dtype)
            self.down_bias = weights[f"{n}.down_proj.bias"].to(runtime.dtype)

    def weight_bytes(self) -> int:
        return (self.gate_up.numel() + self.down.numel()) * self.down.element_size()

    def forward(self, x: torch.Tensor, ctx, into: IntoNorm | None = None) -> torch.Tensor:
        if self.is_swiglu:
            hidden = ops.gate_up_swiglu(x, self.gate_up, self.gate_up_bias, self.block)
        else:
            hidden = ops.gate_up_glu(x, self.gate_up, self.gate_up_bias, self.block, self.alpha, self.limit or 0.0,
                                     self.up_shift)
        if into is not None:
            return into.close(hidden, self.down, self.down_bias)
        return ops.linear(hidden, self.down, self.down_bias)


# The same part under the name of the general unit: a model whose activation is not SwiGLU builds a `GatedFeedForward`.
GatedFeedForward = FEED_FORWARDS.register("gated_linear_unit")(SwiGLUFeedForward)


def _softplus(z: float) -> float:
    import math
    return z if z > 30.0 else math.log1p(math.exp(z))


@FEED_FORWARDS.register("activated")
class ActivatedFeedForward(FeedForward):
    """A feed-forward without a gate branch: ``down(act(up(x)))``.

    ``activation`` "xielu": with two learned numbers p, q (the tensor ``act``, [2]),
    ``act(z) = softplus(p) z^2 + z / 2`` for z > 0 and ``(1/2 + softplus(q)) (exp(z) - 1 - z) + z / 2`` elsewhere; the two
    coefficients are formed once where the weights are bound, in double precision.  ``activation`` "relu2":
    ``act(z) = relu(z)^2``, no tensor.  ``names``: the checkpoint's tensor names by
    role (up, down, act)."""

    cuda_graph_safe = True
    takes_into = True
    takes_pending_norm = True

    def __init__(self, name: str, hidden_size: int, intermediate_size: int, activation: str = "xielu",
                 names: dict[str, str] | None = None) -> None:
        if activation not in ("xielu", "relu2"):
            raise ValueError(f"unknown activation {activation!r} (known: xielu, relu2)")
        self.name, self.hidden_size, self.intermediate_size, self.activation = name, hidden_size, intermediate_size, activation
        self.names = {role: f"{name}.{role}" for role in ("up", "down", "act")}
        self.names.update(names or {})

    def weight_specs(self) -> list[WeightSpec]:
        n = self.names
        specs = [WeightSpec(n["up"], (self.intermediate_size, self.hidden_size)),
                 WeightSpec(n["down"], (self.hidden_size, self.intermediate_size))]
        if self.activation == "xielu":
            specs.append(WeightSpec(n["act"], (2,), kind="vector", init=("normal", 0.5)))
        return specs

    def bind(self, weights: dict[str, torch.Tensor], runtime: Runtime) -> None:
        super().bind(weights, runtime)
        self.up, self.down = weights[self.names["up"]], weights[self.names["down"]]
        if self.activation == "xielu":
            p, q = (float(v) for v in weights[self.names["act"]].to(torch.float64).cpu())
            self.square_coeff, self.tail_coeff = _softplus(p), 0.5 + _softplus(q)

    def weight_bytes(self) -> int:
        return (self.up.numel() + self.down.numel()) * self.down.element_size()

    def forward(self, x: torch.Tensor, ctx, into: IntoNorm | None = None) -> torch.Tensor:
        if self.activation == "relu2":
            hidden = ops.relu_square(ops.linear(x, self.up))
        else:
            hidden = ops.xielu(ops.linear(x, self.up), self.square_coeff, self.tail_coeff)
        if into is not None:
            return into.close(hidden, self.down, None)
        return ops.linear(hidden, self.down)
