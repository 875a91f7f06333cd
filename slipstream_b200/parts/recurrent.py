"""Recurrent mixers with fixed-size per-request state, and a short convolution laid over any mixer's input.

`MatrixMemoryMixer`: the matrix memory of xLSTM (mLSTM).  Per head, with q, k of ``dim`` elements (q times
``dim ** -0.5``), v of ``value_dim`` elements and two scalar gates a token,

    i = cap tanh((w_i . x + b_i) / cap),   f = logsigmoid(cap tanh((w_f . x + b_f) / cap)),
    m' = max(f + m, i),   S <- exp(f + m - m') S + exp(i - m') k v^T,   n <- likewise with k alone,
    o = S^T q / (max(|n . q|, exp(-m')) + 1e-6),

m starting at 0 and S, n at zero.  Every head of o is divided by its root mean square, the concatenated heads are
multiplied by a weight and by ``sigmoid(W_g x)``, and projected back.  S, n and m live in the request's state slot.

`GatedRecurrenceMixer`: minGRU.  ``z = sigmoid(W_z x + b_z)``, ``u = W_x x + b_x``, candidate ``u + 1/2`` where
``u >= 0`` and ``sigmoid(u)`` below, ``S <- (1 - z) S + z candidate`` element by element, output
``W_o (S silu(W_g x))``.  S lives in the request's state slot.

`ConvolvedInput`: wraps a mixer so that it reads ``x + conv(x)`` instead of ``x``, a causal convolution per channel
over ``taps`` tokens whose last ``taps - 1`` inputs live in the request's state slot.

`DecayedLinearAttention`: linear attention with a fixed decay per head.  With q, k of ``dim`` elements and v of
``value_dim`` per head, all three under silu: ``S <- decay_h S + k v^T``, ``o = S^T q`` (no other scale).  The
concatenated heads of o pass one RMS norm with a weight, are multiplied by ``sigmoid(W_g x)`` and projected back.  S
lives in the request's state slot.

`GatedLinearRecurrenceMixer`: the recurrent block around a real-gated linear recurrent unit.  Two branches of
``width`` channels: ``y = gelu_tanh(W_y x + b_y)`` and ``u = conv(W_x x + b_x)``, a causal convolution per channel with a
bias and no activation.  u is cut into ``blocks`` equal parts; in part b ``r = sigmoid(A_b u_b + a_b)`` and
``i = sigmoid(B_b u_b + b_b)`` with square matrices A_b, B_b; ``a = exp(-rate r softplus(lam))``,
``S <- a S + sqrt(1 - a^2) (i u)`` element by element from S = 0; output ``W_o (S y)``.  S and the convolution's last
inputs live in the request's state slot.

`ParallelMixers`: two mixers that read the same input; the result is ``left_scale * left + right_scale * right``.

Gates, biases, decays, states and norms are float32; the projections are in the compute dtype, except the two
gate rows of the matrix memory, whose product leaves in float32.
"""

from __future__ import annotations

import torch

from slipstream_b200 import ops

from .base import MIXERS, CacheSpec, IntoNorm, LayerBinding, Mixer, Part, Runtime, StateSpec, WeightSpec


def _f32(t: torch.Tensor) -> torch.Tensor:
    return t.to(torch.float32).contiguous()  # exact: the stored values are kept


def _pad_rows(w: torch.Tensor, multiple: int = 8) -> torch.Tensor:
    """Rows of zeros behind a stacked projection, so that every token's output row starts on a 16-byte boundary."""
    pad = -w.shape[0] % multiple
    return torch.cat([w, w.new_zeros((pad, w.shape[1]))]).contiguous() if pad else w.contiguous()


@MIXERS.register("matrix_memory")
class MatrixMemoryMixer(Mixer):
    cuda_graph_safe = True
    takes_into = True
    takes_pending_norm = False  # two products read the input

    def __init__(self, name: str, hidden_size: int, heads: int, dim: int, value_dim: int, gate_cap: float,
                 norm_eps: float = 1e-6, names: dict[str, str] | None = None) -> None:
        """``names``: the checkpoint's tensor names by role (q, k, v, g, o, norm, i, i_bias, f, f_bias)."""
        if heads < 1 or not 1 <= dim <= 256 or value_dim < 1 or not gate_cap > 0.0:
            raise ValueError("heads and value_dim must be >= 1, dim between 1 and 256, gate_cap positive")
        self.name, self.hidden_size = name, hidden_size
        self.heads, self.dim, self.value_dim = heads, dim, value_dim
        self.gate_cap, self.norm_eps = float(gate_cap), float(norm_eps)
        self.names = {role: f"{name}.{role}" for role in ("q", "k", "v", "g", "o", "norm", "i", "f")}
        self.names.update({"i_bias": f"{name}.i.b", "f_bias": f"{name}.f.b"})
        self.names.update(names or {})

    def weight_specs(self) -> list[WeightSpec]:
        n, w, h, d, v = self.names, self.hidden_size, self.heads, self.dim, self.value_dim
        return [WeightSpec(n["q"], (h * d, w)), WeightSpec(n["k"], (h * d, w)), WeightSpec(n["v"], (h * v, w)),
                WeightSpec(n["g"], (h * v, w)), WeightSpec(n["o"], (w, h * v)),
                WeightSpec(n["norm"], (h * v,), kind="vector", init=("one_plus_normal", 0.1)),
                WeightSpec(n["i"], (h, w)), WeightSpec(n["i_bias"], (h,), kind="vector", init=("normal", 0.5)),
                WeightSpec(n["f"], (h, w)), WeightSpec(n["f_bias"], (h,), kind="vector", init=("one_plus_normal", 1.0))]

    def state_specs(self) -> list[StateSpec]:
        # S column by column with n as one more column, and the running maximum m
        return [StateSpec("memory", (self.heads, self.value_dim + 1, self.dim)), StateSpec("peak", (self.heads,))]

    def bind(self, weights: dict[str, torch.Tensor], runtime: Runtime) -> None:
        super().bind(weights, runtime)
        n = self.names
        self.qkvg_weight = _pad_rows(torch.cat([weights[n[r]] for r in ("q", "k", "v", "g")], dim=0))
        self.gate_weight = torch.cat([weights[n["i"]], weights[n["f"]]], dim=0).contiguous()
        self.bias_i, self.bias_f = _f32(weights[n["i_bias"]]), _f32(weights[n["f_bias"]])
        self.norm_weight = _f32(weights[n["norm"]])
        self.o_weight = weights[n["o"]]

    def weight_bytes(self) -> int:
        return (self.qkvg_weight.numel() + self.gate_weight.numel() + self.o_weight.numel()) * self.o_weight.element_size()

    def forward(self, x: torch.Tensor, ctx, layer: LayerBinding, into: IntoNorm | None = None) -> torch.Tensor:
        h, d, v = self.heads, self.dim, self.value_dim
        proj = ops.linear(x, self.qkvg_weight)
        gates = ops.linear(x, self.gate_weight, None, out_dtype=torch.float32)
        num, nq, peaks = ops.matrix_cell(proj, gates, self.bias_i, self.bias_f, self.gate_cap, d ** -0.5,
                                         layer.state["memory"], layer.state["peak"], ctx, h, d, v)
        g0 = h * (2 * d + v)
        out = ops.cell_output(num, nq, peaks, self.norm_weight, proj[:, g0: g0 + h * v], h, v, self.norm_eps,
                              self.runtime.dtype)
        if into is not None:
            return into.close(out, self.o_weight, None)
        return ops.linear(out, self.o_weight)


@MIXERS.register("gated_recurrence")
class GatedRecurrenceMixer(Mixer):
    cuda_graph_safe = True
    takes_into = True
    takes_pending_norm = True  # the input goes to one product and nowhere else

    def __init__(self, name: str, hidden_size: int, width: int, names: dict[str, str] | None = None) -> None:
        """``names``: the checkpoint's tensor names by role (z, z_bias, x, x_bias, g, o)."""
        if width < 1:
            raise ValueError("width must be >= 1")
        self.name, self.hidden_size, self.width = name, hidden_size, width
        self.names = {"z": f"{name}.z", "z_bias": f"{name}.z.b", "x": f"{name}.x", "x_bias": f"{name}.x.b",
                      "g": f"{name}.g", "o": f"{name}.o"}
        self.names.update(names or {})

    def weight_specs(self) -> list[WeightSpec]:
        n, w, r = self.names, self.hidden_size, self.width
        return [WeightSpec(n["z"], (r, w)), WeightSpec(n["z_bias"], (r,), kind="vector", init=("normal", 0.5)),
                WeightSpec(n["x"], (r, w)), WeightSpec(n["x_bias"], (r,), kind="vector", init=("normal", 0.5)),
                WeightSpec(n["g"], (r, w)), WeightSpec(n["o"], (w, r))]

    def state_specs(self) -> list[StateSpec]:
        return [StateSpec("cell", (self.width,))]

    def bind(self, weights: dict[str, torch.Tensor], runtime: Runtime) -> None:
        super().bind(weights, runtime)
        n = self.names
        self.in_weight = _pad_rows(torch.cat([weights[n[r]] for r in ("z", "x", "g")], dim=0))
        self.bias = torch.cat([_f32(weights[n["z_bias"]]), _f32(weights[n["x_bias"]])]).contiguous()
        self.o_weight = weights[n["o"]]

    def weight_bytes(self) -> int:
        return (self.in_weight.numel() + self.o_weight.numel()) * self.o_weight.element_size()

    def forward(self, x: torch.Tensor, ctx, layer: LayerBinding, into: IntoNorm | None = None) -> torch.Tensor:
        proj = ops.linear(x, self.in_weight)
        out = ops.gated_recurrence(proj, self.width, layer.state["cell"], ctx, bias=self.bias)
        if into is not None:
            return into.close(out, self.o_weight, None)
        return ops.linear(out, self.o_weight)


@MIXERS.register("convolved_input")
class ConvolvedInput(Mixer):
    """``inner(x + conv(x))``: ``conv(x)_t = sum_j taps[:, j] * x_(t - T + 1 + j)`` per channel, zeros in front of a
    request's first token, no bias and no activation.  The sum is formed in float32 and rounded to the compute dtype
    once.  Pages and state are the inner mixer's, which is also the part that is asked about captured forms."""

    takes_pending_norm = False  # the convolution reads the normed input itself

    def __init__(self, inner: Mixer, hidden_size: int, taps: int, tensor: str) -> None:
        if not 1 <= taps <= 8:
            raise ValueError("between 1 and 8 taps")
        self.inner, self.hidden_size, self.taps, self.tensor = inner, hidden_size, int(taps), tensor
        self.takes_into = inner.takes_into
        self.cuda_graph_safe = getattr(inner, "cuda_graph_safe", False)

    def children(self) -> list[Part]:
        return [self.inner]

    def weight_specs(self) -> list[WeightSpec]:
        return [WeightSpec(self.tensor, (self.hidden_size, self.taps), kind="vector", init=("normal", 0.3))]

    def cache_spec(self) -> CacheSpec | None:
        return self.inner.cache_spec()

    def state_specs(self) -> list[StateSpec]:
        return [*self.inner.state_specs(), StateSpec("input_taps", (max(self.taps - 1, 0), self.hidden_size))]

    def bind(self, weights: dict[str, torch.Tensor], runtime: Runtime) -> None:
        super().bind(weights, runtime)
        self.tap_weights = _f32(weights[self.tensor])

    def forward(self, x: torch.Tensor, ctx, layer: LayerBinding, into: IntoNorm | None = None) -> torch.Tensor:
        x = ops.conv_silu(x, 0, self.hidden_size, self.tap_weights, None, layer.state["input_taps"], ctx, plus_input=True)
        if self.takes_into:
            return self.inner.forward(x, ctx, layer, into=into)
        return self.inner.forward(x, ctx, layer)


@MIXERS.register("decayed_linear_attention")
class DecayedLinearAttention(Mixer):
    cuda_graph_safe = True
    takes_into = True
    takes_pending_norm = True  # the input goes to one product and nowhere else

    def __init__(self, name: str, hidden_size: int, heads: int, dim: int, value_dim: int, decay: "tuple[float, ...]",
                 norm_eps: float = 1e-6, names: dict[str, str] | None = None) -> None:
        """``decay``: one number per head.  ``names``: the checkpoint's tensor names by role (q, k, v, g, o, norm)."""
        if heads < 1 or not 1 <= dim <= 256 or value_dim < 1 or len(decay) != heads:
            raise ValueError("heads and value_dim must be >= 1, dim between 1 and 256, one decay per head")
        self.name, self.hidden_size = name, hidden_size
        self.heads, self.dim, self.value_dim = heads, dim, value_dim
        self.decay, self.norm_eps = tuple(float(d) for d in decay), float(norm_eps)
        self.names = {role: f"{name}.{role}" for role in ("q", "k", "v", "g", "o", "norm")}
        self.names.update(names or {})

    def weight_specs(self) -> list[WeightSpec]:
        n, w, h, d, v = self.names, self.hidden_size, self.heads, self.dim, self.value_dim
        return [WeightSpec(n["q"], (h * d, w)), WeightSpec(n["k"], (h * d, w)), WeightSpec(n["v"], (h * v, w)),
                WeightSpec(n["g"], (h * v, w)), WeightSpec(n["o"], (w, h * v)),
                WeightSpec(n["norm"], (h * v,), kind="vector", init=("one_plus_normal", 0.1))]

    def state_specs(self) -> list[StateSpec]:
        return [StateSpec("memory", (self.heads, self.dim, self.value_dim))]  # S, row by row

    def bind(self, weights: dict[str, torch.Tensor], runtime: Runtime) -> None:
        super().bind(weights, runtime)
        n = self.names
        self.qkvg_weight = _pad_rows(torch.cat([weights[n[r]] for r in ("q", "k", "v", "g")], dim=0))
        self.decay_weight = torch.tensor(self.decay, dtype=torch.float64).to(torch.float32).to(runtime.device)
        self.norm_weight = _f32(weights[n["norm"]])
        self.o_weight = weights[n["o"]]

    def weight_bytes(self) -> int:
        return (self.qkvg_weight.numel() + self.o_weight.numel()) * self.o_weight.element_size()

    def forward(self, x: torch.Tensor, ctx, layer: LayerBinding, into: IntoNorm | None = None) -> torch.Tensor:
        h, d, v = self.heads, self.dim, self.value_dim
        proj = ops.linear(x, self.qkvg_weight)
        mixed = ops.decay_attention(proj, self.decay_weight, layer.state["memory"], ctx, h, d, v)
        g0 = h * (2 * d + v)
        out = ops.gated_rmsnorm(mixed, proj[:, g0: g0 + h * v], self.norm_weight, self.norm_eps, self.runtime.dtype)
        if into is not None:
            return into.close(out, self.o_weight, None)
        return ops.linear(out, self.o_weight)


@MIXERS.register("gated_linear_recurrence")
class GatedLinearRecurrenceMixer(Mixer):
    cuda_graph_safe = True
    takes_into = True
    takes_pending_norm = True  # the input goes to one product and nowhere else

    def __init__(self, name: str, hidden_size: int, width: int, blocks: int, taps: int, rate: float = 8.0,
                 names: dict[str, str] | None = None) -> None:
        """``rate``: the constant in ``a = exp(-rate r softplus(lam))``.  ``names``: the checkpoint's tensor names by role
        (y, y_bias, x, x_bias, conv, conv_bias, ra, ra_bias, ri, ri_bias, lam, o)."""
        if width < 1 or blocks < 1 or width % blocks or not 1 <= taps <= 8:
            raise ValueError("width must split into blocks equal parts, taps between 1 and 8")
        self.name, self.hidden_size, self.width, self.blocks, self.taps = name, hidden_size, width, blocks, int(taps)
        self.rate = float(rate)
        self.names = {role: f"{name}.{role}" for role in ("y", "x", "conv", "ra", "ri", "lam", "o")}
        self.names.update({f"{role}_bias": f"{name}.{role}.b" for role in ("y", "x", "conv", "ra", "ri")})
        self.names.update(names or {})

    def weight_specs(self) -> list[WeightSpec]:
        n, w, r, b = self.names, self.hidden_size, self.width, self.blocks
        bs = r // b
        return [WeightSpec(n["y"], (r, w)), WeightSpec(n["y_bias"], (r,), kind="vector", init=("normal", 0.2)),
                WeightSpec(n["x"], (r, w)), WeightSpec(n["x_bias"], (r,), kind="vector", init=("normal", 0.2)),
                WeightSpec(n["conv"], (r, self.taps), init=("normal", 0.3)),
                WeightSpec(n["conv_bias"], (r,), kind="vector", init=("normal", 0.2)),
                WeightSpec(n["ra"], (b, bs, bs), init=("normal", 0.1)), WeightSpec(n["ra_bias"], (b, bs), kind="vector", init=("normal", 0.5)),
                WeightSpec(n["ri"], (b, bs, bs), init=("normal", 0.1)), WeightSpec(n["ri_bias"], (b, bs), kind="vector", init=("normal", 0.5)),
                WeightSpec(n["lam"], (r,), kind="vector", init=("normal", 1.0)), WeightSpec(n["o"], (w, r))]

    def state_specs(self) -> list[StateSpec]:
        return [StateSpec("conv", (self.taps - 1, self.width)), StateSpec("cell", (self.width,))]

    def bind(self, weights: dict[str, torch.Tensor], runtime: Runtime) -> None:
        super().bind(weights, runtime)
        n = self.names
        self.in_weight = _pad_rows(torch.cat([weights[n["y"]], weights[n["x"]]], dim=0))
        bias = torch.cat([weights[n["y_bias"]], weights[n["x_bias"]]]).to(runtime.dtype)
        self.in_bias = torch.cat([bias, bias.new_zeros(self.in_weight.shape[0] - bias.numel())]).contiguous()
        self.conv_taps, self.conv_bias = _f32(weights[n["conv"]]), _f32(weights[n["conv_bias"]])
        # per block the first gate's rows, then the second's: one product for both
        self.gate_weight = torch.cat([weights[n["ra"]], weights[n["ri"]]], dim=1).to(runtime.dtype).contiguous()
        self.gate_bias = torch.cat([_f32(weights[n["ra_bias"]]), _f32(weights[n["ri_bias"]])], dim=1).contiguous()
        self.lam = _f32(weights[n["lam"]])
        self.o_weight = weights[n["o"]]

    def weight_bytes(self) -> int:
        return (self.in_weight.numel() + self.gate_weight.numel() + self.o_weight.numel()) * self.o_weight.element_size()

    def forward(self, x: torch.Tensor, ctx, layer: LayerBinding, into: IntoNorm | None = None) -> torch.Tensor:
        r = self.width
        proj = ops.linear(x, self.in_weight, self.in_bias)
        u = ops.conv_silu(proj, r, r, self.conv_taps, self.conv_bias, layer.state["conv"], ctx, activation=False)
        pre = ops.block_gates(u, self.gate_weight)
        out = ops.gated_linear_recurrence(pre, self.gate_bias, u, proj[:, :r], self.lam, self.rate, layer.state["cell"], ctx)
        if into is not None:
            return into.close(out, self.o_weight, None)
        return ops.linear(out, self.o_weight)


@MIXERS.register("parallel_mixers")
class ParallelMixers(Mixer):
    """``left_scale * left(x) + right_scale * right(x)``: two mixers side by side on the same input.  At most one of
    them keeps pages (its `cache_spec` is the pair's); both may keep state, which the pair declares under the names
    ``left.<name>`` and ``right.<name>`` and hands to each side under its own names.  The sum is formed in float32 and
    rounded once."""

    takes_into = False
    takes_pending_norm = False  # two products read the input

    def __init__(self, left: Mixer, right: Mixer, left_scale: float = 1.0, right_scale: float = 1.0) -> None:
        if left.cache_spec() is not None and right.cache_spec() is not None:
            raise ValueError("at most one side of a pair of mixers keeps pages")
        self.left, self.right = left, right
        self.left_scale, self.right_scale = float(left_scale), float(right_scale)
        self.cuda_graph_safe = all(getattr(m, "cuda_graph_safe", False) for m in (left, right))

    def children(self) -> list[Part]:
        return [self.left, self.right]

    def cache_spec(self) -> CacheSpec | None:
        return self.left.cache_spec() or self.right.cache_spec()

    def state_specs(self) -> list[StateSpec]:
        return [StateSpec(f"{side}.{s.name}", s.shape, s.dtype)
                for side, m in (("left", self.left), ("right", self.right)) for s in m.state_specs()]

    @staticmethod
    def _side(layer: LayerBinding, side: str, keeps_pages: bool) -> LayerBinding:
        state = {k[len(side) + 1:]: v for k, v in layer.state.items() if k.startswith(side + ".")}
        if keeps_pages:
            return LayerBinding(kv=layer.kv, group=layer.group, writes_cache=layer.writes_cache, state=state)
        return LayerBinding(state=state)

    def forward(self, x: torch.Tensor, ctx, layer: LayerBinding) -> torch.Tensor:
        left_pages = self.left.cache_spec() is not None
        a = self.left.forward(x, ctx, self._side(layer, "left", left_pages))
        b = self.right.forward(x, ctx, self._side(layer, "right", not left_pages and self.right.cache_spec() is not None))
        return ops.scaled_sum(a, self.left_scale, b, self.right_scale)
