"""Several residual streams per token, joined by hyper-connections.

A model of this kind keeps S copies x_0 .. x_{S-1} of the residual stream (float32 ``[tokens, S, hidden]``), all
equal to the embedding output at first.  A branch (a mixer or a feed-forward) with connection weights
``in`` [S], ``out`` [S] and ``mix`` [S, S] (indexed [from, to])

    reads    u = sum_s in[s] * x_s,   runs  y = branch(norm(u)),
    writes   x_t <- sum_s mix[s, t] * x_s + out[t] * y     for all t at once, from the old streams.

The model's output is the plain sum of the streams.  With S = 1 and in = out = mix = 1 this is the ordinary
pre-norm residual block, which is how a model without the connections runs through the same parts.

``ConnectedNorm`` is the read + norm of one branch, fused with the WRITE OF THE BRANCH IN FRONT (one kernel per
branch boundary, `ops.hc_norm`): a branch's output travels as a ``StreamWrite`` until the next norm applies it, the
way a plain block's output stays pending until the next add + norm.  ``HyperConnectionBlock`` arranges a mixer and
an optional feed-forward around the streams.
"""

from __future__ import annotations

from dataclasses import dataclass

import numpy as np
import torch

from slipstream_b200 import ops

from .base import BLOCKS, NORMS, Block, FeedForward, IntoNorm, LayerBinding, Mixer, Norm, Part, Runtime, WeightSpec, settle


@dataclass
class StreamWrite:
    """A branch output that has not been written into the streams yet, with its branch's write weights.  ``y2``: the
    output of a second branch that read the same input; the two are added (in float32) where they are written."""

    y: torch.Tensor
    mix: torch.Tensor  # float32 [S, S], [from, to]
    out: torch.Tensor  # float32 [S]
    y2: torch.Tensor | None = None


@dataclass
class IntoStreams(IntoNorm):
    """`IntoNorm` for hyper-connected streams: the branch's last projection is written into the streams with the
    weights of ``writer`` (the branch's own norm) and ``norm`` (the next branch's) reads and norms what results."""

    writer: "ConnectedNorm" = None

    def close(self, x: torch.Tensor, weight: torch.Tensor, bias: torch.Tensor | None):
        return self.norm.write_linear_then_norm(self.residual, x, weight, bias, self.writer)


@NORMS.register("connected_rmsnorm")
class ConnectedNorm(Norm):
    """RMS norm of a weighted sum of the streams, and the connection weights of the branch behind it.

    ``tensor``: the norm's weight vector.  ``connection``: prefix of the branch's ``.in``, ``.out`` and ``.mix``
    tensors; None stands for in = 1 (the plain sum) and, for `write_of`, out = 1 and mix = identity, which needs
    no tensors.  ``offset``: the tensor holds the weight's difference from ``offset`` and the norm multiplies by ``offset + weight``
    (formed once, in float32).  All arithmetic is float32; the result is rounded once."""

    cuda_graph_safe = True

    def __init__(self, tensor: str, size: int, eps: float, streams: int = 1, connection: str | None = None,
                 offset: float = 0.0) -> None:
        if not 1 <= streams <= 8:
            raise ValueError("between 1 and 8 residual streams")
        self.offset = float(offset)
        self.tensor = tensor
        self.size = size
        self.eps = float(eps)
        self.streams = int(streams)
        self.connection = connection

    def weight_specs(self) -> list[WeightSpec]:
        specs = [WeightSpec(self.tensor, (self.size,), kind="vector",
                            init=("normal", 0.1) if self.offset else ("one_plus_normal", 0.1))]
        if self.connection is not None:
            s = self.streams
            specs += [WeightSpec(f"{self.connection}.in", (s,), kind="vector", init=("one_plus_normal", 0.2)),
                      WeightSpec(f"{self.connection}.out", (s,), kind="vector", init=("one_plus_normal", 0.2)),
                      WeightSpec(f"{self.connection}.mix", (s, s), kind="vector", init=("normal", 0.5))]
        return specs

    def bind(self, weights: dict[str, torch.Tensor], runtime: Runtime) -> None:
        super().bind(weights, runtime)
        self.weight = weights[self.tensor]
        if self.offset:
            self.weight = (self.weight.to(torch.float32) + self.offset).contiguous()
        s, dev = self.streams, runtime.device
        if self.connection is not None:
            self.w_in = weights[f"{self.connection}.in"].to(torch.float32).contiguous()
            self.w_out = weights[f"{self.connection}.out"].to(torch.float32).contiguous()
            self.mix = weights[f"{self.connection}.mix"].to(torch.float32).contiguous()
        else:
            self.w_in = None
            self.w_out = torch.ones(s, dtype=torch.float32, device=dev)
            self.mix = torch.eye(s, dtype=torch.float32, device=dev)
        # the same weights on the host: a product that writes into the streams itself takes them as launch arguments
        self.host_write = np.concatenate([self.mix.cpu().numpy().reshape(-1), self.w_out.cpu().numpy().reshape(-1)])
        self.host_in = self.w_in.cpu().numpy().reshape(-1) if self.w_in is not None else np.ones(s, dtype=np.float32)
        self._fused: dict[int, np.ndarray] = {}

    def weight_bytes(self) -> int:
        return self.weight.numel() * self.weight.element_size()

    def write_of(self, y: torch.Tensor, y2: torch.Tensor | None = None) -> StreamWrite:
        """``y`` (plus ``y2``, a second branch's) as the output of the branch behind this norm."""
        return StreamWrite(y, self.mix, self.w_out, y2)

    def add_norm(self, residual: torch.Tensor, delta: "StreamWrite | None",
                 rows: torch.Tensor | None = None) -> torch.Tensor:
        """Apply the pending write ``delta`` to the streams (in place; not with ``rows``), read this branch's
        input out of them and norm it."""
        streams = residual if residual.dim() == 3 else residual.view(residual.shape[0], 1, residual.shape[1])
        if streams.shape[1] != self.streams:
            raise ValueError(f"{streams.shape[1]} streams where the norm expects {self.streams}")
        if delta is None:
            return ops.hc_norm(streams, None, None, None, self.w_in, self.weight, self.eps, self.runtime.dtype, rows=rows)
        return ops.hc_norm(streams, delta.y, delta.mix, delta.out, self.w_in, self.weight, self.eps, self.runtime.dtype,
                           rows=rows, y2=delta.y2)

    def write_linear_then_norm(self, residual: torch.Tensor, x: torch.Tensor, weight: torch.Tensor,
                               bias: torch.Tensor | None, writer: "ConnectedNorm"):
        """``add_norm(residual, writer.write_of(x @ weight.T + bias))``: a branch's last projection, its write into the
        streams and this norm's read; may come back as an ``ops.PendingNorm`` (see `ops.linear_hc_rmsnorm`)."""
        streams = residual if residual.dim() == 3 else residual.view(residual.shape[0], 1, residual.shape[1])
        host = self._fused.get(id(writer))
        if host is None:
            host = self._fused[id(writer)] = np.ascontiguousarray(
                np.concatenate([writer.host_write, self.host_in]).astype(np.float32))
        return ops.linear_hc_rmsnorm(x, weight, bias, streams, writer.mix, writer.w_out, self.w_in, host, self.weight,
                                     self.eps, self.runtime.dtype)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        return self.add_norm(x, None)


@BLOCKS.register("hyper_connection")
class HyperConnectionBlock(Block):
    """A mixer and an optional feed-forward, each reading from and writing to the residual streams through its
    `ConnectedNorm`.  The last branch's output leaves the block as a pending `StreamWrite`; the next block's first
    norm (or the model's final norm, a `ConnectedNorm` without a connection: the plain sum) applies it."""

    cuda_graph_safe = True

    def __init__(self, mixer: Mixer, feed_forward: FeedForward | None, mixer_norm: ConnectedNorm,
                 ffn_norm: ConnectedNorm | None) -> None:
        if (feed_forward is None) != (ffn_norm is None):
            raise ValueError("a feed-forward and its norm come together")
        self.mixer = mixer
        self.feed_forward = feed_forward
        self.mixer_norm = mixer_norm
        self.ffn_norm = ffn_norm

    def children(self) -> list[Part]:
        parts: list[Part] = [self.mixer_norm, self.mixer]
        if self.feed_forward is not None:
            parts += [self.ffn_norm, self.feed_forward]
        return parts

    def forward(self, residual: torch.Tensor, pending: "StreamWrite | None", ctx,
                layer: LayerBinding) -> "tuple[torch.Tensor, StreamWrite]":
        residual, pending, _ = self.forward_chained(residual, pending, None, None, ctx, layer)
        return residual, pending

    def first_norm(self) -> Norm:
        return self.mixer_norm

    def forward_chained(self, residual: torch.Tensor, pending: "StreamWrite | None", normed, following: Norm | None, ctx,
                        layer: LayerBinding):
        """A branch whose last operation is a projection hands that projection, its write into the streams and the
        next norm to one call (`IntoStreams`); the next norm is this block's second one, the next block's first one
        (``following``) or the model's last one."""
        chain = following if isinstance(following, ConnectedNorm) else None
        x = settle(normed, self.mixer) if normed is not None else self.mixer_norm.add_norm(residual, pending)
        after_mixer = self.ffn_norm if self.feed_forward is not None else chain
        if self.mixer.takes_into and after_mixer is not None:
            x = self.mixer.forward(x, ctx, layer, into=IntoStreams(after_mixer, residual, self.mixer_norm))
            if self.feed_forward is None:
                return residual, None, x
            x = settle(x, self.feed_forward)
        else:
            pending = self.mixer_norm.write_of(self.mixer.forward(x, ctx, layer))
            if self.feed_forward is None:
                return residual, pending, None
            x = self.ffn_norm.add_norm(residual, pending)
        if chain is not None and self.feed_forward.takes_into:
            return residual, None, self.feed_forward.forward(x, ctx, into=IntoStreams(chain, residual, self.ffn_norm))
        return residual, self.ffn_norm.write_of(self.feed_forward.forward(x, ctx)), None
