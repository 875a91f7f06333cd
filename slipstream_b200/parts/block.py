"""Pre-norm residual block: ``x + mixer(norm(x))`` then ``x + ffn(norm(x))``
(slipstream/models/causal_lm.py:47-48,58-61), on a float32 residual stream with
each add fused into the norm that follows it, and that norm handed to the branch
before it (`IntoNorm`), whose last projection may do both in its own launch."""

from __future__ import annotations

import torch

from .base import BLOCKS, Block, FeedForward, IntoNorm, LayerBinding, Mixer, Norm, Part, settle


@BLOCKS.register("pre_norm")
class PreNormBlock(Block):
    cuda_graph_safe = True

    def __init__(self, mixer: Mixer, feed_forward: FeedForward, mixer_norm: Norm, ffn_norm: Norm) -> None:
        self.mixer = mixer
        self.feed_forward = feed_forward
        self.mixer_norm = mixer_norm
        self.ffn_norm = ffn_norm

    def children(self) -> list[Part]:
        return [self.mixer_norm, self.mixer, self.ffn_norm, self.feed_forward]

    def forward(self, residual: torch.Tensor, pending: torch.Tensor | None, ctx,
                layer: LayerBinding) -> tuple[torch.Tensor, torch.Tensor | None]:
        residual, pending, _ = self.forward_chained(residual, pending, None, None, ctx, layer)
        return residual, pending

    def first_norm(self) -> Norm:
        return self.mixer_norm

    def forward_chained(self, residual: torch.Tensor, pending: torch.Tensor | None, normed: torch.Tensor | None,
                        following: Norm | None, ctx, layer: LayerBinding):
        x = settle(normed, self.mixer) if normed is not None else self.mixer_norm.add_norm(residual, pending)
        if self.mixer.takes_into:
            x = settle(self.mixer.forward(x, ctx, layer, into=IntoNorm(self.ffn_norm, residual)), self.feed_forward)
        else:
            x = self.ffn_norm.add_norm(residual, self.mixer.forward(x, ctx, layer))
        if following is not None and self.feed_forward.takes_into:
            return residual, None, self.feed_forward.forward(x, ctx, into=IntoNorm(following, residual))
        return residual, self.feed_forward.forward(x, ctx), None


@BLOCKS.register("branch_norm")
class BranchNormBlock(Block):
    """``x + norm1(mixer(x))`` then ``x + norm2(ffn(x))``: the norm stands on each branch's OUTPUT and the branches
    read the stream itself (in the compute dtype).  ``feed_forward`` may be None.  The kernel that adds a normed
    output also writes the new stream in the compute dtype, so the next branch, of this block or of the next one, has
    its input without a launch of its own."""

    cuda_graph_safe = True

    def __init__(self, mixer: Mixer, feed_forward: FeedForward | None, mixer_norm: Norm, ffn_norm: Norm | None) -> None:
        from .norm import StreamRounding
        if (feed_forward is None) != (ffn_norm is None):
            raise ValueError("a feed-forward and its norm come together")
        self.mixer = mixer
        self.feed_forward = feed_forward
        self.mixer_norm = mixer_norm
        self.ffn_norm = ffn_norm
        self.reader = StreamRounding()

    def children(self) -> list[Part]:
        return [p for p in (self.reader, self.mixer, self.mixer_norm, self.feed_forward, self.ffn_norm) if p is not None]

    def forward(self, residual: torch.Tensor, pending: torch.Tensor | None, ctx,
                layer: LayerBinding) -> tuple[torch.Tensor, torch.Tensor | None]:
        residual, pending, _ = self.forward_chained(residual, pending, None, None, ctx, layer)
        return residual, pending

    def first_norm(self) -> Norm:
        return self.reader

    def forward_chained(self, residual: torch.Tensor, pending: torch.Tensor | None, normed: torch.Tensor | None,
                        following: Norm | None, ctx, layer: LayerBinding):
        from .norm import StreamRounding
        x = normed if normed is not None else self.reader.add_norm(residual, pending)
        hand_over = isinstance(following, StreamRounding)  # the next block reads the rounded stream too
        last = self.feed_forward is None
        x = self.mixer_norm.add_branch(residual, self.mixer.forward(x, ctx, layer), want_out=hand_over or not last)
        if not last:
            if getattr(self.feed_forward, "can_return_terms", False):
                out = self.feed_forward.forward(x, ctx, as_terms=True)
            else:
                out = self.feed_forward.forward(x, ctx)
            if isinstance(out, dict):  # a feed-forward whose output is a sum it has not formed: the norm's kernel does
                x = self.ffn_norm.add_branch(residual, out["terms"], terms=out["count"], extra=out.get("extra"),
                                             term_rows=out.get("term_rows"), want_out=hand_over)
            else:
                x = self.ffn_norm.add_branch(residual, out, want_out=hand_over)
        return residual, None, (x if hand_over else None)


@BLOCKS.register("parallel_branches")
class ParallelBlock(Block):
    """``x + (mixer(norm(x)) + ffn(norm(x)))``: ONE norm whose output both branches read; their outputs are added to the
    stream together.  ``feed_forward`` may be None.  ``norm`` is a `ConnectedNorm` (one stream: the plain residual
    sum), whose kernel applies the block's pending pair of outputs where the next norm reads the stream."""

    cuda_graph_safe = True

    def __init__(self, mixer: Mixer, feed_forward: FeedForward | None, norm: Norm) -> None:
        self.mixer = mixer
        self.feed_forward = feed_forward
        self.norm = norm

    def children(self) -> list[Part]:
        return [p for p in (self.norm, self.mixer, self.feed_forward) if p is not None]

    def forward(self, residual: torch.Tensor, pending, ctx, layer: LayerBinding):
        residual, pending, _ = self.forward_chained(residual, pending, None, None, ctx, layer)
        return residual, pending

    def first_norm(self) -> Norm:
        return self.norm

    def forward_chained(self, residual: torch.Tensor, pending, normed, following: Norm | None, ctx, layer: LayerBinding):
        if normed is not None:
            x = normed if isinstance(normed, torch.Tensor) else normed.materialize()  # two branches read it
        else:
            x = self.norm.add_norm(residual, pending)
        mixed = self.mixer.forward(x, ctx, layer)
        fed = self.feed_forward.forward(x, ctx) if self.feed_forward is not None else None
        return residual, self.norm.write_of(mixed, fed), None
