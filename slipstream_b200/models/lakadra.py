"""Builder of the Lakadra decoder from ``LakadraConfig``: which parts stand in which layer, with which constants and
tensor names.

Embedding ``embed``.  Per layer ``l<i>`` a `ParallelBlock`: ONE norm (``l<i>.norm1``, weight stored as its
difference from one) whose output the mixer and the feed-forward both read, their outputs added to the stream
together.  The mixer, by ``type``:

* ``lightning``: a `DecayedLinearAttention` (``l<i>.mix.{q,k,v,g,o,norm}``), whose matrix state lives in the
  request's state slot;
* ``latent_attention``: a `LatentAttention` without sinks and gates (``l<i>.mix.{dq,dq.norm,uq,dkv,dkv.norm,uk,uv,o}``)
  with pairs of neighbours in the rotated part.  A layer whose mixer names ``kv_from`` has no ``dkv``: its entry in the
  model's order reads the pages of that layer;
* ``parallel``: `ParallelMixers` of a `PagedAttention` (``l<i>.mix.left.{q,k,v,o}`` with biases ``.b``, a gate per head
  ``l<i>.mix.left.g``, half-split rotary pairs with stretched positions, a sliding window, one more 1 in the softmax's
  denominator) and a `GatedLinearRecurrenceMixer` (``l<i>.mix.right.{y,x,conv,ra,ri}`` with biases ``.b``,
  ``l<i>.mix.right.{lam,o}``), each side times its scale.

The feed-forward, unless ``mlp`` is null: `RoutedExperts` in their un-gated form (``l<i>.mlp.e<k>.{up,down}``) with a
softmax router (``l<i>.mlp.router``), a correction on the choice (``l<i>.mlp.correction``), groups, experts that hand
their input on, and a shared expert (``l<i>.mlp.shared.{up,down}``) under a gate per token (``l<i>.mlp.shared.sg``).
``final.norm`` (weight around zero), ``head``, the logits times a constant and under a soft cap.
"""

from __future__ import annotations

from slipstream_b200.config.lakadra_config import LakadraConfig
from slipstream_b200.parts import (ActivatedFeedForward, ConnectedNorm, DecayedLinearAttention, GatedLinearRecurrenceMixer,
                                   LatentAttention, LMHead, NoPositionEncoding, PagedAttention, ParallelBlock,
                                   ParallelMixers, RotaryEncoding, RoutedExperts, TokenEmbedding, YarnRotaryEncoding)

from .decoder import DecoderLM, ExecEntry

NORM_OFFSET = 1.0  # the norms multiply by 1 + the stored weight
RECURRENCE_RATE = 8.0  # a = exp(-8 r softplus(lam))


def _latent_rotary(rot, rot_dim: int, made: dict):
    """One encoding object per distinct rotation of a latent layer's shared key part (pairs of neighbours)."""
    key = ("latent", rot, rot_dim)
    if key not in made:
        if rot is None or rot_dim == 0:
            made[key] = NoPositionEncoding()
        elif rot.scaling is None:
            made[key] = RotaryEncoding(rot_dim, rot.base, rot.dims, interleaved=True, exact_table=True)
        else:
            factor, original, fast, slow = rot.scaling
            made[key] = YarnRotaryEncoding(rot_dim, rot.base, rot.dims, interleaved=True, factor=factor, original=original,
                                           fast=fast, slow=slow)
    return made[key]


def _head_rotary(rot, head_dim: int, made: dict):
    key = ("heads", rot, head_dim)
    if key not in made:
        made[key] = (NoPositionEncoding() if rot is None
                     else RotaryEncoding(head_dim, rot.base, rot.dims, exact_table=True, stretch=rot.factor))
    return made[key]


def build_lakadra(config: LakadraConfig) -> DecoderLM:
    c = config
    width = c.hidden_size
    blocks, order, rotaries = [], [], {}

    def norm(tensor: str) -> ConnectedNorm:
        return ConnectedNorm(tensor, width, c.norm_eps, 1, None, offset=NORM_OFFSET)

    for i, layer in enumerate(c.layers):
        p, m = f"l{i}", layer.mixer
        kv_from = None
        if layer.type == "lightning":
            mixer = DecayedLinearAttention(f"{p}.mix", width, m.heads, m.dim, m.vdim, m.decay, c.norm_eps)
        elif layer.type == "latent_attention":
            kv_from = m.kv_from
            mixer = LatentAttention(f"{p}.mix", width, m.heads, m.dim, m.rot_dim, m.vdim, m.q_rank, m.kv_rank, m.scale,
                                    _latent_rotary(m.rot, m.rot_dim, rotaries), c.norm_eps, sinks=False, gate=False,
                                    has_kv=kv_from is None)
        else:
            a, r = m.left, m.right
            left = PagedAttention(
                f"{p}.mix.left", width, a.heads, a.kv_heads, a.dim, _head_rotary(a.rot, a.dim, rotaries), qkv_bias=True,
                out_bias=True, window=a.window, scale=a.scale, value_dim=a.vdim, head_gate=True, unit_sink=True,
                names={**{role: f"{p}.mix.left.{role}" for role in "qkvog"},
                       **{f"{role}_bias": f"{p}.mix.left.{role}.b" for role in "qkvo"}})
            right = GatedLinearRecurrenceMixer(f"{p}.mix.right", width, r.width, r.blocks, r.conv, RECURRENCE_RATE)
            mixer = ParallelMixers(left, right, m.left_scale, m.right_scale)
        ffn = None
        if layer.mlp is not None:
            f = layer.mlp
            shared = (ActivatedFeedForward(f"{p}.mlp.shared", width, f.shared_ff, "relu2")
                      if f.shared_ff is not None else None)
            ffn = RoutedExperts(f"{p}.mlp", width, f.ff, f.experts, f.top, shared=shared, renormalize=False,
                                weight_on_input=False, router_tensor=f"{p}.mlp.router",
                                expert_names=f"{p}.mlp.e{{e}}.{{role}}", gated=False, scores="softmax",
                                correction=f"{p}.mlp.correction",
                                groups=(f.group_count, f.group_keep) if f.group_count is not None else None,
                                identity=f.identity, shared_gate=f"{p}.mlp.shared.sg" if shared is not None else None)
        blocks.append(ParallelBlock(mixer, ffn, norm(f"{p}.norm1")))
        order.append(ExecEntry(i, cache_of=kv_from))  # layer j is entry j of the order
    return DecoderLM(
        c,
        TokenEmbedding("embed", c.vocab_size, width, tensor="embed"),
        blocks,
        norm("final.norm"),
        LMHead("head", c.vocab_size, width, tied_to=None, tensor="head", softcap=c.logit_softcap, scale=c.logit_scale),
        order=order)
