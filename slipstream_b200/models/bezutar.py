"""Builder of the Bezutar decoder from ``BezutarConfig``: which parts stand in which layer, with which constants and
tensor names.

Embedding: the sum of the token's row (``embed``), a hashed row of token pairs (``bigram``, when the configuration has
``embedding.bigram``) and a learned position row (``pos``, when it has ``max_positions``), copied into every residual
stream.  Per layer ``l<i>`` a `HyperConnectionBlock` (``l<i>.hc1.*`` around the mixer, ``l<i>.hc2.*`` around the
feed-forward; without ``streams`` the plain residual sum) whose norms store their weights as the difference from one
(``l<i>.norm1``, ``l<i>.norm2``).  The mixer, by ``type``:

* ``mlstm``: a `MatrixMemoryMixer` (``l<i>.mix.{q,k,v,g,o,norm,i,i.b,f,f.b}``);
* ``mingru``: a `GatedRecurrenceMixer` (``l<i>.mix.{z,z.b,x,x.b,g,o}``);
* ``latent_attention``: a `LatentAttention` (``l<i>.mix.{dq,dq.norm,uq,dkv,dkv.norm,uk,uv,sink,g,o}``) with half-split
  rotary pairs on the shared key part and the queries' rotated part, YaRN-stretched when ``rot.scaling`` is given.  A
  layer whose mixer names ``kv_from`` has no ``dkv``: its entry in the model's order reads the pages of that layer;

each behind a `ConvolvedInput` (``l<i>.canon1``) when the configuration has ``canon.taps``.  The feed-forward, unless
``mlp`` is null: an `ActivatedFeedForward` with xIELU (``l<i>.mlp.{up,down,act}``).  ``final.norm`` (weight around
zero) over the sum of the streams, then ``head``.
"""

from __future__ import annotations

from slipstream_b200.config.bezutar_config import BezutarConfig
from slipstream_b200.config.fokedra_config import RotaryConfig
from slipstream_b200.parts import (ActivatedFeedForward, ConnectedNorm, ConvolvedInput, GatedRecurrenceMixer,
                                   HyperConnectionBlock, LatentAttention, LMHead, MatrixMemoryMixer, NoPositionEncoding,
                                   RotaryEncoding, SummedEmbedding, YarnRotaryEncoding)

from .decoder import DecoderLM, ExecEntry

NORM_OFFSET = 1.0  # the norms multiply by 1 + the stored weight


def _rotary(rot: RotaryConfig | None, rot_dim: int, made: dict):
    """One encoding object per distinct rotation (layers that rotate alike share the table)."""
    if rot not in made:
        if rot is None or rot_dim == 0:
            made[rot] = NoPositionEncoding()
        elif rot.scaling is None:
            made[rot] = RotaryEncoding(rot_dim, rot.base, rot.dims, exact_table=True)
        else:
            factor, original, fast, slow = rot.scaling
            made[rot] = YarnRotaryEncoding(rot_dim, rot.base, rot.dims, factor=factor, original=original, fast=fast,
                                           slow=slow)
    return made[rot]


def build_bezutar(config: BezutarConfig) -> DecoderLM:
    c = config
    streams = c.streams or 1
    connected = c.streams is not None  # without the key there are no connection tensors: the plain residual sum
    blocks, order, rotaries = [], [], {}

    def norm(tensor: str, connection: str | None) -> ConnectedNorm:
        return ConnectedNorm(tensor, c.hidden_size, c.norm_eps, streams, connection if connected else None,
                             offset=NORM_OFFSET)

    for i, layer in enumerate(c.layers):
        p, m = f"l{i}", layer.mixer
        kv_from = None
        if layer.type == "mlstm":
            mixer = MatrixMemoryMixer(f"{p}.mix", c.hidden_size, m.heads, m.dim, m.vdim, m.gate_cap, c.norm_eps)
        elif layer.type == "mingru":
            mixer = GatedRecurrenceMixer(f"{p}.mix", c.hidden_size, m.width)
        else:
            kv_from = m.kv_from
            mixer = LatentAttention(f"{p}.mix", c.hidden_size, m.heads, m.dim, m.rot_dim, m.vdim, m.q_rank, m.kv_rank,
                                    m.scale, _rotary(m.rot, m.rot_dim, rotaries), c.norm_eps, has_kv=kv_from is None)
        if c.canon_taps is not None:
            mixer = ConvolvedInput(mixer, c.hidden_size, c.canon_taps, f"{p}.canon1")
        ffn = ffn_norm = None
        if layer.mlp is not None:
            ffn = ActivatedFeedForward(f"{p}.mlp", c.hidden_size, layer.mlp.ff, "xielu")
            ffn_norm = norm(f"{p}.norm2", f"{p}.hc2")
        blocks.append(HyperConnectionBlock(mixer, ffn, norm(f"{p}.norm1", f"{p}.hc1"), ffn_norm))
        order.append(ExecEntry(i, cache_of=kv_from))  # layer j is entry j of the order
    pair = c.pair_hash
    return DecoderLM(
        c,
        SummedEmbedding("embed", c.vocab_size, c.hidden_size, copies=streams,
                        pair_hash=(pair.buckets, pair.mul_prev, pair.mul_cur) if pair else None,
                        positions=c.position_rows, names={"token": "embed", "pair": "bigram", "position": "pos"}),
        blocks,
        ConnectedNorm("final.norm", c.hidden_size, c.norm_eps, streams, None, offset=NORM_OFFSET),
        LMHead("head", c.vocab_size, c.hidden_size, tied_to=None, tensor="head"),
        order=order)
