"""Latent attention over the paged cache: keys and values are carried up from one small latent per token, and only
that latent and a rotated key part shared by all heads are cached.

With H heads of ``dim`` unrotated and ``rot_dim`` rotated query/key elements and ``value_dim`` values:

    c_q = rmsnorm(W_dq x) * w_dq_norm,   q_h = (W_uq c_q)_h = [q_h^plain: dim | q_h^turn: rot_dim]
    [c_raw: kv_rank | s_raw: rot_dim] = W_dkv x,   c = rmsnorm(c_raw) * w_dkv_norm,   s = rotate(s_raw, position)
    k_h^plain = W_uk,h c,   v_h = W_uv,h c
    score_h(i, j) = (q_h^plain(i) . k_h^plain(j) + rotate(q_h^turn(i), i) . s(j)) * scale,   j <= i

a softmax whose denominator also holds ``exp(sink_h)`` (one learned number per head with neither key nor value, which the scale does not touch),
each head's output times ``sigmoid(w_g,h . x)``, and the output projection on the concatenated heads.

How it runs.  The products with W_uk and W_uv move to the query's side, so that the cache holds every token once,
whatever the number of heads: ``q_h^plain . (W_uk,h c) = (W_uk,h^T q_h^plain) . c``, and
``sum_j p_j W_uv,h c_j = W_uv,h sum_j p_j c_j``.  A cached token is one key row ``[s | c]`` and one value row ``[c]``
of a single key/value head (padded to a multiple of 16 elements); every query head becomes
``[rotate(q^turn) | W_uk,h^T q^plain]``, the paged attention kernels run with H query heads over that one head, and
the latent-sized outputs go up through W_uv,h with the gate.  A layer with ``has_kv`` False has no W_dkv: the model's
order lets it read the pages of the layer that has (its own W_uk, W_uv, queries, sinks and gate apply).

Norms, angles, scores and the softmax are float32; products are in the compute dtype with float32 accumulation.
"""

from __future__ import annotations

import torch

from slipstream_b200 import ops

from .base import MIXERS, CacheSpec, IntoNorm, LayerBinding, Mixer, PositionEncoding, Runtime, WeightSpec


@MIXERS.register("latent_attention")
class LatentAttention(Mixer):
    cuda_graph_safe = True
    takes_into = True
    takes_pending_norm = True  # the input goes to one product and nowhere else

    def __init__(self, name: str, hidden_size: int, heads: int, dim: int, rot_dim: int, value_dim: int, q_rank: int,
                 kv_rank: int, scale: float, position_encoding: PositionEncoding, norm_eps: float = 1e-6, *,
                 sinks: bool = True, gate: bool = True, has_kv: bool = True, page_size: int | None = None,
                 names: dict[str, str] | None = None) -> None:
        """``position_encoding``: rotates the ``rot_dim`` part (its table holds ``rot_dim / 2`` frequencies; pairs of
        halves, or of neighbours when the encoding says ``interleaved``); a part without a table leaves it unrotated.  ``names``: the checkpoint's tensor names by role
        (dq, dq_norm, uq, dkv, dkv_norm, uk, uv, sink, g, o)."""
        if min(heads, dim, value_dim, q_rank, kv_rank) < 1 or rot_dim < 0 or rot_dim % 2:
            raise ValueError("heads, dim, value_dim, q_rank and kv_rank must be >= 1, rot_dim even and >= 0")
        self.row = -(-(kv_rank + rot_dim) // 16) * 16  # elements of a cached row as the kernels see it
        if self.row > 256:
            raise ValueError("kv_rank + rot_dim must be at most 256")
        # pairs of neighbours (2i, 2i + 1): the rows of the rotated part are reordered where the weights are bound, so that
        # pair i sits at (i, i + rot_dim / 2); queries and keys are reordered alike, which leaves every score as it was
        self.neighbour_pairs = bool(getattr(position_encoding, "interleaved", False))
        self.name, self.hidden_size = name, hidden_size
        self.heads, self.dim, self.rot_dim, self.value_dim = heads, dim, rot_dim, value_dim
        self.q_rank, self.kv_rank = q_rank, kv_rank
        self.scale, self.norm_eps = float(scale), float(norm_eps)
        self.position_encoding = position_encoding
        self.has_sinks, self.gate, self.has_kv, self.page_size = bool(sinks), bool(gate), bool(has_kv), page_size
        self.names = {role: f"{name}.{role}" for role in ("dq", "uq", "dkv", "uk", "uv", "sink", "g", "o")}
        self.names.update({"dq_norm": f"{name}.dq.norm", "dkv_norm": f"{name}.dkv.norm"})
        self.names.update(names or {})

    def weight_specs(self) -> list[WeightSpec]:
        n, w, h = self.names, self.hidden_size, self.heads
        specs = [WeightSpec(n["dq"], (self.q_rank, w)),
                 WeightSpec(n["dq_norm"], (self.q_rank,), kind="vector", init=("one_plus_normal", 0.1)),
                 WeightSpec(n["uq"], (h * (self.dim + self.rot_dim), self.q_rank)),
                 WeightSpec(n["uk"], (h * self.dim, self.kv_rank)), WeightSpec(n["uv"], (h * self.value_dim, self.kv_rank)),
                 WeightSpec(n["o"], (w, h * self.value_dim))]
        if self.has_kv:
            specs += [WeightSpec(n["dkv"], (self.kv_rank + self.rot_dim, w)),
                      WeightSpec(n["dkv_norm"], (self.kv_rank,), kind="vector", init=("one_plus_normal", 0.1))]
        if self.has_sinks:
            specs.append(WeightSpec(n["sink"], (h,), kind="vector", init=("normal", 1.0)))
        if self.gate:
            specs.append(WeightSpec(n["g"], (h, w)))
        return specs

    def cache_spec(self) -> CacheSpec:
        return CacheSpec(1, self.row, None, self.page_size, None)

    def bind(self, weights: dict[str, torch.Tensor], runtime: Runtime) -> None:
        super().bind(weights, runtime)
        n, h = self.names, self.heads
        if self.neighbour_pairs and self.rot_dim:
            order = torch.cat([torch.arange(0, self.rot_dim, 2), torch.arange(1, self.rot_dim, 2)])
            weights = dict(weights)
            uq = weights[n["uq"]].reshape(h, self.dim + self.rot_dim, -1).clone()
            uq[:, self.dim:] = uq[:, self.dim:][:, order.to(uq.device)]
            weights[n["uq"]] = uq.reshape(h * (self.dim + self.rot_dim), -1)
            if self.has_kv:
                dkv = weights[n["dkv"]].clone()
                dkv[self.kv_rank:] = dkv[self.kv_rank:][order.to(dkv.device)]
                weights[n["dkv"]] = dkv
        # one product of the input: [query latent | key/value latent, shared key part | gates], padded to rows of
        # 16-byte multiples
        stacked = [weights[n["dq"]]] + ([weights[n["dkv"]]] if self.has_kv else []) + ([weights[n["g"]]] if self.gate else [])
        w_in = torch.cat(stacked, dim=0)
        pad = -w_in.shape[0] % 8
        self.in_weight = torch.cat([w_in, w_in.new_zeros((pad, w_in.shape[1]))]).contiguous() if pad else w_in.contiguous()
        self.gate_col = self.q_rank + (self.kv_rank + self.rot_dim if self.has_kv else 0)
        as_f32 = lambda t: t.to(torch.float32).contiguous()  # noqa: E731  (exact: the stored values are kept)
        self.q_norm_weight = as_f32(weights[n["dq_norm"]])
        self.kv_norm_weight = as_f32(weights[n["dkv_norm"]]) if self.has_kv else None
        self.sinks = as_f32(weights[n["sink"]]) if self.has_sinks else None
        self.uq_weight = weights[n["uq"]]
        # per head: [dim, kv_rank] carries a query into the latent space; [kv_rank, value_dim] a latent-sized output up
        self.to_latent = weights[n["uk"]].reshape(h, self.dim, self.kv_rank).contiguous()
        self.to_value = weights[n["uv"]].reshape(h, self.value_dim, self.kv_rank).transpose(1, 2).contiguous()
        self.o_weight = weights[n["o"]]
        self.position_encoding.bind(weights, runtime)
        inv_freq, rotary_dim = self.position_encoding.rotary_table()
        if inv_freq is not None and rotary_dim != self.rot_dim:
            raise ValueError(f"{self.name}: the position encoding rotates {rotary_dim} elements, the layer has {self.rot_dim}")
        ops.attention_library(self.row)  # compile now, not inside the first step

    def weight_bytes(self) -> int:
        n = sum(t.numel() for t in (self.in_weight, self.uq_weight, self.to_latent, self.to_value, self.o_weight))
        return n * self.o_weight.element_size()

    def capture_variant(self, longest: int, plan: object = None) -> object:
        return None  # layers with sinks run one form of the decode kernel

    def capture_group(self) -> object:
        return ("latent_attention",)

    def prepare_capture(self, ctx, variant: object, max_model_len: int) -> None:
        if not ctx.is_decode_only:
            return
        ctx.extras["static_max_seq_len"] = max_model_len  # the number of slices must not follow the captured step
        ctx.extras.setdefault("decode_wide", False)
        rows = ctx.num_requests
        ctx.set_query_tiles(16, 1, torch.arange(rows, dtype=torch.int32, device=ctx.device),
                            torch.zeros(rows, dtype=torch.int32, device=ctx.device))

    def forward(self, x: torch.Tensor, ctx, layer: LayerBinding, into: IntoNorm | None = None) -> torch.Tensor:
        if self.has_kv != layer.writes_cache:
            raise ValueError(f"{self.name}: a layer with a latent of its own writes its pages, one without reads another's")
        meta = ctx.groups[layer.group]
        h, row = self.heads, self.row
        inv_freq, _ = self.position_encoding.rotary_table()
        mscale = getattr(self.position_encoding, "mscale", 1.0)
        down = ops.linear(x, self.in_weight)
        cq = ops.latent_rows(down, ctx.positions, meta.slot_mapping if self.has_kv else None,
                             layer.kv if self.has_kv else None, self.q_norm_weight, self.kv_norm_weight, inv_freq, mscale,
                             self.q_rank, self.kv_rank if self.has_kv else 0, self.rot_dim, self.norm_eps)
        q = ops.linear(cq, self.uq_weight)
        n = q.shape[0]
        q_latent = torch.empty((n, h * row), dtype=q.dtype, device=q.device)
        ops.head_product(q, self.dim + self.rot_dim, self.to_latent, q_latent, row, turn=self.rot_dim, pad_to=row,
                         positions=ctx.positions, inv_freq=inv_freq, mscale=mscale)
        mixed = torch.empty_like(q_latent)
        ops.paged_attention(q_latent, mixed, layer.kv, meta.block_tables, ctx, h, 1, row, self.scale, sinks=self.sinks)
        out = torch.empty((n, h * self.value_dim), dtype=q.dtype, device=q.device)
        ops.head_product(mixed, row, self.to_value, out, self.value_dim,
                         gates=down[:, self.gate_col: self.gate_col + h] if self.gate else None)
        if into is not None:
            return into.close(out, self.o_weight, None)
        return ops.linear(out, self.o_weight)
