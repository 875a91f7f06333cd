"""Grouped-query attention over the paged key/value cache.

Biased q/k/v projections (stacked into one product at load), rotary encoding of
queries and keys, the write of keys and values to their pages, causal attention
of the step's rows over each request's pages, and the output projection
(slipstream/models/layers/attention.py:98-191).  ``window`` None attends over all
earlier keys; an integer W over the last W.  ``page_size`` asks for cache pages of
that many tokens for this layer (layers that ask alike share a pool).  Every size is
a constructor parameter; the part does not know which model it is in.

Options beyond that (all off by default):
``chunk`` C: a query sees only the earlier keys of its own chunk of C positions, chunks counted from the
request's first token.  ``value_dim``: values (and the heads' outputs) of another size than queries and keys.
``unit_norm_eps``: after the rotation every query and key head is divided by its root mean square
(``x / sqrt(mean(x^2) + eps)``, no weight); the pages hold the keys in that form.  ``gate``: the concatenated
heads are multiplied by ``sigmoid(W_g x)`` before the output projection (``W_g`` reads the same input as q/k/v).
``has_kv`` False: the layer has no key/value projections and attends over pages that another layer wrote (the
model's order names it).  ``qk_norm_eps``: BEFORE the rotation every query and key head passes an RMS norm over its
elements with a weight of the head's size that all heads share (tensors ``q_norm`` / ``k_norm``).  ``rotate_values``:
the value of position j is rotated by j over all its elements, with the pairing of the position encoding and the
frequencies ``theta^(-2m / value_dim)``, and cached so; a head's output at position i (the weighted sum of such
values) is turned back by -i before any gate, so that what is summed depends on i - j only.  ``softcap`` c: a scaled
score s enters the softmax as ``c tanh(s / c)``.  ``head_gate``: head h's output is multiplied by
``sigmoid(w_g,h . x)``, one number per head and token (``W_g`` [heads, hidden] rides in the stacked product).
``unit_sink``: the softmax's denominator holds one more 1 (a key whose score is 0 and which has no value).  ``names``: the checkpoint's tensor names by role (q, k, v, o, g,
q_bias, k_bias, v_bias, o_bias, q_norm, k_norm).

Heads of a size the kernels do not take (they take multiples of 16), or values of another size than keys, are
padded with zeros where the weights are bound: q/k/v/g rows and o columns of the padding are zero, so the
products, the scores and the outputs are what they would be without it, and no kernel knows.
"""

from __future__ import annotations

import torch

from slipstream_b200 import ops

from .base import MIXERS, CacheSpec, IntoNorm, LayerBinding, Mixer, PositionEncoding, Runtime, WeightSpec


@MIXERS.register("paged_attention")
class PagedAttention(Mixer):
    cuda_graph_safe = True
    takes_into = True
    takes_pending_norm = True

    def __init__(self, name: str, hidden_size: int, num_heads: int, num_kv_heads: int, head_dim: int,
                 position_encoding: PositionEncoding, qkv_bias: bool = True, out_bias: bool = False,
                 window: int | None = None, scale: float | None = None, page_size: int | None = None, *,
                 chunk: int | None = None, value_dim: int | None = None, unit_norm_eps: float | None = None,
                 gate: bool = False, has_kv: bool = True, names: dict[str, str] | None = None,
                 qk_norm_eps: float | None = None, rotate_values: bool = False, softcap: float | None = None,
                 head_gate: bool = False, unit_sink: bool = False) -> None:
        if num_heads % num_kv_heads != 0:
            raise ValueError(f"num_heads ({num_heads}) must be divisible by num_kv_heads ({num_kv_heads})")
        value_dim = head_dim if value_dim is None else int(value_dim)
        if head_dim % 2 or not 2 <= head_dim <= 256 or not 1 <= value_dim <= 256:
            raise ValueError(f"head sizes are even and at most 256 (values: at most 256), not {head_dim} / {value_dim}")
        if window is not None and window < 1:
            raise ValueError("window must be >= 1")
        if chunk is not None and chunk < 1:
            raise ValueError("chunk must be >= 1")
        if window is not None and chunk is not None:
            raise ValueError("a layer has a window or a chunk, not both")
        self.name = name
        self.hidden_size = hidden_size
        self.num_heads = num_heads
        self.num_kv_heads = num_kv_heads
        self.key_dim = head_dim  # what the checkpoint's q and k heads hold
        self.value_dim = value_dim
        # what the kernels and the pages see: one size for keys and values, a multiple of 16
        self.head_dim = -(-max(head_dim, value_dim) // 16) * 16
        self.position_encoding = position_encoding
        self.qkv_bias = qkv_bias
        self.out_bias = out_bias
        self.window = window
        self.chunk = chunk
        self.unit_norm_eps = None if unit_norm_eps is None else float(unit_norm_eps)
        self.gate = bool(gate)
        self.qk_norm_eps = None if qk_norm_eps is None else float(qk_norm_eps)
        self.rotate_values = bool(rotate_values)
        self.softcap = float(softcap) if softcap else None
        if self.rotate_values and (value_dim % 2 or getattr(position_encoding, "theta", None) is None):
            raise ValueError("rotated values need an even value size and a rotary position encoding")
        if self.rotate_values and (gate or head_gate):
            raise ValueError("a gate on rotated values is not built")
        if gate and head_gate:
            raise ValueError("a layer gates its heads element by element or head by head, not both")
        self.head_gate, self.unit_sink = bool(head_gate), bool(unit_sink)
        if self.qk_norm_eps is not None and unit_norm_eps is not None:
            raise ValueError("a layer norms its heads before the rotation or after it, not both")
        self.has_kv = bool(has_kv)
        self.page_size = page_size  # tokens per cache page this layer wants; None: the engine's default
        self.scale = head_dim ** -0.5 if scale is None else float(scale)
        n = name
        self.names = {"q": f"{n}.q_proj.weight", "k": f"{n}.k_proj.weight", "v": f"{n}.v_proj.weight",
                      "o": f"{n}.o_proj.weight", "g": f"{n}.g_proj.weight", "q_bias": f"{n}.q_proj.bias",
                      "k_bias": f"{n}.k_proj.bias", "v_bias": f"{n}.v_proj.bias", "o_bias": f"{n}.o_proj.bias",
                      "q_norm": f"{n}.q_norm.weight", "k_norm": f"{n}.k_norm.weight"}
        self.names.update(names or {})

    @property
    def plain(self) -> bool:
        """The layer as the fused kernels of the plain path know it: q/k/v stacked in a row and nothing after the
        rotation (half-split pairs, unscaled sines, no unit norm, no gate, keys and values of its own)."""
        rotary_plain = getattr(self.position_encoding, "plain", True)
        return (rotary_plain and self.unit_norm_eps is None and not self.gate and self.has_kv
                and not self.head_gate and not self.unit_sink
                and self.qk_norm_eps is None and not self.rotate_values and self.softcap is None
                and self.key_dim == self.value_dim == self.head_dim)

    def weight_specs(self) -> list[WeightSpec]:
        h, d, dv, names = self.hidden_size, self.key_dim, self.value_dim, self.names
        specs = [WeightSpec(names["q"], (self.num_heads * d, h)), WeightSpec(names["o"], (h, self.num_heads * dv))]
        if self.has_kv:
            specs += [WeightSpec(names["k"], (self.num_kv_heads * d, h)), WeightSpec(names["v"], (self.num_kv_heads * dv, h))]
        if self.gate:
            specs.append(WeightSpec(names["g"], (self.num_heads * dv, h)))
        if self.head_gate:
            specs.append(WeightSpec(names["g"], (self.num_heads, h)))
        if self.qkv_bias:
            specs.append(WeightSpec(names["q_bias"], (self.num_heads * d,), kind="vector"))
            if self.has_kv:
                specs += [WeightSpec(names["k_bias"], (self.num_kv_heads * d,), kind="vector"),
                          WeightSpec(names["v_bias"], (self.num_kv_heads * dv,), kind="vector")]
        if self.out_bias:
            specs.append(WeightSpec(names["o_bias"], (h,), kind="vector"))
        if self.qk_norm_eps is not None:
            specs.append(WeightSpec(names["q_norm"], (d,), kind="vector", init=("one_plus_normal", 0.1)))
            if self.has_kv:
                specs.append(WeightSpec(names["k_norm"], (d,), kind="vector", init=("one_plus_normal", 0.1)))
        return specs

    def cache_spec(self) -> CacheSpec:
        return CacheSpec(self.num_kv_heads, self.head_dim, self.window, self.page_size, self.chunk)

    def _pad_heads(self, t: torch.Tensor, heads: int, size: int) -> torch.Tensor:
        """[heads * size, ...] -> [heads * head_dim, ...] with zeros behind each head's ``size`` rows."""
        if size == self.head_dim:
            return t
        out = t.new_zeros((heads, self.head_dim, *t.shape[1:]))
        out[:, :size] = t.reshape(heads, size, *t.shape[1:])
        return out.reshape(heads * self.head_dim, *t.shape[1:])

    def bind(self, weights: dict[str, torch.Tensor], runtime: Runtime) -> None:
        super().bind(weights, runtime)
        names, nq, nkv = self.names, self.num_heads, self.num_kv_heads
        # one stacked product: [q | k | v | g]; k and v only if the layer has them, g only with a gate
        roles = [("q", nq, self.key_dim)]
        if self.has_kv:
            roles += [("k", nkv, self.key_dim), ("v", nkv, self.value_dim)]
        if self.gate:
            roles.append(("g", nq, self.value_dim))
        stacked = [self._pad_heads(weights[names[r]], heads, size) for r, heads, size in roles]
        self.head_gate_col = sum(t.shape[0] for t in stacked)
        extra_rows = 0
        if self.head_gate:  # one row per head behind the heads themselves, then zeros up to a row of 16-byte multiples
            extra_rows = -(-nq // 8) * 8
            g = weights[names["g"]]
            stacked.append(torch.cat([g, g.new_zeros((extra_rows - nq, g.shape[1]))]))
        self.qkv_weight = torch.cat(stacked, dim=0).contiguous()
        self.qkv_b = None
        if self.qkv_bias:
            biases = [self._pad_heads(weights[names[f"{r}_bias"]], heads, size) if r != "g"
                      else weights[names["q"]].new_zeros(heads * self.head_dim) for r, heads, size in roles]
            if extra_rows:
                biases.append(weights[names["q"]].new_zeros(extra_rows))
            self.qkv_b = torch.cat(biases).to(runtime.dtype).contiguous()
        o = weights[names["o"]]
        if self.value_dim != self.head_dim:
            o = self._pad_heads(o.t().contiguous(), nq, self.value_dim).t().contiguous()
        self.o_weight = o
        self.o_b = weights[names["o_bias"]].to(runtime.dtype) if self.out_bias else None
        self.position_encoding.bind(weights, runtime)
        self.q_norm_weight = self.k_norm_weight = self.value_inv_freq = None
        if self.qk_norm_eps is not None:
            self.q_norm_weight = weights[names["q_norm"]].to(torch.float32).contiguous()
            if self.has_kv:
                self.k_norm_weight = weights[names["k_norm"]].to(torch.float32).contiguous()
        if self.rotate_values:  # formed in double precision, rounded once
            pairs = torch.arange(0, self.value_dim, 2, dtype=torch.float64)
            self.value_inv_freq = (float(self.position_encoding.theta) ** (-pairs / self.value_dim)).to(torch.float32).to(runtime.device)
        self.sinks = torch.zeros(nq, dtype=torch.float32, device=runtime.device) if self.unit_sink else None
        ops.attention_library(self.head_dim)  # compile now, not inside the first step

    # ------------------------------------------------------------------ decode steps replayed from a graph
    def capture_variant(self, longest: int, plan: object = None) -> object:
        """Decode steps: long contexts of few requests want the keys cut into more slices than fit one thread-block
        cluster (``ops.decode_slices``).  Steps with prompt portions: into how many parts the tcgen05 prefill kernel
        cuts the keys of a query tile (``ops.prefill_key_parts``).  Each form is captured as a graph of its own."""
        bf16 = self.runtime.dtype == torch.bfloat16
        if plan is None or plan.is_decode_only:
            return bool(bf16 and ops.is_long_context(longest))
        group = self.num_heads // self.num_kv_heads
        if not bf16 or not ops.tcgen05_prefill_fits(self.head_dim, self.num_heads, self.num_kv_heads, self.page_size or 16):
            return None
        return int(ops.prefill_key_parts(plan.q_lens, plan.seq_lens, 128 // group, self.num_kv_heads,
                                         ops.sm_count(self.runtime.device), self.window or self.chunk or 0))

    def capture_group(self) -> object:
        # layers that see equally far answer `capture_variant` alike
        return ("paged_attention", self.window or self.chunk or 0)

    def prepare_capture(self, ctx, variant: object, max_model_len: int) -> None:
        if not ctx.is_decode_only:
            # a captured step with prompt portions: the number of key parts is the variant's (the choice follows the
            # lengths of the step, which a replay does not know on the host)
            ctx.extras[("prefill_key_parts", 128 // (self.num_heads // self.num_kv_heads), self.num_kv_heads,
                        self.window or self.chunk or 0)] = int(variant or 1)
            return
        # the number of slices must not follow the lengths of the step that happens to be captured
        ctx.extras["static_max_seq_len"] = max_model_len
        ctx.extras["decode_wide"] = bool(variant)
        # the float32 kernel's list of query tiles: one tile per row of the batch
        rows = ctx.num_requests
        ctx.set_query_tiles(16, 1, torch.arange(rows, dtype=torch.int32, device=ctx.device),
                            torch.zeros(rows, dtype=torch.int32, device=ctx.device))

    def weight_bytes(self) -> int:
        return (self.qkv_weight.numel() + self.o_weight.numel()) * self.o_weight.element_size()

    def after_projection(self, qkv: torch.Tensor, ctx) -> None:
        """Hook for subclasses: change the stacked projection output [N, (n_q + 2 n_kv) * D] in place before
        queries and keys are rotated and keys and values go to their pages (a norm over each query and key head,
        say).  A subclass that overrides it keeps every attention kernel; only the fusion of rotation and page
        write into the decode kernel is off for it, since that kernel takes the projection output as it is."""
        return None

    def forward(self, x: torch.Tensor, ctx, layer: LayerBinding, into: IntoNorm | None = None) -> torch.Tensor:
        meta = ctx.groups[layer.group]
        qkv = ops.linear(x, self.qkv_weight, self.qkv_b)
        plain_projection = type(self).after_projection is PagedAttention.after_projection
        if not plain_projection:
            self.after_projection(qkv, ctx)
        inv_freq, rotary_dim = self.position_encoding.rotary_table()
        # a decode step's attention kernel rotates and writes the newest key and value itself
        fused = (plain_projection and self.plain and layer.writes_cache
                 and ops.fuses_rope(qkv, ctx, self.head_dim, self.num_heads, self.num_kv_heads, layer.kv.shape[3]))
        early_norm = self.qk_norm_eps is not None or self.rotate_values
        if early_norm:
            if getattr(self.position_encoding, "mscale", 1.0) != 1.0:
                raise ValueError(f"{self.name}: scaled sines are not built for layers that norm before the rotation")
            if self.has_kv != layer.writes_cache:
                raise ValueError(f"{self.name}: a layer with keys and values of its own writes its pages, one without "
                                 "reads another layer's")
            ops.norm_rope_cache(qkv, ctx.positions, meta.slot_mapping, layer.kv, self.num_heads,
                                self.num_kv_heads if self.has_kv else 0, self.head_dim, inv_freq=inv_freq,
                                rotary_dim=rotary_dim, value_inv_freq=self.value_inv_freq,
                                value_rotary_dim=self.value_dim if self.rotate_values else 0,
                                interleaved=getattr(self.position_encoding, "interleaved", False),
                                q_weight=self.q_norm_weight, k_weight=self.k_norm_weight,
                                norm_dim=self.key_dim if self.qk_norm_eps is not None else 0, eps=self.qk_norm_eps or 0.0,
                                write_cache=layer.writes_cache)
        elif not self.plain:
            if self.has_kv != layer.writes_cache:
                raise ValueError(f"{self.name}: a layer with keys and values of its own writes its pages, one without "
                                 "reads another layer's")
            encoding = self.position_encoding
            ops.rope_norm_cache(qkv, ctx.positions, meta.slot_mapping, inv_freq, layer.kv, self.num_heads,
                                self.num_kv_heads if self.has_kv else 0, self.head_dim, rotary_dim,
                                interleaved=getattr(encoding, "interleaved", False),
                                mscale=getattr(encoding, "mscale", 1.0),
                                norm_dim=self.key_dim if self.unit_norm_eps is not None else 0,
                                eps=self.unit_norm_eps or 0.0, write_cache=layer.writes_cache)
        elif not fused:
            ops.rope_and_cache(qkv, ctx.positions, meta.slot_mapping, inv_freq, layer.kv, self.num_heads,
                               self.num_kv_heads, self.head_dim, rotary_dim, write_cache=layer.writes_cache)
        out = torch.empty((x.shape[0], self.num_heads * self.head_dim), dtype=x.dtype, device=x.device)
        ops.paged_attention(qkv, out, layer.kv, meta.block_tables, ctx, self.num_heads, self.num_kv_heads,
                            self.head_dim, self.scale, self.window or 0,
                            rope=(inv_freq, rotary_dim) if fused else None, chunk=self.chunk or 0,
                            gate=qkv[:, qkv.shape[1] - out.shape[1]:] if self.gate else None, softcap=self.softcap or 0.0,
                            sinks=self.sinks)
        if self.head_gate:
            ops.head_gate(out, qkv[:, self.head_gate_col: self.head_gate_col + self.num_heads], self.num_heads, self.head_dim)
        if self.rotate_values:
            ops.turn_heads(out, ctx.positions, self.value_inv_freq, self.num_heads, self.head_dim, self.value_dim,
                           interleaved=getattr(self.position_encoding, "interleaved", False), sign=-1.0)
        if into is not None:
            return into.close(out, self.o_weight, self.o_b)
        return ops.linear(out, self.o_weight, self.o_b)
