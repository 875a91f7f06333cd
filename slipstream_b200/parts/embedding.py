"""Token embedding into the float32 residual stream, and the LM head that gives
float32 logits for the wanted rows only (slipstream/models/causal_lm.py:93,140;
tied weights: slipstream/models/loader.py:91-93)."""

from __future__ import annotations

import torch

from slipstream_b200 import ops

from .base import EMBEDDINGS, HEADS, Embedding, Head, Runtime, StateSpec, WeightSpec


@EMBEDDINGS.register("token_table")
class TokenEmbedding(Embedding):
    cuda_graph_safe = True

    def __init__(self, name: str, vocab_size: int, hidden_size: int, scale: float = 1.0, copies: int = 1,
                 tensor: str | None = None) -> None:
        """``scale``: a constant the table's rows are multiplied by (in float32).  ``copies``: how many residual
        streams the model keeps; above 1 the result is [N, copies, hidden], every stream starting as the same
        row.  ``tensor``: the checkpoint's name of the table (default ``<name>.weight``)."""
        self.name = name
        self.vocab_size = vocab_size
        self.hidden_size = hidden_size
        self.scale = float(scale)
        self.copies = int(copies)
        self.tensor = tensor or f"{name}.weight"

    def weight_specs(self) -> list[WeightSpec]:
        return [WeightSpec(self.tensor, (self.vocab_size, self.hidden_size))]

    def bind(self, weights: dict[str, torch.Tensor], runtime: Runtime) -> None:
        super().bind(weights, runtime)
        self.weight = weights[self.tensor]

    def forward(self, token_ids: torch.Tensor) -> torch.Tensor:
        return ops.embedding(token_ids, self.weight, scale=self.scale, copies=self.copies)


@EMBEDDINGS.register("summed_tables")
class SummedEmbedding(Embedding):
    """An embedding that is a sum of rows of up to three tables, formed in float32:

    * the token's row of the token table (times ``scale``);
    * with ``pair_hash`` = (buckets, mul_prev, mul_cur): row ``(previous * mul_prev + token * mul_cur) mod buckets`` of
      a table of ``buckets + 1`` rows, whose last row serves a request's first token.  The previous token of a step's
      first row is per-request state (``last_token``, an int32 per slot), so a request may be cut anywhere;
    * with ``positions``: row ``position`` of a learned table of that many rows (added as it is).

    ``copies``: how many residual streams the model keeps (see `TokenEmbedding`).  ``names``: the checkpoint's tensor
    names by role (token, pair, position)."""

    cuda_graph_safe = True

    def __init__(self, name: str, vocab_size: int, hidden_size: int, *, scale: float = 1.0, copies: int = 1,
                 pair_hash: tuple[int, int, int] | None = None, positions: int | None = None,
                 names: dict[str, str] | None = None) -> None:
        self.name = name
        self.vocab_size = vocab_size
        self.hidden_size = hidden_size
        self.scale = float(scale)
        self.copies = int(copies)
        self.pair_hash = None if pair_hash is None else tuple(int(v) for v in pair_hash)
        self.positions = None if positions is None else int(positions)
        if self.pair_hash is not None and (self.pair_hash[0] < 1 or min(self.pair_hash[1:]) < 0):
            raise ValueError("pair_hash is (buckets >= 1, mul_prev >= 0, mul_cur >= 0)")
        self.names = {"token": f"{name}.weight", "pair": f"{name}.pair.weight", "position": f"{name}.position.weight"}
        self.names.update(names or {})

    def weight_specs(self) -> list[WeightSpec]:
        specs = [WeightSpec(self.names["token"], (self.vocab_size, self.hidden_size))]
        if self.pair_hash is not None:
            specs.append(WeightSpec(self.names["pair"], (self.pair_hash[0] + 1, self.hidden_size)))
        if self.positions is not None:
            specs.append(WeightSpec(self.names["position"], (self.positions, self.hidden_size)))
        return specs

    def state_specs(self) -> list[StateSpec]:
        return [StateSpec("last_token", (), torch.int32)] if self.pair_hash is not None else []

    def bind(self, weights: dict[str, torch.Tensor], runtime: Runtime) -> None:
        super().bind(weights, runtime)
        self.weight = weights[self.names["token"]]
        self.pair_table = weights[self.names["pair"]] if self.pair_hash is not None else None
        self.position_table = weights[self.names["position"]] if self.positions is not None else None

    def forward(self, token_ids: torch.Tensor) -> torch.Tensor:
        raise RuntimeError(f"{self.name}: this embedding needs the step's positions and state (forward_step)")

    def forward_step(self, token_ids: torch.Tensor, ctx, state: dict[str, torch.Tensor]) -> torch.Tensor:
        return ops.embed_sum(token_ids, self.weight, ctx, pair_table=self.pair_table, pair_hash=self.pair_hash,
                             last_token=state.get("last_token"), position_table=self.position_table, scale=self.scale,
                             copies=self.copies)


@HEADS.register("linear")
class LMHead(Head):
    cuda_graph_safe = True
    takes_pending_norm = True  # ``forward`` hands x to ``ops.linear`` as it is

    def __init__(self, name: str, vocab_size: int, hidden_size: int, tied_to: str | None,
                 tensor: str | None = None, softcap: float | None = None, scale: float = 1.0) -> None:
        """``scale``: the head's output is multiplied by it.  ``softcap`` c: the (scaled) logits leave as
        ``c * tanh(logits / c)``."""
        self.softcap = float(softcap) if softcap else None
        self.scale = float(scale)
        self.name = name
        self.vocab_size = vocab_size
        self.hidden_size = hidden_size
        self.tied_to = tied_to
        self.tensor = tensor or f"{name}.weight"

    def weight_specs(self) -> list[WeightSpec]:
        return [WeightSpec(self.tensor, (self.vocab_size, self.hidden_size), alias_of=self.tied_to)]

    def bind(self, weights: dict[str, torch.Tensor], runtime: Runtime) -> None:
        super().bind(weights, runtime)
        self.weight = weights[self.tensor]

    def weight_bytes(self) -> int:
        return self.weight.numel() * self.weight.element_size()

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        logits = ops.linear(x, self.weight, None, out_dtype=torch.float32)
        if self.softcap or self.scale != 1.0:
            return ops.soft_cap(logits, self.softcap, self.scale)
        return logits
