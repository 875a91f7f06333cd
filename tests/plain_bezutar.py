"""A plain, slow implementation of the Bezutar decoder on the CPU, one function per mechanism.

Written from the design's equations alone, in double precision, over a whole sequence at a time (no cache, no
batching, no portions: the recurrent mixers are literal loops over the tokens).  It shares no code with the
package: the tests compare the engine's logits against it.

Notation: ``x`` is [tokens, width]; ``p`` is a token's position in its sequence, from 0.  Weights come as a dict
name -> tensor; a layer's tensor ``foo`` of its mixer is ``<layer>.mix.foo``.  ``config`` is the dictionary of the
model's config.json.
"""

from __future__ import annotations

import math

import torch

F64 = torch.float64


def rms_unit(x: torch.Tensor, eps: float) -> torch.Tensor:
    return x / torch.sqrt((x * x).mean(dim=-1, keepdim=True) + eps)


def softplus(z: torch.Tensor) -> torch.Tensor:
    return torch.where(z > 30.0, z, torch.log1p(torch.exp(torch.minimum(z, torch.full_like(z, 30.0)))))


def log_sigmoid(z: torch.Tensor) -> torch.Tensor:
    return -softplus(-z)


def silu(z: torch.Tensor) -> torch.Tensor:
    return z * torch.sigmoid(z)


# --------------------------------------------------------------------------- embedding

def bigram_rows(tokens: list[int], bigram: dict) -> list[int]:
    """Row of the pair table for every token: a hash of (previous, current); the first token takes the last row."""
    buckets, a, b = bigram["buckets"], bigram["mul_prev"], bigram["mul_cur"]
    return [buckets if i == 0 else (tokens[i - 1] * a + t * b) % buckets for i, t in enumerate(tokens)]


def embed(config: dict, w: dict, tokens: list[int]) -> torch.Tensor:
    x = w["embed"].to(F64)[tokens]
    bigram = (config.get("embedding") or {}).get("bigram")
    if bigram:
        x = x + w["bigram"].to(F64)[bigram_rows(tokens, bigram)]
    if "pos" in w:
        x = x + w["pos"].to(F64)[: len(tokens)]
    return x


# --------------------------------------------------------------------------- norms, streams, the short convolution

def offset_norm(x: torch.Tensor, weight: torch.Tensor, eps: float) -> torch.Tensor:
    """RMS norm whose tensor holds the weight's difference from one."""
    return rms_unit(x, eps) * (1.0 + weight.to(F64))


def input_convolution(h: torch.Tensor, taps: torch.Tensor) -> torch.Tensor:
    """h + conv(h): per channel, tap j of ``taps`` [width, T] meets the input T - 1 - j tokens back; zeros in front."""
    n, t = h.shape[0], taps.shape[1]
    padded = torch.cat([torch.zeros((t - 1, h.shape[1]), dtype=F64), h])
    out = h.clone()
    for j in range(t):
        out = out + taps.to(F64)[:, j] * padded[j: j + n]
    return out


def streams_read(streams: torch.Tensor, w_in: torch.Tensor) -> torch.Tensor:
    """streams [S, tokens, width] -> sum_s in[s] x_s."""
    return torch.einsum("s,snw->nw", w_in.to(F64), streams)


def streams_write(streams: torch.Tensor, y: torch.Tensor, mix: torch.Tensor, w_out: torch.Tensor) -> torch.Tensor:
    """x_t <- sum_s mix[s, t] x_s + out[t] y, all t from the old streams."""
    return torch.einsum("st,snw->tnw", mix.to(F64), streams) + w_out.to(F64)[:, None, None] * y[None]


# --------------------------------------------------------------------------- mixers

def matrix_memory(h: torch.Tensor, w: dict, p: str, m: dict, eps: float) -> torch.Tensor:
    """The matrix-memory recurrence with exponential input gates and a running maximum that starts at 0."""
    H, D, V, cap = m["heads"], m["dim"], m["vdim"], float(m["gate_cap"])
    n = h.shape[0]
    g = lambda name: w[f"{p}.{name}"].to(F64)  # noqa: E731
    q = (h @ g("q").T).reshape(n, H, D) * D ** -0.5
    k = (h @ g("k").T).reshape(n, H, D)
    v = (h @ g("v").T).reshape(n, H, V)
    gi = cap * torch.tanh((h @ g("i").T + g("i.b")) / cap)
    gf = log_sigmoid(cap * torch.tanh((h @ g("f").T + g("f.b")) / cap))
    S = torch.zeros((H, D, V), dtype=F64)
    nn = torch.zeros((H, D), dtype=F64)
    mx = torch.zeros(H, dtype=F64)
    out = torch.zeros((n, H, V), dtype=F64)
    for t in range(n):
        new = torch.maximum(gf[t] + mx, gi[t])
        keep, take = torch.exp(gf[t] + mx - new), torch.exp(gi[t] - new)
        S = keep[:, None, None] * S + take[:, None, None] * k[t][:, :, None] * v[t][:, None, :]
        nn = keep[:, None] * nn + take[:, None] * k[t]
        mx = new
        num = torch.einsum("hdv,hd->hv", S, q[t])
        den = torch.maximum((nn * q[t]).sum(-1).abs(), torch.exp(-mx)) + 1e-6
        out[t] = num / den[:, None]
    out = rms_unit(out, eps).reshape(n, H * V) * g("norm")
    return (out * torch.sigmoid(h @ g("g").T)) @ g("o").T


def gated_recurrence(h: torch.Tensor, w: dict, p: str, m: dict) -> torch.Tensor:
    """A gated recurrence per channel whose gates read the current token only."""
    g = lambda name: w[f"{p}.{name}"].to(F64)  # noqa: E731
    z = torch.sigmoid(h @ g("z").T + g("z.b"))
    u = h @ g("x").T + g("x.b")
    cand = torch.where(u >= 0, u + 0.5, torch.sigmoid(u))
    S = torch.zeros(m["width"], dtype=F64)
    rows = []
    for t in range(h.shape[0]):
        S = (1.0 - z[t]) * S + z[t] * cand[t]
        rows.append(S)
    return (torch.stack(rows) * silu(h @ g("g").T)) @ g("o").T


def rotary_frequencies(rot: dict) -> tuple[torch.Tensor, float]:
    """Frequencies of the rotated pairs and the factor on cosines and sines."""
    dims, base = rot["dims"], float(rot["base"])
    i = torch.arange(dims // 2, dtype=F64)
    f = base ** (-2.0 * i / dims)
    scaling = rot.get("scaling")
    if not scaling:
        return f, 1.0
    factor, original = float(scaling["factor"]), float(scaling["original"])
    at = lambda turns: dims * math.log(original / (2.0 * math.pi * turns)) / (2.0 * math.log(base))  # noqa: E731
    lo = max(math.floor(at(float(scaling["fast"]))), 0)
    hi = min(math.ceil(at(float(scaling["slow"]))), dims - 1)
    ramp = ((i - lo) / max(hi - lo, 0.001)).clamp(0.0, 1.0)
    return f / factor * ramp + f * (1.0 - ramp), 0.1 * math.log(factor) + 1.0


def rotate_halves(x: torch.Tensor, positions: torch.Tensor, rot: dict) -> torch.Tensor:
    """x [tokens, ..., size]: element i < dims/2 pairs with i + dims/2 among the first ``dims`` elements."""
    dims = rot["dims"]
    half = dims // 2
    f, factor = rotary_frequencies(rot)
    angle = positions.to(F64)[:, None] * f[None, :]
    shape = [x.shape[0]] + [1] * (x.dim() - 2) + [half]
    cos, sin = (torch.cos(angle) * factor).reshape(shape), (torch.sin(angle) * factor).reshape(shape)
    a, b = x[..., :half], x[..., half:dims]
    out = x.clone()
    out[..., :half] = a * cos - b * sin
    out[..., half:dims] = b * cos + a * sin
    return out


def latent_keys(h: torch.Tensor, w: dict, p: str, m: dict, eps: float, positions: torch.Tensor):
    """What a latent-attention layer caches: the normed latent c and the rotated key part shared by its heads."""
    g = lambda name: w[f"{p}.{name}"].to(F64)  # noqa: E731
    down = h @ g("dkv").T
    r = m["kv_rank"]
    c = rms_unit(down[:, :r], eps) * g("dkv.norm")
    shared = down[:, r:]
    if m.get("rot"):
        shared = rotate_halves(shared, positions, m["rot"])
    return c, shared


def latent_attention(h: torch.Tensor, w: dict, p: str, m: dict, eps: float, positions: torch.Tensor,
                     cached: tuple[torch.Tensor, torch.Tensor]) -> torch.Tensor:
    """Queries through a latent, keys and values up from the cached latent, causal softmax with a sink, a gate per head."""
    g = lambda name: w[f"{p}.{name}"].to(F64)  # noqa: E731
    n, H, D, R, V = h.shape[0], m["heads"], m["dim"], m["rot_dim"], m["vdim"]
    c, shared = cached
    cq = rms_unit(h @ g("dq").T, eps) * g("dq.norm")
    q = (cq @ g("uq").T).reshape(n, H, D + R)
    q_plain, q_turn = q[..., :D], q[..., D:]
    if m.get("rot"):
        q_turn = rotate_halves(q_turn, positions, m["rot"])
    k_plain = (c @ g("uk").T).reshape(n, H, D)
    v = (c @ g("uv").T).reshape(n, H, V)
    scores = (torch.einsum("ihd,jhd->hij", q_plain, k_plain) + torch.einsum("ihr,jr->hij", q_turn, shared)) * float(m["scale"])
    i, j = torch.arange(n)[:, None], torch.arange(n)[None, :]
    scores = scores.masked_fill(~(j <= i), -math.inf)
    sink = g("sink")[:, None, None]
    top = torch.maximum(scores.max(dim=-1, keepdim=True).values, sink)
    e = torch.exp(scores - top)
    weights = e / (e.sum(dim=-1, keepdim=True) + torch.exp(sink - top))
    out = torch.einsum("hij,jhv->ihv", weights, v)
    out = out * torch.sigmoid(h @ g("g").T)[:, :, None]
    return out.reshape(n, H * V) @ g("o").T


# --------------------------------------------------------------------------- feed-forward

def xielu(z: torch.Tensor, p: torch.Tensor, q: torch.Tensor) -> torch.Tensor:
    pos = softplus(p) * z * z + 0.5 * z
    neg = (0.5 + softplus(q)) * torch.expm1(torch.minimum(z, torch.zeros_like(z))) - (0.5 + softplus(q)) * z + 0.5 * z
    return torch.where(z > 0, pos, neg)


def dense_ff(h: torch.Tensor, w: dict, p: str) -> torch.Tensor:
    act = w[f"{p}.act"].to(F64)
    return xielu(h @ w[f"{p}.up"].to(F64).T, act[0], act[1]) @ w[f"{p}.down"].to(F64).T


# --------------------------------------------------------------------------- the model

def layer_streams(config: dict, weights: dict, tokens: list[int]) -> tuple[list[torch.Tensor], torch.Tensor]:
    """(the sum of the streams after every layer, the streams at the end [S, tokens, width])."""
    w = weights
    eps = float(config["norm"]["eps"])
    S = config.get("streams")
    x = embed(config, w, tokens)
    streams = x[None].repeat(S or 1, 1, 1)
    positions = torch.arange(len(tokens))
    one = torch.ones(1, dtype=F64)
    caches: dict[int, tuple] = {}
    after = []
    for i, layer in enumerate(config["layers"]):
        p, m = f"l{i}", layer["mixer"]
        for q, branch in ((1, "mixer"), (2, "mlp")):
            if branch == "mlp" and layer.get("mlp") is None:
                continue
            hc = f"{p}.hc{q}"
            w_in, w_out, mix = (w[f"{hc}.in"], w[f"{hc}.out"], w[f"{hc}.mix"]) if S else (one, one, one[None])
            h = offset_norm(streams_read(streams, w_in), w[f"{p}.norm{q}"], eps)
            if branch == "mixer":
                if config.get("canon"):
                    h = input_convolution(h, w[f"{p}.canon1"])
                if layer["type"] == "mlstm":
                    y = matrix_memory(h, w, f"{p}.mix", m, eps)
                elif layer["type"] == "mingru":
                    y = gated_recurrence(h, w, f"{p}.mix", m)
                else:
                    src = m.get("kv_from")
                    if src is None:
                        caches[i] = latent_keys(h, w, f"{p}.mix", m, eps, positions)
                    y = latent_attention(h, w, f"{p}.mix", m, eps, positions, caches[i if src is None else src])
            else:
                y = dense_ff(h, w, f"{p}.mlp")
            streams = streams_write(streams, y, mix, w_out)
        after.append(streams.sum(dim=0))
    return after, streams


def logits(config: dict, weights: dict, tokens: list[int]) -> torch.Tensor:
    _, streams = layer_streams(config, weights, tokens)
    x = offset_norm(streams.sum(dim=0), weights["final.norm"], float(config["norm"]["eps"]))
    return x @ weights["head"].to(F64).T
