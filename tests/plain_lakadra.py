"""A plain, slow implementation of the Lakadra decoder in double precision on the CPU: one function per mechanism,
written from the design's equations, sharing no code with the package.  Tests compare the engine with it.

``config`` is the design's nested dictionary (what its config.json holds), ``weights`` a dictionary from tensor name
to a float64 tensor.  A whole sequence is run at once: ``forward(config, weights, tokens)`` returns the logits of
every position and, on request, the residual stream after every layer.
"""

from __future__ import annotations

import math

import torch

F64 = torch.float64


def rms(x: torch.Tensor, eps: float) -> torch.Tensor:
    return x / torch.sqrt((x * x).mean(dim=-1, keepdim=True) + eps)


def offset_norm(x: torch.Tensor, w: torch.Tensor, eps: float) -> torch.Tensor:
    """The layers' norm: the tensor holds the weight's distance from one."""
    return rms(x, eps) * (1.0 + w)


def plain_norm(x: torch.Tensor, w: torch.Tensor, eps: float) -> torch.Tensor:
    return rms(x, eps) * w


def silu(z: torch.Tensor) -> torch.Tensor:
    return z * torch.sigmoid(z)


def gelu_tanh(z: torch.Tensor) -> torch.Tensor:
    return 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def rotate(x: torch.Tensor, positions: torch.Tensor, base: float, dims: int, interleaved: bool,
           factor: float = 1.0) -> torch.Tensor:
    """``x`` [T, heads, D]: the first ``dims`` elements of every head turned by position * f_i, f_i = base^(-2i/dims)
    / factor; pairs (2i, 2i+1) when ``interleaved``, else (i, i + dims/2)."""
    half = dims // 2
    i = torch.arange(half, dtype=F64)
    freq = base ** (-2.0 * i / dims) / factor
    angle = positions.to(F64)[:, None] * freq[None, :]  # [T, half]
    cos, sin = torch.cos(angle)[:, None, :], torch.sin(angle)[:, None, :]
    out = x.clone()
    if interleaved:
        u, v = x[..., 0:dims:2], x[..., 1:dims:2]
        out[..., 0:dims:2] = u * cos - v * sin
        out[..., 1:dims:2] = v * cos + u * sin
    else:
        u, v = x[..., :half], x[..., half:dims]
        out[..., :half] = u * cos - v * sin
        out[..., half:dims] = v * cos + u * sin
    return out


# --------------------------------------------------------------------------- mixers

def lightning(m: dict, w: dict, p: str, h: torch.Tensor, eps: float) -> torch.Tensor:
    """Linear attention with a fixed decay per head, token by token."""
    t, heads, d, dv = h.shape[0], m["heads"], m["dim"], m.get("vdim", m["dim"])
    q = silu(h @ w[f"{p}.q"].T).reshape(t, heads, d)
    k = silu(h @ w[f"{p}.k"].T).reshape(t, heads, d)
    v = silu(h @ w[f"{p}.v"].T).reshape(t, heads, dv)
    decay = torch.tensor(m["decay"], dtype=F64)
    state = torch.zeros(heads, d, dv, dtype=F64)
    out = torch.zeros(t, heads, dv, dtype=F64)
    for i in range(t):
        state = decay[:, None, None] * state + k[i][:, :, None] * v[i][:, None, :]
        out[i] = torch.einsum("hdv,hd->hv", state, q[i])
    o = plain_norm(out.reshape(t, heads * dv), w[f"{p}.norm"], eps) * torch.sigmoid(h @ w[f"{p}.g"].T)
    return o @ w[f"{p}.o"].T


def latent_cache(m: dict, w: dict, p: str, h: torch.Tensor, eps: float) -> tuple[torch.Tensor, torch.Tensor]:
    """What a latent-attention layer with a down projection of its own caches: the normed latent and the rotated
    shared key part."""
    t, rank, rot_dim = h.shape[0], m["kv_rank"], m["rot_dim"]
    down = h @ w[f"{p}.dkv"].T
    c = plain_norm(down[:, :rank], w[f"{p}.dkv.norm"], eps)
    shared = down[:, rank:]
    if rot_dim and m.get("rot"):
        shared = rotate(shared.reshape(t, 1, rot_dim), torch.arange(t), m["rot"]["base"], m["rot"]["dims"], True).reshape(t, rot_dim)
    return c, shared


def latent_attention(m: dict, w: dict, p: str, h: torch.Tensor, eps: float, cached) -> torch.Tensor:
    t, heads, d, rot_dim, dv = h.shape[0], m["heads"], m["dim"], m["rot_dim"], m.get("vdim", m["dim"])
    c, shared = cached
    cq = plain_norm(h @ w[f"{p}.dq"].T, w[f"{p}.dq.norm"], eps)
    q = (cq @ w[f"{p}.uq"].T).reshape(t, heads, d + rot_dim)
    q_plain, q_turn = q[..., :d], q[..., d:]
    if rot_dim and m.get("rot"):
        q_turn = rotate(q_turn, torch.arange(t), m["rot"]["base"], m["rot"]["dims"], True)
    k_plain = (c @ w[f"{p}.uk"].T).reshape(t, heads, d)
    v = (c @ w[f"{p}.uv"].T).reshape(t, heads, dv)
    scores = (torch.einsum("ihd,jhd->hij", q_plain, k_plain) + torch.einsum("ihd,jd->hij", q_turn, shared)) * m["scale"]
    visible = torch.tril(torch.ones(t, t, dtype=torch.bool))
    scores = scores.masked_fill(~visible, -math.inf)
    out = torch.einsum("hij,jhv->ihv", torch.softmax(scores, dim=-1), v).reshape(t, heads * dv)
    return out @ w[f"{p}.o"].T


def windowed_attention(m: dict, w: dict, p: str, h: torch.Tensor) -> torch.Tensor:
    """Grouped-query attention with biases, half-split rotation with stretched positions, a sliding window, a softmax
    whose denominator holds one more 1, and a gate per head."""
    t, heads, groups, d, dv = h.shape[0], m["heads"], m.get("kv_heads", m["heads"]), m["dim"], m.get("vdim", m["dim"])
    q = (h @ w[f"{p}.q"].T + w[f"{p}.q.b"]).reshape(t, heads, d)
    k = (h @ w[f"{p}.k"].T + w[f"{p}.k.b"]).reshape(t, groups, d)
    v = (h @ w[f"{p}.v"].T + w[f"{p}.v.b"]).reshape(t, groups, dv)
    rot = m.get("rot")
    if rot:
        factor = (rot.get("scaling") or {}).get("factor", 1.0)
        q = rotate(q, torch.arange(t), rot["base"], rot["dims"], False, factor)
        k = rotate(k, torch.arange(t), rot["base"], rot["dims"], False, factor)
    per = heads // groups
    k, v = k.repeat_interleave(per, dim=1), v.repeat_interleave(per, dim=1)
    scores = torch.einsum("ihd,jhd->hij", q, k) * m["scale"]
    i, j = torch.arange(t)[:, None], torch.arange(t)[None, :]
    visible = j <= i
    if m.get("mask"):
        visible = visible & (i - j < m["mask"]["size"])
    e = torch.exp(scores.masked_fill(~visible, -math.inf))
    prob = e / (1.0 + e.sum(dim=-1, keepdim=True))
    out = torch.einsum("hij,jhv->ihv", prob, v)
    out = out * torch.sigmoid(h @ w[f"{p}.g"].T)[:, :, None]
    return out.reshape(t, heads * dv) @ w[f"{p}.o"].T + w[f"{p}.o.b"]


def causal_conv(x: torch.Tensor, taps: torch.Tensor, bias: torch.Tensor) -> torch.Tensor:
    """``taps`` [channels, T]: the last column multiplies the current token; zeros in front of the sequence."""
    t, n = x.shape[0], taps.shape[1]
    padded = torch.cat([torch.zeros(n - 1, x.shape[1], dtype=F64), x])
    out = bias.expand(t, -1).clone()
    for j in range(n):
        out = out + padded[j: j + t] * taps[:, j]
    return out


def gated_linear_recurrence(m: dict, w: dict, p: str, h: torch.Tensor) -> torch.Tensor:
    """The recurrent block with a real-gated linear recurrent unit."""
    t, width, blocks = h.shape[0], m["width"], m["blocks"]
    y = gelu_tanh(h @ w[f"{p}.y"].T + w[f"{p}.y.b"])
    u = causal_conv(h @ w[f"{p}.x"].T + w[f"{p}.x.b"], w[f"{p}.conv"], w[f"{p}.conv.b"])
    ub = u.reshape(t, blocks, width // blocks)
    r = torch.sigmoid(torch.einsum("boi,tbi->tbo", w[f"{p}.ra"], ub) + w[f"{p}.ra.b"]).reshape(t, width)
    i = torch.sigmoid(torch.einsum("boi,tbi->tbo", w[f"{p}.ri"], ub) + w[f"{p}.ri.b"]).reshape(t, width)
    a = torch.exp(-8.0 * r * torch.nn.functional.softplus(w[f"{p}.lam"]))
    state = torch.zeros(width, dtype=F64)
    out = torch.zeros(t, width, dtype=F64)
    for s in range(t):
        state = a[s] * state + torch.sqrt(1.0 - a[s] ** 2) * i[s] * u[s]
        out[s] = state
    return (out * y) @ w[f"{p}.o"].T


def parallel_mixers(m: dict, w: dict, p: str, h: torch.Tensor) -> torch.Tensor:
    left = windowed_attention(m["left"], w, f"{p}.left", h)
    right = gated_linear_recurrence(m["right"], w, f"{p}.right", h)
    return m["left_scale"] * left + m["right_scale"] * right


# --------------------------------------------------------------------------- feed-forward

def expert(w: dict, p: str, h: torch.Tensor) -> torch.Tensor:
    return (torch.relu(h @ w[f"{p}.up"].T) ** 2) @ w[f"{p}.down"].T


def route(mlp: dict, w: dict, p: str, h: torch.Tensor) -> tuple[torch.Tensor, torch.Tensor]:
    """(chosen experts [T, top], their weights [T, top]); ids from ``experts`` on are identity experts."""
    r = mlp["router"]
    s = torch.softmax(h @ w[f"{p}.router"].T, dim=-1)
    choice = s + w[f"{p}.correction"]
    g = r.get("groups")
    if g:
        per = choice.shape[1] // g["count"]
        best = choice.reshape(-1, g["count"], per).max(dim=-1).values
        kept = best.topk(g["keep"], dim=-1).indices
        allowed = torch.zeros_like(best, dtype=torch.bool).scatter_(1, kept, True).repeat_interleave(per, dim=1)
        choice = choice.masked_fill(~allowed, -math.inf)
    ids = choice.topk(r["top"], dim=-1).indices
    return ids, s.gather(1, ids)


def routed_experts(mlp: dict, w: dict, p: str, h: torch.Tensor) -> torch.Tensor:
    ids, weights = route(mlp, w, p, h)
    real = mlp["router"]["experts"]
    out = torch.zeros_like(h)
    for t in range(h.shape[0]):
        for e, s in zip(ids[t].tolist(), weights[t]):
            out[t] += s * (expert(w, f"{p}.e{e}", h[t: t + 1])[0] if e < real else h[t])
    if mlp.get("shared"):
        out = out + expert(w, f"{p}.shared", h) * torch.sigmoid(h @ w[f"{p}.shared.sg"].T)
    return out


# --------------------------------------------------------------------------- the model

def forward(config: dict, weights: dict, tokens: list[int], want_layers: bool = False):
    eps = config["norm"]["eps"]
    w = weights
    x = w["embed"][torch.tensor(tokens)]
    caches: dict[int, tuple] = {}
    layers = []
    for i, layer in enumerate(config["layers"]):
        p, m = f"l{i}", layer["mixer"]
        h = offset_norm(x, w[f"{p}.norm1"], eps)
        if layer["type"] == "lightning":
            mixed = lightning(m, w, f"{p}.mix", h, eps)
        elif layer["type"] == "latent_attention":
            src = m.get("kv_from")
            if src is None:
                caches[i] = latent_cache(m, w, f"{p}.mix", h, eps)
            mixed = latent_attention(m, w, f"{p}.mix", h, eps, caches[i if src is None else src])
        elif layer["type"] == "parallel":
            mixed = parallel_mixers(m, w, f"{p}.mix", h)
        else:
            raise ValueError(layer["type"])
        if layer.get("mlp"):
            mixed = mixed + routed_experts(layer["mlp"], w, f"{p}.mlp", h)
        x = x + mixed
        layers.append(x)
    logits = offset_norm(x, w["final.norm"], eps) @ w["head"].T * config.get("logit_scale", 1.0)
    cap = config.get("logit_softcap")
    if cap:
        logits = cap * torch.tanh(logits / cap)
    return (logits, torch.stack(layers)) if want_layers else logits
