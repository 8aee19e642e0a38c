"""A plain, slow restatement of the Basitar decoder in float64: one function per mechanism, whole sequences,
no cache, no state, no batching.  It shares no code with the engine and is what the engine's results are
compared with.  ``weights`` maps tensor names to tensors (any dtype); ``config`` is the parsed ``config.json``.
"""

from __future__ import annotations

import math

import torch

F64 = torch.float64


def _w(weights, name):
    return weights[name].to(F64)


def unit_rms(x, eps):
    return x / torch.sqrt((x * x).mean(dim=-1, keepdim=True) + eps)


def offset_norm(x, weight, eps):
    """RMS norm whose weight is stored around zero."""
    return unit_rms(x, eps) * (1.0 + weight)


def plain_norm(x, weight, eps):
    return unit_rms(x, eps) * weight


def silu(z):
    return z * torch.sigmoid(z)


# ------------------------------------------------------------------ embedding
def bigram_rows(tokens, buckets, mul_prev, mul_cur):
    rows = []
    for place, token in enumerate(tokens):
        rows.append(buckets if place == 0 else (tokens[place - 1] * mul_prev + token * mul_cur) % buckets)
    return rows


def embed(tokens, weights, config):
    ids = torch.tensor(list(tokens), dtype=torch.long)
    x = _w(weights, "embed")[ids]
    bigram = (config.get("embedding") or {}).get("bigram")
    if bigram:
        rows = bigram_rows(list(tokens), int(bigram["buckets"]), int(bigram["mul_prev"]), int(bigram["mul_cur"]))
        x = x + _w(weights, "bigram")[torch.tensor(rows, dtype=torch.long)]
    if "pos" in weights:
        x = x + _w(weights, "pos")[: len(tokens)]
    return x


# ------------------------------------------------------------------ rotation
def rotary_frequencies(dims, base, scaling=None):
    """``(frequencies [dims / 2], factor on cos and sin)``."""
    half = dims // 2
    freq = torch.tensor([base ** (-2.0 * i / dims) for i in range(half)], dtype=F64)
    if not scaling:
        return freq, 1.0
    factor, original = float(scaling["factor"]), float(scaling["original"])

    def turn(t):
        return dims * math.log(original / (2.0 * math.pi * t)) / (2.0 * math.log(base))

    lo = max(math.floor(turn(float(scaling["fast"]))), 0)
    hi = min(math.ceil(turn(float(scaling["slow"]))), dims - 1)
    ramp = torch.tensor([min(max((i - lo) / max(hi - lo, 0.001), 0.0), 1.0) for i in range(half)], dtype=F64)
    return freq / factor * ramp + freq * (1.0 - ramp), 0.1 * math.log(factor) + 1.0


def rotate(x, positions, freq, magnitude, interleaved):
    """x ``[T, ..., dims]``: all ``dims`` entries rotate; pairs ``(i, i + dims/2)`` or ``(2i, 2i + 1)``."""
    dims = x.shape[-1]
    half = dims // 2
    angle = positions.to(F64)[:, None] * freq[None, :]
    cos, sin = torch.cos(angle) * magnitude, torch.sin(angle) * magnitude
    while cos.dim() < x.dim():
        cos, sin = cos.unsqueeze(1), sin.unsqueeze(1)
    if interleaved:
        u, v = x[..., 0::2], x[..., 1::2]
        out = torch.empty_like(x)
        out[..., 0::2] = u * cos - v * sin
        out[..., 1::2] = v * cos + u * sin
        return out
    u, v = x[..., :half], x[..., half:]
    return torch.cat([u * cos - v * sin, v * cos + u * sin], dim=-1)


# ------------------------------------------------------------------ latent attention
def latent_attention(h, weights, prefix, sizes, eps, second):
    """Both kinds: ``second`` has interleaved pairs, scaled frequencies and a gate per head."""
    T = h.shape[0]
    H, dim, rot_dim, vdim, rank = (int(sizes[k]) for k in ("heads", "dim", "rot_dim", "vdim", "kv_rank"))
    rot = sizes["rot"]
    freq, magnitude = rotary_frequencies(rot_dim, float(rot["base"]), rot.get("scaling") if second else None)
    positions = torch.arange(T)
    cq = plain_norm(h @ _w(weights, prefix + "dq").T, _w(weights, prefix + "dq.norm"), eps)
    q = (cq @ _w(weights, prefix + "uq").T).view(T, H, dim + rot_dim)
    q_flat, q_rot = q[..., :dim], rotate(q[..., dim:], positions, freq, magnitude, second)
    down = h @ _w(weights, prefix + "dkv").T
    c = plain_norm(down[:, :rank], _w(weights, prefix + "dkv.norm"), eps)
    k_rot = rotate(down[:, rank:], positions, freq, magnitude, second)                 # one for all heads
    k_flat = (c @ _w(weights, prefix + "uk").T).view(T, H, dim)
    v = (c @ _w(weights, prefix + "uv").T).view(T, H, vdim)
    scores = torch.einsum("thd,shd->hts", q_flat, k_flat) + torch.einsum("thd,sd->hts", q_rot, k_rot)
    scores = scores * float(sizes["scale"])
    hidden = torch.ones(T, T, dtype=torch.bool).triu(1)
    scores = scores.masked_fill(hidden[None], float("-inf"))
    out = torch.einsum("hts,shd->thd", torch.softmax(scores, dim=-1), v)
    if second:
        gate = torch.sigmoid(h @ _w(weights, prefix + "g").T)                           # [T, H]
        out = out * gate[:, :, None]
    return out.reshape(T, H * vdim) @ _w(weights, prefix + "o").T


# ------------------------------------------------------------------ wkv
def wkv(h, weights, prefix, sizes, eps):
    T = h.shape[0]
    H, dim = int(sizes["heads"]), int(sizes["dim"])
    before = torch.cat([torch.zeros_like(h[:1]), h[:-1]], dim=0)

    def mixed(which):
        return h + (before - h) * _w(weights, prefix + "mu." + which)

    r = (mixed("r") @ _w(weights, prefix + "r").T).view(T, H, dim)
    k = (mixed("k") @ _w(weights, prefix + "k").T).view(T, H, dim)
    v = (mixed("v") @ _w(weights, prefix + "v").T).view(T, H, dim)
    gate = silu(mixed("g") @ _w(weights, prefix + "g").T)
    low = torch.tanh(mixed("w") @ _w(weights, prefix + "w1").T)
    decay = torch.exp(-torch.exp(low @ _w(weights, prefix + "w2").T + _w(weights, prefix + "w0"))).view(T, H, dim)
    bonus = _w(weights, prefix + "u").view(H, dim)
    out = torch.zeros(T, H, dim, dtype=F64)
    S = torch.zeros(H, dim, dim, dtype=F64)               # [head, key channel, value channel]
    for t in range(T):
        kv = k[t][:, :, None] * v[t][:, None, :]
        out[t] = torch.einsum("hkv,hk->hv", S + bonus[:, :, None] * kv, r[t])
        S = decay[t][:, :, None] * S + kv
    out = unit_rms(out, eps).reshape(T, H * dim) * _w(weights, prefix + "norm") * gate
    return out @ _w(weights, prefix + "o").T


# ------------------------------------------------------------------ feed-forwards
def gated_unit(h, gate, up, down):
    return (silu(h @ gate.T) * (h @ up.T)) @ down.T


def dense_feed_forward(h, weights, prefix):
    return gated_unit(h, _w(weights, prefix + "gate"), _w(weights, prefix + "up"), _w(weights, prefix + "down"))


def router_choice(h, weights, prefix, top):
    """``(chosen experts [T, top], their weights [T, top], logits [T, E])``; largest logits first, ties to the lower index."""
    logits = h @ _w(weights, prefix + "router").T + _w(weights, prefix + "router.b")
    order = torch.sort(logits, dim=-1, descending=True, stable=True).indices[:, :top]
    chosen = torch.gather(logits, 1, order)
    return order, torch.softmax(chosen, dim=-1), logits


def routed_feed_forward(h, weights, prefix, mlp, margins=None):
    experts, top = int(mlp["router"]["experts"]), int(mlp["router"]["top"])
    order, share, logits = router_choice(h, weights, prefix, top)
    if margins is not None and top < experts:
        # how clearly the last chosen expert beats the first one left out, in units of the logits' spread
        ranked = torch.sort(logits, dim=-1, descending=True).values
        margins.append(float(((ranked[:, top - 1] - ranked[:, top]) / logits.std()).min()))
    out = torch.zeros_like(h)
    for e in range(experts):
        name = f"{prefix}e{e}."
        each = gated_unit(h, _w(weights, name + "gate"), _w(weights, name + "up"), _w(weights, name + "down"))
        out = out + each * (share * (order == e)).sum(dim=-1, keepdim=True)
    return out


# ------------------------------------------------------------------ the model
def layer_prefix(config, index):
    """Where layer ``index``'s tensors live: its own prefix, or that of the layer whose weights it uses."""
    owner = config["layers"][index].get("weights_of")
    return f"l{index if owner is None else int(owner)}."


def run_mixer(kind, h, weights, prefix, sizes, eps):
    if kind == "wkv":
        return wkv(h, weights, prefix, sizes, eps)
    if kind in ("latent_attention", "latent_attention_2"):
        return latent_attention(h, weights, prefix, sizes, eps, second=kind == "latent_attention_2")
    raise ValueError(kind)


def forward(tokens, weights, config, return_layers=False, margins=None):
    """Logits ``[T, vocab]`` (float64) of a whole sequence; with ``return_layers`` also the stream after every layer.
    ``margins`` (a list) receives the narrowest router decision of every routed layer."""
    eps = float(config["norm"]["eps"])
    x = embed(tokens, weights, config)
    streams = []
    for index, layer in enumerate(config["layers"]):
        p = layer_prefix(config, index)
        h = offset_norm(x, _w(weights, p + "norm1"), eps)
        x = x + offset_norm(run_mixer(layer["type"], h, weights, p + "mix.", layer["mixer"], eps), _w(weights, p + "norm1b"), eps)
        mlp = layer.get("mlp")
        if mlp is not None:
            h = offset_norm(x, _w(weights, p + "norm2"), eps)
            wide = dense_feed_forward(h, weights, p + "mlp.") if mlp["kind"] == "dense" else routed_feed_forward(h, weights, p + "mlp.", mlp, margins)
            x = x + offset_norm(wide, _w(weights, p + "norm2b"), eps)
        streams.append(x)
    logits = offset_norm(x, _w(weights, "final.norm"), eps) @ _w(weights, "embed").T
    return (logits, torch.stack(streams)) if return_layers else logits


def greedy(tokens, weights, config, steps: int) -> list[int]:
    """The ``steps`` tokens that always taking the largest logit produces after ``tokens``."""
    tokens = list(tokens)
    start = len(tokens)
    for _ in range(steps):
        tokens.append(int(forward(tokens, weights, config)[-1].argmax()))
    return tokens[start:]


def clear_margin(tokens, weights, config) -> float:
    """The narrowest router decision of the sequence (infinite for a model without routers)."""
    margins: list = []
    forward(tokens, weights, config, margins=margins)
    return min(margins) if margins else math.inf
