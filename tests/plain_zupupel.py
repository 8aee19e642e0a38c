"""A plain, slow restatement of the Zupupel decoder in float64: one function per mechanism, whole sequences only,
no cache, no state, no batch.  It shares no code with the engine; the engine's tests compare against it.

Notation: ``x [T, W]`` rows of one sequence at positions ``0 .. T-1``; weights are ``[out, in]`` and applied as
``x @ W.T``; ``tensors`` maps checkpoint names to float64 tensors.
"""

from __future__ import annotations

import math

import torch

F64 = torch.float64


# ---------------------------------------------------------------- norms -- #
def rms_norm(x: torch.Tensor, weight: torch.Tensor, eps: float) -> torch.Tensor:
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps) * weight


def layer_norm(x: torch.Tensor, weight: torch.Tensor, bias: torch.Tensor, eps: float) -> torch.Tensor:
    mean = x.mean(-1, keepdim=True)
    var = ((x - mean) ** 2).mean(-1, keepdim=True)
    return (x - mean) / torch.sqrt(var + eps) * weight + bias


# ------------------------------------------------------------- rotation -- #
def rotate(rows: torch.Tensor, positions: torch.Tensor, dims: int, base: float, layout: str) -> torch.Tensor:
    """Rotate the first ``dims`` entries of ``rows [T, heads, n]``; ``layout`` ``"halves"`` pairs entry ``i`` with
    ``i + dims/2``, ``"neighbours"`` pairs ``2i`` with ``2i + 1``; the angle of pair ``i`` is ``p * base^(-2i/dims)``."""
    if dims == 0:
        return rows
    half = dims // 2
    freq = torch.tensor([base ** (-2.0 * i / dims) for i in range(half)], dtype=F64)
    angle = positions.to(F64)[:, None] * freq[None, :]            # [T, half]
    cos, sin = torch.cos(angle)[:, None, :], torch.sin(angle)[:, None, :]
    out = rows.clone()
    if layout == "halves":
        u, v = rows[..., :half], rows[..., half:dims]
        out[..., :half] = u * cos - v * sin
        out[..., half:dims] = v * cos + u * sin
    else:
        u, v = rows[..., 0:dims:2], rows[..., 1:dims:2]
        out[..., 0:dims:2] = u * cos - v * sin
        out[..., 1:dims:2] = v * cos + u * sin
    return out


# ------------------------------------------------------------ attention -- #
def softmax_attention(q, k, v, scale: float, window: int) -> torch.Tensor:
    """``q [T, H, d]``, ``k [T, H, d]``, ``v [T, H, dv]`` (keys already expanded to the query heads); position ``i``
    sees ``j <= i`` and, with ``window > 0``, only ``i - j < window``."""
    T = q.shape[0]
    scores = torch.einsum("ihd,jhd->hij", q, k) * scale
    i = torch.arange(T)[:, None]
    j = torch.arange(T)[None, :]
    visible = j <= i
    if window > 0:
        visible = visible & (i - j < window)
    scores = scores.masked_fill(~visible[None], -math.inf)
    weights = torch.softmax(scores, dim=-1)
    return torch.einsum("hij,jhd->ihd", weights, v)


def attention_keys_values(h, tensors, prefix: str, sizes: dict, eps: float):
    """What a windowed-attention layer caches: keys after the norm over the whole projection and the rotation,
    ``[T, G, dim]``, and values ``[T, G, vdim]``."""
    T = h.shape[0]
    G, dim, vdim = sizes["kv_heads"], sizes["dim"], sizes["vdim"]
    rot = sizes.get("rot") or {}
    k = rms_norm(h @ tensors[prefix + "k"].T, tensors[prefix + "k.norm"], eps).view(T, G, dim)
    k = rotate(k, torch.arange(T), int(rot.get("dims", 0)), float(rot.get("base", 1.0)), "halves")
    v = (h @ tensors[prefix + "v"].T).view(T, G, vdim)
    return k, v


def attention_mixer(h, tensors, prefix: str, sizes: dict, eps: float, keys_values=None):
    """Grouped-query attention with a sliding window, a norm over the whole q and k projections, partial rotation
    by halves and a sigmoid gate on the heads side by side.  ``keys_values``: another layer's, for a layer that has
    none of its own.  Returns ``(output, (keys, values))``."""
    T = h.shape[0]
    H, G, dim, vdim = sizes["heads"], sizes["kv_heads"], sizes["dim"], sizes["vdim"]
    rot = sizes.get("rot") or {}
    window = int((sizes.get("mask") or {}).get("size", 0))
    q = rms_norm(h @ tensors[prefix + "q"].T, tensors[prefix + "q.norm"], eps).view(T, H, dim)
    q = rotate(q, torch.arange(T), int(rot.get("dims", 0)), float(rot.get("base", 1.0)), "halves")
    if keys_values is None:
        keys_values = attention_keys_values(h, tensors, prefix, sizes, eps)
    k, v = keys_values
    group = H // G
    k_wide = k.repeat_interleave(group, dim=1)       # query head h reads key/value head h // group
    v_wide = v.repeat_interleave(group, dim=1)
    mixed = softmax_attention(q, k_wide, v_wide, float(sizes["scale"]), window).reshape(T, H * vdim)
    mixed = mixed * torch.sigmoid(h @ tensors[prefix + "g"].T)
    return mixed @ tensors[prefix + "o"].T, keys_values


def latent_attention_mixer(h, tensors, prefix: str, sizes: dict, eps: float):
    """Attention over keys and values that are products of a normed latent; one rotated key part is shared by all
    heads; rotation pairs neighbours; causal; a sigmoid gate on the heads side by side."""
    T = h.shape[0]
    H, dim, rd, vdim, rank = sizes["heads"], sizes["dim"], sizes["rot_dim"], sizes["vdim"], sizes["kv_rank"]
    rot = sizes.get("rot") or {}
    base = float(rot.get("base", 1.0))
    positions = torch.arange(T)
    q = (h @ tensors[prefix + "q"].T).view(T, H, dim + rd)
    q_plain, q_rot = q[..., :dim], rotate(q[..., dim:], positions, rd, base, "neighbours")
    down = h @ tensors[prefix + "dkv"].T
    c = rms_norm(down[:, :rank], tensors[prefix + "dkv.norm"], eps)
    k_rot = rotate(down[:, None, rank:], positions, rd, base, "neighbours")        # [T, 1, rd]
    k_plain = (c @ tensors[prefix + "uk"].T).view(T, H, dim)
    v = (c @ tensors[prefix + "uv"].T).view(T, H, vdim)
    k = torch.cat([k_plain, k_rot.expand(T, H, rd)], dim=-1)
    mixed = softmax_attention(torch.cat([q_plain, q_rot], dim=-1), k, v, float(sizes["scale"]), 0).reshape(T, H * vdim)
    mixed = mixed * torch.sigmoid(h @ tensors[prefix + "g"].T)
    return mixed @ tensors[prefix + "o"].T


# -------------------------------------------------------------- experts -- #
def clamped_expert(h, gate_w, up_w, down_w, limit: float) -> torch.Tensor:
    g = torch.clamp(h @ gate_w.T, max=limit)
    u = torch.clamp(h @ up_w.T, min=-limit, max=limit)
    return (g * torch.sigmoid(1.702 * g) * (u + 1.0)) @ down_w.T


def route(h, router_w, correction, top: int, groups: int, keep: int, margins: list | None = None):
    """``(chosen [T, top], weights [T, top], scores [T, E])``: softmax over all router rows; the choice is made on
    scores plus ``correction`` among the rows of the ``keep`` best of ``groups`` equal groups of neighbours (a group's
    rank is its largest corrected score); weights are the chosen rows' plain scores over their sum."""
    scores = torch.softmax(h @ router_w.T, dim=-1)
    choice = scores + correction
    T, E = choice.shape
    if groups > 1:
        per = E // groups
        best = choice.view(T, groups, per).max(-1).values                   # [T, groups]
        kept = torch.topk(best, keep, dim=-1).indices
        if margins is not None and keep < groups:
            ranked = best.sort(-1, descending=True).values
            margins.extend(((ranked[:, keep - 1] - ranked[:, keep]) / scores.std(-1)).tolist())
        allowed = torch.zeros(T, groups, dtype=torch.bool)
        allowed.scatter_(1, kept, True)
        choice = choice.masked_fill(~allowed.repeat_interleave(per, dim=1), -math.inf)
    chosen = torch.topk(choice, top, dim=-1).indices
    if margins is not None and top < E:
        ranked = choice.sort(-1, descending=True).values
        gap = ranked[:, top - 1] - ranked[:, top]                            # infinite where no other row was allowed
        margins.extend((gap / scores.std(-1)).tolist())
    picked = torch.gather(scores, 1, chosen)
    return chosen, picked / (picked.sum(-1, keepdim=True) + 1e-20), scores


def routed_experts(h, tensors, prefix: str, mlp: dict, margins: list | None = None) -> torch.Tensor:
    router = mlp["router"]
    experts, identity, top = int(router["experts"]), int(router.get("identity", 0)), int(router["top"])
    groups = router.get("groups") or {}
    limit = float(mlp["expert"]["limit"])
    chosen, weights, _ = route(h, tensors[prefix + "router"], tensors[prefix + "correction"], top,
                               int(groups.get("count", 1)), int(groups.get("keep", 1)), margins)
    out = torch.zeros_like(h)
    for t in range(h.shape[0]):
        for e, w in zip(chosen[t].tolist(), weights[t]):
            if e >= experts:                   # the last router rows have no tensors: the input itself
                assert e < experts + identity
                out[t] += w * h[t]
            else:
                p = f"{prefix}e{e}."
                out[t] += w * clamped_expert(h[t], tensors[p + "gate"], tensors[p + "up"], tensors[p + "down"], limit)
    return out


# ---------------------------------------------------------------- model -- #
def forward(config: dict, tensors: dict, tokens, collect_layers: bool = False, margins: list | None = None):
    """Logits ``[T, vocab]`` of one sequence (and, with ``collect_layers``, the stream after every layer).  ``margins``
    collects how clearly every router decision fell, in units of the scores' spread."""
    eps, alpha = float(config["norm"]["eps"]), float(config["postln_alpha"])
    x = tensors["embed"][torch.as_tensor(tokens)] * float(config["embedding"]["scale"])
    kept: dict[int, tuple] = {}
    streams = []
    for index, layer in enumerate(config["layers"]):
        p = f"l{index}."
        sizes = layer["mixer"]
        if layer["type"] == "latent_attention":
            mixed = latent_attention_mixer(x, tensors, p + "mix.", sizes, eps)
        else:
            source = sizes.get("kv_from")
            mixed, kept[index] = attention_mixer(x, tensors, p + "mix.", sizes, eps,
                                                 None if source is None else kept[int(source)])
        x = layer_norm(alpha * x + mixed, tensors[p + "norm1"], tensors[p + "norm1.b"], eps)
        if layer.get("mlp") is not None:
            wide = routed_experts(x, tensors, p + "mlp.", layer["mlp"], margins)
            x = layer_norm(alpha * x + wide, tensors[p + "norm2"], tensors[p + "norm2.b"], eps)
        streams.append(x)
    x = layer_norm(x, tensors["final.norm"], tensors["final.norm.b"], eps)
    logits = x @ tensors["head"].T * float(config["logit_scale"])
    return (logits, torch.stack(streams)) if collect_layers else logits


def greedy(config: dict, tensors: dict, tokens, steps: int) -> list[int]:
    """The ``steps`` tokens that always taking the largest logit produces after ``tokens``."""
    tokens = list(tokens)
    start = len(tokens)
    for _ in range(steps):
        tokens.append(int(forward(config, tensors, tokens)[-1].argmax()))
    return tokens[start:]


def clear_margin(config: dict, tensors: dict, tokens) -> float:
    """The narrowest router decision of the sequence (infinite for a model without routers)."""
    margins: list = []
    forward(config, tensors, tokens, margins=margins)
    return min(margins) if margins else math.inf
