"""Small Zupupel configurations and seeded weights for the tests.

The weights are drawn so that every mechanism carries weight: norm weights spread around one with biases of their
size, sharp attention, router corrections of the size of a score, limits that clamp a good share of the experts'
products.  Every value is rounded to bfloat16 once, so a folder written in either precision and the float64 plain
implementation hold the same numbers.
"""

from __future__ import annotations

import copy
import json
import math
from pathlib import Path

import torch


def moe(experts=6, top=2, ff=24, identity=2, groups=2, keep=1, limit=0.6):
    return {"kind": "moe", "expert": {"ff": ff, "limit": limit},
            "router": {"experts": experts, "identity": identity, "top": top, "groups": {"count": groups, "keep": keep}}}


def attention_layer(*, heads=4, kv_heads=2, dim=16, vdim=16, window=12, rot_dims=8, base=100.0, scale=0.3, kv_from=None,
                    mlp=None):
    mixer = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale}
    if window:
        mixer["mask"] = {"size": window}
    if rot_dims:
        mixer["rot"] = {"base": base, "dims": rot_dims}
    if kv_from is not None:
        mixer["kv_from"] = kv_from
    return {"type": "attention", "mixer": mixer, "mlp": mlp}


def latent_layer(*, heads=3, dim=16, rot_dim=8, vdim=24, kv_rank=40, base=100.0, scale=0.3, mlp=None):
    return {"type": "latent_attention",
            "mixer": {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "kv_rank": kv_rank, "scale": scale,
                      "rot": {"base": base, "dims": rot_dim}}, "mlp": mlp}


def make_config(layers, *, width=64, vocab=97, eps=1e-5, alpha=2.0, embedding_scale=0.7, logit_scale=0.75) -> dict:
    return {"architecture": "Zupupel", "vocab": vocab, "width": width, "norm": {"eps": eps},
            "embedding": {"scale": embedding_scale}, "postln_alpha": alpha, "logit_scale": logit_scale,
            "layers": copy.deepcopy(list(layers))}


CONFIGS = {
    # one mechanism a model
    "window": make_config([attention_layer(mlp=None)]),
    "latent": make_config([latent_layer(mlp=None)], width=48, vocab=61, alpha=1.0, logit_scale=1.0),
    "experts": make_config([attention_layer(heads=2, kv_heads=2, dim=8, vdim=8, window=0, rot_dims=0, mlp=moe())],
                           width=40, vocab=70, embedding_scale=1.0),
    # a reader of another layer's keys and values with a window of its own (narrower, wider, none), the latent layer
    # first, layers without a feed-forward, heads whose value size is below and above their key size, the whole head
    # rotated, one group of experts, no identity expert, every expert taken
    "stack": make_config([
        latent_layer(heads=2, dim=32, rot_dim=16, vdim=16, kv_rank=48, mlp=moe(experts=4, top=4, ff=16, identity=0, groups=1, keep=1)),
        attention_layer(heads=6, kv_heads=3, dim=16, vdim=32, window=9, rot_dims=16, mlp=moe(experts=5, top=1, ff=16, identity=1, groups=3, keep=2)),
        attention_layer(heads=6, kv_heads=3, dim=16, vdim=32, window=20, rot_dims=16, kv_from=1, mlp=None),
        attention_layer(heads=4, kv_heads=1, dim=32, vdim=16, window=0, rot_dims=4, base=1.0e4, scale=0.2, mlp=moe()),
        attention_layer(heads=6, kv_heads=3, dim=16, vdim=32, window=5, rot_dims=16, kv_from=1, mlp=moe(experts=3, top=2, ff=8, identity=3, groups=3, keep=3)),
        latent_layer(heads=5, dim=8, rot_dim=4, vdim=8, kv_rank=24, base=1.0e4, scale=0.5, mlp=None),
        attention_layer(heads=4, kv_heads=1, dim=32, vdim=16, window=7, rot_dims=4, base=1.0e4, scale=0.2, kv_from=3, mlp=None),
    ], width=72, vocab=130, alpha=2.5, embedding_scale=0.6, logit_scale=0.4),
    # nothing is a multiple of 4 or 8: every kernel's element-by-element path
    "narrow": make_config([
        attention_layer(heads=3, kv_heads=3, dim=10, vdim=6, window=3, rot_dims=6, scale=0.7, mlp=moe(experts=7, top=3, ff=10, identity=2, groups=3, keep=2)),
        latent_layer(heads=3, dim=10, rot_dim=6, vdim=6, kv_rank=14, scale=0.7, mlp=moe(experts=1, top=1, ff=14, identity=0, groups=1, keep=1)),
        attention_layer(heads=3, kv_heads=3, dim=10, vdim=6, window=1, rot_dims=6, scale=0.7, kv_from=0, mlp=None),
    ], width=50, vocab=83, eps=1e-6, alpha=1.5, embedding_scale=1.3, logit_scale=1.7),
}


def tensor_shapes(config: dict) -> dict[str, tuple[int, ...]]:
    width = config["width"]
    shapes = {"embed": (config["vocab"], width), "final.norm": (width,), "final.norm.b": (width,), "head": (config["vocab"], width)}
    for index, layer in enumerate(config["layers"]):
        p, m = f"l{index}.", layer["mixer"]
        shapes.update({p + "norm1": (width,), p + "norm1.b": (width,)})
        h = m["heads"]
        if layer["type"] == "attention":
            shapes.update({p + "mix.q": (h * m["dim"], width), p + "mix.q.norm": (h * m["dim"],),
                           p + "mix.g": (h * m["vdim"], width), p + "mix.o": (width, h * m["vdim"])})
            if m.get("kv_from") is None:
                g = m["kv_heads"]
                shapes.update({p + "mix.k": (g * m["dim"], width), p + "mix.k.norm": (g * m["dim"],), p + "mix.v": (g * m["vdim"], width)})
        else:
            shapes.update({p + "mix.q": (h * (m["dim"] + m["rot_dim"]), width), p + "mix.dkv": (m["kv_rank"] + m["rot_dim"], width),
                           p + "mix.dkv.norm": (m["kv_rank"],), p + "mix.uk": (h * m["dim"], m["kv_rank"]),
                           p + "mix.uv": (h * m["vdim"], m["kv_rank"]), p + "mix.g": (h * m["vdim"], width),
                           p + "mix.o": (width, h * m["vdim"])})
        mlp = layer.get("mlp")
        if mlp is None:
            continue
        shapes.update({p + "norm2": (width,), p + "norm2.b": (width,)})
        ff, router = mlp["expert"]["ff"], mlp["router"]
        for e in range(router["experts"]):
            shapes.update({f"{p}mlp.e{e}.gate": (ff, width), f"{p}mlp.e{e}.up": (ff, width), f"{p}mlp.e{e}.down": (width, ff)})
        rows = router["experts"] + router.get("identity", 0)
        shapes.update({p + "mlp.router": (rows, width), p + "mlp.correction": (rows,)})
    return shapes


def make_weights(config: dict, seed: int) -> dict[str, torch.Tensor]:
    """Float32 tensors whose values are exact in bfloat16."""
    generator = torch.Generator().manual_seed(seed)
    weights = {}
    for name, shape in tensor_shapes(config).items():
        draw = torch.randn(shape, generator=generator)
        last = name.rsplit(".", 1)[-1]
        if name == "embed":
            value = draw
        elif last == "b":
            value = 0.3 * draw
        elif last in ("norm1", "norm2") or name == "final.norm" or last == "norm":
            value = 1.0 + 0.25 * draw
        elif last == "correction":
            value = 0.15 * draw
        elif last == "router":
            value = 2.0 * draw / math.sqrt(shape[-1])
        elif last == "q":
            value = 2.5 * draw / math.sqrt(shape[-1])             # sharp scores
        elif last in ("gate", "up"):
            value = 1.5 * draw / math.sqrt(shape[-1])             # a good share beyond the limit
        else:
            value = draw / math.sqrt(shape[-1])
        weights[name] = value.to(torch.bfloat16).to(torch.float32)
    return weights


def write_folder(folder: Path, config: dict, weights: dict[str, torch.Tensor], dtype: torch.dtype) -> Path:
    from rapid_llm_b200.weights.safetensors_io import write_safetensors

    folder.mkdir(parents=True, exist_ok=True)
    (folder / "config.json").write_text(json.dumps(config))
    write_safetensors(folder / "model.safetensors", {name: value.to(dtype) for name, value in weights.items()})
    return folder


def as_double(weights: dict[str, torch.Tensor]) -> dict[str, torch.Tensor]:
    return {name: value.double() for name, value in weights.items()}
