"""Small Basitar configurations and seeded weights for the tests.

The weights are drawn so that every mechanism carries weight: token-pair and position rows of the token rows' size,
norm weights spread around zero, decays from nearly none to nearly total, bonuses and router biases of the size of
what they are added to, sharp attention.  Every value is rounded to bfloat16 once, so a folder written in either
precision and the float64 plain implementation hold the same numbers.
"""

from __future__ import annotations

import copy
import json
import math
from pathlib import Path

import torch


def dense(ff=40):
    return {"kind": "dense", "ff": ff}


def moe(experts=5, top=2, ff=24):
    return {"kind": "moe", "router": {"experts": experts, "top": top}, "expert": {"ff": ff}}


def latent_layer(*, heads=3, dim=16, rot_dim=8, vdim=24, kv_rank=40, q_rank=24, base=100.0, scale=0.3, second=False,
                 scaling=None, mlp=None, weights_of=None):
    rot = {"base": base, "dims": rot_dim}
    if scaling:
        rot["scaling"] = dict(scaling)
    layer = {"type": "latent_attention_2" if second else "latent_attention",
             "mixer": {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "kv_rank": kv_rank, "q_rank": q_rank,
                       "rot": rot, "scale": scale}, "mlp": mlp}
    if weights_of is not None:
        layer["weights_of"] = weights_of
    return layer


def wkv_layer(*, heads=2, dim=16, rank=6, mlp=None, weights_of=None):
    """``rank`` is not part of the file's configuration (the tensors' shapes give it); the tests keep it beside the
    mixer's sizes under a key of their own and strip it when a folder is written without it."""
    layer = {"type": "wkv", "mixer": {"heads": heads, "dim": dim, "decay_rank": rank}, "mlp": mlp}
    if weights_of is not None:
        layer["weights_of"] = weights_of
    return layer


YARN = {"factor": 8.0, "original": 64, "fast": 16.0, "slow": 2.0}


def make_config(layers, *, width=64, vocab=97, eps=1e-5, max_positions=512, buckets=53, mul_prev=7, mul_cur=3) -> dict:
    return {"architecture": "Basitar", "vocab": vocab, "width": width, "max_positions": max_positions,
            "norm": {"eps": eps}, "embedding": {"bigram": {"buckets": buckets, "mul_prev": mul_prev, "mul_cur": mul_cur}},
            "layers": copy.deepcopy(list(layers))}


CONFIGS = {
    # one mechanism a model
    "latent": make_config([latent_layer(mlp=dense())]),
    "latent2": make_config([latent_layer(heads=2, dim=24, rot_dim=16, vdim=16, kv_rank=32, q_rank=16, second=True, scaling=YARN,
                                         mlp=dense(ff=36))], width=48, vocab=61),
    "wkv": make_config([wkv_layer(mlp=dense(ff=24))], width=40, vocab=70, buckets=1),
    "experts": make_config([wkv_layer(heads=1, dim=8, rank=3, mlp=moe())], width=40, vocab=70, mul_prev=1, mul_cur=1),
    # the layers in another order, a looped layer of each kind, a layer without a feed-forward, one and all experts,
    # the second attention without stretched frequencies, rows of the cache that are and are not multiples of 16
    "stack": make_config([
        wkv_layer(heads=3, dim=16, rank=5, mlp=moe(experts=3, top=1, ff=16)),
        latent_layer(heads=2, dim=32, rot_dim=16, vdim=32, kv_rank=48, q_rank=32, second=True, mlp=None),
        latent_layer(heads=5, dim=8, rot_dim=4, vdim=8, kv_rank=24, q_rank=16, base=1.0e4, scale=0.5, mlp=moe(experts=4, top=4, ff=8)),
        wkv_layer(heads=3, dim=16, rank=5, mlp=moe(experts=3, top=1, ff=16), weights_of=0),
        latent_layer(heads=1, dim=48, rot_dim=32, vdim=64, kv_rank=96, q_rank=40, second=True, scaling=YARN, mlp=dense(ff=24)),
        latent_layer(heads=5, dim=8, rot_dim=4, vdim=8, kv_rank=24, q_rank=16, base=1.0e4, scale=0.5, mlp=moe(experts=4, top=4, ff=8),
                     weights_of=2),
    ], width=72, vocab=130, buckets=211, mul_prev=13, mul_cur=29),
    # nothing is a multiple of 4 or 8: every kernel's element-by-element path
    "narrow": make_config([
        latent_layer(heads=3, dim=10, rot_dim=6, vdim=6, kv_rank=14, q_rank=10, scale=0.7, mlp=moe(experts=7, top=3, ff=10)),
        wkv_layer(heads=3, dim=6, rank=3, mlp=dense(ff=22)),
        latent_layer(heads=2, dim=14, rot_dim=2, vdim=22, kv_rank=22, q_rank=6, second=True,
                     scaling={"factor": 2.0, "original": 32, "fast": 4.0, "slow": 1.0}, mlp=moe(experts=1, top=1, ff=14)),
    ], width=50, vocab=83, eps=1e-6, buckets=17, mul_prev=5, mul_cur=11),
}


def bare(config: dict) -> dict:
    """The configuration as a model's folder holds it: without the decays' ranks."""
    out = copy.deepcopy(config)
    for layer in out["layers"]:
        layer["mixer"].pop("decay_rank", None)
    return out


def tensor_shapes(config: dict) -> dict[str, tuple[int, ...]]:
    width = config["width"]
    shapes = {"embed": (config["vocab"], width), "bigram": (config["embedding"]["bigram"]["buckets"] + 1, width),
              "pos": (config["max_positions"], width), "final.norm": (width,)}
    for index, layer in enumerate(config["layers"]):
        if layer.get("weights_of") is not None:
            continue
        p, m = f"l{index}.", layer["mixer"]
        for name in ("norm1", "norm1b"):
            shapes[p + name] = (width,)
        if layer["type"] == "wkv":
            c = m["heads"] * m["dim"]
            for which in "rkvgw":
                shapes[f"{p}mix.mu.{which}"] = (width,)
            for which in "rkvg":
                shapes[f"{p}mix.{which}"] = (c, width)
            shapes.update({p + "mix.w1": (m["decay_rank"], width), p + "mix.w2": (c, m["decay_rank"]), p + "mix.w0": (c,),
                           p + "mix.u": (m["heads"], m["dim"]), p + "mix.norm": (c,), p + "mix.o": (width, c)})
        else:
            h = m["heads"]
            shapes.update({p + "mix.dq": (m["q_rank"], width), p + "mix.dq.norm": (m["q_rank"],),
                           p + "mix.uq": (h * (m["dim"] + m["rot_dim"]), m["q_rank"]),
                           p + "mix.dkv": (m["kv_rank"] + m["rot_dim"], width), p + "mix.dkv.norm": (m["kv_rank"],),
                           p + "mix.uk": (h * m["dim"], m["kv_rank"]), p + "mix.uv": (h * m["vdim"], m["kv_rank"]),
                           p + "mix.o": (width, h * m["vdim"])})
            if layer["type"] == "latent_attention_2":
                shapes[p + "mix.g"] = (h, width)
        mlp = layer.get("mlp")
        if mlp is None:
            continue
        for name in ("norm2", "norm2b"):
            shapes[p + name] = (width,)
        if mlp["kind"] == "dense":
            shapes.update({p + "mlp.gate": (mlp["ff"], width), p + "mlp.up": (mlp["ff"], width), p + "mlp.down": (width, mlp["ff"])})
            continue
        ff = mlp["expert"]["ff"]
        for e in range(mlp["router"]["experts"]):
            shapes.update({f"{p}mlp.e{e}.gate": (ff, width), f"{p}mlp.e{e}.up": (ff, width), f"{p}mlp.e{e}.down": (width, ff)})
        shapes[p + "mlp.router"] = (mlp["router"]["experts"], width)
        shapes[p + "mlp.router.b"] = (mlp["router"]["experts"],)
    return shapes


def make_weights(config: dict, seed: int) -> dict[str, torch.Tensor]:
    """Float32 tensors whose values are exact in bfloat16."""
    generator = torch.Generator().manual_seed(seed)
    weights = {}
    for name, shape in tensor_shapes(config).items():
        draw = torch.randn(shape, generator=generator)
        last = name.rsplit(".", 1)[-1]
        if name in ("embed", "bigram", "pos"):
            value = draw * (1.0 if name == "embed" else 0.7)
        elif last in ("norm1", "norm1b", "norm2", "norm2b") or name == "final.norm":
            value = 0.25 * draw                                   # stored around zero
        elif name.endswith("dq.norm") or name.endswith("dkv.norm") or name.endswith("mix.norm"):
            value = 1.0 + 0.2 * draw
        elif ".mu." in name:
            value = torch.rand(shape, generator=generator)
        elif last == "w0":
            value = -2.0 + 2.0 * draw                             # decays from about 0.2 to nearly 1
        elif last == "u":
            value = draw
        elif last == "b":
            value = 0.5 * draw
        elif last == "uq":
            value = 3.0 * draw / math.sqrt(shape[-1])             # sharp scores
        else:
            value = draw / math.sqrt(shape[-1])
        weights[name] = value.to(torch.bfloat16).to(torch.float32)
    return weights


def write_folder(folder: Path, config: dict, weights: dict[str, torch.Tensor], dtype: torch.dtype, keep_ranks: bool = False) -> Path:
    from rapid_llm_b200.weights.safetensors_io import write_safetensors

    folder.mkdir(parents=True, exist_ok=True)
    (folder / "config.json").write_text(json.dumps(config if keep_ranks else bare(config)))
    write_safetensors(folder / "model.safetensors", {name: value.to(dtype) for name, value in weights.items()})
    return folder


def as_double(weights: dict[str, torch.Tensor]) -> dict[str, torch.Tensor]:
    return {name: value.double() for name, value in weights.items()}
