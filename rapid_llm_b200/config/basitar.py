"""Configuration of the Basitar decoder: a list of layers, each with a linear-attention mixer with input-made
decays or one of two latent-attention mixers, and a dense or routed feed-forward (or none).

``config.json`` gives ``vocab``, ``width``, ``max_positions``, ``norm.eps``, ``embedding.bigram`` (``buckets``,
``mul_prev``, ``mul_cur``) and ``layers``: one entry a layer, ``type`` names the mixer (``wkv``,
``latent_attention`` or ``latent_attention_2``), ``mixer`` its sizes and constants, ``mlp`` the feed-forward
(``kind`` ``dense`` or ``moe``) or ``null``.  Layer ``i``'s tensors start with ``l<i>.``; a layer with
``weights_of: j`` has none of its own and runs layer ``j``'s parts on a cache and state of its own.  The rank of
the ``wkv`` mixer's decay product is not in the file: it is the first extent of the tensor ``mix.w1``, so the
configuration is read from a folder (:meth:`BasitarConfig.from_folder`) or given ``decay_rank`` per mixer.

What the parts are built from:

* the embedding is ``summed_embedding``: token row + token-pair row + learned position row, opening the float32 stream;
* every layer is the arrangement ``sandwich``: a norm in front of and behind each sublayer, all ``rmsnorm`` with
  ``unit_offset`` (the file stores the weight minus one);
* ``wkv`` -> ``wkv`` (:class:`~rapid_llm_b200.parts.recurrent.ShiftedDecay`);
* ``latent_attention`` -> ``latent_attention`` with ``rotation="halves"`` and plain frequencies;
  ``latent_attention_2`` -> the same mixer with ``rotation="neighbours"``, ``yarn_frequencies`` where ``rot.scaling``
  is given, and a sigmoid gate per head;
* ``dense`` -> ``swiglu``; ``moe`` -> ``routed_experts`` with a router bias, weights that are the softmax
  over the chosen logits, applied to the experts' outputs;
* the head is tied to the embedding table.
"""

from __future__ import annotations

import copy
from dataclasses import dataclass, field
from pathlib import Path
from typing import Any, Mapping

from .model_spec import LayerSpec, ModelSpec, PartSpec, ScheduleEntry

MIXER_TYPES = ("wkv", "latent_attention", "latent_attention_2")
MLP_KINDS = ("dense", "moe")


@dataclass
class BasitarConfig:
    architecture = "Basitar"
    model_type = "basitar"

    vocab: int
    width: int
    max_positions: int
    norm_eps: float
    bigram: dict[str, int]
    layers: list[dict[str, Any]]
    raw: dict[str, Any] = field(default_factory=dict)

    # -------------------------------------------------------------- reading #
    @classmethod
    def from_folder(cls, model_dir, raw: Mapping[str, Any], overrides: Mapping[str, Any] | None = None) -> "BasitarConfig":
        """As :meth:`from_dict`, with every ``wkv`` mixer's ``decay_rank`` read from the shape of its ``mix.w1``."""
        raw = copy.deepcopy(dict(raw))
        shapes = None
        for index, layer in enumerate(raw.get("layers") or []):
            if layer.get("type") != "wkv" or "decay_rank" in (layer.get("mixer") or {}):
                continue
            if shapes is None:
                from ..weights.safetensors_io import SafetensorsFile

                shapes = {}
                for path in sorted(Path(model_dir).glob("*.safetensors")):
                    handle = SafetensorsFile(path)
                    shapes.update({name: handle.shape(name) for name in handle.keys()})
                    handle.close()
            owner = layer.get("weights_of", index)
            name = f"l{owner}.mix.w1"
            if name not in shapes:
                raise ValueError(f"layer {index}: the decay's rank is the first extent of {name!r}, which is missing")
            layer.setdefault("mixer", {})["decay_rank"] = int(shapes[name][0])
        return cls.from_dict(raw, overrides)

    @classmethod
    def from_dict(cls, raw: Mapping[str, Any], overrides: Mapping[str, Any] | None = None) -> "BasitarConfig":
        raw = copy.deepcopy(dict(raw))
        raw.update(copy.deepcopy(dict(overrides or {})))
        for key in ("vocab", "width", "layers", "norm", "max_positions", "embedding"):
            if key not in raw:
                raise ValueError(f"config.json of a Basitar model lacks {key!r}")
        bigram = (raw["embedding"] or {}).get("bigram")
        if not bigram:
            raise ValueError("config.json of a Basitar model lacks 'embedding.bigram'")
        config = cls(vocab=int(raw["vocab"]), width=int(raw["width"]), max_positions=int(raw["max_positions"]),
                     norm_eps=float(raw["norm"]["eps"]),
                     bigram={key: int(bigram[key]) for key in ("buckets", "mul_prev", "mul_cur")},
                     layers=list(raw["layers"]), raw=raw)
        config.validate()
        return config

    def validate(self) -> None:
        if not self.layers:
            raise ValueError("a Basitar model needs at least one layer")
        for index, layer in enumerate(self.layers):
            if layer.get("type") not in MIXER_TYPES:
                raise ValueError(f"layer {index}: unknown mixer type {layer.get('type')!r}")
            mixer = layer.get("mixer") or {}
            wanted = ("heads", "dim", "decay_rank") if layer["type"] == "wkv" else (
                "heads", "dim", "rot_dim", "vdim", "kv_rank", "q_rank", "scale")
            for key in wanted:
                if key not in mixer:
                    raise ValueError(f"layer {index}: the {layer['type']} mixer lacks {key!r}")
            mlp = layer.get("mlp")
            if mlp is not None and mlp.get("kind") not in MLP_KINDS:
                raise ValueError(f"layer {index}: unknown feed-forward kind {mlp.get('kind')!r}")
            owner = layer.get("weights_of")
            if owner is not None:
                if not 0 <= int(owner) < len(self.layers) or int(owner) == index:
                    raise ValueError(f"layer {index}: weights_of names layer {owner}, which is not another layer")
                if self.layers[int(owner)].get("weights_of") is not None:
                    raise ValueError(f"layer {index}: weights_of names layer {owner}, which has no tensors of its own")
                if self.layers[int(owner)].get("type") != layer["type"]:
                    raise ValueError(f"layer {index}: it is a {layer['type']} layer, the layer whose weights it uses is not")

    def to_dict(self) -> dict[str, Any]:
        return {"architecture": self.architecture, "vocab": self.vocab, "width": self.width,
                "max_positions": self.max_positions, "norm": {"eps": self.norm_eps},
                "embedding": {"bigram": dict(self.bigram)}, "layers": copy.deepcopy(self.layers)}

    # ----------------------------------------------------------------- spec #
    def _mixer(self, layer: Mapping[str, Any]) -> PartSpec:
        sizes = layer["mixer"]
        if layer["type"] == "wkv":
            return PartSpec("wkv", {"hidden_size": self.width, "num_heads": int(sizes["heads"]),
                                    "key_dim": int(sizes["dim"]), "decay_rank": int(sizes["decay_rank"]),
                                    "norm_eps": self.norm_eps})
        rot = sizes.get("rot") or {}
        rot_dim = int(sizes["rot_dim"])
        if int(rot.get("dims", rot_dim)) != rot_dim:
            raise ValueError("a latent-attention mixer rotates its whole rotated part: rot.dims must equal rot_dim")
        frequencies = {"rotary_dim": rot_dim, "theta": float(rot.get("base", 10000.0)), "max_positions": self.max_positions}
        scaling = rot.get("scaling") if layer["type"] == "latent_attention_2" else None
        if scaling:
            position = PartSpec("yarn_frequencies", {**frequencies, "factor": float(scaling["factor"]),
                                                     "original": float(scaling["original"]),
                                                     "fast": float(scaling["fast"]), "slow": float(scaling["slow"])})
        else:
            position = PartSpec("rotary_frequencies", frequencies)
        second = layer["type"] == "latent_attention_2"
        return PartSpec("latent_attention", {
            "hidden_size": self.width, "num_heads": int(sizes["heads"]), "head_dim": int(sizes["dim"]), "rot_dim": rot_dim,
            "value_dim": int(sizes["vdim"]), "kv_rank": int(sizes["kv_rank"]), "q_rank": int(sizes["q_rank"]),
            "scale": float(sizes["scale"]), "norm_eps": self.norm_eps, "position": position,
            "rotation": "neighbours" if second else "halves", "head_gate": second,
        })

    def _feed_forward(self, mlp: Mapping[str, Any] | None) -> PartSpec | None:
        if mlp is None:
            return None
        if mlp["kind"] == "dense":
            return PartSpec("swiglu", {"hidden_size": self.width, "intermediate_size": int(mlp["ff"]),
                                       "gate_name": "gate", "up_name": "up", "down_name": "down", "suffix": ""})
        return PartSpec("routed_experts", {
            "hidden_size": self.width, "num_experts": int(mlp["router"]["experts"]), "top_k": int(mlp["router"]["top"]),
            "expert_size": int(mlp["expert"]["ff"]), "scale_input": False, "router_bias": True,
            "weighting": "softmax_chosen",
        })

    def to_spec(self) -> ModelSpec:
        norm = PartSpec("rmsnorm", {"size": self.width, "eps": self.norm_eps, "name": "", "unit_offset": True})
        owners = [index for index, layer in enumerate(self.layers) if layer.get("weights_of") is None]
        place = {index: at for at, index in enumerate(owners)}
        layers = [LayerSpec(arrangement="sandwich", mixer=self._mixer(self.layers[index]),
                            feed_forward=self._feed_forward(self.layers[index].get("mlp")), norm=norm, prefix=f"l{index}.")
                  for index in owners]
        schedule = tuple(ScheduleEntry(place[int(layer.get("weights_of", index)) if layer.get("weights_of") is not None else index])
                         for index, layer in enumerate(self.layers))
        spec = ModelSpec(
            architecture=self.architecture, vocab_size=self.vocab, hidden_size=self.width, max_positions=self.max_positions,
            embedding=PartSpec("summed_embedding", {
                "vocab_size": self.vocab, "hidden_size": self.width, "pair_buckets": self.bigram["buckets"],
                "pair_mul_prev": self.bigram["mul_prev"], "pair_mul_cur": self.bigram["mul_cur"],
                "max_positions": self.max_positions, "name": "embed", "pair_name": "bigram", "position_name": "pos"}),
            layers=tuple(layers), schedule=schedule, final_norm=norm,
            head=PartSpec("lm_head", {"vocab_size": self.vocab, "hidden_size": self.width, "tied": True, "name": ""}),
            final_norm_prefix="final.norm", embedding_prefix="", head_prefix="head",
        )
        spec.validate()
        return spec
