"""Configuration of the Zupupel decoder: a list of layers, each a windowed grouped-query attention or an attention
over a cached latent, followed by routed experts (or nothing), with the norm BEHIND every sum.

``config.json`` gives ``vocab``, ``width``, ``norm.eps``, ``embedding.scale``, ``postln_alpha``, ``logit_scale`` and
``layers``: one entry a layer, ``type`` names the mixer (``attention`` or ``latent_attention``), ``mixer`` its sizes
and constants, ``mlp`` the feed-forward (``kind`` ``moe``) or ``null``.  Layer ``i``'s tensors start with ``l<i>.``.

What the parts are built from:

* every layer is the arrangement ``postnorm``: ``x <- norm1(alpha x + mixer(x)); x <- norm2(alpha x + ff(x))`` with
  ``alpha = postln_alpha`` and layer norms (mean, variance, weight, bias ``<name>.b``); the float32 stream is opened
  by the scaled embedding;
* ``attention`` -> ``gqa_attention``: ``heads`` query heads over ``kv_heads`` key/value heads of ``dim`` (values
  ``vdim``), q and k RMS-normed over their WHOLE projection (weights ``q.norm``, ``k.norm``), the first ``rot.dims``
  entries of a head rotated by halves from frequencies ``rot.base^(-2i / dims)``, ``scale`` on the scores, a window
  of ``mask.size`` positions (none: all), a sigmoid gate ``g`` on the heads side by side.  ``kv_from: j`` makes the
  layer read layer ``j``'s cache (keys as cached, values) with queries, window and gate of its own: in the run order
  its entry names entry ``j`` as ``cache_from``, and layer ``j`` keeps as many positions as its widest reader needs;
* ``latent_attention`` -> ``latent_attention`` without a query latent (``q`` straight from the input), neighbouring
  entries rotated together, and the same kind of gate;
* ``moe`` -> ``routed_experts`` with ``weighting="softmax_all"``: ``router.experts`` clamped units of ``expert.ff``
  (``expert.limit``) and ``router.identity`` identity experts behind them, ``router.top`` chosen on the corrected
  scores within the ``groups.keep`` best of ``groups.count`` groups, weights renormalised;
* the model ends in a layer norm (``final.norm``) and an untied head whose logits are multiplied by ``logit_scale``:
  the constant is the last norm's ``gain``, ``W (n * c) = (W n) * c``.
"""

from __future__ import annotations

import copy
from dataclasses import dataclass, field
from typing import Any, Mapping

from .model_spec import LayerSpec, ModelSpec, PartSpec, ScheduleEntry

MAX_POSITIONS = 1 << 20     # nothing tabulated bounds a sequence; the engine's max_seq_len does

MIXER_TYPES = ("attention", "latent_attention")
EXPERT_ALPHA = 1.702        # the design fixes it: an expert is g * sigmoid(1.702 g) * (u + 1)


@dataclass
class ZupupelConfig:
    architecture = "Zupupel"
    model_type = "zupupel"

    vocab: int
    width: int
    norm_eps: float
    embedding_scale: float
    postln_alpha: float
    logit_scale: float
    layers: list[dict[str, Any]]
    raw: dict[str, Any] = field(default_factory=dict)

    # -------------------------------------------------------------- reading #
    @classmethod
    def from_dict(cls, raw: Mapping[str, Any], overrides: Mapping[str, Any] | None = None) -> "ZupupelConfig":
        raw = copy.deepcopy(dict(raw))
        raw.update(copy.deepcopy(dict(overrides or {})))
        for key in ("vocab", "width", "layers", "norm"):
            if key not in raw:
                raise ValueError(f"config.json of a Zupupel model lacks {key!r}")
        config = cls(vocab=int(raw["vocab"]), width=int(raw["width"]), norm_eps=float(raw["norm"]["eps"]),
                     embedding_scale=float((raw.get("embedding") or {}).get("scale", 1.0)),
                     postln_alpha=float(raw.get("postln_alpha", 1.0)), logit_scale=float(raw.get("logit_scale", 1.0)),
                     layers=list(raw["layers"]), raw=raw)
        config.validate()
        return config

    def validate(self) -> None:
        if not self.layers:
            raise ValueError("a Zupupel model needs at least one layer")
        for index, layer in enumerate(self.layers):
            if layer.get("type") not in MIXER_TYPES:
                raise ValueError(f"layer {index}: unknown mixer type {layer.get('type')!r}")
            mixer = layer.get("mixer") or {}
            if layer["type"] == "attention":
                for key in ("heads", "kv_heads", "dim", "vdim", "scale"):
                    if key not in mixer:
                        raise ValueError(f"layer {index}: the attention mixer lacks {key!r}")
                source = mixer.get("kv_from")
                if source is not None:
                    source = int(source)
                    if not 0 <= source < index or self.layers[source].get("type") != "attention":
                        raise ValueError(f"layer {index}: kv_from must name an earlier attention layer, got {source}")
                    theirs = self.layers[source]["mixer"]
                    if theirs.get("kv_from") is not None:
                        raise ValueError(f"layer {index}: layer {source} has no keys and values of its own")
                    for key in ("kv_heads", "dim", "vdim"):
                        if int(theirs[key]) != int(mixer[key]):
                            raise ValueError(f"layer {index}: {key} differs from layer {source}'s, whose cache it reads")
            else:
                for key in ("heads", "dim", "rot_dim", "vdim", "kv_rank", "scale"):
                    if key not in mixer:
                        raise ValueError(f"layer {index}: the latent attention mixer lacks {key!r}")
                rot = mixer.get("rot") or {}
                if int(mixer["rot_dim"]) and int(rot.get("dims", mixer["rot_dim"])) != int(mixer["rot_dim"]):
                    raise ValueError(f"layer {index}: rot.dims must equal rot_dim")
            mlp = layer.get("mlp")
            if mlp is not None and mlp.get("kind") != "moe":
                raise ValueError(f"layer {index}: unknown feed-forward kind {mlp.get('kind')!r}")

    def to_dict(self) -> dict[str, Any]:
        return {"architecture": self.architecture, "vocab": self.vocab, "width": self.width,
                "norm": {"eps": self.norm_eps}, "embedding": {"scale": self.embedding_scale},
                "postln_alpha": self.postln_alpha, "logit_scale": self.logit_scale, "layers": copy.deepcopy(self.layers)}

    # ----------------------------------------------------------------- spec #
    @staticmethod
    def _window(sizes: Mapping[str, Any]) -> int:
        return int((sizes.get("mask") or {}).get("size", 0) or 0)

    def _kept(self, index: int) -> int:
        """Positions layer ``index`` must keep cached: the widest window among itself and the layers that read its
        cache; 0 (everything) as soon as one of them has no window."""
        windows = [self._window(self.layers[index]["mixer"])]
        for other in self.layers[index + 1:]:
            source = other["mixer"].get("kv_from") if other["type"] == "attention" else None
            if source is not None and int(source) == index:
                windows.append(self._window(other["mixer"]))
        return 0 if 0 in windows else max(windows)

    def _mixer(self, index: int) -> PartSpec:
        layer = self.layers[index]
        sizes = layer["mixer"]
        rot = sizes.get("rot") or {}
        if layer["type"] == "latent_attention":
            return PartSpec("latent_attention", {
                "hidden_size": self.width, "num_heads": int(sizes["heads"]), "head_dim": int(sizes["dim"]),
                "rot_dim": int(sizes["rot_dim"]), "value_dim": int(sizes["vdim"]), "kv_rank": int(sizes["kv_rank"]),
                "q_rank": None, "scale": float(sizes["scale"]), "norm_eps": self.norm_eps, "rotation": "neighbours",
                "wide_gate": True,
                "position": PartSpec("rotary_frequencies", {
                    "rotary_dim": int(sizes["rot_dim"]), "theta": float(rot.get("base", 10000.0)),
                    "max_positions": MAX_POSITIONS}),
            })
        shares = sizes.get("kv_from") is not None
        return PartSpec("gqa_attention", {
            "hidden_size": self.width, "num_heads": int(sizes["heads"]), "num_kv_heads": int(sizes["kv_heads"]),
            "head_dim": int(sizes["dim"]), "value_dim": int(sizes["vdim"]), "scale": float(sizes["scale"]),
            "qk_norm": True, "qk_norm_over": "row", "qk_norm_eps": self.norm_eps, "window": self._window(sizes),
            "cache_window": None if shares else self._kept(index), "shares_cache": shares, "gate": "sigmoid",
            "position": PartSpec("rotary_frequencies", {
                "rotary_dim": int(rot.get("dims", 0)), "theta": float(rot.get("base", 10000.0)),
                "max_positions": MAX_POSITIONS}),
            "names": {"q_proj.weight": "q", "k_proj.weight": "k", "v_proj.weight": "v", "o_proj.weight": "o",
                      "g_proj.weight": "g", "q_norm.weight": "q.norm", "k_norm.weight": "k.norm"},
        })

    def _feed_forward(self, mlp: Mapping[str, Any] | None) -> PartSpec | None:
        if mlp is None:
            return None
        router = mlp["router"]
        groups = router.get("groups") or {}
        return PartSpec("routed_experts", {
            "hidden_size": self.width, "num_experts": int(router["experts"]), "top_k": int(router["top"]),
            "expert_size": int(mlp["expert"]["ff"]), "scale_input": False, "weighting": "softmax_all",
            "num_groups": int(groups.get("count", 1)), "group_keep": int(groups.get("keep", 1)),
            "identity_experts": int(router.get("identity", 0)), "expert_limit": float(mlp["expert"]["limit"]),
            "expert_alpha": EXPERT_ALPHA,
        })

    def to_spec(self) -> ModelSpec:
        norm = PartSpec("layernorm", {"size": self.width, "eps": self.norm_eps, "name": "", "bias_suffix": ".b"})
        names = {"mixer_norm": "norm1", "mixer": "mix.", "feed_forward_norm": "norm2", "feed_forward": "mlp."}
        layers, schedule = [], []
        for index, layer in enumerate(self.layers):
            layers.append(LayerSpec(arrangement="postnorm", mixer=self._mixer(index),
                                    feed_forward=self._feed_forward(layer.get("mlp")), norm=norm, prefix=f"l{index}.",
                                    names=names, arrangement_params={"alpha": self.postln_alpha}))
            source = layer["mixer"].get("kv_from") if layer["type"] == "attention" else None
            schedule.append(ScheduleEntry(index, cache_from=None if source is None else int(source)))
        spec = ModelSpec(
            architecture=self.architecture, vocab_size=self.vocab, hidden_size=self.width, max_positions=MAX_POSITIONS,
            embedding=PartSpec("token_embedding", {"vocab_size": self.vocab, "hidden_size": self.width, "name": "",
                                                   "scale": self.embedding_scale, "opens_stream": True}),
            layers=tuple(layers), schedule=tuple(schedule),
            final_norm=norm.with_params(gain=self.logit_scale),
            head=PartSpec("lm_head", {"vocab_size": self.vocab, "hidden_size": self.width, "tied": False, "name": ""}),
            final_norm_prefix="final.norm", embedding_prefix="embed", head_prefix="head",
        )
        spec.validate()
        return spec
