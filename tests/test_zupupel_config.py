"""Zupupel's configuration on the CPU: parts and their parameters, expected tensors, the run order, what a layer
keeps cached for its readers, refusals; the plain implementation against second forms of the same equations; and that
every mechanism of the plain implementation moves the logits of the test models (so a comparison with it has teeth)."""

from __future__ import annotations

import copy
import math

import pytest
import torch
from plain_zupupel import (attention_mixer, clamped_expert, forward, latent_attention_mixer, layer_norm, rms_norm, rotate,
                           route, softmax_attention)
from zupupel_models import CONFIGS, as_double, attention_layer, latent_layer, make_config, make_weights, moe, tensor_shapes

from rapid_llm_b200.config import ZupupelConfig, resolve_architecture
from rapid_llm_b200.models.causal_lm import CausalLM


def test_the_registry_finds_the_architecture():
    assert resolve_architecture({"architecture": "Zupupel"}) is ZupupelConfig


@pytest.mark.parametrize("name", list(CONFIGS))
def test_the_model_expects_the_files_tensors(name):
    config = CONFIGS[name]
    model = CausalLM(ZupupelConfig.from_dict(config).to_spec(), torch.float32, "cpu")
    assert {n: tuple(s.shape) for n, s in model.tensor_specs().items()} == tensor_shapes(config)


def test_parts_run_order_and_what_a_layer_keeps_for_its_readers():
    spec = ZupupelConfig.from_dict(CONFIGS["stack"]).to_spec()
    assert [layer.arrangement for layer in spec.layers] == ["postnorm"] * 7
    assert all(layer.arrangement_params == {"alpha": 2.5} for layer in spec.layers)
    assert [layer.mixer.kind for layer in spec.layers] == ["latent_attention", "gqa_attention", "gqa_attention", "gqa_attention",
                                                            "gqa_attention", "latent_attention", "gqa_attention"]
    assert [entry.cache_from for entry in spec.schedule] == [None, None, 1, None, 1, None, 3]
    # layer 1 (window 9) is read through windows of 20 and 5: it keeps 20; layer 3 has no window at all
    assert [layer.mixer.params.get("window") for layer in spec.layers] == [None, 9, 20, 0, 5, None, 7]
    assert [layer.mixer.params.get("cache_window") for layer in spec.layers] == [None, 20, None, 0, None, None, None]
    first = spec.layers[1].mixer.params
    assert (first["qk_norm"], first["qk_norm_over"], first["gate"], first["shares_cache"]) == (True, "row", "sigmoid", False)
    assert first["position"].kind == "rotary_frequencies" and first["position"].params["rotary_dim"] == 16
    latent = spec.layers[0].mixer.params
    assert (latent["q_rank"], latent["rotation"], latent["wide_gate"]) == (None, "neighbours", True)
    experts = spec.layers[1].feed_forward.params
    assert (experts["num_experts"], experts["identity_experts"], experts["top_k"], experts["num_groups"], experts["group_keep"],
            experts["weighting"], experts["scale_input"], experts["expert_alpha"]) == (5, 1, 1, 3, 2, "softmax_all", False, 1.702)
    assert spec.layers[2].feed_forward is None
    assert spec.embedding.params["scale"] == 0.6 and spec.embedding.params["opens_stream"]
    assert spec.final_norm.kind == "layernorm" and spec.final_norm.params["gain"] == 0.4
    model = CausalLM(spec, torch.float32, "cpu")
    needs = model.cache_needs()
    assert [need is not None for need in needs] == [True, True, False, True, False, True, False]
    assert (needs[1].kind, needs[1].window, needs[3].kind) == ("window", 20, "full")
    assert needs[0].token_shape == (64,) and needs[5].token_shape == (32,)
    # a reader with a window behind a layer without one keeps that layer's cache whole
    config = make_config([attention_layer(window=6), attention_layer(window=0, kv_from=0)])
    assert ZupupelConfig.from_dict(config).to_spec().layers[0].mixer.params["cache_window"] == 0
    # no mask, no rotation, no groups, no identity experts in the file
    bare = make_config([attention_layer(window=0, rot_dims=0, mlp=moe())])
    del bare["layers"][0]["mlp"]["router"]["groups"], bare["layers"][0]["mlp"]["router"]["identity"]
    params = ZupupelConfig.from_dict(bare).to_spec().layers[0]
    assert params.mixer.params["window"] == 0 and params.mixer.params["position"].params["rotary_dim"] == 0
    assert (params.feed_forward.params["num_groups"], params.feed_forward.params["identity_experts"]) == (1, 0)


def test_refusals():
    config = copy.deepcopy(CONFIGS["window"])
    config["layers"][0]["type"] = "lightning"
    with pytest.raises(ValueError, match="unknown mixer type"):
        ZupupelConfig.from_dict(config)
    config = copy.deepcopy(CONFIGS["experts"])
    config["layers"][0]["mlp"]["kind"] = "dense"
    with pytest.raises(ValueError, match="unknown feed-forward kind"):
        ZupupelConfig.from_dict(config)
    with pytest.raises(ValueError, match="kv_from"):
        ZupupelConfig.from_dict(make_config([attention_layer(kv_from=0)]))
    with pytest.raises(ValueError, match="kv_from"):
        ZupupelConfig.from_dict(make_config([latent_layer(), attention_layer(kv_from=0)]))
    with pytest.raises(ValueError, match="no keys and values of its own"):
        ZupupelConfig.from_dict(make_config([attention_layer(), attention_layer(kv_from=0), attention_layer(kv_from=1)]))
    with pytest.raises(ValueError, match="differs"):
        ZupupelConfig.from_dict(make_config([attention_layer(), attention_layer(vdim=8, kv_from=0)]))
    config = copy.deepcopy(CONFIGS["latent"])
    del config["width"]
    with pytest.raises(ValueError, match="width"):
        ZupupelConfig.from_dict(config)
    config = make_config([attention_layer(mlp=moe(experts=5, identity=2, groups=2))])      # 7 rows in 2 groups
    with pytest.raises(ValueError, match="groups"):
        CausalLM(ZupupelConfig.from_dict(config).to_spec(), torch.float32, "cpu")
    config = make_config([attention_layer(mlp=moe(experts=6, identity=2, groups=4, keep=1, top=3))])     # 2 rows to choose 3 from
    with pytest.raises(ValueError, match="top_k"):
        CausalLM(ZupupelConfig.from_dict(config).to_spec(), torch.float32, "cpu")


# ----------------------------------------------------------- second forms of the plain equations -- #
def test_the_two_rotations_are_one_rotation_in_two_layouts():
    generator = torch.Generator().manual_seed(0)
    rows = torch.randn(7, 3, 12, generator=generator, dtype=torch.float64)
    positions = torch.arange(7)
    halves = rotate(rows, positions, 8, 50.0, "halves")
    # entry i of the first half and entry i of the second, side by side, are neighbours 2i and 2i + 1
    shuffled = rows.clone()
    shuffled[..., 0:8:2], shuffled[..., 1:8:2] = rows[..., :4], rows[..., 4:8]
    neighbours = rotate(shuffled, positions, 8, 50.0, "neighbours")
    assert torch.allclose(neighbours[..., 0:8:2], halves[..., :4]) and torch.allclose(neighbours[..., 1:8:2], halves[..., 4:8])
    assert torch.equal(halves[..., 8:], rows[..., 8:]) and torch.allclose(halves[0], rows[0])
    # a score depends on the distance alone
    q, k = rows[:, :1], torch.randn(7, 1, 12, generator=generator, dtype=torch.float64)
    one = (rotate(q[2:3].expand(7, 1, 12), positions, 8, 50.0, "halves")[5] * rotate(k[1:2].expand(7, 1, 12), positions, 8, 50.0, "halves")[3]).sum()
    two = (rotate(q[2:3].expand(7, 1, 12), positions, 8, 50.0, "halves")[4] * rotate(k[1:2].expand(7, 1, 12), positions, 8, 50.0, "halves")[2]).sum()
    assert torch.allclose(one, two)


def test_the_latent_mixer_with_queries_moved_into_the_latent():
    """The form the engine computes: ``W_uk`` on the query side and ``W_uv`` behind the attention over the cached rows
    ``[c | rotated key part]`` gives what the expanded keys and values give."""
    config = CONFIGS["latent"]
    sizes = config["layers"][0]["mixer"]
    weights = as_double(make_weights(config, seed=2))
    generator = torch.Generator().manual_seed(1)
    h = torch.randn(19, config["width"], generator=generator, dtype=torch.float64)
    want = latent_attention_mixer(h, weights, "l0.mix.", sizes, 1e-5)
    H, dim, rd, vdim, rank = sizes["heads"], sizes["dim"], sizes["rot_dim"], sizes["vdim"], sizes["kv_rank"]
    positions = torch.arange(19)
    q = (h @ weights["l0.mix.q"].T).view(19, H, dim + rd)
    down = h @ weights["l0.mix.dkv"].T
    c = rms_norm(down[:, :rank], weights["l0.mix.dkv.norm"], 1e-5)
    row = torch.cat([c, rotate(down[:, None, rank:], positions, rd, sizes["rot"]["base"], "neighbours")[:, 0]], dim=-1)
    uk = weights["l0.mix.uk"].view(H, dim, rank)
    wide_q = torch.cat([torch.einsum("thd,hdr->thr", q[..., :dim], uk),
                        rotate(q[..., dim:], positions, rd, sizes["rot"]["base"], "neighbours")], dim=-1)
    shared = row[:, None, :].expand(19, H, rank + rd)
    attended = softmax_attention(wide_q, shared, shared, sizes["scale"], 0)[..., :rank]
    values = torch.einsum("thr,hvr->thv", attended, weights["l0.mix.uv"].view(H, vdim, rank)).reshape(19, H * vdim)
    got = (values * torch.sigmoid(h @ weights["l0.mix.g"].T)) @ weights["l0.mix.o"].T
    assert torch.allclose(got, want, atol=1e-10)


def test_the_window_and_the_groups_of_heads_by_hand():
    config = CONFIGS["window"]
    sizes = config["layers"][0]["mixer"]
    weights = as_double(make_weights(config, seed=4))
    h = torch.randn(30, config["width"], generator=torch.Generator().manual_seed(2), dtype=torch.float64)
    want, (k, v) = attention_mixer(h, weights, "l0.mix.", sizes, 1e-5)
    H, G, dim, vdim, window = sizes["heads"], sizes["kv_heads"], sizes["dim"], sizes["vdim"], sizes["mask"]["size"]
    q = rotate(rms_norm(h @ weights["l0.mix.q"].T, weights["l0.mix.q.norm"], 1e-5).view(30, H, dim), torch.arange(30),
               sizes["rot"]["dims"], sizes["rot"]["base"], "halves")
    rows = []
    for i in range(30):
        heads = []
        for head in range(H):
            seen = list(range(max(0, i - window + 1), i + 1))
            scores = torch.stack([(q[i, head] * k[j, head // (H // G)]).sum() * sizes["scale"] for j in seen])
            heads.append((torch.softmax(scores, 0)[:, None] * torch.stack([v[j, head // (H // G)] for j in seen])).sum(0))
        rows.append(torch.cat(heads))
    got = (torch.stack(rows) * torch.sigmoid(h @ weights["l0.mix.g"].T)) @ weights["l0.mix.o"].T
    assert torch.allclose(got, want, atol=1e-10)
    # the norm runs over the whole projection: one head's entries scale every other head's
    bent = dict(weights)
    bent["l0.mix.q"] = weights["l0.mix.q"].clone()
    bent["l0.mix.q"][:dim] *= 3.0
    other, _ = attention_mixer(h, bent, "l0.mix.", sizes, 1e-5)
    per_head = (other - want).abs().amax()
    assert per_head > 1e-3


def test_the_router_by_hand():
    generator = torch.Generator().manual_seed(7)
    h = torch.randn(50, 12, generator=generator, dtype=torch.float64)
    w = torch.randn(9, 12, generator=generator, dtype=torch.float64)
    correction = 0.2 * torch.randn(9, generator=generator, dtype=torch.float64)
    chosen, weights, scores = route(h, w, correction, top=2, groups=3, keep=2)
    for t in range(50):
        s = torch.softmax(h[t] @ w.T, 0)
        c = s + correction
        ranked = sorted(range(3), key=lambda g: -float(c[3 * g : 3 * g + 3].max()))[:2]
        allowed = [e for e in range(9) if e // 3 in ranked]
        best = sorted(allowed, key=lambda e: -float(c[e]))[:2]
        assert chosen[t].tolist() == best
        assert torch.allclose(weights[t], s[best] / (s[best].sum() + 1e-20))
    assert torch.allclose(scores.sum(-1), torch.ones(50, dtype=torch.float64))
    # a correction can lift a row with a small score; the weight stays the score's
    lifted = correction.clone()
    lifted[4] = 5.0
    chosen, weights, scores = route(h, w, lifted, top=1, groups=1, keep=1)
    assert set(chosen.view(-1).tolist()) == {4} and torch.allclose(weights, torch.ones_like(weights))


def test_norms_and_the_expert_by_hand():
    generator = torch.Generator().manual_seed(9)
    x = torch.randn(4, 10, generator=generator, dtype=torch.float64)
    w, b = torch.randn(10, generator=generator, dtype=torch.float64), torch.randn(10, generator=generator, dtype=torch.float64)
    assert torch.allclose(layer_norm(x, w, b, 1e-5), torch.nn.functional.layer_norm(x, (10,), w, b, 1e-5))
    assert torch.allclose(rms_norm(x, w, 0.0).pow(2).div(w * w).mean(-1), torch.ones(4, dtype=torch.float64))
    gate, up, down = (torch.randn(*shape, generator=generator, dtype=torch.float64) for shape in ((6, 10), (6, 10), (10, 6)))
    y = clamped_expert(x, gate, up, down, 0.5)
    for t in range(4):
        g = [min(float(gate[i] @ x[t]), 0.5) for i in range(6)]
        u = [max(-0.5, min(0.5, float(up[i] @ x[t]))) for i in range(6)]
        act = torch.tensor([g[i] / (1.0 + math.exp(-1.702 * g[i])) * (u[i] + 1.0) for i in range(6)], dtype=torch.float64)
        assert torch.allclose(y[t], down @ act)


def test_every_mechanism_moves_the_logits():
    """Leaving one mechanism out of the plain implementation changes the logits by far more than the engine's bound."""
    config = CONFIGS["stack"]
    weights = as_double(make_weights(config, seed=11))
    tokens = torch.randint(0, config["vocab"], (40,), generator=torch.Generator().manual_seed(3)).tolist()
    reference = forward(config, weights, tokens)

    def moved(other_config=None, other_weights=None):
        logits = forward(other_config or config, other_weights or weights, tokens)
        return float((logits - reference).abs().max())

    def changed(path, value):
        other = copy.deepcopy(config)
        node = other
        for key in path[:-1]:
            node = node[key]
        node[path[-1]] = value
        return other

    def without(suffix, fill):
        return {name: (torch.full_like(value, fill) if name.endswith(suffix) else value) for name, value in weights.items()}

    assert moved(other_weights=without("correction", 0.0)) > 0.05
    assert moved(other_weights=without(".b", 0.0)) > 0.05
    assert moved(other_weights=without("q.norm", 1.0)) > 0.05
    assert moved(other_weights=without("dkv.norm", 1.0)) > 0.05
    assert moved(other_weights=without("mix.g", 0.0)) > 0.05
    assert moved(changed(("postln_alpha",), 1.0)) > 0.05
    assert moved(changed(("logit_scale",), 1.0)) > 0.05
    assert moved(changed(("embedding", "scale"), 1.0)) > 0.05
    assert moved(changed(("layers", 1, "mixer", "mask", "size"), 10)) > 0.01          # the layer's own window
    assert moved(changed(("layers", 4, "mixer", "mask", "size"), 6)) > 0.01           # a reader's window
    assert moved(changed(("layers", 1, "mixer", "rot", "dims"), 8)) > 0.02
    assert moved(changed(("layers", 0, "mixer", "rot", "base"), 10.0)) > 0.02
    assert moved(changed(("layers", 3, "mlp", "expert", "limit"), 100.0)) > 0.02
    assert moved(changed(("layers", 3, "mlp", "router", "groups", "keep"), 2)) > 0.02
    assert moved(changed(("layers", 3, "mlp", "router", "groups", "count"), 1)) > 0.02
    own_keys = changed(("layers", 2, "mixer", "kv_from"), None)
    del own_keys["layers"][2]["mixer"]["kv_from"]
    shapes = tensor_shapes(own_keys)
    extra = dict(weights)
    for name in ("l2.mix.k", "l2.mix.k.norm", "l2.mix.v"):
        extra[name] = torch.ones(shapes[name], dtype=torch.float64) * 0.1
    assert moved(own_keys, extra) > 0.05
    assert math.isfinite(moved())


def test_a_random_model_folder_is_written_and_read_back(tmp_path):
    """``random-init`` takes the architecture from the file like every other entry point: the folder it writes holds
    exactly the tensors the model expects, and loads as this architecture."""
    import json

    from rapid_llm_b200.cli import main
    from rapid_llm_b200.config import load_config
    from rapid_llm_b200.weights.safetensors_io import SafetensorsFile

    (tmp_path / "config.json").write_text(json.dumps(CONFIGS["narrow"]))
    assert main(["random-init", "--config", str(tmp_path / "config.json"), "--out", str(tmp_path / "model"), "--seed", "3"]) == 0
    assert isinstance(load_config(tmp_path / "model"), ZupupelConfig)
    written = SafetensorsFile(tmp_path / "model" / "model.safetensors")
    shapes = {name: written.shape(name) for name in written.keys()}
    assert shapes == tensor_shapes(CONFIGS["narrow"])
