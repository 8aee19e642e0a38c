"""Basitar's configuration on the CPU: parts and their parameters, expected tensors, the decay's rank from the file,
refusals; the plain implementation's mechanisms against second forms of the same equations; and that every mechanism
of the plain implementation moves the logits of the test models (so a comparison with it has teeth)."""

from __future__ import annotations

import copy
import math

import pytest
import torch
from basitar_models import CONFIGS, YARN, as_double, bare, latent_layer, make_config, make_weights, tensor_shapes, write_folder
from plain_basitar import F64, bigram_rows, forward, latent_attention, rotary_frequencies, rotate, router_choice, wkv

from rapid_llm_b200.config import BasitarConfig, load_config, resolve_architecture
from rapid_llm_b200.models.causal_lm import CausalLM


def test_the_registry_finds_the_architecture():
    assert resolve_architecture({"architecture": "Basitar"}) is BasitarConfig


@pytest.mark.parametrize("name", list(CONFIGS))
def test_the_model_expects_the_files_tensors(name):
    config = CONFIGS[name]
    model = CausalLM(BasitarConfig.from_dict(config).to_spec(), torch.float32, "cpu")
    # the head is the token table: a tensor of its own may be there and is not expected
    assert {n: tuple(s.shape) for n, s in model.tensor_specs().items() if not s.optional} == tensor_shapes(config)


def test_parts_and_their_parameters():
    spec = BasitarConfig.from_dict(CONFIGS["stack"]).to_spec()
    # six layer runs on four layers' tensors
    assert len(spec.layers) == 4 and [entry.layer for entry in spec.schedule] == [0, 1, 2, 0, 3, 2]
    assert [layer.arrangement for layer in spec.layers] == ["sandwich"] * 4
    assert [layer.prefix for layer in spec.layers] == ["l0.", "l1.", "l2.", "l4."]
    assert [layer.mixer.kind for layer in spec.layers] == ["wkv", "latent_attention", "latent_attention", "latent_attention"]
    assert [layer.mixer.params.get("rotation") for layer in spec.layers] == [None, "neighbours", "halves", "neighbours"]
    assert [layer.mixer.params.get("head_gate") for layer in spec.layers] == [None, True, False, True]
    assert [None if layer.mixer.kind == "wkv" else layer.mixer.params["position"].kind for layer in spec.layers] == [
        None, "rotary_frequencies", "rotary_frequencies", "yarn_frequencies"]
    assert [None if layer.feed_forward is None else layer.feed_forward.kind for layer in spec.layers] == [
        "routed_experts", None, "routed_experts", "swiglu"]
    routed = spec.layers[2].feed_forward.params
    assert (routed["num_experts"], routed["top_k"], routed["expert_size"], routed["router_bias"], routed["weighting"]) == (
        4, 4, 8, True, "softmax_chosen")
    assert spec.embedding.kind == "summed_embedding"
    assert (spec.embedding.params["pair_buckets"], spec.embedding.params["pair_mul_prev"], spec.embedding.params["pair_mul_cur"]) == (211, 13, 29)
    assert spec.head.params["tied"]
    model = CausalLM(spec, torch.float32, "cpu")
    # a cache or a state per layer run: the looped layers have their own
    assert [need is not None for need in model.cache_needs()] == [False, True, True, False, True, True]
    # ... and behind the layer runs' states stands the embedding's: the request's latest token
    assert [need is not None for need in model.state_needs()] == [True, False, False, True, False, False, True]
    assert model.state_needs()[-1].shape == (1,)
    assert [need.token_shape for need in model.cache_needs() if need is not None] == [(64,), (32,), (128,), (32,)]


def test_the_decays_rank_comes_from_the_file(tmp_path):
    config = CONFIGS["stack"]
    folder = write_folder(tmp_path / "model", config, make_weights(config, seed=1), torch.float32)
    assert "decay_rank" not in (tmp_path / "model" / "config.json").read_text()
    loaded = load_config(folder)
    assert isinstance(loaded, BasitarConfig)
    assert [layer["mixer"].get("decay_rank") for layer in loaded.layers] == [5, None, None, 5, None, None]
    with pytest.raises(ValueError, match="decay_rank"):
        BasitarConfig.from_dict(bare(config))


def test_refusals():
    config = copy.deepcopy(CONFIGS["latent"])
    config["layers"][0]["type"] = "window"
    with pytest.raises(ValueError, match="unknown mixer type"):
        BasitarConfig.from_dict(config)
    config = copy.deepcopy(CONFIGS["latent"])
    config["layers"][0]["mlp"]["kind"] = "sparse"
    with pytest.raises(ValueError, match="unknown feed-forward kind"):
        BasitarConfig.from_dict(config)
    config = copy.deepcopy(CONFIGS["latent"])
    del config["width"]
    with pytest.raises(ValueError, match="width"):
        BasitarConfig.from_dict(config)
    config = copy.deepcopy(CONFIGS["stack"])
    config["layers"][3]["weights_of"] = 1                      # a wkv layer on an attention layer's tensors
    with pytest.raises(ValueError, match="weights"):
        BasitarConfig.from_dict(config)
    config = copy.deepcopy(CONFIGS["stack"])
    config["layers"][5]["weights_of"] = 5
    with pytest.raises(ValueError, match="not another layer"):
        BasitarConfig.from_dict(config)


# ------------------------------------------------------------------ the plain implementation, checked by other forms
def test_token_pair_rows():
    assert bigram_rows([4, 9, 9, 0], buckets=7, mul_prev=3, mul_cur=5) == [7, (12 + 45) % 7, (27 + 45) % 7, 27 % 7]
    assert bigram_rows([3], buckets=1, mul_prev=2, mul_cur=2) == [1]
    assert bigram_rows([3, 5], buckets=1, mul_prev=2, mul_cur=2) == [1, 0]


def test_rotation_by_both_pairings_is_a_rotation_by_the_position_difference():
    """Scores of rotated queries and keys depend on the difference of the positions only, and the two pairings
    agree once one's entries are reordered."""
    generator = torch.Generator().manual_seed(2)
    freq, magnitude = rotary_frequencies(8, 50.0)
    assert magnitude == 1.0 and torch.allclose(freq, torch.tensor([1.0, 50.0 ** -0.25, 50.0 ** -0.5, 50.0 ** -0.75], dtype=F64))
    q, k = torch.randn(1, 8, generator=generator, dtype=F64), torch.randn(1, 8, generator=generator, dtype=F64)
    for interleaved in (False, True):
        near = (rotate(q, torch.tensor([9]), freq, 1.0, interleaved) * rotate(k, torch.tensor([4]), freq, 1.0, interleaved)).sum()
        far = (rotate(q, torch.tensor([105]), freq, 1.0, interleaved) * rotate(k, torch.tensor([100]), freq, 1.0, interleaved)).sum()
        assert abs(float(near - far)) < 1e-9
    order = torch.tensor([0, 4, 1, 5, 2, 6, 3, 7])             # halves -> neighbours
    halves = rotate(q, torch.tensor([13]), freq, 1.0, False)
    neighbours = rotate(q[:, order], torch.tensor([13]), freq, 1.0, True)
    assert torch.allclose(halves[:, order], neighbours)


def test_stretched_frequencies():
    """Fast turns keep their frequency, slow ones are divided by the factor, the ramp lies between; cosine and sine
    carry the magnitude."""
    dims, base = 16, 100.0
    plainly, _ = rotary_frequencies(dims, base)
    freq, magnitude = rotary_frequencies(dims, base, YARN)
    assert magnitude == pytest.approx(0.1 * math.log(8.0) + 1.0)
    turn = lambda t: dims * math.log(64 / (2 * math.pi * t)) / (2 * math.log(base))
    lo, hi = max(math.floor(turn(16.0)), 0), min(math.ceil(turn(2.0)), dims - 1)
    assert 0 <= lo < hi
    for i in range(dims // 2):
        if i <= lo:
            assert float(freq[i]) == pytest.approx(float(plainly[i]))
        elif i >= hi:
            assert float(freq[i]) == pytest.approx(float(plainly[i]) / 8.0)
        else:
            assert float(plainly[i]) / 8.0 < float(freq[i]) < float(plainly[i])
    x = torch.ones(1, dims, dtype=F64)
    assert float(rotate(x, torch.tensor([0]), freq, magnitude, True)[0, 0]) == pytest.approx(magnitude)


def test_latent_attention_equals_attention_over_expanded_keys_and_values():
    """The other order of the same products: keys and values expanded per token and head, scores key by key."""
    config = CONFIGS["latent2"]
    weights = as_double(make_weights(config, seed=3))
    sizes, eps = config["layers"][0]["mixer"], config["norm"]["eps"]
    H, dim, rot, vdim, rank = (sizes[k] for k in ("heads", "dim", "rot_dim", "vdim", "kv_rank"))
    T = 9
    h = torch.randn(T, config["width"], generator=torch.Generator().manual_seed(4), dtype=F64)
    got = latent_attention(h, weights, "l0.mix.", sizes, eps, second=True)
    freq, magnitude = rotary_frequencies(rot, sizes["rot"]["base"], sizes["rot"]["scaling"])
    rms = lambda x: x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)
    out = torch.zeros(T, H, vdim, dtype=F64)
    for t in range(T):
        q = weights["l0.mix.uq"] @ (rms(weights["l0.mix.dq"] @ h[t]) * weights["l0.mix.dq.norm"])
        gate = torch.sigmoid(weights["l0.mix.g"] @ h[t])
        for head in range(H):
            mine = q[head * (dim + rot) : (head + 1) * (dim + rot)]
            mine = torch.cat([mine[:dim], rotate(mine[None, dim:], torch.tensor([t]), freq, magnitude, True)[0]])
            scores, values = [], []
            for s in range(t + 1):
                down = weights["l0.mix.dkv"] @ h[s]
                c = rms(down[:rank]) * weights["l0.mix.dkv.norm"]
                key = torch.cat([(weights["l0.mix.uk"] @ c)[head * dim : (head + 1) * dim],
                                 rotate(down[None, rank:], torch.tensor([s]), freq, magnitude, True)[0]])
                scores.append((mine * key).sum() * sizes["scale"])
                values.append((weights["l0.mix.uv"] @ c)[head * vdim : (head + 1) * vdim])
            share = torch.softmax(torch.stack(scores), dim=0)
            out[t, head] = gate[head] * (share[:, None] * torch.stack(values)).sum(0)
    assert torch.allclose(got, out.reshape(T, -1) @ weights["l0.mix.o"].T, atol=1e-10)


def test_the_recurrence_equals_its_sum_over_earlier_tokens():
    """``o_t = sum_(s<t) (r_t . (prod_(s<j<t) w_j) k_s) v_s + (r_t . u k_t) v_t``, written out."""
    config = CONFIGS["wkv"]
    weights = as_double(make_weights(config, seed=5))
    sizes, eps = config["layers"][0]["mixer"], config["norm"]["eps"]
    H, dim, T = sizes["heads"], sizes["dim"], 7
    h = torch.randn(T, config["width"], generator=torch.Generator().manual_seed(6), dtype=F64)
    got = wkv(h, weights, "l0.mix.", sizes, eps)
    before = torch.cat([torch.zeros(1, config["width"], dtype=F64), h[:-1]])
    mixed = lambda which: h + (before - h) * weights["l0.mix.mu." + which]
    r, k, v = ((mixed(s) @ weights["l0.mix." + s].T).view(T, H, dim) for s in "rkv")
    gate = mixed("g") @ weights["l0.mix.g"].T
    gate = gate * torch.sigmoid(gate)
    decay = torch.exp(-torch.exp(torch.tanh(mixed("w") @ weights["l0.mix.w1"].T) @ weights["l0.mix.w2"].T + weights["l0.mix.w0"])).view(T, H, dim)
    out = torch.zeros(T, H, dim, dtype=F64)
    for t in range(T):
        for head in range(H):
            out[t, head] = (r[t, head] * weights["l0.mix.u"][head] * k[t, head]).sum() * v[t, head]
            for s in range(t):
                kept = torch.ones(dim, dtype=F64)
                for j in range(s + 1, t):
                    kept = kept * decay[j, head]
                out[t, head] += (r[t, head] * kept * k[s, head]).sum() * v[s, head]
    out = out / torch.sqrt((out * out).mean(-1, keepdim=True) + eps)
    want = (out.reshape(T, -1) * weights["l0.mix.norm"] * gate) @ weights["l0.mix.o"].T
    assert torch.allclose(got, want, atol=1e-10)


def test_the_routers_choice():
    weights = {"p.router": torch.tensor([[1.0, 0.0], [0.0, 1.0], [1.0, 1.0], [-1.0, 0.0]], dtype=F64),
               "p.router.b": torch.tensor([0.0, 0.0, -0.5, 5.0], dtype=F64)}
    h = torch.tensor([[2.0, 1.0], [-3.0, 0.5]], dtype=F64)
    order, share, logits = router_choice(h, weights, "p.", 2)
    assert logits.tolist() == [[2.0, 1.0, 2.5, 3.0], [-3.0, 0.5, -3.0, 8.0]]
    assert order.tolist() == [[3, 2], [3, 1]]
    assert torch.allclose(share[0], torch.softmax(torch.tensor([3.0, 2.5], dtype=F64), 0)) and float(share.sum()) == pytest.approx(2.0)


def test_every_mechanism_moves_the_logits():
    """Leaving one mechanism out of the plain implementation changes the logits by far more than the engine's bound."""
    config = CONFIGS["stack"]
    weights = as_double(make_weights(config, seed=11))
    tokens = torch.randint(0, config["vocab"], (40,), generator=torch.Generator().manual_seed(3)).tolist()
    reference = forward(tokens, weights, config)

    def moved(other_config=None, other_weights=None):
        logits = forward(tokens, other_weights or weights, other_config or config)
        return float((logits - reference).abs().max())

    def changed(path, value):
        other = copy.deepcopy(config)
        node = other
        for key in path[:-1]:
            node = node[key]
        node[path[-1]] = value
        return other

    def without(ending, value=0.0):
        return {name: (torch.full_like(tensor, value) if name.endswith(ending) else tensor) for name, tensor in weights.items()}

    assert moved(other_weights=without("bigram")) > 0.05
    assert moved(other_weights=without("pos")) > 0.05
    assert moved(other_weights=without("mix.u")) > 0.05
    assert moved(other_weights=without("mix.w0", -20.0)) > 0.05          # no decay at all
    assert moved(other_weights=without("mu.k")) > 0.05
    assert moved(other_weights=without("mix.g", 0.0)) > 0.05             # both gates: SiLU of zero, sigmoid of zero
    assert moved(other_weights=without("router.b")) > 0.02
    assert moved(other_weights=without("norm1b")) > 0.05
    assert moved(changed(("layers", 4, "mixer", "rot", "scaling"), None)) > 0.02
    assert moved(changed(("layers", 2, "mixer", "rot", "base"), 10.0)) > 0.05
    assert moved(changed(("layers", 1, "mixer", "scale"), 0.05)) > 0.05
    assert moved(changed(("layers", 0, "mlp", "router", "top"), 2)) > 0.05
    assert moved(changed(("embedding", "bigram", "mul_prev"), 14)) > 0.05
    assert math.isfinite(moved())
