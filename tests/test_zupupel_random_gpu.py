"""Zupupel configurations drawn by seed against the plain implementation: the two mixers in any order, head counts,
key, value and rotated sizes, windows from one position to none, bases, latent ranks, layers that read an earlier
layer's keys and values through a window of their own, experts, identity experts, groups and how many are kept,
layers without a feed-forward, the model's constants.  Each draw replays a mixed trace (portions of prompts beside
decoded tokens on few pages and three slots) in float32 and bfloat16."""

from __future__ import annotations

import random

import pytest
from plain_zupupel import forward
from test_kopatar_gpu import DTYPES, _replay, _runner
from test_zupupel_gpu import _check, _sequences
from trace_tools import mixed
from zupupel_models import as_double, attention_layer, latent_layer, make_config, make_weights, moe, write_folder

DRAWS = 10


def _feed_forward(rng):
    if rng.random() < 0.25:
        return None
    groups = rng.choice([1, 1, 2, 3, 4])
    per = rng.randint(1, 4)
    rows = groups * per
    identity = rng.randint(0, rows - 1)
    keep = rng.randint(1, groups)
    return moe(experts=rows - identity, identity=identity, top=rng.randint(1, min(4, keep * per)), ff=rng.choice([8, 12, 32, 40]),
               groups=groups, keep=keep, limit=rng.choice([0.3, 1.0, 7.0]))


def draw_config(seed: int) -> dict:
    rng = random.Random(7000 + seed)
    layers = []
    for _ in range(rng.randint(2, 6)):
        mlp = _feed_forward(rng)
        owners = [i for i, layer in enumerate(layers) if layer["type"] == "attention" and "kv_from" not in layer["mixer"]]
        if owners and rng.random() < 0.35:                      # its own queries and window over an earlier layer's cache
            owner = rng.choice(owners)
            mixer = dict(layers[owner]["mixer"])
            mixer.pop("mask", None)
            window = rng.choice([0, 1, 2, 7, 16, 33])
            if window:
                mixer["mask"] = {"size": window}
            mixer["kv_from"] = owner
            layers.append({"type": "attention", "mixer": mixer, "mlp": mlp})
            continue
        if rng.random() < 0.35:
            layers.append(latent_layer(heads=rng.randint(1, 6), dim=rng.choice([8, 16, 24, 64]), rot_dim=rng.choice([2, 4, 8, 16, 32]),
                                       vdim=rng.choice([8, 16, 40, 64]), kv_rank=rng.choice([12, 16, 40, 64, 96, 250]),
                                       base=rng.choice([50.0, 1.0e4, 5.0e5]), scale=rng.uniform(0.1, 0.5), mlp=mlp))
            continue
        kv_heads = rng.choice([1, 2, 3, 4])
        dim = rng.choice([8, 12, 16, 32, 64, 128])
        layers.append(attention_layer(heads=kv_heads * rng.choice([1, 2, 4]), kv_heads=kv_heads, dim=dim,
                                      vdim=rng.choice([8, 16, 24, 64, 128]), window=rng.choice([0, 1, 3, 8, 17, 41]),
                                      rot_dims=rng.choice([0, 2, dim // 2, dim]), base=rng.choice([50.0, 1.0e4, 1.0e6]),
                                      scale=rng.uniform(0.1, 0.5), mlp=mlp))
    return make_config(layers, width=rng.choice([32, 40, 48, 64, 72, 96]), vocab=rng.randint(50, 200), eps=rng.choice([1e-6, 1e-5]),
                       alpha=rng.choice([1.0, 2.0, 3.5]), embedding_scale=rng.choice([0.5, 1.0, 1.7]),
                       logit_scale=rng.choice([0.3, 1.0, 2.0]))


def test_the_draws_differ():
    drawn = [draw_config(seed) for seed in range(DRAWS)]
    kinds = [tuple((layer["type"], "kv_from" in layer["mixer"], layer["mlp"] is None) for layer in config["layers"]) for config in drawn]
    assert len(set(kinds)) >= DRAWS - 2
    assert {"attention", "latent_attention"} <= {k for order in kinds for k, _, _ in order}
    assert any(shares for order in kinds for _, shares, _ in order) and any(bare for order in kinds for _, _, bare in order)
    routers = [layer["mlp"]["router"] for config in drawn for layer in config["layers"] if layer["mlp"]]
    assert any(r["identity"] == 0 for r in routers) and any(r["identity"] > 0 for r in routers)
    assert any(r["groups"]["count"] > 1 and r["groups"]["keep"] < r["groups"]["count"] for r in routers)


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", list(DTYPES))
@pytest.mark.parametrize("seed", range(DRAWS))
def test_a_drawn_configuration_in_mixed_batches(seed, dtype, tmp_path):
    config = draw_config(seed)
    weights = make_weights(config, seed=100 + seed)
    folder = write_folder(tmp_path / "model", config, weights, DTYPES[dtype])
    lengths = [33, 70, 12, 58, 91, 6] if dtype == "float32" else [17, 30, 12, 25, 36, 6]
    sequences = _sequences(config, weights, lengths, seed=seed, dtype=dtype, deep=True)
    double = as_double(weights)
    plain = {rid: forward(config, double, tokens) for rid, tokens in sequences.items()}
    records, peak = mixed(sequences, seed=seed, max_live=3, page=8)
    runner = _runner(folder, config, dtype, peak, page=8, slots=3)
    _check(_replay(runner, records), plain, dtype, f"seed {seed} {dtype}: {config}", True)


def draw_large_config(seed: int) -> dict:
    """Sizes nearer to a real model's: widths of a few hundred, heads of 32 to 128, windows of tens of positions, latents
    of up to 256, router rows in groups of several."""
    rng = random.Random(400 + seed)
    layers = []
    for _ in range(rng.randint(4, 7)):
        groups, per = rng.choice([1, 2, 4]), rng.choice([3, 4, 5, 8])
        rows = groups * per
        identity, keep = rng.randint(0, rows // 3), rng.randint(1, groups)
        mlp = None if rng.random() < 0.15 else moe(experts=rows - identity, identity=identity, top=rng.randint(1, min(6, keep * per)),
                                                   ff=rng.choice([32, 48, 96]), groups=groups, keep=keep, limit=rng.choice([0.5, 2.0]))
        owners = [i for i, layer in enumerate(layers) if layer["type"] == "attention" and "kv_from" not in layer["mixer"]]
        if owners and rng.random() < 0.35:
            owner = rng.choice(owners)
            mixer = dict(layers[owner]["mixer"])
            mixer.pop("mask", None)
            window = rng.choice([0, 24, 56, 100])
            if window:
                mixer["mask"] = {"size": window}
            mixer["kv_from"] = owner
            layers.append({"type": "attention", "mixer": mixer, "mlp": mlp})
            continue
        if rng.random() < 0.3:
            layers.append(latent_layer(heads=rng.choice([4, 6, 8]), dim=rng.choice([32, 48, 64]), rot_dim=rng.choice([16, 32]),
                                       vdim=rng.choice([32, 64]), kv_rank=rng.choice([64, 96, 192, 256]), base=rng.choice([1e4, 2.5e5]),
                                       scale=rng.uniform(0.08, 0.2), mlp=mlp))
            continue
        kv_heads, dim = rng.choice([1, 2, 4]), rng.choice([32, 96, 128])
        layers.append(attention_layer(heads=kv_heads * rng.choice([1, 2, 4]), kv_heads=kv_heads, dim=dim, vdim=rng.choice([32, 64, 128]),
                                      window=rng.choice([0, 24, 33, 48]), rot_dims=rng.choice([16, 32, dim]), base=rng.choice([1e4, 1e6]),
                                      scale=rng.uniform(0.08, 0.2), mlp=mlp))
    return make_config(layers, width=rng.choice([128, 192, 320]), vocab=rng.randint(300, 900), eps=1e-6, alpha=rng.choice([1.0, 2.0, 4.0]),
                       embedding_scale=rng.choice([1.0, 2.0]), logit_scale=rng.choice([0.3, 1.0]))


@pytest.mark.gpu
@pytest.mark.parametrize("seed", range(3))
def test_a_larger_drawn_model_over_hundreds_of_tokens(seed, tmp_path):
    """Float32, a 700-token request whole, with its tail decoded, in portions of changing size, and mixed with shorter
    requests on four slots: every row within 5e-5 of the logits' spread (difference with its mean removed, root mean
    square over the vocabulary), which a key lost far back, a window off by one or a wrong expert would exceed a
    thousandfold."""
    import torch
    from trace_tools import portions, tail_one_by_one, whole

    config = draw_large_config(seed)
    weights = make_weights(config, seed=500 + seed)
    folder = write_folder(tmp_path / "model", config, weights, torch.float32)
    generator = torch.Generator().manual_seed(seed)
    sequences = {f"r{i}": torch.randint(0, config["vocab"], (n,), generator=generator).tolist() for i, n in enumerate([700, 260, 90, 33, 1])}
    double = as_double(weights)
    plain = {rid: forward(config, double, tokens) for rid, tokens in sequences.items()}
    records, peak = mixed(sequences, seed=seed, max_live=4, page=16)
    runner = _runner(folder, config, "float32", max(peak, 704), page=16, slots=4)
    first = sequences["r0"]
    for label, trace in (("whole", whole("r0", first)), ("tail", tail_one_by_one("r0", first, tail=70)),
                         ("portions", portions("r0", first, [37, 37, 14, 19, 6, 2, 128, 1, 1, 64])), ("mixed", records)):
        for rid, by_position in _replay(runner, trace).items():
            positions = sorted(by_position)
            got = torch.stack([by_position[p] for p in positions]).double()
            want = plain[rid][positions]
            error = got - want
            share = (error - error.mean(-1, keepdim=True)).pow(2).mean(-1).sqrt() / want.std()
            assert float(share.max()) < 5e-5, f"seed {seed} ({label}): request {rid!r}, position {positions[int(share.argmax())]}: {float(share.max()):.2e}"
