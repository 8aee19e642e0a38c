"""Basitar configurations drawn by seed against the plain implementation: layer kinds in any order, head counts, plain,
rotated and value sizes, latent ranks, decay ranks, bases and stretched frequencies, experts and how many a token takes,
layers without a feed-forward, layers that run another layer's tensors, token-pair constants.  Each draw replays a
mixed trace (portions of prompts beside decoded tokens on few pages and three state slots) in float32 and bfloat16."""

from __future__ import annotations

import random

import pytest
import plain_basitar
import torch
from basitar_models import as_double, dense, latent_layer, make_config, make_weights, moe, wkv_layer, write_folder
from plain_basitar import forward
from test_basitar_gpu import _check, _sequences
from test_kopatar_gpu import DTYPES, _replay, _runner
from tolerances import at_scale
from trace_tools import mixed

DRAWS = 8


def _feed_forward(rng):
    pick = rng.random()
    if pick < 0.2:
        return None
    if pick < 0.5:
        return dense(ff=rng.choice([20, 33, 48, 64]))
    experts = rng.randint(1, 9)
    return moe(experts=experts, top=rng.randint(1, min(experts, 4)), ff=rng.choice([8, 12, 32]))


def draw_config(seed: int) -> dict:
    rng = random.Random(9000 + seed)
    layers = []
    for _ in range(rng.randint(2, 5)):
        if layers and rng.random() < 0.25:                      # once more through an earlier layer's tensors
            owner = rng.choice([i for i, layer in enumerate(layers) if "weights_of" not in layer])
            layers.append({**layers[owner], "weights_of": owner})
            continue
        mlp = _feed_forward(rng)
        if rng.random() < 0.35:
            layers.append(wkv_layer(heads=rng.randint(1, 4), dim=rng.choice([6, 8, 16, 32]), rank=rng.randint(1, 9), mlp=mlp))
            continue
        second = rng.random() < 0.5
        rot_dim = rng.choice([2, 4, 8, 16, 32])
        scaling = None
        if second and rng.random() < 0.7:
            scaling = {"factor": rng.choice([2.0, 4.0, 32.0]), "original": rng.choice([16, 64, 256]),
                       "fast": rng.choice([8.0, 32.0]), "slow": rng.choice([1.0, 2.0])}
        layers.append(latent_layer(heads=rng.randint(1, 6), dim=rng.choice([8, 16, 24, 64]), rot_dim=rot_dim,
                                   vdim=rng.choice([8, 16, 40, 64]), kv_rank=rng.choice([12, 16, 40, 64, 96]),
                                   q_rank=rng.choice([8, 20, 48]), base=rng.choice([50.0, 1.0e4, 5.0e5]),
                                   scale=rng.uniform(0.1, 0.6), second=second, scaling=scaling, mlp=mlp))
    return make_config(layers, width=rng.choice([32, 40, 48, 64, 72, 96]), vocab=rng.randint(50, 200), eps=rng.choice([1e-6, 1e-5]),
                       buckets=rng.choice([1, 13, 100, 509]), mul_prev=rng.randint(1, 40), mul_cur=rng.randint(1, 40))


def _forward_in_float32(tokens, weights, config):
    """The plain implementation's own equations with float32 numbers (its dtype is a module constant)."""
    plain_basitar.F64 = torch.float32
    try:
        return forward(tokens, {name: value.float() for name, value in weights.items()}, config)
    finally:
        plain_basitar.F64 = torch.float64


def _compare_float32(rows, plain, sequences, weights, config, label):
    """A drawn model has rows that float32 itself cannot hold to the usual bound (a norm of a small vector, sharp
    scores): the plain implementation run in float32 misses its own float64 result there by many times its median
    error.  A row is held to the usual bound plus eight times that miss, which is what another order of the same
    float32 sums may differ by; the rows that float32 computes well keep the usual bound alone."""
    for request_id, by_position in rows.items():
        positions = sorted(by_position)
        got = torch.stack([by_position[p] for p in positions]).float()
        want = plain[request_id][positions]
        single = _forward_in_float32(sequences[request_id], weights, config)[positions].double()
        miss = (single - want).abs().amax(-1, keepdim=True).float()
        bound = at_scale("float32", want.float())
        excess = (got - want.float()).abs() - bound["rtol"] * want.float().abs() - bound["atol"] - 8.0 * miss
        assert float(excess.max()) <= 0.0, (
            f"{label}: request {request_id!r}, position {positions[int(excess.amax(-1).argmax())]}: off by "
            f"{float((got - want.float()).abs().amax(-1)[int(excess.amax(-1).argmax())]):.3g}, float32 itself by {float(miss[int(excess.amax(-1).argmax())]):.3g}")


def test_the_draws_differ():
    drawn = [draw_config(seed) for seed in range(DRAWS)]
    kinds = [tuple((layer["type"], (layer["mlp"] or {}).get("kind")) for layer in config["layers"]) for config in drawn]
    assert len(set(kinds)) >= DRAWS - 2
    assert {"wkv", "latent_attention", "latent_attention_2"} <= {k for order in kinds for k, _ in order}
    assert {"dense", "moe", None} <= {m for order in kinds for _, m in order}
    assert any("weights_of" in layer for config in drawn for layer in config["layers"])


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
    plain = {rid: forward(tokens, double, config) for rid, tokens in sequences.items()}
    records, peak = mixed(sequences, seed=seed, max_live=3, page=8)
    runner = _runner(folder, config, dtype, peak, page=8, slots=3)
    rows = _replay(runner, records)
    if dtype == "float32":
        return _compare_float32(rows, plain, sequences, weights, config, f"seed {seed} {dtype}: {config}")
    _check(rows, plain, dtype, f"seed {seed} {dtype}: {config}", True)
