"""The Zupupel decoder in the engine against the plain implementation (``plain_zupupel.py``).

Every configuration of ``zupupel_models.CONFIGS`` runs whole, with its tail decoded token by token, in portions of
changing size down to two tokens, and mixed with other requests on pages and slots that are used again; then the
edges: a far key that stands out among hundreds (before, on and behind a page's border) for both mixers, the keys
just inside and just outside a window (the layer's own and a reader's of another layer's cache) in prompts and while
decoding, windows that let a small pool serve a long sequence, the first tokens of a sequence on slots used again,
long decoding from captured graphs, latent rows wider than the tensor-core tiles, many experts, greedy generation
through ``LLM.generate``, the command line and the trace runner.
"""

from __future__ import annotations

import pytest
import torch
from plain_zupupel import clear_margin, forward, greedy
from test_basitar_gpu import MARGIN, _compare_deep_bfloat16
from test_kopatar_gpu import DTYPES, _compare, _replay, _runner
from tolerances import assert_rows_close_by_size
from trace_tools import mixed, portions, tail_one_by_one, whole
from zupupel_models import CONFIGS, as_double, attention_layer, latent_layer, make_config, make_weights, moe, write_folder

pytestmark = pytest.mark.gpu

DEEP = ("stack", "narrow")        # several layers, small widths, routers on every other layer


def _sequences(config, weights, lengths, seed, dtype, deep=False):
    """Token sequences drawn by seed, each redrawn until no router decision in it is a close call.  A long sequence
    through several routers always holds some call that 16-bit rounding may settle; for the models whose 16-bit run is
    held to a bound over all rows (``deep``), the clearest of forty draws is taken then."""
    generator = torch.Generator().manual_seed(seed)
    double, out = as_double(weights), {}
    relaxed = deep and dtype == "bfloat16"
    for index, length in enumerate(lengths):
        best, best_margin = None, -1.0
        for _ in range(40 if relaxed else 300):
            tokens = torch.randint(0, config["vocab"], (length,), generator=generator).tolist()
            margin = clear_margin(config, double, tokens)
            if margin > best_margin:
                best, best_margin = tokens, margin
            if margin > MARGIN[dtype + (" deep" if relaxed else "")]:
                break
        else:
            if not relaxed:
                raise AssertionError("no sequence without a close router decision was drawn")
        out[f"r{index}"] = best
    return out


def _check(rows, plain, dtype, label, deep):
    if deep and dtype == "bfloat16":
        return _compare_deep_bfloat16(rows, plain, label)
    return _compare(rows, plain, dtype, label)


def _plain(sequences, weights, config):
    double = as_double(weights)
    return {rid: forward(config, double, tokens) for rid, tokens in sequences.items()}


@pytest.mark.parametrize("dtype", list(DTYPES))
@pytest.mark.parametrize("name", list(CONFIGS))
def test_whole_decoded_and_in_portions(name, dtype, tmp_path):
    config = CONFIGS[name]
    weights = make_weights(config, seed=11)
    folder = write_folder(tmp_path / "model", config, weights, DTYPES[dtype])
    tokens = _sequences(config, weights, [61], seed=3, dtype=dtype, deep=name in DEEP)["r0"]
    plain = _plain({"a": tokens}, weights, config)
    runner = _runner(folder, config, dtype, 160)
    for label, records in (
        ("whole", whole("a", tokens)),
        ("tail one by one", tail_one_by_one("a", tokens, tail=40)),
        ("portions", portions("a", tokens, [2, 3, 16, 2, 7, 8, 1, 5])),
        ("portions of two", portions("a", tokens, [2])),
        ("token by token", portions("a", tokens, [1])),
    ):
        _check(_replay(runner, records), plain, dtype, f"{name} {dtype} ({label})", name in DEEP)


@pytest.mark.parametrize("dtype", list(DTYPES))
@pytest.mark.parametrize("name", ["stack", "narrow"])
def test_mixed_batches_on_reused_pages_and_slots(name, dtype, tmp_path):
    config = CONFIGS[name]
    weights = make_weights(config, seed=5)
    folder = write_folder(tmp_path / "model", config, weights, DTYPES[dtype])
    lengths = [37, 90, 18, 75, 131, 52, 9] if dtype == "float32" else [21, 40, 12, 33, 48, 9]
    sequences = _sequences(config, weights, lengths, seed=8, dtype=dtype, deep=True)
    plain = _plain(sequences, weights, config)
    records, peak = mixed(sequences, seed=2, max_live=3, page=8)
    runner = _runner(folder, config, dtype, peak, page=8, slots=3)
    mixed_rows = _replay(runner, records)
    _check(mixed_rows, plain, dtype, f"{name} {dtype} (mixed)", True)
    # the same requests alone: what else is in the batch, and which slot and pages serve, changes nothing but rounding
    if dtype == "float32":
        for rid in ("r1", "r4"):
            alone = _replay(runner, whole(rid, sequences[rid]))[rid]
            for position, row in mixed_rows[rid].items():
                torch.testing.assert_close(row, alone[position], rtol=2e-5, atol=2e-5)


# ------------------------------------------------------------------ keys that stand out -- #
def pointing(config, seed, gain=3.0):
    """Weights in which token 0's query points at token 1's key and at no other.  Every row of the table has mean
    zero and variance one, and token 1's row is token 0's with its entries moved one place on; the query projection
    is the key projection with its columns moved one place back, so ``W_q x_0 = W_k x_1``.  The norm weight of k is
    one, that of q the gain, and the rotated share of a head is small, so positions hardly move a score.  For the
    latent mixer the unrotated query is ``gain * W_uk W_dkv x_1``, which is parallel to the key ``W_uk norm(W_dkv x_1)``.
    In a model of two layers the SECOND layer reads the first one's keys and values: the first layer's output
    projection is zero and its closing norm has weight one and no bias, so the second layer's input is the table's
    row again (the norm of a standardised row is the row), and it is the second layer's query that points."""
    weights = make_weights(config, seed=seed)
    rows = weights["embed"]
    rows = (rows - rows.mean(-1, keepdim=True)) / rows.std(-1, unbiased=False, keepdim=True)
    rows[1] = torch.roll(rows[0], 1)
    weights["embed"] = (rows / config["embedding"]["scale"]).bfloat16().float()
    sizes = config["layers"][0]["mixer"]
    heads, dim = sizes["heads"], sizes["dim"]
    if config["layers"][0]["type"] == "attention":
        last = len(config["layers"]) - 1
        if last:
            weights["l0.mix.o"] = torch.zeros_like(weights["l0.mix.o"])
            weights["l0.norm1"] = torch.ones_like(weights["l0.norm1"])
            weights["l0.norm1.b"] = torch.zeros_like(weights["l0.norm1.b"])
        group = heads // sizes["kv_heads"]
        keys = torch.roll(weights["l0.mix.k"], -1, dims=1).view(sizes["kv_heads"], dim, -1)
        weights[f"l{last}.mix.q"] = keys.repeat_interleave(group, dim=0).reshape(heads * dim, -1).clone()
        weights[f"l{last}.mix.q.norm"] = torch.full_like(weights[f"l{last}.mix.q.norm"], gain)
        weights["l0.mix.k.norm"] = torch.ones_like(weights["l0.mix.k.norm"])
    else:
        rank, rot = sizes["kv_rank"], sizes["rot_dim"]
        weights["l0.mix.dkv.norm"] = torch.ones_like(weights["l0.mix.dkv.norm"])
        q = torch.zeros(heads, dim + rot, config["width"])
        q[:, :dim] = gain * (weights["l0.mix.uk"] @ torch.roll(weights["l0.mix.dkv"][:rank], -1, dims=1)).view(heads, dim, -1)
        weights["l0.mix.q"] = q.view(heads * (dim + rot), -1).bfloat16().float()
    return weights


POINTING = {
    "attention": make_config([attention_layer(heads=4, kv_heads=2, dim=32, vdim=24, window=0, rot_dims=4, scale=0.25, mlp=None)],
                             width=32, vocab=40),
    "latent": make_config([latent_layer(heads=2, dim=32, rot_dim=8, vdim=24, kv_rank=32, scale=0.25, mlp=None)], width=32, vocab=40),
}


@pytest.mark.parametrize("dtype", list(DTYPES))
@pytest.mark.parametrize("far", [2, 15, 16, 33])
@pytest.mark.parametrize("kind", list(POINTING))
def test_a_far_key_stands_out_among_hundreds(kind, far, dtype, tmp_path):
    """The last token is token 0 and its query points at token 1's key, which stands at one far place among 400
    (before, on and behind a border of the 16-token pages).  Replacing that far token must change the last logits as
    the plain implementation says: in a whole prompt, with the tail decoded, and in portions."""
    config = POINTING[kind]
    weights = pointing(config, seed=31)
    folder = write_folder(tmp_path / "model", config, weights, DTYPES[dtype])
    generator = torch.Generator().manual_seed(far)
    base = torch.randint(2, config["vocab"], (400,), generator=generator).tolist()
    base[far], base[-1] = 1, 0                      # tokens 0 and 1 nowhere else
    other = list(base)
    other[far] = 2
    last = len(base) - 1
    want = [forward(config, as_double(weights), tokens)[last].float() for tokens in (base, other)]
    effect = float((want[0] - want[1]).abs().max())
    assert effect > 0.2, "the test's weights do not make the far key count"
    runner = _runner(folder, config, dtype, 416, page=16)
    for records_of in (lambda t: whole("a", t), lambda t: tail_one_by_one("a", t, tail=20), lambda t: portions("a", t, [150, 2, 99, 17])):
        got = [_replay(runner, records_of(tokens))["a"][last] for tokens in (base, other)]
        error = float(((got[0] - got[1]) - (want[0] - want[1])).abs().max())
        assert error < (2e-3 if dtype == "float32" else 0.15) * effect


WINDOW = 21


def _window_model(reader: bool):
    """One windowed layer whose last query points at one key; with ``reader`` a second layer that reads the first
    one's keys and values through a NARROWER window of its own, the first layer's window being wide."""
    own = attention_layer(heads=2, kv_heads=2, dim=32, vdim=16, window=60 if reader else WINDOW, rot_dims=4, scale=0.25, mlp=None)
    layers = [own]
    if reader:
        layers.append(attention_layer(heads=2, kv_heads=2, dim=32, vdim=16, window=WINDOW, rot_dims=4, scale=0.25, kv_from=0, mlp=None))
    return make_config(layers, width=32, vocab=40, alpha=1.0)


@pytest.mark.parametrize("dtype", list(DTYPES))
@pytest.mark.parametrize("reader", [False, True])
def test_the_keys_just_inside_and_just_outside_a_window(reader, dtype, tmp_path):
    """The query at position ``p`` sees ``p - window + 1`` and not ``p - window``.  The last token is token 0, whose
    query points at token 1's key, which stands at one place: just inside the window it must change the last logits
    as the plain implementation says, just outside it must change nothing; in a whole prompt, with the tail decoded,
    and in portions that cut the window.  The second model's window belongs to a layer that reads another layer's
    cache, which keeps more than that layer's own window."""
    config = _window_model(reader)
    weights = pointing(config, seed=37)
    folder = write_folder(tmp_path / "model", config, weights, DTYPES[dtype])
    double = as_double(weights)
    generator = torch.Generator().manual_seed(5)
    length = 130
    last = length - 1
    runner = _runner(folder, config, dtype, 144, page=16)
    schedules = (lambda t: whole("a", t), lambda t: tail_one_by_one("a", t, tail=WINDOW + 9),
                 lambda t: portions("a", t, [40, 2, 61, 7, 3]))
    for place, inside in ((last - WINDOW + 1, True), (last - WINDOW, False)):
        base = torch.randint(2, config["vocab"], (length,), generator=generator).tolist()
        base[place], base[-1] = 1, 0
        other = list(base)
        other[place] = 2
        want = [forward(config, double, tokens)[last].float() for tokens in (base, other)]
        effect = float((want[0] - want[1]).abs().max())
        assert (effect > 0.3) == inside, "the plain implementation's window is off by one, or the weights do not point"
        for records_of in schedules:
            got = [_replay(runner, records_of(tokens))["a"][last] for tokens in (base, other)]
            moved = got[0] - got[1]
            if inside:
                assert float((moved - (want[0] - want[1])).abs().max()) < (2e-3 if dtype == "float32" else 0.15) * effect
            else:
                assert float(moved.abs().max()) == 0.0, "a key outside the window reached the logits"


@pytest.mark.parametrize("dtype", list(DTYPES))
def test_windows_give_pages_back_while_a_sequence_grows(dtype, tmp_path):
    """A model of windowed layers only (one reads the other's cache through a wider window) runs a sequence several
    times longer than the pool: the pages the windows have passed are handed out again, in portions and while
    decoding, and the logits stay those of the plain implementation."""
    config = make_config([attention_layer(window=9, mlp=None), attention_layer(window=14, kv_from=0, mlp=None)], width=48)
    weights = make_weights(config, seed=19)
    folder = write_folder(tmp_path / "model", config, weights, DTYPES[dtype])
    tokens = torch.randint(0, config["vocab"], (150,), generator=torch.Generator().manual_seed(1)).tolist()
    plain = _plain({"a": tokens}, weights, config)
    import dataclasses

    from rapid_llm_b200.config import load_config
    from rapid_llm_b200.engine.runner import ModelRunner
    from rapid_llm_b200.replay import engine_config_for

    engine = dataclasses.replace(engine_config_for(load_config(folder), dtype, 160, 8, 2), num_pages=6)    # 48 of 150 tokens
    runner = ModelRunner.from_folder(folder, engine)
    records = portions("a", tokens[:60], [9, 2, 16, 5])
    records[-1]["end"] = []
    for offset, token in enumerate(tokens[60:]):
        records.append({"step": 100 + offset, "entries": [{"id": "a", "tokens": [token], "want": [0]}], "end": []})
    records[-1]["end"] = ["a"]
    rows = _replay(runner, records)
    _compare(rows, plain, dtype, f"windows on a small pool {dtype}")
    assert len(rows["a"]) == len(tokens)


@pytest.mark.parametrize("dtype", list(DTYPES))
def test_the_first_tokens_of_a_sequence(dtype, tmp_path):
    """Positions 0 to 5 alone: a position sees few keys, a window is not yet full, a group of experts may hold only
    identity experts.  Every slot is used several times."""
    config = make_config([attention_layer(window=3, mlp=moe(experts=2, top=2, ff=8, identity=2, groups=2, keep=1)),
                          latent_layer(mlp=None), attention_layer(window=2, kv_from=0, mlp=None)], width=48)
    weights = make_weights(config, seed=41)
    folder = write_folder(tmp_path / "model", config, weights, DTYPES[dtype])
    sequences = _sequences(config, weights, [6, 1, 3, 2, 5, 4, 1, 2], seed=9, dtype=dtype)
    plain = _plain(sequences, weights, config)
    runner = _runner(folder, config, dtype, 32, page=8, slots=2)
    for rid, tokens in sequences.items():
        _compare(_replay(runner, portions(rid, tokens, [1, 2])), plain, dtype, f"first tokens {dtype}")
    records, peak = mixed(sequences, seed=4, max_live=2, page=8)
    _compare(_replay(_runner(folder, config, dtype, peak, page=8, slots=2), records), plain, dtype, f"first tokens {dtype} (mixed)")


@pytest.mark.parametrize("dtype", list(DTYPES))
def test_wide_rows_and_many_heads(dtype, tmp_path):
    """A cached latent row of the tensor-core tiles' widest size (256 numbers) and one beyond it (which the
    one-warp-per-row kernel serves in either precision), sixteen heads, heads of 128 with a window over several
    blocks of keys, long prompts, portions behind cached keys."""
    config = make_config([
        latent_layer(heads=16, dim=24, rot_dim=64, vdim=40, kv_rank=192, base=1.0e6, scale=0.15, mlp=None),
        attention_layer(heads=4, kv_heads=2, dim=128, vdim=128, window=150, rot_dims=32, base=1.0e4, scale=0.09, mlp=None),
        latent_layer(heads=3, dim=64, rot_dim=32, vdim=16, kv_rank=288, scale=0.07, mlp=None),
        attention_layer(heads=4, kv_heads=2, dim=128, vdim=128, window=0, rot_dims=32, base=1.0e4, scale=0.09, kv_from=1, mlp=None),
    ], width=128, vocab=150)
    weights = make_weights(config, seed=61)
    folder = write_folder(tmp_path / "model", config, weights, DTYPES[dtype])
    sequences = _sequences(config, weights, [300, 45, 170], seed=5, dtype=dtype)
    plain = _plain(sequences, weights, config)
    runner = _runner(folder, config, dtype, 320, page=16)
    tokens = sequences["r0"]
    _compare(_replay(runner, whole("r0", tokens)), plain, dtype, f"wide rows {dtype} (whole)")
    _compare(_replay(runner, portions("r0", tokens, [130, 2, 90, 1, 40])), plain, dtype, f"wide rows {dtype} (portions)")
    _compare(_replay(runner, tail_one_by_one("r0", tokens, tail=12)), plain, dtype, f"wide rows {dtype} (tail)")
    records, peak = mixed(sequences, seed=3, max_live=3, page=16)
    _compare(_replay(_runner(folder, config, dtype, peak, page=16, slots=3), records), plain, dtype, f"wide rows {dtype} (mixed)")


@pytest.mark.parametrize("dtype", list(DTYPES))
def test_long_decoding_from_captured_graphs(dtype, tmp_path):
    from rapid_llm_b200.engine.runner import StepEntry

    config = CONFIGS["stack"]
    weights = make_weights(config, seed=13)
    folder = write_folder(tmp_path / "model", config, weights, DTYPES[dtype])
    lengths = [150, 171, 160] if dtype == "float32" else [60, 75, 66]
    sequences = _sequences(config, weights, lengths, seed=12, dtype=dtype, deep=True)
    plain = _plain(sequences, weights, config)
    runner = _runner(folder, config, dtype, 3 * 176, page=16, slots=4, graphs=True)
    heads = {"r0": 5, "r1": 40, "r2": 2}
    fed = {}
    for rid, head in heads.items():
        assert runner.admit(rid)
        runner.step([StepEntry(rid, sequences[rid][:head], [])])
        fed[rid] = head
    rows = {rid: {} for rid in sequences}
    while any(fed[rid] < len(sequences[rid]) for rid in sequences):
        live = [rid for rid in sequences if fed[rid] < len(sequences[rid])]
        logits = runner.step_decode([StepEntry(rid, [sequences[rid][fed[rid]]], [0]) for rid in live]).float().cpu()
        for row, rid in enumerate(live):
            rows[rid][fed[rid]] = logits[row].clone()
            fed[rid] += 1
    runner.check_fault()
    _check(rows, plain, dtype, f"long decoding {dtype}", True)


def test_greedy_generation_through_the_entry_point(tmp_path):
    """More prompts than slots, so requests wait, and slots and pages change hands; float32 picks the same tokens."""
    from rapid_llm_b200 import LLM, SamplingParams

    config = CONFIGS["stack"]
    weights = make_weights(config, seed=17)
    folder = write_folder(tmp_path / "model", config, weights, torch.float32)
    prompts = list(_sequences(config, weights, [5, 23, 2, 41, 12], seed=14, dtype="float32").values())
    llm = LLM(folder, dtype="float32", max_seq_len=96, max_gpu_num_blocks=24, page_size=8, max_num_seqs=2, max_chunk_size=16)
    outputs = llm.generate(prompts, SamplingParams.greedy(max_gen_len=12))
    for prompt, output in zip(prompts, outputs):
        assert output.outputs[0].token_ids == greedy(config, as_double(weights), prompt, 12)


def test_many_experts_and_long_portions(tmp_path):
    """More pairs of one expert than a tile of the grouped products holds, more router rows than a warp has lanes,
    more groups than one, a portion of hundreds of tokens (float32; in bfloat16 a sequence of this length always holds
    a router decision that rounding settles, so there a layer of two experts and two identity experts runs)."""
    config = make_config([attention_layer(mlp=moe(experts=37, top=3, ff=24, identity=3, groups=5, keep=2)),
                          latent_layer(mlp=moe(experts=2, top=1, ff=40, identity=0, groups=1, keep=1))], width=64, vocab=90)
    weights = make_weights(config, seed=51)
    folder = write_folder(tmp_path / "float32", config, weights, torch.float32)
    tokens = _sequences(config, weights, [300], seed=2, dtype="float32")["r0"]
    plain = _plain({"a": tokens}, weights, config)
    runner = _runner(folder, config, "float32", 320, page=16)
    _compare(_replay(runner, whole("a", tokens)), plain, "float32", "many experts float32")
    _compare(_replay(runner, portions("a", tokens, [70, 2, 33])), plain, "float32", "many experts float32 (portions)")
    config = make_config([latent_layer(mlp=moe(experts=2, top=1, ff=40, identity=2, groups=2, keep=1))], width=64, vocab=90)
    weights = make_weights(config, seed=52)
    folder = write_folder(tmp_path / "bfloat16", config, weights, torch.bfloat16)
    tokens = _sequences(config, weights, [90], seed=2, dtype="bfloat16")["r0"]
    plain = _plain({"a": tokens}, weights, config)
    runner = _runner(folder, config, "bfloat16", 96, page=16)
    _compare(_replay(runner, whole("a", tokens)), plain, "bfloat16", "two experts bfloat16")


def test_the_command_line_and_the_trace_runner_take_a_zupupel_folder(tmp_path):
    """``batch`` generates from token-id prompts; ``bin/trace_run`` replays steps and writes the same logits as the
    plain implementation computes."""
    import json
    import subprocess
    import sys
    from pathlib import Path

    import numpy as np

    root = Path(__file__).resolve().parents[1]
    config = CONFIGS["stack"]
    weights = make_weights(config, seed=23)
    folder = write_folder(tmp_path / "model", config, weights, torch.float32)
    prompts = tmp_path / "prompts.txt"
    prompts.write_text("5 9 12 80 3\n7 7 1\n")
    done = subprocess.run([sys.executable, "-m", "rapid_llm_b200.cli", "batch", "--model-dir", str(folder), "--dtype", "float32",
                           "--prompt-ids-file", str(prompts), "--max-gen-len", "6", "--temperature", "0", "--repetition-penalty", "1.0", "--max-seq-len", "64",
                           "--max-gpu-num-blocks", "16"], cwd=root, capture_output=True, text=True)
    assert done.returncode == 0, done.stderr
    lines = [line for line in done.stdout.splitlines() if line and not line.startswith("---")]
    assert [int(t) for t in lines[0].split()] == greedy(config, as_double(weights), [5, 9, 12, 80, 3], 6)

    tokens = _sequences(config, weights, [30], seed=2, dtype="float32")["r0"]
    steps = [{"step": 0, "entries": [{"id": "x", "tokens": tokens[:17], "want": [16]}], "end": []},
             {"step": 1, "entries": [{"id": "x", "tokens": tokens[17:], "want": [0, 12]}], "end": ["x"]}]
    out = tmp_path / "out"
    done = subprocess.run([str(root / "bin" / "trace_run"), "--model", str(folder), "--dtype", "float32", "--out", str(out),
                           "--max-tokens", "64"], input="".join(json.dumps(s) + "\n" for s in steps), cwd=tmp_path,
                          capture_output=True, text=True)
    assert done.returncode == 0, done.stderr
    assert [line for line in done.stdout.splitlines() if line.startswith("done")] == ["done 0", "done 1"]
    plain = forward(config, as_double(weights), tokens).float()
    got = torch.from_numpy(np.fromfile(out / "1.f32", dtype="<f4").reshape(2, -1).copy())
    assert_rows_close_by_size(got, plain[[17, 29]], "float32")
