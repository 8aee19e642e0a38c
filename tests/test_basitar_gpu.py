"""The Basitar decoder in the engine against the plain implementation (``plain_basitar.py``).

Every configuration of ``basitar_models.CONFIGS`` runs whole, with its tail decoded token by token, in portions of
changing size down to two tokens, and mixed with other requests on pages and state slots that are used again; then
the edges: a far token whose key is the only one the last query points at (before, on and behind a page's border),
a far token under a decay of nearly one, the first tokens of a sequence (the token-pair table's last row, the zero
row before the first token, slots that had another owner), long decoding from captured graphs, wide latents and
many heads, many experts, greedy generation through ``LLM.generate``, the command line and the trace runner.
"""

from __future__ import annotations

import pytest
import torch
from basitar_models import CONFIGS, YARN, as_double, dense, latent_layer, make_config, make_weights, moe, wkv_layer, write_folder
from plain_basitar import clear_margin, forward, greedy
from test_kopatar_gpu import DTYPES, _compare, _replay, _runner
from tolerances import BF16_ROW_RMS, assert_rows_close_by_size
from trace_tools import mixed, portions, tail_one_by_one, whole

pytestmark = pytest.mark.gpu

# how clearly every router decision of a test sequence must fall, in units of the router logits' spread: bfloat16
# rounds the stream the router reads, and a decision narrower than that rounding is no test of the engine
MARGIN = {"float32": 1e-4, "bfloat16": 0.04, "bfloat16 deep": 0.02}


def _sequences(config, weights, lengths, seed, dtype, deep=False):
    """Token sequences drawn by seed, each redrawn until no router decision in it is a close call."""
    generator = torch.Generator().manual_seed(seed)
    double, out = as_double(weights), {}
    for index, length in enumerate(lengths):
        for _ in range(200):
            tokens = torch.randint(0, config["vocab"], (length,), generator=generator).tolist()
            if clear_margin(tokens, double, config) > MARGIN[dtype + (" deep" if deep and dtype == "bfloat16" else "")]:
                break
        else:
            raise AssertionError("no sequence without a close router decision was drawn")
        out[f"r{index}"] = tokens
    return out


DEEP = ("stack", "narrow")        # several layers, small widths, routers that take one expert of few


def _compare_deep_bfloat16(rows, plain, label):
    """A model of several layers, few columns and sharp mechanisms multiplies rounding errors: in float32 these models
    are off by tens of the format's steps, and in bfloat16 by several hundredths of a row's size, which also settles a
    router decision here and there although the sequences were drawn clear of the closest calls (such a row, and to a
    lesser degree the rows behind it, then differ as a whole).  So the 16-bit run of such a model is held to the
    bound by the row's size at its median row, to four times the bound at nine rows in ten, and may be off by more
    than a quarter of a row's size in one row of twenty; a wrong kernel moves every row by its size.  The one-layer
    models hold the bound at every row in 16 bits, and these models hold the float32 bound at every position."""
    shares = []
    for request_id, by_position in rows.items():
        for position, got in by_position.items():
            want = plain[request_id][position].float()
            error = got.float() - want
            size = (want - want.mean()).pow(2).mean().sqrt()
            shares.append(float((error - error.mean()).pow(2).mean().sqrt() / size))
    shares.sort()
    count = len(shares)
    assert shares[count // 2] <= BF16_ROW_RMS, f"{label}: the median row is off by {shares[count // 2]:.3f} of its size"
    assert shares[(9 * count) // 10 - 1] <= 4 * BF16_ROW_RMS, f"{label}: one row in ten is off by {shares[(9 * count) // 10 - 1]:.3f} of its size"
    beyond = sum(share > 0.25 for share in shares)
    assert beyond <= max(1, count // 20), f"{label}: {beyond} of {count} rows are off by more than a quarter of their size"


def _check(rows, plain, dtype, label, deep):
    if deep and dtype == "bfloat16":
        return _compare_deep_bfloat16(rows, plain, label)
    return _compare(rows, plain, dtype, label)


def _plain(sequences, weights, config):
    double = as_double(weights)
    return {rid: forward(tokens, double, config) for rid, tokens in sequences.items()}


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


def pointing_weights(config, seed, gain=1.0):
    """Weights of a one-layer latent-attention model in which token 0's query points at token 1's key and at no
    other: token 1's row of the table is token 0's with its entries moved one place on, the query's down-projection
    is the latent's with its columns moved one place back (so token 0's query latent is token 1's key latent), and
    the queries' unrotated up-projection is the keys'.  The rotated parts of the queries are zero."""
    weights = make_weights(config, seed=seed)
    sizes = config["layers"][0]["mixer"]
    heads, dim, rot, rank = sizes["heads"], sizes["dim"], sizes["rot_dim"], sizes["kv_rank"]
    assert sizes["q_rank"] == rank
    weights["embed"][1] = torch.roll(weights["embed"][0], 1)
    weights["l0.norm1"] = torch.zeros_like(weights["l0.norm1"])
    weights["pos"] = (0.3 * weights["pos"]).bfloat16().float()
    weights["bigram"] = (0.3 * weights["bigram"]).bfloat16().float()
    weights["l0.mix.dq"] = torch.roll(weights["l0.mix.dkv"][:rank], -1, dims=1)
    weights["l0.mix.dq.norm"] = weights["l0.mix.dkv.norm"].clone()
    uq = torch.zeros(heads, dim + rot, rank)
    uq[:, :dim] = gain * weights["l0.mix.uk"].view(heads, dim, rank)
    weights["l0.mix.uq"] = uq.view(heads * (dim + rot), rank).bfloat16().float()
    return weights


@pytest.mark.parametrize("dtype", list(DTYPES))
@pytest.mark.parametrize("far", [2, 15, 16, 33])
@pytest.mark.parametrize("second", [False, True])
def test_a_far_key_stands_out_among_hundreds(second, far, dtype, tmp_path):
    """The last token is token 0 and its query points at token 1's key, which stands at one far place among 400
    (before, on and behind a border of the 16-token pages).  Replacing that far token must change the last logits as
    the plain implementation says: in a whole prompt, with the tail decoded, and in portions."""
    config = make_config([latent_layer(heads=2, dim=32, rot_dim=8, vdim=24, kv_rank=32, q_rank=32, scale=0.25, second=second,
                                       scaling=YARN if second else None, mlp=None)], width=32, vocab=40)
    weights = pointing_weights(config, seed=31)
    folder = write_folder(tmp_path / "model", config, weights, DTYPES[dtype])
    generator = torch.Generator().manual_seed(far)
    base = torch.randint(2, config["vocab"], (400,), generator=generator).tolist()
    base[far], base[-1] = 1, 0                      # tokens 0 and 1 nowhere else
    other = list(base)
    other[far] = 2
    last = len(base) - 1
    want = [forward(tokens, as_double(weights), config)[last].float() for tokens in (base, other)]
    effect = float((want[0] - want[1]).abs().max())
    assert effect > 0.5, "the test's weights do not make the far key count"
    runner = _runner(folder, config, dtype, 416, page=16)
    for records_of in (lambda t: whole("a", t), lambda t: tail_one_by_one("a", t, tail=20), lambda t: portions("a", t, [150, 2, 99, 17])):
        got = [_replay(runner, records_of(tokens))["a"][last] for tokens in (base, other)]
        error = float(((got[0] - got[1]) - (want[0] - want[1])).abs().max())
        assert error < (2e-3 if dtype == "float32" else 0.15) * effect


@pytest.mark.parametrize("dtype", list(DTYPES))
def test_a_far_token_under_a_decay_of_nearly_one(dtype, tmp_path):
    """With decays of about 0.9999 the first token still weighs at position 300: what changing it does to the last
    logits must match the plain implementation (a state that was lost or restarted on the way would show here)."""
    config = make_config([wkv_layer(heads=2, dim=16, rank=4, mlp=None)], width=32, vocab=50)
    weights = make_weights(config, seed=9)
    weights["l0.mix.w0"] = torch.full_like(weights["l0.mix.w0"], -9.0)
    weights["l0.mix.w2"] = torch.zeros_like(weights["l0.mix.w2"])
    folder = write_folder(tmp_path / "model", config, weights, DTYPES[dtype])
    generator = torch.Generator().manual_seed(6)
    base = torch.randint(0, config["vocab"], (300,), generator=generator).tolist()
    other = [(base[0] + 7) % config["vocab"]] + base[1:]
    runner = _runner(folder, config, dtype, 320, page=16)
    last = len(base) - 1
    got = [_replay(runner, portions("a", tokens, [64, 2, 31, 1, 90]))["a"][last] for tokens in (base, other)]
    want = [forward(tokens, as_double(weights), config)[last].float() for tokens in (base, other)]
    effect = float((want[0] - want[1]).abs().max())
    assert effect > 5e-3, "the test's weights do not make the far token count"
    tolerance = 1e-2 if dtype == "float32" else 0.25
    assert float(((got[0] - got[1]) - (want[0] - want[1])).abs().max()) < tolerance * effect + (0 if dtype == "float32" else 0.05)


@pytest.mark.parametrize("dtype", list(DTYPES))
def test_the_first_tokens_of_a_sequence(dtype, tmp_path):
    """Positions 0 to 5 alone: the first token takes the token-pair table's last row and blends with a row of zeros,
    whatever the slot kept from its last owner; a position sees few keys.  Every slot is used several times."""
    config = make_config([wkv_layer(heads=2, dim=8, rank=3, mlp=dense()), latent_layer(mlp=None),
                          latent_layer(heads=2, dim=8, rot_dim=8, vdim=8, kv_rank=16, q_rank=8, second=True, scaling=YARN, mlp=None)],
                         width=48, buckets=7, mul_prev=3, mul_cur=2)
    weights = make_weights(config, seed=41)
    folder = write_folder(tmp_path / "model", config, weights, DTYPES[dtype])
    sequences = _sequences(config, weights, [6, 1, 3, 2, 5, 4, 1, 2], seed=9, dtype=dtype)
    plain = _plain(sequences, weights, config)
    runner = _runner(folder, config, dtype, 32, page=8, slots=2)
    for rid, tokens in sequences.items():
        _compare(_replay(runner, portions(rid, tokens, [1, 2])), plain, dtype, f"first tokens {dtype}")
    records, peak = mixed(sequences, seed=4, max_live=2, page=8)
    _compare(_replay(_runner(folder, config, dtype, peak, page=8, slots=2), records), plain, dtype, f"first tokens {dtype} (mixed)")


def test_the_token_before_belongs_to_the_request(tmp_path):
    """Two requests fed in alternating steps, and a third that takes over a freed slot: the token-pair row and the
    blends with the row before follow each request's own last token, not the batch's or the slot's."""
    config = make_config([wkv_layer(heads=1, dim=8, rank=2, mlp=None)], width=24, vocab=30, buckets=11, mul_prev=1, mul_cur=1)
    weights = make_weights(config, seed=43)
    folder = write_folder(tmp_path / "model", config, weights, torch.float32)
    sequences = _sequences(config, weights, [9, 8, 7], seed=1, dtype="float32")
    plain = _plain(sequences, weights, config)
    a, b, c = (sequences[r] for r in ("r0", "r1", "r2"))
    every = lambda tokens: list(range(len(tokens)))
    entry = lambda rid, tokens: {"id": rid, "tokens": tokens, "want": every(tokens)}
    records = [
        {"step": 0, "entries": [entry("r0", a[:3])], "end": []},
        {"step": 1, "entries": [entry("r1", b[:2])], "end": []},
        {"step": 2, "entries": [entry("r1", b[2:3]), entry("r0", a[3:4])], "end": []},
        {"step": 3, "entries": [entry("r0", a[4:])], "end": ["r0"]},
        {"step": 4, "entries": [entry("r2", c[:1]), entry("r1", b[3:5])], "end": []},
        {"step": 5, "entries": [entry("r1", b[5:]), entry("r2", c[1:])], "end": ["r1", "r2"]},
    ]
    runner = _runner(folder, config, "float32", 32, page=8, slots=2)
    _compare(_replay(runner, records), plain, "float32", "the token before")


@pytest.mark.parametrize("dtype", list(DTYPES))
def test_wide_latents_and_many_heads(dtype, tmp_path):
    """A cached row of the attention kernels' widest head (256 numbers), sixteen heads, heads whose unrotated size is
    below and above their value size, long prompts over several blocks of keys, portions behind cached keys."""
    config = make_config([
        latent_layer(heads=16, dim=24, rot_dim=64, vdim=40, kv_rank=192, q_rank=48, base=1.0e6, scale=0.15, mlp=dense(ff=96)),
        latent_layer(heads=3, dim=128, rot_dim=32, vdim=16, kv_rank=80, q_rank=160, scale=0.07, second=True,
                     scaling={"factor": 16.0, "original": 128, "fast": 32.0, "slow": 1.0}, mlp=None),
    ], width=128, vocab=150)
    weights = make_weights(config, seed=61)
    folder = write_folder(tmp_path / "model", config, weights, DTYPES[dtype])
    sequences = _sequences(config, weights, [300, 45, 170], seed=5, dtype=dtype)
    plain = _plain(sequences, weights, config)
    runner = _runner(folder, config, dtype, 320, page=16)
    tokens = sequences["r0"]
    _compare(_replay(runner, whole("r0", tokens)), plain, dtype, f"wide latents {dtype} (whole)")
    _compare(_replay(runner, portions("r0", tokens, [130, 2, 90, 1, 40])), plain, dtype, f"wide latents {dtype} (portions)")
    _compare(_replay(runner, tail_one_by_one("r0", tokens, tail=12)), plain, dtype, f"wide latents {dtype} (tail)")
    records, peak = mixed(sequences, seed=3, max_live=3, page=16)
    _compare(_replay(_runner(folder, config, dtype, peak, page=16, slots=3), records), plain, dtype, f"wide latents {dtype} (mixed)")


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
        assert output.outputs[0].token_ids == greedy(prompt, as_double(weights), config, 12)


def test_many_experts_and_long_portions(tmp_path):
    """More pairs of one expert than a tile of the grouped products holds, more experts than a warp has lanes, and a
    portion of hundreds of tokens (float32; in bfloat16 a sequence of this length always holds a router decision
    that rounding settles, so there a layer of two experts runs)."""
    config = make_config([wkv_layer(heads=2, dim=16, rank=4, mlp=moe(experts=40, top=3, ff=24)),
                          latent_layer(mlp=moe(experts=2, top=1, ff=40))], width=64, vocab=90)
    weights = make_weights(config, seed=51)
    folder = write_folder(tmp_path / "float32", config, weights, torch.float32)
    tokens = _sequences(config, weights, [300], seed=2, dtype="float32")["r0"]
    plain = _plain({"a": tokens}, weights, config)
    runner = _runner(folder, config, "float32", 320, page=16)
    _compare(_replay(runner, whole("a", tokens)), plain, "float32", "many experts float32")
    _compare(_replay(runner, portions("a", tokens, [70, 2, 33])), plain, "float32", "many experts float32 (portions)")
    config = make_config([latent_layer(mlp=moe(experts=2, top=1, ff=40))], width=64, vocab=90)
    weights = make_weights(config, seed=52)
    folder = write_folder(tmp_path / "bfloat16", config, weights, torch.bfloat16)
    tokens = _sequences(config, weights, [90], seed=2, dtype="bfloat16")["r0"]
    plain = _plain({"a": tokens}, weights, config)
    runner = _runner(folder, config, "bfloat16", 96, page=16)
    _compare(_replay(runner, whole("a", tokens)), plain, "bfloat16", "two experts bfloat16")


def test_the_command_line_and_the_trace_runner_take_a_basitar_folder(tmp_path):
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
    assert [int(t) for t in lines[0].split()] == greedy([5, 9, 12, 80, 3], as_double(weights), config, 6)

    tokens = _sequences(config, weights, [30], seed=2, dtype="float32")["r0"]
    steps = [{"step": 0, "entries": [{"id": "x", "tokens": tokens[:17], "want": [16]}], "end": []},
             {"step": 1, "entries": [{"id": "x", "tokens": tokens[17:], "want": [0, 12]}], "end": ["x"]}]
    out = tmp_path / "out"
    done = subprocess.run([str(root / "bin" / "trace_run"), "--model", str(folder), "--dtype", "float32", "--out", str(out),
                           "--max-tokens", "64"], input="".join(json.dumps(s) + "\n" for s in steps), cwd=tmp_path,
                          capture_output=True, text=True)
    assert done.returncode == 0, done.stderr
    assert [line for line in done.stdout.splitlines() if line.startswith("done")] == ["done 0", "done 1"]
    plain = forward(tokens, as_double(weights), config).float()
    got = torch.from_numpy(np.fromfile(out / "1.f32", dtype="<f4").reshape(2, -1).copy())
    assert_rows_close_by_size(got, plain[[17, 29]], "float32")
