"""Prefill and decode throughput of Basitar models at layer sizes of real models, beside Mezadra and Qwen3 of equal
width and depth, and the kernels that came with the design alone against their rooflines.

    python bench.py --workload basitar [--sizes 2048,4096]
    python -m rapid_llm_b200.ops.basitar_compare [--sizes 2048,4096]
    python -m rapid_llm_b200.ops.basitar_compare --alone --sizes 2048      # the kernels a few times each, for ncu

Random weights, bfloat16, one GPU.  A model of width ``W`` has six layers, ``latent_attention, latent_attention_2,
wkv, latent_attention, latent_attention_2, wkv`` with the feed-forwards ``dense, experts, experts, dense, experts,
experts``: ``W / 128`` attention heads of 128 plain, 64 rotated and 128 value entries over a latent of 192 (a cached
row of 256 numbers, the attention tiles' widest) and a query latent of ``3 W / 8``; ``W / 64`` recurrent heads of 64
with a decay product of rank 64; a dense feed-forward of ``8 W / 3`` (rounded to 256) and 16 experts of ``W / 4`` of
which a token takes two.  Mezadra and Qwen3 beside it have six layers of the same width.  Prefill is one 2,048-token
step (best of three, CUDA events around the step function); decode is batch 8 behind 1,024-token prompts, replayed
from the captured graph (median of 32 steps).  Kernels are timed alone with CUDA events, L2 flushed between runs (a
write of 256 MB), on one 2,048-token prompt and on 64 single tokens behind 1,024 cached ones; ``frac`` is (bytes the
kernel must move) / time / measured copy bandwidth, ``tflops`` the products' arithmetic over the same time.
"""

from __future__ import annotations

import argparse
import json
import statistics
from types import SimpleNamespace

import torch

from .mezadra_compare import mezadra_raw
from .recurrent_compare import PREFILL, _events, model_figures, qwen3_raw

EXPERTS, TOP = 16, 2
PLAIN, ROT, VDIM, KV_RANK = 128, 64, 128, 192
WKV_DIM, DECAY_RANK = 64, 64


def basitar_raw(width: int) -> dict:
    heads = width // 128
    first = {"heads": heads, "dim": PLAIN, "rot_dim": ROT, "vdim": VDIM, "kv_rank": KV_RANK, "q_rank": 3 * width // 8,
             "rot": {"base": 1.0e4, "dims": ROT}, "scale": (PLAIN + ROT) ** -0.5}
    second = {**first, "rot": {"base": 1.0e4, "dims": ROT, "scaling": {"factor": 40.0, "original": 4096, "fast": 32.0, "slow": 1.0}}}
    wkv = {"heads": width // WKV_DIM, "dim": WKV_DIM, "decay_rank": DECAY_RANK}
    dense = {"kind": "dense", "ff": (8 * width // 3 + 255) // 256 * 256}
    experts = {"kind": "moe", "router": {"experts": EXPERTS, "top": TOP}, "expert": {"ff": width // 4}}
    order = [("latent_attention", first, dense), ("latent_attention_2", second, experts), ("wkv", wkv, experts),
             ("latent_attention", first, dense), ("latent_attention_2", second, experts), ("wkv", wkv, experts)]
    return {"architecture": "Basitar", "vocab": 32000, "width": width, "max_positions": 4096, "norm": {"eps": 1e-6},
            "embedding": {"bigram": {"buckets": 65521, "mul_prev": 31, "mul_cur": 17}},
            "layers": [{"type": kind, "mixer": dict(mixer), "mlp": dict(mlp)} for kind, mixer, mlp in order]}


def kernel_figures(width: int, hbm_gbs: float) -> dict:
    """The design's own kernels alone, on a 2,048-token prompt and on 64 single tokens."""
    import numpy as np

    from ..parts.attention import AttentionItems
    from ..parts.base import StepShape
    from . import gemm, kernels

    device = "cuda:0"
    heads, d, q_rank = width // 128, 256, 3 * width // 8
    flush = torch.empty(64 << 20, dtype=torch.float32, device=device)
    out = {}

    def timed(label, tokens, entries, moved, run, flops=0.0):
        times = []
        for _ in range(5):
            flush.zero_()
            begin, end = _events()
            begin.record()
            run()
            end.record()
            torch.cuda.synchronize()
            times.append(begin.elapsed_time(end) * 1e3)
        us = statistics.median(times[1:])
        row = {"us": round(us, 1), "mb": round(moved / 1e6, 2), "frac": round(moved / (us * 1e-6) / (hbm_gbs * 1e9), 3)}
        if flops:
            row["tflops"] = round(flops / (us * 1e-6) / 1e12, 1)
        out[f"{label} ({'prompt of ' + str(tokens) if entries == 1 else str(entries) + ' single tokens'})"] = row

    bf = lambda *shape: torch.randn(*shape, device=device).to(torch.bfloat16)      # noqa: E731
    f32 = lambda *shape: torch.randn(*shape, device=device)                        # noqa: E731
    fault = torch.zeros(1, dtype=torch.int32, device=device)
    page, context = 16, 1024
    for tokens, entries in ((PREFILL, 1), (64, 64)):
        per = tokens // entries
        start = 0 if entries == 1 else context
        batch = SimpleNamespace(
            cu_seqlens=torch.arange(0, tokens + 1, per, dtype=torch.int32, device=device),
            entry_slot=torch.arange(entries, dtype=torch.int32, device=device),
            entry_start=torch.full((entries,), start, dtype=torch.int32, device=device), num_entries=entries, fault=fault)
        positions = (start + torch.arange(per, dtype=torch.int32, device=device)).repeat(entries)
        # -- latent attention: both latents' norms and the cache row, the per-head products, the rotation, the tiles
        c_col0 = q_rank
        down_rows = c_col0 + d + 8 * ((heads + 7) // 8)
        down = bf(tokens, down_rows)
        pages_per = -(-(start + per) // page)
        cache = torch.zeros(entries * pages_per + 1, page, d, dtype=torch.bfloat16, device=device)
        cache.normal_()
        table = (1 + torch.arange(entries * pages_per, dtype=torch.int32, device=device)).view(entries, pages_per)
        slot_of = torch.arange(entries, dtype=torch.int32, device=device).repeat_interleave(per)
        dest = (table[slot_of.long(), (positions // page).long()] * page + positions % page).to(torch.int32)
        c_q = torch.empty(tokens, q_rank, dtype=torch.bfloat16, device=device)
        q_weight, c_weight, freq = f32(q_rank), f32(KV_RANK), torch.rand(ROT // 2, device=device)
        timed("latent_norm_write", tokens, entries, tokens * (q_rank + d) * 4,
              lambda: kernels.latent_norm_write(down, q_col0=0, q_rank=q_rank, c_col0=c_col0, kv_rank=KV_RANK, rot=ROT,
                                                q_weight=q_weight, c_weight=c_weight, eps=1e-6, q_out=c_q, cache=cache,
                                                kv_dest=dest, positions=positions, freq=freq, magnitude=1.2,
                                                layout=kernels.ROTATE_NEIGHBOURS, fault=fault))
        q, wide = bf(tokens, heads * (PLAIN + ROT)), torch.empty(tokens, heads * d, dtype=torch.bfloat16, device=device)
        uk_t, uv = bf(heads, KV_RANK, PLAIN), bf(heads, VDIM, KV_RANK)
        timed("heads_linear, queries into the latent", tokens, entries,
              tokens * heads * (PLAIN + KV_RANK) * 2 + uk_t.numel() * 2,
              lambda: gemm.heads_linear(q, uk_t, wide), flops=2.0 * tokens * heads * PLAIN * KV_RANK)
        timed("latent_rotate_queries", tokens, entries, tokens * heads * (ROT + d - KV_RANK) * 2,
              lambda: kernels.latent_rotate_queries(q, wide, heads=heads, dim=PLAIN, rot=ROT, kv_rank=KV_RANK, positions=positions,
                                                    freq=freq, magnitude=1.2, layout=kernels.ROTATE_NEIGHBOURS))
        planner = AttentionItems(heads, 1, d, tensor_core=False)
        plan = planner.plan(StepShape(lengths=np.full(entries, per, dtype=np.int32), starts=np.full(entries, start, dtype=np.int32),
                                      decode_only=per == 1, page_size=page))
        chunk = torch.from_numpy(plan["chunk_items"]).to(device)
        decode = torch.from_numpy(plan["decode_items"]).to(device)
        splits = plan["splits"]
        rows = tokens * heads * splits
        part_out = torch.empty(rows, d, device=device) if splits > 1 else None
        part_lse = torch.empty(rows, 1, device=device) if splits > 1 else None
        attended = torch.empty_like(wide)
        keys = sum(range(start + 1, start + per + 1)) * entries
        timed("attention tiles over one cached row per token", tokens, entries,
              entries * (start + per) * d * 2 + tokens * heads * d * 4,
              lambda: kernels.attention_mma(
                  wide, cache.view(cache.shape[0], 1, 1, page, d), attended, chunk_items=chunk, decode_items=decode, splits=splits,
                  part_out=part_out, part_lse=part_lse, cu_seqlens=batch.cu_seqlens, entry_start=batch.entry_start,
                  entry_slot=batch.entry_slot, block_table=table, num_heads=heads, num_kv_heads=1, head_dim=d, window=0,
                  scale=(PLAIN + ROT) ** -0.5, fault=fault, decode_kernel="mma", decode_rows=plan.get("decode_rows", 0),
                  chunk_rows=kernels.CHUNK_TILE_ROWS),
              flops=4.0 * keys * heads * d)
        values = torch.empty(tokens, heads * VDIM, dtype=torch.bfloat16, device=device)
        timed("heads_linear, values out of the latent", tokens, entries,
              tokens * heads * (KV_RANK + VDIM) * 2 + uv.numel() * 2,
              lambda: gemm.heads_linear(attended, uv, values), flops=2.0 * tokens * heads * VDIM * KV_RANK)
        timed("sigmoid_scale_heads", tokens, entries, tokens * heads * VDIM * 4,
              lambda: kernels.sigmoid_scale_heads(values, down[:, c_col0 + d :], heads=heads))
        # -- the recurrent mixer: blends, decay, the walk with a bonus, norm and gate
        wkv_heads, c = width // WKV_DIM, width
        x, mu = bf(tokens, width), torch.rand(5, width, device=device)
        blends = torch.empty(5 * tokens, width, dtype=torch.bfloat16, device=device)
        state = torch.zeros(entries, wkv_heads * WKV_DIM * WKV_DIM + width, device=device)
        S, kept = state[:, : wkv_heads * WKV_DIM * WKV_DIM], state[:, wkv_heads * WKV_DIM * WKV_DIM :]
        timed("shift_mix, five blends", tokens, entries, tokens * width * 12 + 2 * kept.numel() * 4,
              lambda: kernels.shift_mix(x, mu, blends, kept, batch))
        low = bf(tokens, DECAY_RANK)
        timed("tanh_rows", tokens, entries, tokens * DECAY_RANK * 4, lambda: kernels.tanh_rows(low, low))
        high, w0, decay = bf(tokens, c), f32(c), torch.empty(tokens, c, device=device)
        timed("exp_decay", tokens, entries, tokens * c * 6, lambda: kernels.exp_decay(high, w0, decay))
        decay.uniform_(0.9, 1.0)
        r, k, v, read = f32(tokens, c), f32(tokens, c), f32(tokens, c), f32(tokens, c)
        bonus = f32(wkv_heads, WKV_DIM)
        timed("linear_scan, row decays and a bonus", tokens, entries, 2 * S.numel() * 4 + 5 * tokens * c * 4,
              lambda: kernels.linear_scan(r, k, v, decay, read, S, batch, heads=wkv_heads, kv_heads=wkv_heads, dim=WKV_DIM,
                                          vdim=WKV_DIM, bonus=bonus))
        normed, weight, gate = torch.empty(tokens, c, dtype=torch.bfloat16, device=device), f32(c), bf(tokens, c)
        timed("gated_norm, heads of 64, SiLU gate", tokens, entries, tokens * c * 8,
              lambda: kernels.gated_norm(read, normed, group=WKV_DIM, gate=gate, act=kernels.GATE_SILU, weight=weight, eps=1e-6))
        # -- the layer's norms, the router, the weighted sum over a token's experts
        stream, closing, opening = f32(tokens, width), f32(width), f32(width)
        timed("join_then_rmsnorm", tokens, entries, tokens * width * 12,
              lambda: kernels.join_then_rmsnorm(x, stream, closing, opening, normed, 1e-6))
        router, bias = f32(EXPERTS, width), f32(EXPERTS)
        ids = torch.empty(tokens, TOP, dtype=torch.int32, device=device)
        shares = torch.empty(tokens, TOP, device=device)
        timed("router_topk, bias, softmax over the chosen", tokens, entries, tokens * width * 2 + router.numel() * 4,
              lambda: kernels.router_topk(x, router, experts=EXPERTS, top=TOP, ids=ids, weights=shares, bias=bias, softmax_chosen=True))
        each, combined = f32(tokens * TOP, width), torch.empty(tokens, width, dtype=torch.bfloat16, device=device)
        timed("moe_combine, weights on the outputs", tokens, entries, tokens * TOP * width * 4 + tokens * width * 2,
              lambda: kernels.moe_combine(each, TOP, combined, weights=shares.view(-1)))
    assert int(fault.item()) == 0, "a kernel reported a fault"
    return out


def alone(width: int = 2048) -> None:
    """Every kernel of :func:`kernel_figures` a few times and nothing else: the case a profiler captures, picking its
    kernel by name."""
    kernel_figures(width, 6650.0)
    torch.cuda.synchronize()


def run(sizes: list[int], hbm_gbs: float) -> dict:
    from ..config import BasitarConfig, MezadraConfig, Qwen3Config

    result = {"workload": "basitar beside mezadra and qwen3, equal sizes", "dtype": "bf16", "data": "synthetic",
              "prefill_tokens": PREFILL, "decode_batch": 8, "decode_context": 1024, "sizes": {}}
    for width in sizes:
        result["sizes"][str(width)] = {
            "basitar": model_figures(BasitarConfig.from_dict(basitar_raw(width))),
            "mezadra": model_figures(MezadraConfig.from_dict(mezadra_raw(width))),
            "qwen3": model_figures(Qwen3Config.from_dict(qwen3_raw(width, layers=6))),
            "kernels": kernel_figures(width, hbm_gbs),
        }
    return result


def main() -> int:
    parser = argparse.ArgumentParser(description=__doc__.splitlines()[0])
    parser.add_argument("--sizes", default="2048,4096")
    parser.add_argument("--hbm-gbs", type=float, default=6650.0)
    parser.add_argument("--alone", action="store_true", help="only launch the kernels a few times (for a profiler)")
    args = parser.parse_args()
    if args.alone:
        alone(int(args.sizes.split(",")[0]))
        return 0
    print(json.dumps(run([int(s) for s in args.sizes.split(",") if s], args.hbm_gbs)))
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
