"""Prefill and decode throughput of Zupupel models at layer sizes of real models, beside Basitar, Mezadra and Qwen3 of
equal width and depth, and the kernels that came with the design alone, each next to the like kernel of the closest
model in the same harness.

    python bench.py --workload zupupel [--sizes 2048,4096]
    python -m rapid_llm_b200.ops.zupupel_compare [--sizes 2048,4096]
    python -m rapid_llm_b200.ops.zupupel_compare --alone --sizes 2048      # the kernels a few times each, for ncu

Random weights, bfloat16, one GPU.  A model of width ``W`` has six layers, ``attention, attention (reads layer 0's
cache), latent_attention, attention, attention (reads layer 3's cache), latent_attention``, each followed by routed
experts: ``W / 128`` attention heads of 128 over ``W / 512`` key/value heads, 64 rotated entries, a window of 512
positions, a gate over the heads; latent attention with 128 plain, 64 rotated and 128 value entries over a latent of
192 (a cached row of 256 numbers); 16 clamped experts of ``W / 4`` and 8 identity experts in 4 groups of which 2 are
kept, a token taking two.  Basitar, Mezadra and Qwen3 beside it have six layers of the same width.  Prefill is one
2,048-token step (best of three, CUDA events around the step function); decode is batch 8 behind 1,024-token prompts,
replayed from the captured graph (median of 32 steps).  Kernels are timed alone with CUDA events, L2 flushed between
runs (a write of 256 MB), on one 2,048-token prompt and on 64 single tokens; ``frac`` is (bytes the kernel must move)
/ time / measured copy bandwidth, ``tflops`` the products' arithmetic over the same time.
"""

from __future__ import annotations

import argparse
import json
import statistics

import torch

from .basitar_compare import basitar_raw
from .mezadra_compare import mezadra_raw
from .recurrent_compare import PREFILL, _events, model_figures, qwen3_raw

EXPERTS, IDENTITY, TOP, GROUPS, KEEP = 16, 8, 2, 4, 2
PLAIN, ROT, VDIM, KV_RANK, WINDOW = 128, 64, 128, 192, 512


def zupupel_raw(width: int) -> dict:
    heads = width // 128
    attention = {"heads": heads, "kv_heads": max(heads // 4, 1), "dim": 128, "vdim": 128, "mask": {"size": WINDOW},
                 "rot": {"dims": 64, "base": 1.0e6}, "scale": 128 ** -0.5}
    latent = {"heads": heads, "dim": PLAIN, "rot_dim": ROT, "vdim": VDIM, "kv_rank": KV_RANK,
              "rot": {"base": 1.0e4, "dims": ROT}, "scale": (PLAIN + ROT) ** -0.5}
    experts = {"kind": "moe", "expert": {"ff": width // 4, "limit": 7.0},
               "router": {"experts": EXPERTS, "identity": IDENTITY, "top": TOP, "groups": {"count": GROUPS, "keep": KEEP}}}
    order = [("attention", attention), ("attention", {**attention, "kv_from": 0}), ("latent_attention", latent),
             ("attention", attention), ("attention", {**attention, "kv_from": 3}), ("latent_attention", latent)]
    return {"architecture": "Zupupel", "vocab": 32000, "width": width, "norm": {"eps": 1e-6}, "embedding": {"scale": 1.0},
            "postln_alpha": 2.0, "logit_scale": 0.25,
            "layers": [{"type": kind, "mixer": dict(mixer), "mlp": dict(experts)} for kind, mixer in order]}


def kernel_figures(width: int, hbm_gbs: float) -> dict:
    """The design's own kernels alone, and beside each the like kernel of the closest model, on a 2,048-token prompt
    and on 64 single tokens."""
    from . import kernels

    device = "cuda:0"
    heads, kv_heads, d, inter = width // 128, max(width // 512, 1), 128, width // 4
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
    page = 16
    for tokens, entries in ((PREFILL, 1), (64, 64)):
        x = bf(tokens, width)
        # -- the norm behind the sum, beside the norm that joins the stream (Mezadra's)
        stream, weight, bias = f32(tokens, width), f32(width), f32(width)
        rounded = torch.empty(tokens, width, dtype=torch.bfloat16, device=device)
        timed("layernorm behind the sum", tokens, entries, tokens * width * 12,
              lambda: kernels.layernorm(x, stream, weight, bias, rounded, 1e-6, residual_scale=2.0, store=kernels.LAYERNORM_STORE_NORM))
        timed("join_rmsnorm (like kernel)", tokens, entries, tokens * width * 12,
              lambda: kernels.join_rmsnorm(x, stream, weight, rounded, 1e-6))
        # -- norm over the whole projection, rotation and cache write, beside the per-head norm from tables (Qwen3's)
        channels = (heads + 2 * kv_heads) * d
        qkv = bf(tokens, channels)
        q_out = torch.empty(tokens, heads * d, dtype=torch.bfloat16, device=device)
        pages = -(-tokens // page) + 1
        cache = torch.zeros(pages, 2, kv_heads, page, d, dtype=torch.bfloat16, device=device)
        positions = torch.arange(tokens, dtype=torch.int32, device=device)
        dest = (positions + page).to(torch.int32)
        q_weight, k_weight, freq = f32(heads * d), f32(kv_heads * d), torch.rand(32, device=device)
        timed("row_norm_rope_write", tokens, entries, tokens * channels * 4,
              lambda: kernels.row_norm_rope_write(qkv, q_out, num_heads=heads, num_kv_heads=kv_heads, head_dim=d, q_weight=q_weight,
                                                  k_weight=k_weight, q_count=heads * d, k_count=kv_heads * d, inv_freq=freq,
                                                  positions=positions, eps=1e-6, fault=fault, kv_dest=dest, cache=cache, page_size=page))
        cos, sin, head_weight = torch.rand(tokens, 32, device=device), torch.rand(tokens, 32, device=device), f32(d)
        timed("qk_norm_rope_write (like kernel)", tokens, entries, tokens * channels * 4,
              lambda: kernels.qk_norm_rope_write(qkv, q_out, num_heads=heads, num_kv_heads=kv_heads, head_dim=d, rotary_dim=64, cos=cos,
                                                 sin=sin, positions=positions, eps=1e-6, fault=fault, q_weight=head_weight,
                                                 k_weight=head_weight, kv_dest=dest, cache=cache, page_size=page))
        # -- the router over all rows with corrections and groups, beside the sigmoid router (Mezadra's)
        rows = EXPERTS + IDENTITY
        router, correction = f32(rows, width), 0.1 * f32(rows)
        ids = torch.empty(tokens, TOP, dtype=torch.int32, device=device)
        weights = torch.empty(tokens, TOP, device=device)
        timed("router_topk, softmax over all rows, groups", tokens, entries, tokens * width * 2 + router.numel() * 4,
              lambda: kernels.router_topk(x, router, experts=rows, top=TOP, ids=ids, weights=weights, softmax_all=True,
                                          correction=correction, groups=GROUPS, keep=KEEP))
        plain_ids = torch.empty_like(ids)
        timed("router_topk, sigmoid (like kernel)", tokens, entries, tokens * width * 2 + router.numel() * 4,
              lambda: kernels.router_topk(x, router, experts=rows, top=TOP, ids=plain_ids, weights=weights))
        kernels.router_topk(x, router, experts=rows, top=TOP, ids=ids, weights=weights, softmax_all=True, correction=correction,
                            groups=GROUPS, keep=KEEP)
        # -- clamped experts over the pairs that chose one, beside SiLU experts over the same plan; the weighted sum
        pairs = tokens * TOP
        order, place = (torch.empty(pairs, dtype=torch.int32, device=device) for _ in range(2))
        meta = torch.zeros(1 + 3 * kernels.moe_max_tiles(pairs, EXPERTS, True), dtype=torch.int32, device=device)
        max_tiles = kernels.moe_plan(ids, EXPERTS, order, place, meta, fault, wide=True)
        gate_up, down = bf(EXPERTS, 2 * inter, width) / width ** 0.5, bf(EXPERTS, width, inter)
        act, each = torch.zeros(pairs, inter, dtype=torch.bfloat16, device=device), torch.zeros(pairs, width, device=device)
        real = int((ids < EXPERTS).sum())
        touched = min(EXPERTS, real)
        moved = touched * 2 * inter * width * 2 + tokens * width * 2 + real * inter * 2
        timed("grouped_linear, gate and up, clamped unit", tokens, entries, moved,
              lambda: kernels.grouped_linear(x, gate_up, order, meta, top=TOP, by_token=True, max_tiles=max_tiles, out_act=act,
                                             wide=True, clamp=(7.0, 1.702)), flops=2.0 * real * 2 * inter * width)
        timed("grouped_linear, gate and up, SiLU (like kernel)", tokens, entries, moved,
              lambda: kernels.grouped_linear(x, gate_up, order, meta, top=TOP, by_token=True, max_tiles=max_tiles, out_act=act,
                                             wide=True), flops=2.0 * real * 2 * inter * width)
        kernels.grouped_linear(act, down, order, meta, top=TOP, by_token=False, max_tiles=max_tiles, out_y=each, wide=True)
        combined = torch.empty(tokens, width, dtype=torch.bfloat16, device=device)
        timed("moe_combine, weights and identity experts", tokens, entries, pairs * width * 4 + tokens * width * 4,
              lambda: kernels.moe_combine(each, TOP, combined, weights=weights.view(-1), ids=ids, experts=EXPERTS, x=x))
        timed("moe_combine, weights (like kernel)", tokens, entries, pairs * width * 4 + tokens * width * 2,
              lambda: kernels.moe_combine(each, TOP, combined, weights=weights.view(-1)))
        timed("moe_combine_layernorm: the sum, the stream and the norm behind them", tokens, entries,
              pairs * width * 4 + tokens * width * 12,
              lambda: kernels.moe_combine_layernorm(each, TOP, stream, weight, bias, combined, 1e-6, stream_scale=2.0,
                                                    weights=weights.view(-1), ids=ids.view(-1), experts=EXPERTS, x=x))
        # -- the gate over the heads side by side, entry by entry, beside the gate of one number a head (Basitar's)
        attended, gate = bf(tokens, heads * d), bf(tokens, heads * d)
        gated = torch.empty_like(attended)
        timed("sigmoid_gate, entry by entry", tokens, entries, tokens * heads * d * 6,
              lambda: kernels.sigmoid_gate(attended, gate, gated))
        timed("sigmoid_scale_heads (like kernel)", tokens, entries, tokens * heads * d * 4,
              lambda: kernels.sigmoid_scale_heads(attended, gate, heads=heads))
    assert int(fault.item()) == 0, "a kernel reported a fault"
    return out


def alone(width: int = 2048) -> None:
    """Every kernel of :func:`kernel_figures` a few times and nothing else: the case a profiler captures, picking its
    kernel by name."""
    kernel_figures(width, 6650.0)
    torch.cuda.synchronize()


def run(sizes: list[int], hbm_gbs: float) -> dict:
    from ..config import BasitarConfig, MezadraConfig, Qwen3Config, ZupupelConfig

    result = {"workload": "zupupel beside basitar, mezadra and qwen3, equal sizes", "dtype": "bf16", "data": "synthetic",
              "prefill_tokens": PREFILL, "decode_batch": 8, "decode_context": 1024, "sizes": {}}
    for width in sizes:
        result["sizes"][str(width)] = {
            "zupupel": model_figures(ZupupelConfig.from_dict(zupupel_raw(width))),
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
