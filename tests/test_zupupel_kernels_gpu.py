"""The kernels that came with the Zupupel decoder, one by one, against plain PyTorch float32."""

from __future__ import annotations

import math

import pytest
import torch

pytestmark = pytest.mark.gpu

DEVICE = "cuda:0"


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("hidden", [64, 50, 1032])
def test_the_layer_norm_in_front_of_behind_and_of_the_stream(hidden, dtype):
    """Mean, variance as the mean of squared deviations, weight and bias; the sum stored (a norm in front of a
    sublayer), the norm stored (a norm behind the sum, with a weight on the stream), the stream alone through a row
    index with a gain on what is handed on; rows of eight and rows that are not."""
    from rapid_llm_b200.ops import kernels

    g = torch.Generator().manual_seed(hidden)
    y = torch.randn(9, hidden, generator=g).to(dtype).to(DEVICE)
    stream = (5 * torch.randn(9, hidden, generator=g) + 2.0).to(DEVICE)
    weight = (1 + 0.2 * torch.randn(hidden, generator=g)).to(DEVICE)
    bias = (0.3 * torch.randn(hidden, generator=g)).to(DEVICE)

    def norm(r, b=bias):
        out = torch.nn.functional.layer_norm(r.double(), (hidden,), weight.double(), None if b is None else b.double(), 1e-5)
        return out.float()

    # behind the sum: stream <- norm(alpha * stream + y)
    before, out = stream.clone(), torch.empty(9, hidden, dtype=dtype, device=DEVICE)
    kernels.layernorm(y, stream, weight, bias, out, 1e-5, residual_scale=2.5, store=kernels.LAYERNORM_STORE_NORM)
    want = norm(2.5 * before + y.float())
    torch.testing.assert_close(stream, want, rtol=1e-5, atol=1e-5)
    assert torch.equal(out, stream.to(dtype))
    # in front of a sublayer: stream <- stream + y, out = norm(stream), no bias
    before = stream.clone()
    kernels.layernorm(y, stream, weight, None, out, 1e-5, store=kernels.LAYERNORM_STORE_SUM)
    torch.testing.assert_close(stream, before + y.float(), rtol=1e-6, atol=1e-6)
    bound = {"rtol": 1e-5, "atol": 1e-5} if dtype == torch.float32 else {"rtol": 1e-2, "atol": 1e-2}
    torch.testing.assert_close(out.float(), norm(before + y.float(), None), **bound)
    # the stream alone, some rows, with a gain; and x alone
    before = stream.clone()
    index = torch.tensor([7, 0, 7, 3], dtype=torch.int32, device=DEVICE)
    picked = torch.empty(4, hidden, dtype=dtype, device=DEVICE)
    kernels.layernorm(None, stream, weight, bias, picked, 1e-5, row_index=index, gain=0.75)
    torch.testing.assert_close(picked.float(), 0.75 * norm(before[index.long()]), **bound)
    assert torch.equal(stream, before)
    kernels.layernorm(y, None, weight, bias, out, 1e-5)
    torch.testing.assert_close(out.float(), norm(y.float()), **bound)
    # a row whose mean dwarfs its spread: the variance is taken around the mean
    shifted = (1000.0 + 0.01 * torch.randn(2, hidden, generator=g)).to(DEVICE)
    flat = torch.empty(2, hidden, dtype=torch.float32, device=DEVICE)
    kernels.layernorm(None, shifted, weight, bias, flat, 1e-7)
    want = torch.nn.functional.layer_norm(shifted.double(), (hidden,), weight.double(), bias.double(), 1e-7).float()
    torch.testing.assert_close(flat, want, rtol=2e-2, atol=2e-2)


def _rotate_halves(rows, positions, rotary, freq):
    """``rows [T, heads, d]`` float64; entry ``i`` of a head pairs with ``i + rotary / 2``."""
    half = rotary // 2
    angle = (positions.float()[:, None] * freq.float()[None, :]).double()      # the angle itself is a float32 product
    cos, sin = torch.cos(angle)[:, None, :], torch.sin(angle)[:, None, :]
    out = rows.clone()
    u, v = rows[..., :half], rows[..., half:rotary]
    out[..., :half] = u * cos - v * sin
    out[..., half:rotary] = v * cos + u * sin
    return out


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("hq,hkv,d,true_d,rotary,with_kv", [(4, 2, 16, 16, 8, True), (6, 3, 32, 20, 20, True), (3, 3, 16, 10, 6, True),
                                                           (8, 1, 64, 64, 0, True), (5, 5, 48, 48, 48, False)])
def test_norm_over_the_whole_projection_rotation_and_cache_write(hq, hkv, d, true_d, rotary, with_kv, dtype):
    """q (and k) normed over all heads at once with a weight per entry (the mean over the TRUE entries when heads are
    laid out with padding), the first ``rotary`` entries of a head rotated by halves, q out, k and v into their pages."""
    from rapid_llm_b200.ops import kernels

    g = torch.Generator().manual_seed(hq * d)
    tokens, page_size, pages = 23, 8, 9
    width = (hq + 2 * hkv) * d if with_kv else hq * d
    qkv = torch.randn(tokens, width, generator=g)
    pad = torch.arange(d) >= true_d                           # a head's padding holds zeros, as zero weight rows leave it
    qkv.view(tokens, -1, d)[:, :, pad] = 0.0
    qkv = qkv.to(dtype).to(DEVICE)
    q_weight = (1 + 0.3 * torch.randn(hq * d, generator=g)).to(DEVICE)
    k_weight = (1 + 0.3 * torch.randn(hkv * d, generator=g)).to(DEVICE)
    freq = (100.0 ** (-torch.arange(0, rotary, 2, dtype=torch.float64) / max(rotary, 1))).float().to(DEVICE) if rotary else None
    positions = torch.randint(0, 3000, (tokens,), generator=g).to(torch.int32).to(DEVICE)
    dest = torch.randperm(page_size * (pages - 1), generator=g)[:tokens].to(torch.int32).to(DEVICE) + page_size
    cache = torch.zeros(pages, 2, hkv, page_size, d, dtype=dtype, device=DEVICE)
    q_out = torch.empty(tokens, hq * d, dtype=dtype, device=DEVICE)
    fault = torch.zeros(1, dtype=torch.int32, device=DEVICE)
    kernels.row_norm_rope_write(qkv, q_out, num_heads=hq, num_kv_heads=hkv, head_dim=d, q_weight=q_weight,
                                k_weight=k_weight if with_kv else None, q_count=hq * true_d, k_count=hkv * true_d,
                                inv_freq=freq, positions=positions, eps=1e-5, fault=fault,
                                kv_dest=dest if with_kv else None, cache=cache if with_kv else None, page_size=page_size)
    assert int(fault.item()) == 0
    rows = qkv.double()

    def normed(part, weight, count, heads):
        scaled = part * torch.rsqrt((part * part).sum(-1, keepdim=True) / count + 1e-5) * weight.double()
        scaled = scaled.view(tokens, heads, d)
        return _rotate_halves(scaled, positions.cpu(), rotary, freq.cpu()) if rotary else scaled

    bound = {"rtol": 2e-5, "atol": 2e-5} if dtype == torch.float32 else {"rtol": 1e-2, "atol": 1e-2}
    want_q = normed(rows[:, : hq * d].cpu(), q_weight.cpu(), hq * true_d, hq)
    torch.testing.assert_close(q_out.view(tokens, hq, d).double().cpu(), want_q, **bound)
    if not with_kv:
        return
    want_k = normed(rows[:, hq * d : (hq + hkv) * d].cpu(), k_weight.cpu(), hkv * true_d, hkv)
    want_v = rows[:, (hq + hkv) * d :].view(tokens, hkv, d).cpu()
    for t in range(tokens):
        page, offset = divmod(int(dest[t]), page_size)
        torch.testing.assert_close(cache[page, 0, :, offset].double().cpu(), want_k[t], **bound)
        assert torch.equal(cache[page, 1, :, offset].double().cpu(), want_v[t])
    assert int(cache[0].abs().sum()) == 0 and float(cache.float().abs().sum()) > 0


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("rows,top,groups,keep,hidden", [(8, 2, 2, 1, 64), (40, 3, 5, 2, 50), (6, 6, 1, 1, 33), (70, 8, 7, 3, 128),
                                                         (9, 1, 3, 3, 40), (12, 4, 12, 4, 24)])
def test_the_router_over_all_rows_with_corrections_and_groups(rows, top, groups, keep, hidden, dtype):
    from rapid_llm_b200.ops import kernels

    g = torch.Generator().manual_seed(rows)
    tokens = 45
    x = torch.randn(tokens, hidden, generator=g).to(dtype).to(DEVICE)
    w = (2.0 * torch.randn(rows, hidden, generator=g) / math.sqrt(hidden)).to(DEVICE)
    correction = (0.1 * torch.randn(rows, generator=g)).to(DEVICE)
    ids = torch.empty(tokens, top, dtype=torch.int32, device=DEVICE)
    weights = torch.empty(tokens, top, device=DEVICE)
    all_scores = torch.empty(tokens, rows, device=DEVICE)
    kernels.router_topk(x, w, experts=rows, top=top, ids=ids, weights=weights, scores=all_scores, softmax_all=True,
                        correction=correction, groups=groups, keep=keep)
    scores = torch.softmax(x.double() @ w.double().T, dim=-1).cpu()
    torch.testing.assert_close(all_scores.double().cpu(), scores, rtol=1e-5, atol=1e-7)
    choice = scores + correction.double().cpu()
    per = rows // groups
    best = choice.view(tokens, groups, per).max(-1).values
    kept = torch.topk(best, keep, dim=-1).indices
    allowed = torch.zeros(tokens, groups, dtype=torch.bool).scatter_(1, kept, True).repeat_interleave(per, dim=1)
    want = torch.topk(choice.masked_fill(~allowed, -math.inf), top, dim=-1).indices
    assert torch.equal(ids.long().cpu(), want)
    picked = torch.gather(scores, 1, want)
    torch.testing.assert_close(weights.double().cpu(), picked / (picked.sum(-1, keepdim=True) + 1e-20), rtol=1e-5, atol=1e-6)


def test_a_correction_decides_the_choice_and_not_the_weight():
    from rapid_llm_b200.ops import kernels

    x = torch.ones(3, 8, device=DEVICE)
    w = torch.zeros(6, 8, device=DEVICE)
    w[0] = 0.5                                    # row 0 has by far the largest score
    correction = torch.tensor([0.0, 0.0, 0.0, 0.0, 0.0, 2.0], device=DEVICE)      # row 5 is lifted above it
    ids = torch.empty(3, 2, dtype=torch.int32, device=DEVICE)
    weights = torch.empty(3, 2, device=DEVICE)
    kernels.router_topk(x, w, experts=6, top=2, ids=ids, weights=weights, softmax_all=True, correction=correction)
    assert ids.tolist() == [[5, 0]] * 3
    scores = torch.softmax(torch.tensor([4.0, 0, 0, 0, 0, 0], dtype=torch.float64), 0)
    torch.testing.assert_close(weights[0].double().cpu(), torch.stack([scores[5], scores[0]]) / (scores[5] + scores[0]), rtol=1e-5, atol=1e-7)
    # groups of three: the lifted row's group wins, rows of the other group are out although their scores are larger
    kernels.router_topk(x, w, experts=6, top=2, ids=ids, weights=weights, softmax_all=True, correction=correction, groups=2, keep=1)
    assert ids.tolist() == [[5, 3]] * 3           # then the lowest index among equal scores
    # negative corrected scores everywhere: rows outside the kept group must count as minus infinity, not as zero
    correction = torch.tensor([-5.0, -5.0, -5.0, -9.0, -9.0, -9.0], device=DEVICE)
    chosen = torch.empty(3, 3, dtype=torch.int32, device=DEVICE)
    kernels.router_topk(x, w, experts=6, top=3, ids=chosen, weights=weights.new_empty(3, 3), softmax_all=True,
                        correction=correction, groups=2, keep=1)
    assert chosen.tolist() == [[0, 1, 2]] * 3


@pytest.mark.parametrize("wide", [False, True])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("tokens,experts,identity,top,hidden,inter", [(300, 37, 3, 3, 64, 24), (37, 5, 2, 2, 50, 22), (1, 2, 1, 3, 32, 8),
                                                                      (150, 2, 2, 2, 200, 72), (40, 1, 3, 2, 40, 16)])
def test_clamped_experts_and_identity_experts(tokens, experts, identity, top, hidden, inter, dtype, wide):
    """Given choices and weights, plan + clamped gated product + down product + weighted sum equal the experts run pair
    by pair, a choice at or behind ``experts`` being the token's own row; on the plain tiles and the pipelined ones."""
    from rapid_llm_b200.ops import kernels

    if wide and not kernels.moe_wide_takes(dtype, hidden, inter):
        pytest.skip("the pipelined tiles take bfloat16 with 16-byte rows")
    limit, alpha = 0.7, 1.702
    g = torch.Generator().manual_seed(tokens + experts)
    x = torch.randn(tokens, hidden, generator=g).to(dtype).to(DEVICE)
    gate_up = (1.5 * torch.randn(experts, 2 * inter, hidden, generator=g) / hidden ** 0.5).to(dtype).to(DEVICE)
    down = (torch.randn(experts, hidden, inter, generator=g) / inter ** 0.5).to(dtype).to(DEVICE)
    ids = torch.stack([torch.randperm(experts + identity, generator=g)[:top] for _ in range(tokens)]).to(torch.int32).to(DEVICE)
    weights = torch.rand(tokens, top, generator=g).to(DEVICE)
    fault = torch.zeros(1, dtype=torch.int32, device=DEVICE)
    pairs = tokens * top
    order = torch.empty(pairs, dtype=torch.int32, device=DEVICE)
    place = torch.empty(pairs, dtype=torch.int32, device=DEVICE)
    meta = torch.zeros(1 + 3 * kernels.moe_max_tiles(pairs, experts, wide), dtype=torch.int32, device=DEVICE)
    max_tiles = kernels.moe_plan(ids, experts, order, place, meta, fault, wide=wide)
    act = torch.empty(pairs, inter, dtype=dtype, device=DEVICE)
    kernels.grouped_linear(x, gate_up, order, meta, top=top, by_token=True, max_tiles=max_tiles, out_act=act, wide=wide,
                           clamp=(limit, alpha))
    each = torch.full((pairs, hidden), float("nan"), device=DEVICE)       # rows of identity pairs stay as they are
    kernels.grouped_linear(act, down, order, meta, top=top, by_token=False, max_tiles=max_tiles, out_y=each, wide=wide)
    out = torch.empty(tokens, hidden, dtype=dtype, device=DEVICE)
    kernels.moe_combine(each, top, out, weights=weights.view(-1), ids=ids, experts=experts, x=x)
    assert int(fault.item()) == 0
    want = torch.zeros(tokens, hidden, device=DEVICE)
    xf, wf, df = x.float(), gate_up.float(), down.float()
    clamped = 0
    for t in range(tokens):
        for j in range(top):
            e, w = int(ids[t, j]), weights[t, j]
            if e >= experts:
                want[t] += w * xf[t]
                continue
            both = wf[e] @ xf[t]
            clamped += int((both[:inter] > limit).sum()) + int((both[inter:].abs() > limit).sum())
            gate, up = both[:inter].clamp(max=limit), both[inter:].clamp(-limit, limit)
            a = gate * torch.sigmoid(alpha * gate) * (up + 1.0)
            if dtype == torch.bfloat16:
                a = a.to(dtype).float()
            want[t] += w * (df[e] @ a)
    assert clamped > 0 and torch.isfinite(out.float()).all()
    bound = {"rtol": 1e-4, "atol": 1e-5} if dtype == torch.float32 else {"rtol": 2e-2, "atol": 2e-2}
    torch.testing.assert_close(out.float(), want, **bound)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("d", [272, 640])
def test_rows_wider_than_the_tensor_core_tiles(d, dtype):
    """The one-warp-per-row attention over a cache of one plane whose rows are wider than 256 numbers."""
    from rapid_llm_b200.ops import kernels

    g = torch.Generator().manual_seed(d)
    heads, page_size, tokens = 3, 8, 21
    pages = 1 + -(-tokens // page_size)
    cache = torch.zeros(pages, 1, 1, page_size, d, dtype=dtype, device=DEVICE)
    rows = (torch.randn(tokens, d, generator=g) / math.sqrt(d) * 4).to(dtype)
    for t in range(tokens):
        cache[1 + t // page_size, 0, 0, t % page_size] = rows[t].to(DEVICE)
    q = torch.randn(tokens, heads * d, generator=g).to(dtype).to(DEVICE)
    out = torch.empty_like(q)
    table = torch.arange(1, pages, dtype=torch.int32, device=DEVICE).view(1, -1).contiguous()
    positions = torch.arange(tokens, dtype=torch.int32, device=DEVICE)
    fault = torch.zeros(1, dtype=torch.int32, device=DEVICE)
    kernels.attention_generic(q, cache, out, positions=positions, token_slot=torch.zeros(tokens, dtype=torch.int32, device=DEVICE),
                              block_table=table, num_heads=heads, num_kv_heads=1, head_dim=d, window=0, scale=0.5, fault=fault)
    assert int(fault.item()) == 0
    qf, kf = q.double().cpu().view(tokens, heads, d), rows.double()
    scores = torch.einsum("ihd,jd->hij", qf, kf) * 0.5
    scores = scores.masked_fill(torch.arange(tokens)[None, :] > torch.arange(tokens)[:, None], -math.inf)
    want = torch.einsum("hij,jd->ihd", torch.softmax(scores, -1), kf).reshape(tokens, heads * d)
    bound = {"rtol": 1e-4, "atol": 1e-5} if dtype == torch.float32 else {"rtol": 2e-2, "atol": 2e-2}
    torch.testing.assert_close(out.double().cpu(), want, **bound)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("width,stride", [(64, 64), (64, 200), (50, 50), (30, 77)])
def test_a_sigmoid_gate_entry_by_entry(width, stride, dtype):
    from rapid_llm_b200.ops import kernels

    g = torch.Generator().manual_seed(width + stride)
    rows = torch.randn(19, width, generator=g).to(dtype).to(DEVICE)
    wide = (3 * torch.randn(19, stride, generator=g)).to(dtype).to(DEVICE)
    gate = wide[:, stride - width :]                      # a view of the last columns of wider rows
    out = torch.empty_like(rows)
    kernels.sigmoid_gate(rows, gate, out)
    want = rows.float() * torch.sigmoid(gate.float())
    bound = {"rtol": 1e-6, "atol": 1e-6} if dtype == torch.float32 else {"rtol": 1e-2, "atol": 1e-2}
    torch.testing.assert_close(out.float(), want, **bound)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("tokens,top,hidden,identity", [(33, 3, 64, True), (5, 1, 50, False), (70, 4, 1032, True)])
def test_the_sum_over_a_tokens_experts_with_the_norm_behind_it(tokens, top, hidden, identity, dtype):
    """``stream <- LN(alpha * stream + sum_j w_j y_j)`` in one kernel equals the sum's kernel followed by the norm's,
    and the plain formula; identity experts' rows of ``y`` are never read."""
    from rapid_llm_b200.ops import kernels

    g = torch.Generator().manual_seed(tokens)
    experts = 5
    y = torch.randn(tokens * top, hidden, generator=g).to(DEVICE)
    ids = torch.randint(0, experts + (3 if identity else 0), (tokens, top), generator=g).to(torch.int32).to(DEVICE)
    if identity:
        y[(ids.view(-1) >= experts)] = float("nan")
    weights = torch.rand(tokens, top, generator=g).to(DEVICE)
    x = torch.randn(tokens, hidden, generator=g).to(dtype).to(DEVICE)
    stream = (2 * torch.randn(tokens, hidden, generator=g) + 0.5).to(DEVICE)
    ln_w, ln_b = (1 + 0.2 * torch.randn(hidden, generator=g)).to(DEVICE), (0.3 * torch.randn(hidden, generator=g)).to(DEVICE)
    before, out = stream.clone(), torch.empty(tokens, hidden, dtype=dtype, device=DEVICE)
    kernels.moe_combine_layernorm(y, top, stream, ln_w, ln_b, out, 1e-5, stream_scale=1.5, weights=weights.view(-1),
                                  ids=ids.view(-1) if identity else None, experts=experts, x=x if identity else None)
    rows = y.view(tokens, top, hidden).double()
    if identity:
        rows = torch.where((ids >= experts)[:, :, None], x.double()[:, None, :], rows)
    total = (weights.double()[:, :, None] * rows).sum(1)
    want = torch.nn.functional.layer_norm(1.5 * before.double() + total, (hidden,), ln_w.double(), ln_b.double(), 1e-5).float()
    torch.testing.assert_close(stream, want, rtol=2e-5, atol=2e-5)
    assert torch.equal(out, stream.to(dtype))
