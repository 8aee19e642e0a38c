"""The kernels that came with the Basitar decoder, one by one, against plain PyTorch float32."""

from __future__ import annotations

import math

import pytest
import torch

pytestmark = pytest.mark.gpu

DEVICE = "cuda:0"
DTYPES = [torch.float32, torch.bfloat16]


def _tolerance(dtype):
    return dict(rtol=2e-5, atol=2e-5) if dtype == torch.float32 else dict(rtol=1.6e-2, atol=1.6e-2)


def _rotated(x, positions, freq, magnitude, neighbours):
    """x ``[T, ..., R]`` float32."""
    angle = positions.float()[:, None] * freq[None, :]
    cos, sin = torch.cos(angle) * magnitude, torch.sin(angle) * magnitude
    while cos.dim() < x.dim():
        cos, sin = cos.unsqueeze(1), sin.unsqueeze(1)
    out = torch.empty_like(x)
    if neighbours:
        u, v = x[..., 0::2], x[..., 1::2]
        out[..., 0::2], out[..., 1::2] = u * cos - v * sin, v * cos + u * sin
    else:
        half = x.shape[-1] // 2
        u, v = x[..., :half], x[..., half:]
        out[..., :half], out[..., half:] = u * cos - v * sin, v * cos + u * sin
    return out


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("neighbours", [False, True])
@pytest.mark.parametrize("q_rank,kv_rank,rot,width", [(24, 40, 8, 48), (10, 14, 6, 32), (80, 192, 64, 256), (16, 22, 2, 32), (8, 16, 0, 16)])
def test_latent_norm_write(q_rank, kv_rank, rot, width, neighbours, dtype):
    """Both latents are normed, the key part is rotated, and the cache row is ``[c | key part | zeros]`` at the place
    ``kv_dest`` names; a destination below zero writes nothing."""
    from rapid_llm_b200.ops import kernels

    g = torch.Generator().manual_seed(q_rank + kv_rank)
    tokens, page_size, pages = 37, 8, 9
    up8 = lambda n: -(-n // 8) * 8
    c_col0 = up8(q_rank)
    down = torch.randn(tokens, c_col0 + up8(kv_rank + rot) + 8, generator=g).to(dtype).to(DEVICE)
    q_weight = (1 + 0.2 * torch.randn(q_rank, generator=g)).to(DEVICE)
    c_weight = (1 + 0.2 * torch.randn(kv_rank, generator=g)).to(DEVICE)
    positions = torch.randint(0, 500, (tokens,), generator=g).to(torch.int32).to(DEVICE)
    freq = (torch.rand(rot // 2, generator=g) if rot else torch.zeros(1)).to(DEVICE)
    kv_dest = torch.randperm(pages * page_size, generator=g)[:tokens].to(torch.int32).to(DEVICE)
    cache = torch.full((pages, page_size, width), 7.0, dtype=dtype, device=DEVICE)
    q_out = torch.empty(tokens, q_rank, dtype=dtype, device=DEVICE)
    fault = torch.zeros(1, dtype=torch.int32, device=DEVICE)
    eps, magnitude = 1e-5, 1.3
    kernels.latent_norm_write(down, q_col0=0, q_rank=q_rank, c_col0=c_col0, kv_rank=kv_rank, rot=rot, q_weight=q_weight,
                              c_weight=c_weight, eps=eps, q_out=q_out, cache=cache, kv_dest=kv_dest, positions=positions,
                              freq=freq if rot else None, magnitude=magnitude,
                              layout=kernels.ROTATE_NEIGHBOURS if neighbours else kernels.ROTATE_HALVES, fault=fault)
    assert int(fault.item()) == 0
    rms = lambda x: x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)
    f = down.float()
    torch.testing.assert_close(q_out.float(), (rms(f[:, :q_rank]) * q_weight).to(dtype).float(), **_tolerance(dtype))
    rows = cache.view(-1, width)[kv_dest.long()].float()
    torch.testing.assert_close(rows[:, :kv_rank], (rms(f[:, c_col0 : c_col0 + kv_rank]) * c_weight).to(dtype).float(), **_tolerance(dtype))
    if rot:
        want = _rotated(f[:, c_col0 + kv_rank : c_col0 + kv_rank + rot], positions, freq, magnitude, neighbours)
        torch.testing.assert_close(rows[:, kv_rank : kv_rank + rot], want.to(dtype).float(), **_tolerance(dtype))
    assert float(rows[:, kv_rank + rot :].abs().sum()) == 0.0
    untouched = torch.ones(pages * page_size, dtype=torch.bool)
    untouched[kv_dest.long().cpu()] = False
    assert bool((cache.view(-1, width)[untouched.to(DEVICE)] == 7.0).all())


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("neighbours", [False, True])
@pytest.mark.parametrize("heads,dim,rot,kv_rank,width", [(3, 16, 8, 40, 48), (5, 10, 6, 14, 32), (16, 24, 64, 192, 256), (2, 14, 2, 22, 32)])
def test_latent_rotate_queries(heads, dim, rot, kv_rank, width, neighbours, dtype):
    from rapid_llm_b200.ops import kernels

    g = torch.Generator().manual_seed(heads * dim)
    tokens = 29
    q = torch.randn(tokens, heads * (dim + rot), generator=g).to(dtype).to(DEVICE)
    wide = torch.full((tokens, heads * width), 3.0, dtype=dtype, device=DEVICE)
    positions = torch.randint(0, 900, (tokens,), generator=g).to(torch.int32).to(DEVICE)
    freq = torch.rand(rot // 2, generator=g).to(DEVICE)
    kernels.latent_rotate_queries(q, wide, heads=heads, dim=dim, rot=rot, kv_rank=kv_rank, positions=positions, freq=freq,
                                  magnitude=0.8, layout=kernels.ROTATE_NEIGHBOURS if neighbours else kernels.ROTATE_HALVES)
    got = wide.view(tokens, heads, width).float()
    want = _rotated(q.view(tokens, heads, dim + rot)[..., dim:].float(), positions, freq, 0.8, neighbours)
    torch.testing.assert_close(got[..., kv_rank : kv_rank + rot], want.to(dtype).float(), **_tolerance(dtype))
    assert float(got[..., kv_rank + rot :].abs().sum()) == 0.0
    assert bool((got[..., :kv_rank] == 3.0).all())                 # the product's columns are another kernel's


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("tokens,heads,n_out,k,x_width,out_width,x_col0", [
    (33, 3, 40, 16, 24, 48, 0), (1, 5, 14, 10, 16, 32, 0), (200, 16, 192, 24, 88, 256, 0), (17, 2, 24, 32, 48, 24, 0),
    (9, 4, 6, 22, 32, 6, 2), (70, 1, 64, 96, 96, 64, 0), (90, 3, 10, 14, 18, 13, 1), (2048, 8, 192, 128, 192, 256, 0)])
@pytest.mark.parametrize("entry", ["tiles", "by size"])
def test_a_product_per_head(tokens, heads, n_out, k, x_width, out_width, x_col0, dtype, entry):
    """The hand-written tiles at every size, and the entry point that hands large bfloat16 steps to the library's
    batched product over strided views (rows that start at odd columns too)."""
    from rapid_llm_b200.ops import gemm, kernels

    g = torch.Generator().manual_seed(tokens + heads)
    x = torch.randn(tokens, heads * x_width, generator=g).to(dtype).to(DEVICE)
    weight = (torch.randn(heads, n_out, k, generator=g) / math.sqrt(k)).to(dtype).to(DEVICE)
    out = torch.full((tokens, heads * out_width), 5.0, dtype=dtype, device=DEVICE)
    (kernels if entry == "tiles" else gemm).heads_linear(x, weight, out, x_col0=x_col0)
    got = out.view(tokens, heads, out_width).float()
    want = torch.einsum("thk,hnk->thn", x.view(tokens, heads, x_width)[..., x_col0 : x_col0 + k].double(), weight.double()).float()
    torch.testing.assert_close(got[..., :n_out], want.to(dtype).float(), **_tolerance(dtype))
    assert bool((got[..., n_out:] == 5.0).all())


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("heads,width", [(3, 24), (1, 64), (5, 6), (16, 40)])
def test_a_sigmoid_gate_per_head(heads, width, dtype):
    from rapid_llm_b200.ops import kernels

    g = torch.Generator().manual_seed(heads)
    tokens = 21
    rows = torch.randn(tokens, heads * width, generator=g).to(dtype).to(DEVICE)
    wide = torch.randn(tokens, 8 + heads + 3, generator=g).to(dtype).to(DEVICE)
    want = rows.view(tokens, heads, width).float() * torch.sigmoid(wide[:, 8 : 8 + heads].float())[:, :, None]
    kernels.sigmoid_scale_heads(rows, wide[:, 8:], heads=heads)
    torch.testing.assert_close(rows.view(tokens, heads, width).float(), want.to(dtype).float(), **_tolerance(dtype))


@pytest.mark.parametrize("dtype", DTYPES)
def test_decay_from_a_product_and_tanh(dtype):
    from rapid_llm_b200.ops import kernels

    g = torch.Generator().manual_seed(1)
    tokens, channels = 45, 50
    wide = (2 * torch.randn(tokens, channels + 6, generator=g)).to(dtype).to(DEVICE)
    bias = (-2 + 2 * torch.randn(channels, generator=g)).to(DEVICE)
    decay = torch.empty(tokens, channels, device=DEVICE)
    kernels.exp_decay(wide[:, 6:], bias, decay)
    want = torch.exp(-torch.exp(wide[:, 6:].double() + bias.double())).float()
    torch.testing.assert_close(decay, want, rtol=1e-5, atol=1e-6)
    assert decay.dtype == torch.float32 and float(decay.min()) >= 0.0 and float(decay.max()) <= 1.0
    x = (3 * torch.randn(tokens, 7, generator=g)).to(dtype).to(DEVICE)
    out = torch.empty_like(x)
    kernels.tanh_rows(x, out)
    torch.testing.assert_close(out.float(), torch.tanh(x.float()).to(dtype).float(), **_tolerance(dtype))
    kernels.tanh_rows(x, x)
    assert torch.equal(x, out)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("width", [50, 64, 256, 1000])
def test_a_closing_norm_and_the_next_opening_norm_in_one_pass(width, dtype):
    from rapid_llm_b200.ops import kernels

    g = torch.Generator().manual_seed(width)
    tokens, eps = 19, 1e-6
    y = torch.randn(tokens, width, generator=g).to(dtype).to(DEVICE)
    stream = torch.randn(tokens, width, generator=g).to(DEVICE)
    closing, opening = ((1 + 0.25 * torch.randn(width, generator=g)).to(DEVICE) for _ in range(2))
    rms = lambda x: x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)
    want_stream = stream.double() + rms(y.double()) * closing.double()
    want = rms(want_stream) * opening.double()
    out = torch.empty_like(y)
    kernels.join_then_rmsnorm(y, stream, closing, opening, out, eps)
    torch.testing.assert_close(stream, want_stream.float(), rtol=1e-5, atol=1e-5)       # the stream stays float32
    torch.testing.assert_close(out.float(), want.float().to(dtype).float(), **_tolerance(dtype))


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("tokens,experts,top,hidden", [(50, 8, 4, 64), (7, 5, 2, 50), (33, 1, 1, 32), (20, 4, 4, 40), (64, 40, 3, 48)])
def test_a_router_with_a_bias_and_weights_over_the_chosen(tokens, experts, top, hidden, dtype):
    from rapid_llm_b200.ops import kernels

    g = torch.Generator().manual_seed(experts + top)
    x = torch.randn(tokens, hidden, generator=g).to(dtype).to(DEVICE)
    weight = (torch.randn(experts, hidden, generator=g) / math.sqrt(hidden)).to(torch.bfloat16).float().to(DEVICE)
    bias = (2.0 * torch.randn(experts, generator=g)).to(DEVICE)              # large: it decides many choices
    ids = torch.empty(tokens, top, dtype=torch.int32, device=DEVICE)
    shares = torch.empty(tokens, top, device=DEVICE)
    kernels.router_topk(x, weight, experts=experts, top=top, ids=ids, weights=shares, bias=bias, softmax_chosen=True)
    logits = x.double() @ weight.double().T + bias.double()
    order = torch.sort(logits, dim=-1, descending=True, stable=True).indices[:, :top]
    assert torch.equal(ids.long().cpu(), order.cpu())
    without = torch.sort(x.double() @ weight.double().T, dim=-1, descending=True, stable=True).indices[:, :top]
    assert experts == top or not torch.equal(order, without), "the bias decides nothing in this case"
    want = torch.softmax(torch.gather(logits, 1, order), dim=-1).float()
    torch.testing.assert_close(shares, want, rtol=1e-4, atol=1e-5)
    torch.testing.assert_close(shares.sum(-1), torch.ones(tokens, device=DEVICE), rtol=1e-5, atol=1e-5)


@pytest.mark.parametrize("magnitude_of", ["plain", "stretched"])
def test_the_frequencies_the_engine_rotates_by(magnitude_of):
    """The position parts' frequencies against the closed form, in float64."""
    from rapid_llm_b200.config.model_spec import PartSpec
    from rapid_llm_b200.parts.base import POSITION_ENCODINGS

    dims, base = 16, 100.0
    plain = torch.tensor([base ** (-2.0 * i / dims) for i in range(dims // 2)], dtype=torch.float64)
    if magnitude_of == "plain":
        part = POSITION_ENCODINGS.build(PartSpec("rotary_frequencies", {"rotary_dim": dims, "theta": base, "max_positions": 64}),
                                        dtype=torch.float32, device=DEVICE)
        want, magnitude = plain, 1.0
    else:
        factor, original, fast, slow = 8.0, 64.0, 16.0, 2.0
        part = POSITION_ENCODINGS.build(PartSpec("yarn_frequencies", {"rotary_dim": dims, "theta": base, "max_positions": 64, "factor": factor,
                                                                      "original": original, "fast": fast, "slow": slow}),
                                        dtype=torch.float32, device=DEVICE)
        turn = lambda t: dims * math.log(original / (2 * math.pi * t)) / (2 * math.log(base))
        lo, hi = max(math.floor(turn(fast)), 0), min(math.ceil(turn(slow)), dims - 1)
        ramp = torch.tensor([min(max((i - lo) / max(hi - lo, 0.001), 0.0), 1.0) for i in range(dims // 2)], dtype=torch.float64)
        want, magnitude = plain / factor * ramp + plain * (1 - ramp), 0.1 * math.log(factor) + 1.0
    torch.testing.assert_close(part.inv_freq.cpu().double(), want, rtol=1e-6, atol=0)
    assert float(getattr(part, "magnitude", 1.0)) == pytest.approx(magnitude)
