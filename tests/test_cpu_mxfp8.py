"""MXFP8 host-side arithmetic (pure PyTorch, no GPU): block scales, quantisation error, the scale layout the
tensor core reads.  The GPU kernels are checked against these functions in the gpu-marked tests."""
import pytest
import torch

from mintccl_b200.ops import mxfp8 as mx


def test_scale_is_the_smallest_power_of_two_without_saturation():
    g = torch.Generator().manual_seed(0)
    amax = torch.cat([torch.rand(2000, generator=g) * 10 ** torch.randint(-6, 7, (2000,), generator=g).float(),
                      torch.tensor([448.0, 448.0001, 447.9999, 1.75, 1.7500001, 2.0 ** -20, 3.0e4])])
    s = mx.scale_to_float(mx.scale_for_amax(amax))
    assert bool(((torch.log2(s) % 1) == 0).all())                    # powers of two
    assert bool((amax / s <= 448.0).all())                           # the block's largest value fits e4m3
    assert bool((amax / (s / 2) > 448.0).all())                      # and half the scale would not


def test_zero_block_and_roundtrip_shapes():
    x = torch.zeros(64)
    d, s = mx.quantize_mxfp8(x)
    assert d.dtype == torch.uint8 and s.dtype == torch.uint8 and d.numel() == 64 and s.numel() == 2
    assert int(s[0]) == 127 - 8 and bool((mx.dequantize_mxfp8(d, s) == 0).all())
    with pytest.raises(Exception):
        mx.quantize_mxfp8(torch.zeros(33))                           # blocks of 32


@pytest.mark.parametrize("spread", [1.0, 1e-3, 1e3])
def test_quantisation_error_is_bounded_by_the_block_maximum(spread):
    g = torch.Generator().manual_seed(3)
    x = torch.randn(4096, generator=g) * spread * torch.logspace(-2, 2, 4096 // 32).repeat_interleave(32)
    d, s = mx.quantize_mxfp8(x)
    dq = mx.dequantize_mxfp8(d, s)
    assert bool(torch.isfinite(dq).all())                            # e4m3fn has no infinity; NaN would mean saturation
    amax = x.view(-1, 32).abs().amax(dim=1, keepdim=True)
    err = (dq - x).view(-1, 32).abs()
    # 3 mantissa bits: half an ulp is 2^-4 of the value's binade, at most 2^-4 of the block maximum
    assert bool((err <= amax * 2.0 ** -4 + 1e-30).all())
    # elements near the block maximum keep 2^-4 relative accuracy
    big = x.view(-1, 32).abs() >= amax / 2
    assert bool((err[big] <= x.view(-1, 32).abs()[big] * 2.0 ** -4 * 1.0001).all())


def test_quantise_rows_keeps_blocks_inside_rows():
    g = torch.Generator().manual_seed(5)
    x = torch.randn(8, 96, generator=g)
    x[3] *= 1000.0                                                   # one loud row must not change its neighbours' scales
    d, s = mx.quantize_rows_mxfp8(x)
    assert d.shape == (8, 96) and s.shape == (8, 3)
    d2, s2 = mx.quantize_rows_mxfp8(x[2:3])
    assert torch.equal(d[2:3], d2) and torch.equal(s[2:3], s2)


@pytest.mark.parametrize("rows,k", [(128, 128), (256, 384), (384, 1024)])
def test_tiled_scale_layout_matches_the_documented_formula(rows, k):
    """[rows / 128][K / 128][512] bytes with byte (r % 32) * 16 + ((r % 128) / 32) * 4 + kb % 4 for row r and
    32-element block kb: what tcgen05.cp moves into TMEM for kind::mxf8f6f4.block_scale."""
    kb = k // 32
    scale = torch.arange(rows * kb, dtype=torch.int64).remainder(251).to(torch.uint8).view(rows, kb)
    tiled = mx.tile_scales(scale)
    assert tiled.numel() == rows * kb
    g = torch.Generator().manual_seed(rows + k)
    for _ in range(300):
        r = int(torch.randint(0, rows, (1,), generator=g))
        b = int(torch.randint(0, kb, (1,), generator=g))
        off = ((r // 128) * (k // 128) + b // 4) * 512 + (r % 32) * 16 + ((r % 128) // 32) * 4 + b % 4
        assert int(tiled[off]) == int(scale[r, b]), (r, b)
    with pytest.raises(ValueError):
        mx.tile_scales(torch.zeros(100, 4, dtype=torch.uint8))


def test_sum_of_quantised_tensors_requantises_once():
    """The oracle of the block-scaled all-reduce: dequantise every rank's tensor, add in fp32, quantise the sum
    once.  Its error against the exact sum is that of ONE quantisation of the sum plus the inputs' own."""
    g = torch.Generator().manual_seed(9)
    xs = [torch.randn(2048, generator=g) * (r + 1) for r in range(8)]
    qs = [mx.quantize_mxfp8(x) for x in xs]
    total = sum(mx.dequantize_mxfp8(d, s) for d, s in qs)
    d, s = mx.quantize_mxfp8(total)
    out = mx.dequantize_mxfp8(d, s)
    amax = total.view(-1, 32).abs().amax(dim=1, keepdim=True)
    assert bool(((out - total).view(-1, 32).abs() <= amax * 2.0 ** -4).all())
    exact = sum(xs)
    rel = ((out - exact).norm() / exact.norm()).item()
    assert rel < 0.05
