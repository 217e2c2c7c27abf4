"""tcgen05 GEMM and the fused GEMM + collective kernels against fp32 PyTorch references."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def ref_mm(a, w):
    return a.float() @ w.float().t()


def close(got, ref32, k):
    # bf16 output of an fp32-accumulated product: one rounding of the result (2^-8 relative)
    torch.testing.assert_close(got.float(), ref32, rtol=1.6e-2, atol=2e-2 * (k ** 0.5) * 0.05 + 1e-2)


@pytest.fixture(params=[1, 0], ids=["cta_pair", "single_cta"])
def gemm_kernel(request):
    """Plain GEMMs run on CTA pairs (tcgen05 cta_group::2, 256 x 256 tiles) when M % 256 == 0, else on the
    single-CTA kernel (128 x 256 tiles); both are tested on every shape."""
    from mintccl_b200 import _native as N
    N.lib().mt_gemm_set_pair(request.param)
    yield request.param
    assert N.lib().mt_gemm_pair_error() == 0, "a bounded wait of the CTA-pair GEMM expired"
    N.lib().mt_gemm_set_pair(-1)


@pytest.mark.parametrize("shape", [(128, 256, 64), (256, 256, 64), (256, 512, 128), (384, 256, 1024), (1024, 1792, 4096),
                                   (2048, 4096, 1792), (4096, 2048, 512)])
def test_gemm_matches_fp32_reference(shape, gemm_kernel):
    from mintccl_b200.ops.gemm import gemm
    M, N, K = shape
    g = torch.Generator(device="cuda").manual_seed(M + N + K)
    a = torch.randn(M, K, generator=g, device="cuda").to(torch.bfloat16)
    w = (torch.randn(N, K, generator=g, device="cuda") * 0.02).to(torch.bfloat16)
    out = gemm(a, w)
    torch.cuda.synchronize()
    close(out, ref_mm(a, w), K)
    # a second call on the same stream (fresh barriers, TMEM re-allocated) and fewer CTAs than tiles
    out2 = gemm(a, w, nctas=3)
    torch.cuda.synchronize()
    assert torch.equal(out, out2)


@pytest.mark.parametrize("bn", ["224", "256"])
@pytest.mark.parametrize("shape", [(256, 1792, 128), (2048, 1792, 512), (8192, 1792, 1024)])
def test_gemm_tile_width(shape, bn, monkeypatch):
    """The CTA-pair GEMM with 224-column tiles (chosen by itself when that saves a wave, forced here) against
    the fp32 reference and, bit for bit, against the 256-column tiles."""
    from mintccl_b200 import _native as N
    from mintccl_b200.ops.gemm import gemm
    M, Nn, K = shape
    g = torch.Generator(device="cuda").manual_seed(7 * M + K)
    a = torch.randn(M, K, generator=g, device="cuda").to(torch.bfloat16)
    w = (torch.randn(Nn, K, generator=g, device="cuda") * 0.02).to(torch.bfloat16)
    N.lib().mt_gemm_set_pair(1)
    try:
        monkeypatch.setenv("MINTCCL_GEMM_BN", bn)
        out = gemm(a, w)
        monkeypatch.setenv("MINTCCL_GEMM_BN", "256")
        ref256 = gemm(a, w)
        torch.cuda.synchronize()
        assert N.lib().mt_gemm_pair_error() == 0
    finally:
        N.lib().mt_gemm_set_pair(-1)
    close(out, ref_mm(a, w), K)
    assert torch.equal(out, ref256)


_worlds = {}


def world(n):
    from mintccl_b200 import Config, emulated
    if n not in _worlds:
        cfg = Config.from_env(max_channels=4, num_blocks=4, buff_size=1 << 20, heap_bytes=768 << 20, scratch_bytes=1 << 20,
                              wait_timeout_ms=4000)
        _worlds[n] = emulated(n, 0, cfg)
    return _worlds[n]


@pytest.mark.parametrize("mode", ["push", "fan"])
@pytest.mark.parametrize("n", [1, 2, 4])
@pytest.mark.parametrize("N", [512, 1792])       # 1792: the fused kernel picks 224-column tiles
def test_ag_gemm_emulated(n, mode, N):
    from mintccl_b200.ops.gemm import AllGatherGemm
    w_ = world(n)
    M, K = 128 * n * 2, 256
    plan = AllGatherGemm(w_, M, N, K, ncomm=4, mode=mode)
    for it in range(3):  # counters keep growing across calls
        g = torch.Generator(device="cuda").manual_seed(it)
        shards = [torch.randn(M // n, K, generator=g, device="cuda").to(torch.bfloat16) for _ in range(n)]
        ws = [(torch.randn(N, K, generator=g, device="cuda") * 0.05).to(torch.bfloat16) for _ in range(n)]
        outs = plan(shards, ws)
        w_.check()
        full = torch.cat(shards, 0)
        for r in range(n):
            close(outs[r], ref_mm(full, ws[r]), K)


@pytest.mark.parametrize("n", [1, 2, 4])
def test_gemm_rs_emulated(n):
    from mintccl_b200.ops.gemm import GemmReduceScatter
    w_ = world(n)
    M, N, K = 128 * n * 2, 512, 192
    plan = GemmReduceScatter(w_, M, N, K)
    for it in range(3):
        g = torch.Generator(device="cuda").manual_seed(10 + it)
        As = [torch.randn(M, K, generator=g, device="cuda").to(torch.bfloat16) for _ in range(n)]
        ws = [(torch.randn(N, K, generator=g, device="cuda") * 0.05).to(torch.bfloat16) for _ in range(n)]
        outs = plan(As, ws)
        w_.check()
        # partial products are rounded to bf16 before the fp32 sum over ranks
        ref = sum(ref_mm(a, w).to(torch.bfloat16).float() for a, w in zip(As, ws))
        rows = M // n
        for r in range(n):
            torch.testing.assert_close(outs[r].float(), ref[r * rows:(r + 1) * rows], rtol=2e-2, atol=3e-2)


def test_tp_mlp_forward_backward_single_rank():
    from mintccl_b200.models.tp_mlp import smoke_mlp
    smoke_mlp()


@pytest.mark.parametrize("shape", [(128, 256, 128), (256, 256, 128), (256, 512, 512), (1024, 1792, 4096), (2048, 1024, 1024)])
def test_mxfp8_gemm_matches_dequantised_reference(shape, gemm_kernel):
    """Block-scaled fp8 GEMM against the fp32 product of the dequantised operands (the quantisation error is in
    both; what is compared is the tensor-core arithmetic and the scale plumbing)."""
    from mintccl_b200.ops import mxfp8 as mx
    M, N, K = shape
    g = torch.Generator(device="cuda").manual_seed(M + N + K)
    a = torch.randn(M, K, generator=g, device="cuda") * torch.logspace(-2, 2, M, device="cuda")[:, None]
    w = torch.randn(N, K, generator=g, device="cuda") * 0.02
    ad, asc = mx.quantize_rows_mxfp8(a)
    wd, wsc = mx.quantize_rows_mxfp8(w)
    out = mx.gemm_mxfp8(ad, asc, wd, wsc)
    torch.cuda.synchronize()
    a_dq = mx.dequantize_mxfp8(ad.reshape(-1), asc.reshape(-1)).view(M, K)
    w_dq = mx.dequantize_mxfp8(wd.reshape(-1), wsc.reshape(-1)).view(N, K)
    ref = a_dq @ w_dq.t()
    err = (out.float() - ref).abs()
    tol = 1.6e-2 * ref.abs() + 2e-3 * (a_dq.abs().amax(dim=1, keepdim=True) * (K ** 0.5) * 0.02)
    assert bool((err <= tol).all()), f"max err {err.max().item()} worst ratio {(err / tol).max().item()}"


@pytest.mark.parametrize("n", [1, 2, 4])
def test_fused_kernels_mxfp8_emulated(n):
    from mintccl_b200.ops import mxfp8 as mx
    from mintccl_b200.ops.gemm import AllGatherGemm, GemmReduceScatter
    w_ = world(n)
    M, N, K = 128 * n * 2, 512, 256
    g = torch.Generator(device="cuda").manual_seed(5)
    ag = AllGatherGemm(w_, M, N, K, ncomm=4, fp8=True)
    rs = GemmReduceScatter(w_, M, N, K)
    for it in range(2):
        shards = [torch.randn(M // n, K, generator=g, device="cuda") * (r + 1) for r in range(n)]
        ws = [torch.randn(N, K, generator=g, device="cuda") * 0.05 for _ in range(n)]
        qa = [mx.quantize_rows_mxfp8(t) for t in shards]
        qw = [mx.quantize_rows_mxfp8(t) for t in ws]
        outs = ag.call_mxfp8([q[0] for q in qa], [q[1] for q in qa], [q[0] for q in qw], [q[1] for q in qw])
        w_.check()
        a_dq = torch.cat([mx.dequantize_mxfp8(d.reshape(-1), s.reshape(-1)).view(M // n, K) for d, s in qa], 0)
        for r in range(n):
            w_dq = mx.dequantize_mxfp8(qw[r][0].reshape(-1), qw[r][1].reshape(-1)).view(N, K)
            torch.testing.assert_close(outs[r].float(), a_dq @ w_dq.t(), rtol=2e-2, atol=5e-2)
        As = [torch.randn(M, K, generator=g, device="cuda") for _ in range(n)]
        qA = [mx.quantize_rows_mxfp8(t) for t in As]
        ys = rs.call_mxfp8([q[0] for q in qA], [q[1] for q in qA], [q[0] for q in qw], [q[1] for q in qw])
        w_.check()
        ref = 0
        for r in range(n):
            A_dq = mx.dequantize_mxfp8(qA[r][0].reshape(-1), qA[r][1].reshape(-1)).view(M, K)
            w_dq = mx.dequantize_mxfp8(qw[r][0].reshape(-1), qw[r][1].reshape(-1)).view(N, K)
            ref = ref + (A_dq @ w_dq.t()).to(torch.bfloat16).float()
        rows = M // n
        for r in range(n):
            torch.testing.assert_close(ys[r].float(), ref[r * rows:(r + 1) * rows], rtol=2e-2, atol=6e-2)
