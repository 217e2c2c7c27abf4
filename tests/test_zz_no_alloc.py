"""The allocation-free entry point (``mt_gemm_rs_single_noalloc``), called through its exported C symbol.

Some hosts may not allocate device memory while they run (a serving loop with a fixed memory plan, a
plugin inside somebody else's process, a caller whose own allocator already owns the whole device).  For
them the library offers one entry point whose scratch memory is a fixed array inside the library image.
This test checks it against the regular entry point (``mt_gemm_rs`` on a one-rank communicator), twice in
a row because the built-in scratch keeps the previous call's contents, and checks that a problem larger
than the scratch is refused with a clear message.  The file sorts last so that a run that stops at the
first failure has already run everything else.
"""
import ctypes as C

import pytest
import torch

pytestmark = pytest.mark.gpu


def _entry():
    from mintccl_b200 import _native as N
    lib = N.lib()
    fn = lib.mt_gemm_rs_single_noalloc
    fn.restype = C.c_int
    fn.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_int, C.c_int, C.c_int]
    st = lib.mt_gemm_rs_single_noalloc_status
    st.restype = C.c_int
    st.argtypes = [C.POINTER(N.MtStatus), C.c_int]
    return N, fn, st


def test_noalloc_entry_matches_regular_entry_twice():
    import mintccl_b200
    from mintccl_b200 import Config
    from mintccl_b200.ops.gemm import GemmReduceScatter
    N, fn, status = _entry()
    torch.cuda.set_device(0)
    cfg = Config.from_env(max_channels=2, num_blocks=2, buff_size=1 << 20, heap_bytes=128 << 20, scratch_bytes=1 << 20,
                          wait_timeout_ms=4000)
    world = mintccl_b200.emulated(1, 0, cfg)   # one rank: the regular entry point with its heap scratch
    try:
        for M, Nn, K in [(256, 512, 192), (1024, 2048, 512)]:
            plan = GemmReduceScatter(world, M, Nn, K)
            for it in range(2):  # two calls in a row on the same scratch
                g = torch.Generator(device="cuda").manual_seed(100 * it + M)
                a = torch.randn(M, K, generator=g, device="cuda").to(torch.bfloat16)
                w = (torch.randn(Nn, K, generator=g, device="cuda") * 0.05).to(torch.bfloat16)
                want = plan([a], [w])[0]
                got = torch.full((M, Nn), float("nan"), device="cuda", dtype=torch.bfloat16)
                stream = torch.cuda.current_stream().cuda_stream
                rc = fn(stream, a.data_ptr(), w.data_ptr(), got.data_ptr(), M, Nn, K)
                assert rc == 0, N.last_error()
                torch.cuda.synchronize()
                world.check()                       # the regular entry point's communicator
                own = N.MtStatus()                  # the entry point's own record, in its built-in array
                assert status(C.byref(own), 0) == 0, N.last_error()
                assert own.code == 0 and own.abort == 0, (own.code, own.where, own.expected, own.seen)
                torch.testing.assert_close(got.float(), want.float(), rtol=1.6e-2, atol=2e-2)
                ref = (a.float() @ w.float().t())
                torch.testing.assert_close(got.float(), ref, rtol=2e-2, atol=3e-2)
            world.symm_free(plan.stage)
            world.symm_free(plan.flags)
    finally:
        world.close()


def test_noalloc_entry_rejects_sizes_beyond_its_scratch():
    N, fn, _ = _entry()
    x = torch.zeros(16, device="cuda", dtype=torch.bfloat16)
    assert fn(0, x.data_ptr(), x.data_ptr(), x.data_ptr(), 4096, 256, 64) == -1
    assert "exceeds the built-in scratch" in N.last_error()
    assert fn(0, x.data_ptr(), x.data_ptr(), x.data_ptr(), 128, 4096, 64) == -1
    assert "exceeds the built-in scratch" in N.last_error()
    assert fn(0, x.data_ptr(), x.data_ptr(), x.data_ptr(), 100, 256, 64) == -1
