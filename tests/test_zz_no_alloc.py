"""The allocation-free GEMM entry point (vla_op_gemm_noalloc) against the allocating one (vla_op_gemm).

Some users of this library run it where device allocation is off limits: inside a robot's real-time control
loop with a fixed memory budget, or from a thread that must never block on the allocator.  For them the
library offers one GEMM call whose split-K scratch lives in a static device array instead of cudaMalloc'd
memory.  This test drives it through the C ABI twice in a row (the scratch keeps the previous call's
contents, so the second call also shows that stale partial tiles do no harm) and expects the same bf16
output as the existing entry point: both run the same kernel with the same fixed-order reduction, so the
tolerance of the other GEMM tests (bf16 rounding, 6e-3 relative) is met with room to spare.

Collected last on purpose, so that a run stopping at the first failure has already run every other test."""
import ctypes as C

import pytest
import torch

pytestmark = pytest.mark.gpu


def _call(lib, capi, x, w_nk, N, bias, out, split):
    d = capi.GemmNoAllocDesc()
    d.x, d.tokens, d.K = x.data_ptr(), x.shape[0], x.shape[1]
    d.w_nk, d.N, d.n_pad, d.k_pad = w_nk.data_ptr(), N, w_nk.shape[0], w_nk.shape[1]
    d.bias, d.out_bf16, d.split = bias.data_ptr(), out.data_ptr(), split
    return lib.vla_op_gemm_noalloc(C.byref(d), None)


@pytest.mark.parametrize("tokens,K,N,split", [(51, 2048, 1024, 8), (51, 1024, 2560, 4), (200, 1152, 1152, 2),
                                              (512, 4352, 1152, 0)])   # split 0: the library's choice, cut down to fit
def test_noalloc_matches_allocating_entry_point(tokens, K, N, split):
    if not torch.cuda.is_available():
        pytest.skip("needs a GPU")
    import _capi
    import vla_ops
    lib = _capi.lib()
    dev = torch.device("cuda")
    g = torch.Generator().manual_seed(77)
    x = torch.randn(tokens, K, generator=g).to(torch.bfloat16).to(dev)
    w = (torch.randn(K, N, generator=g) * 0.05).to(torch.bfloat16).to(dev)
    bias = torch.randn(N, generator=g).to(dev)
    want = vla_ops.gemm(x, w, bias=bias, split=split)                # existing entry point (allocates)
    n_pad, k_pad = (N + 127) // 128 * 128, (K + 63) // 64 * 64
    w_nk = torch.zeros(n_pad, k_pad, dtype=torch.bfloat16, device=dev)
    w_nk[:N, :K] = w.t()
    ref = x.float() @ w.float() + bias
    for call in range(2):                                            # two calls in a row share the scratch
        out = torch.full((tokens, N), float("nan"), dtype=torch.bfloat16, device=dev)
        rc = _call(lib, _capi, x, w_nk, N, bias, out, split)
        assert rc == 0, lib.vla_last_error(None)
        torch.cuda.synchronize()
        assert torch.isfinite(out.float()).all()
        err = (out.float() - want.float()).abs().max().item()
        assert err <= 6e-3 * want.float().abs().max().item(), "call %d: differs from vla_op_gemm by %g" % (call, err)
        assert (out.float() - ref).abs().max().item() <= 6e-3 * ref.abs().max().item()
    # no bounded wait ran out inside the kernel: the status word (also a static device symbol) reads zero
    word = C.c_int(-1)
    assert lib.vla_op_gemm_noalloc_status(C.byref(word)) == 0
    assert word.value == 0


def test_noalloc_rejects_oversized_shapes():
    if not torch.cuda.is_available():
        pytest.skip("needs a GPU")
    import _capi
    lib = _capi.lib()
    dev = torch.device("cuda")
    # 788 tokens x 16384 features split 2: far more partial tiles than the 4 MiB built-in scratch holds
    x = torch.zeros(788, 2048, dtype=torch.bfloat16, device=dev)
    w_nk = torch.zeros(16384, 2048, dtype=torch.bfloat16, device=dev)
    bias = torch.zeros(16384, device=dev)
    out = torch.zeros(788, 16384, dtype=torch.bfloat16, device=dev)
    rc = _call(lib, _capi, x, w_nk, 16384, bias, out, 2)
    assert rc == 5                                                   # VLA_ERR_LIMIT
    assert b"scratch" in lib.vla_last_error(None)
