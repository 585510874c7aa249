"""The allocation-free BitLinear entry point (mmf_bitlinear_gemv_static), called through the C ABI.

It serves hosts that cannot allocate device memory when they run a decode step (a serving process whose
memory arena is planned once and owned by another runtime, or a loop where allocation is forbidden): its
split-K scratch is a fixed array inside the library.  The test checks it against the ordinary entry point
(mmf_bitlinear with a caller-provided workspace), bit for bit, on two calls in a row — the second call finds
the array as the first one left it.  The file name sorts last so that a failure here cannot hide any other
test's result in a run that stops at the first failure."""
import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu

STATIC_SCRATCH_BYTES = 1 << 20


def _p(t):
    return ctypes.c_void_p(t.data_ptr())


def _call_static(lib_mod, q, dq, rs, pw, out):
    M = q.shape[0] // pw.groups
    lib_mod.call("mmf_bitlinear_gemv_static", _p(q), _p(dq), _p(rs), _p(pw.packed), _p(pw.scale), pw.groups, _p(out),
                 lib_mod.BF16 if out.dtype == torch.bfloat16 else lib_mod.F32, out.stride(0), M, pw.N, pw.K,
                 ctypes.c_void_p(torch.cuda.current_stream().cuda_stream))


@pytest.mark.parametrize("M,K,N,groups", [(1, 2048, 2048, 1), (3, 2048, 11264, 1), (4, 704, 256, 1), (2, 256, 768, 3)])
def test_static_scratch_matches_workspace_entry_point(M, K, N, groups):
    from matmulfreellm_b200 import _lib, kernels
    assert torch.cuda.is_available()
    g = torch.Generator().manual_seed(M * 1000 + N)
    n_each = N // groups
    pws = [kernels.pack_weight((torch.randn(n_each, K, generator=g) * 0.02).cuda()) for _ in range(groups)]
    pw = pws[0] if groups == 1 else kernels.stack_packed(pws)
    x = torch.randn(M, K, generator=g).bfloat16().cuda()
    parts = [kernels.act_quant(x, (1.0 + 0.1 * torch.randn(K, generator=g)).cuda(), 1e-6) for _ in range(groups)]
    q = torch.cat([p[0] for p in parts]); dq = torch.cat([p[1] for p in parts]); rs = torch.cat([p[2] for p in parts])
    for dtype in (torch.float32, torch.bfloat16):
        want = kernels.bitlinear(q, dq, rs, pw, dtype, kernel=kernels.KERNEL_GEMV)     # existing entry point
        first = torch.full((M, N), float("nan"), dtype=dtype, device="cuda")
        second = torch.full((M, N), float("nan"), dtype=dtype, device="cuda")
        _call_static(_lib, q, dq, rs, pw, first)
        _call_static(_lib, q, dq, rs, pw, second)      # runs on the array as the first call left it
        torch.cuda.synchronize()
        assert torch.equal(first, want) and torch.equal(second, want)


def test_static_scratch_rejects_oversize_and_bad_arguments():
    from matmulfreellm_b200 import _lib, kernels
    lib = _lib.load()
    M, K, N = 8, 2048, 32000                      # needs more split-K scratch than the built-in array holds
    assert lib.mmf_bitlinear_workspace_bytes(M, N, K) > STATIC_SCRATCH_BYTES
    pw = kernels.pack_weight((torch.randn(N, K) * 0.02).cuda())
    q, dq, rs = kernels.act_quant(torch.randn(M, K).bfloat16().cuda(), None, 1e-6)
    out = torch.zeros(M, N, dtype=torch.bfloat16, device="cuda")
    with pytest.raises(_lib.MMFreeError) as e:
        _call_static(_lib, q, dq, rs, pw, out)
    assert e.value.code == -6 and "built-in array" in str(e.value)
    assert int(out.abs().sum()) == 0              # nothing was launched
    with pytest.raises(_lib.MMFreeError) as e:    # null pointer
        _lib.call("mmf_bitlinear_gemv_static", None, _p(dq), _p(rs), _p(pw.packed), _p(pw.scale), 1, _p(out), _lib.BF16, N, 1,
                  N, K, None)
    assert e.value.code == -1
