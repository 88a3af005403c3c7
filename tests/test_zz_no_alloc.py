"""The split-K GEMM entry point that allocates nothing (its scratch is a buffer inside the library
image) against the ordinary entry point with caller-provided scratch, through the C ABI.

It exists for callers that cannot get device memory of their own: hosts whose memory pool already
owns all of HBM, or loops where the device-wide synchronisation of a cudaMalloc is not acceptable.
Collected last on purpose; passes both alone in a fresh process and after the other tests."""
import ctypes as C

import pytest

torch = pytest.importorskip("torch")
pytestmark = pytest.mark.gpu

if not torch.cuda.is_available():
    pytest.skip("needs a CUDA device", allow_module_level=True)

import multigputrainmlp_b200 as mgt  # noqa: E402
from multigputrainmlp_b200 import _lib  # noqa: E402

DEV = "cuda:0"
STATIC_FLOATS = 4 << 20


def _static_check():
    """mgt_static_scratch_check: (status, device code) of the built-in status word, read and cleared."""
    lib = _lib.load()
    lib.mgt_static_scratch_check.argtypes = [C.c_void_p, C.POINTER(C.c_int32)]
    code = C.c_int32(-1)
    st = int(lib.mgt_static_scratch_check(torch.cuda.current_stream().cuda_stream, C.byref(code)))
    return st, int(code.value)


def _static_gemm(a, lda, a_mn, b, ldb, b_mn, d, m, n, k, splits):
    lib = _lib.load()
    lib.mgt_gemm_split_k_static_scratch.argtypes = [C.c_void_p, C.c_uint32, C.c_int32, C.c_void_p, C.c_uint32, C.c_int32, C.c_void_p,
                                                    C.c_uint32, C.c_uint32, C.c_uint32, C.c_uint32, C.c_void_p]
    stream = torch.cuda.current_stream().cuda_stream
    return int(lib.mgt_gemm_split_k_static_scratch(a.data_ptr(), lda, int(a_mn), b.data_ptr(), ldb, int(b_mn), d.data_ptr(), m, n, k, splits, stream))


def test_static_scratch_gemm_matches_the_ordinary_entry_point_twice_in_a_row():
    torch.cuda.set_device(0)
    engine = mgt.Engine(0)
    # two calls in a row with different shapes and data: the second must not see what the first left behind
    for call, (m, n, k, splits) in enumerate([(225, 224, 8192, 37), (130, 40, 1000, 5)]):
        g = torch.Generator(device=DEV).manual_seed(100 + call)
        a_t = (torch.randn(k, m, device=DEV, generator=g) * 0.5).half()   # A stored [K][M]
        b = (torch.randn(k, n, device=DEV, generator=g) * 0.5).half()     # B stored [K][N]
        lda = (m + 7) // 8 * 8
        ldb = (n + 7) // 8 * 8
        a_buf = torch.zeros(k, lda, device=DEV, dtype=torch.half)
        a_buf[:, :m] = a_t
        b_buf = torch.zeros(k, ldb, device=DEV, dtype=torch.half)
        b_buf[:, :n] = b
        want = torch.full((m, n), float("nan"), device=DEV)
        partial = torch.zeros(splits * m * n, device=DEV)
        assert engine.debug_gemm(a_buf, lda, True, b_buf, ldb, True, want, m, n, k, splits, partial) == 0
        got = torch.full((m, n), float("nan"), device=DEV)
        assert _static_gemm(a_buf, lda, True, b_buf, ldb, True, got, m, n, k, splits) == 0
        assert _static_check() == (0, 0)  # no bounded wait of its kernels gave up
        torch.cuda.synchronize()
        assert torch.isfinite(got).all()
        # same kernels, same order of additions: identical; the tolerance of the GEMM tests is the outer bound
        ref = a_t.float().t() @ b.float()
        assert (got - ref).abs().max().item() <= 2e-3 * max(ref.abs().max().item(), 1.0)
        assert torch.equal(got, want)
    engine.close()


def test_static_scratch_gemm_rejects_what_does_not_fit():
    m, n, k = 2048, 2048, 256
    a = torch.zeros(m, k, device=DEV, dtype=torch.half)
    b = torch.zeros(n, k, device=DEV, dtype=torch.half)
    d = torch.zeros(m, n, device=DEV)
    assert 2 * m * n > STATIC_FLOATS
    assert _static_gemm(a, k, False, b, k, False, d, m, n, k, 2) == 3      # capacity_exceeded
    assert _static_gemm(a, k, False, b, k, False, d, m, n, k, 1) == 0      # a single split needs no scratch
    assert _static_gemm(a, k, False, b, k, False, d, 0, n, k, 1) == 1
    # a single split stores 16-byte vectors straight into d when n is a multiple of 4: a d that is only 4-byte aligned is
    # refused before anything is launched (both entry points share the check)
    flat = torch.zeros(m * n + 4, device=DEV)
    odd = flat[1:1 + m * n]
    assert odd.data_ptr() % 16 == 4
    assert _static_gemm(a, k, False, b, k, False, odd, m, n, k, 1) == 1
    engine = mgt.Engine(0)
    assert engine.debug_gemm(a, k, False, b, k, False, odd, m, n, k, 1, None) == 1
    engine.close()
    assert _static_check() == (0, 0)
    torch.cuda.synchronize()
