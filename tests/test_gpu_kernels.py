"""GPU parity tests of the individual kernels, called through the C ABI (ctypes).

GEMM operand forms are pinned against a torch fp32 matmul of the same fp16 inputs; the walk
generator and AdamW against the CPU oracle (bit-exact for the walks)."""
import ctypes as C

import numpy as np
import pytest

torch = pytest.importorskip("torch")
pytestmark = pytest.mark.gpu

if not torch.cuda.is_available():
    pytest.skip("needs a CUDA device", allow_module_level=True)

import multigputrainmlp_b200 as mgt  # noqa: E402
from oracle.binding import WALK_META_DTYPE  # noqa: E402

DEV = "cuda:0"


@pytest.fixture(scope="module")
def engine():
    e = mgt.Engine(0)
    yield e
    e.close()


def _gemm_case(engine, m, n, k, a_mn, b_mn, splits=1, seed=0):
    g = torch.Generator(device=DEV).manual_seed(seed + m * 7 + n * 3 + k)
    a = (torch.randn(m, k, device=DEV, generator=g) * 0.5).half()
    b = (torch.randn(k, n, device=DEV, generator=g) * 0.5).half()
    want = a.float() @ b.float()
    # pitches rounded up to 8 elements so that TMA can address the rows
    def padded(t):
        rows, cols = t.shape
        pitch = (cols + 7) // 8 * 8
        buf = torch.zeros(rows, pitch, device=DEV, dtype=torch.half)
        buf[:, :cols] = t
        return buf, pitch
    a_buf, lda = padded(a.t().contiguous() if a_mn else a)
    b_buf, ldb = padded(b if b_mn else b.t().contiguous())
    d = torch.full((m, n), float("nan"), device=DEV)
    partial = torch.zeros(splits * m * n, device=DEV) if splits > 1 else None
    st = engine.debug_gemm(a_buf, lda, a_mn, b_buf, ldb, b_mn, d, m, n, k, splits, partial)
    assert st == 0, mgt.status_name(st)
    st, code = engine.check()
    assert st == 0, f"device status {code}"
    err = (d - want).abs().max().item()
    scale = want.abs().max().item()
    assert torch.isfinite(d).all(), f"non-finite output for m={m} n={n} k={k} a_mn={a_mn} b_mn={b_mn}"
    assert err <= 2e-3 * max(scale, 1.0), f"m={m} n={n} k={k} a_mn={a_mn} b_mn={b_mn} splits={splits}: max err {err} (scale {scale})"


@pytest.mark.parametrize("a_mn,b_mn", [(False, False), (False, True), (True, True), (True, False)])
def test_gemm_operand_forms_one_tile(engine, a_mn, b_mn):
    _gemm_case(engine, 128, 256, 64, a_mn, b_mn)
    _gemm_case(engine, 128, 256, 256, a_mn, b_mn)


@pytest.mark.parametrize("a_mn,b_mn", [(False, False), (False, True), (True, True), (True, False)])
def test_gemm_ragged_and_multi_tile(engine, a_mn, b_mn):
    _gemm_case(engine, 200, 224, 224, a_mn, b_mn)       # K tail of 32, ragged M
    _gemm_case(engine, 1000, 520, 72, a_mn, b_mn)       # several tiles in M and N, K tail of 8
    _gemm_case(engine, 5, 3, 8, a_mn, b_mn)             # smaller than one MMA in every direction
    _gemm_case(engine, 40000, 224, 96, a_mn, b_mn)      # more tiles than SMs: persistent loop, TMEM double buffering


def test_gemm_split_k(engine):
    _gemm_case(engine, 225, 224, 8192, True, True, splits=37)
    _gemm_case(engine, 130, 40, 1000, True, True, splits=5)


def _walk_gpu(cfg, seed, epoch, step, rank, moves, target):
    n = cfg.sample_count
    d_moves = torch.from_numpy(moves).to(DEV)
    d_target = torch.from_numpy(target).to(DEV)
    states = torch.full((n, 80), 255, dtype=torch.uint8, device=DEV)
    labels = torch.zeros(n, device=DEV)
    meta = torch.zeros(n, 16, dtype=torch.uint8, device=DEV)
    st = mgt.launch_random_walk_kernel(cfg, seed, epoch, step, rank, d_moves, d_target, states, labels, meta)
    assert st == 0
    torch.cuda.synchronize()
    return states.cpu().numpy(), labels.cpu().numpy(), meta.cpu().numpy().view(WALK_META_DTYPE).reshape(-1)


def test_walks_bit_exact_against_golden_and_oracle(oracle, golden):
    w = golden.walks
    moves, target = w["moves"], w["target"]
    for idx, (seed, epoch, step, rank, kmin, kmax, n) in enumerate(w["cases"]):
        cfg = mgt.RandomWalkKernelConfig(int(n), int(kmin), int(kmax))
        states, labels, meta = _walk_gpu(cfg, int(seed), int(epoch), int(step), int(rank), moves, target)
        assert np.array_equal(states, w[f"states_{idx}"])
        assert np.array_equal(labels, w[f"labels_{idx}"])
        assert np.array_equal(meta["depth"], w[f"depth_{idx}"])
        assert np.array_equal(meta["last_move"], w[f"last_move_{idx}"])
        assert np.array_equal(meta["rng_counter"], w[f"rng_{idx}"])
    # full batch of the headline configuration, and a smaller puzzle (11 moves on 31 positions)
    for (n, sl, mc, kmin, kmax, seed, step, rank) in ((53248, 72, 18, 1, 29, 1234, 199, 7), (1234, 31, 11, 2, 5, 99, 3, 1), (1, 72, 18, 29, 29, 5, 0, 0)):
        mv, tg = oracle.cyclic_puzzle(sl, mc)
        cfg = mgt.RandomWalkKernelConfig(n, kmin, kmax, mc, sl, 80)
        states, labels, meta = _walk_gpu(cfg, seed, 0, step, rank, mv, tg)
        st, s2, l2, m2 = oracle.random_walks(mv, tg, seed=seed, epoch=0, step=step, rank=rank, k_min=kmin, k_max=kmax, samples=n,
                                             move_count=mc, state_len=sl)
        assert st == 0
        assert np.array_equal(states, s2) and np.array_equal(labels, l2) and np.array_equal(meta, m2)
        assert (states[:, sl:] == 0).all()


def test_walk_config_errors():
    # native/cuda/random_walk_kernel.cu:68-76
    ok = mgt.RandomWalkKernelConfig(8, 1, 9)
    assert mgt.validate_random_walk_kernel_config(ok) == 0
    for bad in (mgt.RandomWalkKernelConfig(0, 1, 9), mgt.RandomWalkKernelConfig(8, 0, 9), mgt.RandomWalkKernelConfig(8, 9, 1),
                mgt.RandomWalkKernelConfig(8, 1, 9, 19), mgt.RandomWalkKernelConfig(8, 1, 9, 18, 73), mgt.RandomWalkKernelConfig(8, 1, 9, 18, 72, 71),
                mgt.RandomWalkKernelConfig(8, 1, 9, 18, 72, 81)):
        assert mgt.validate_random_walk_kernel_config(bad) == 1
    assert mgt.launch_random_walk_kernel(ok, 1, 0, 0, 0, None, None, None, None, None) == 1
    # the kernel reads the puzzle as words and writes states as 16-byte vectors: arrays that are not aligned for that are
    # refused before anything is launched
    raw = torch.zeros(18 * 80 + 80 + 16, dtype=torch.uint8, device=DEV)
    states = torch.zeros(8 * 80 + 16, dtype=torch.uint8, device=DEV)
    labels = torch.zeros(8, device=DEV)
    meta = torch.zeros(8 * 16, dtype=torch.uint8, device=DEV)
    assert mgt.launch_random_walk_kernel(ok, 1, 0, 0, 0, raw[:1440], raw[1440:1520], states[:640], labels, meta) == 0
    assert mgt.launch_random_walk_kernel(ok, 1, 0, 0, 0, raw[1:1441], raw[1444:1524], states[:640], labels, meta) == 1
    assert mgt.launch_random_walk_kernel(ok, 1, 0, 0, 0, raw[:1440], raw[1442:1522], states[:640], labels, meta) == 1
    assert mgt.launch_random_walk_kernel(ok, 1, 0, 0, 0, raw[:1440], raw[1440:1520], states[8:648], labels, meta) == 1
    torch.cuda.synchronize()


def test_adamw_against_oracle(oracle):
    # tolerances of native/tests/cuda/test_cuda_adamw_smoke.cu:43-81
    rng = np.random.default_rng(5)
    for n, mirror in ((1024, False), (1024, True), (1000003, True), (7, True)):
        w = (rng.standard_normal(n) * 0.1).astype(np.float32)
        m = np.zeros(n, np.float32)
        v = np.zeros(n, np.float32)
        dw, dm, dv = (torch.from_numpy(x.copy()).to(DEV) for x in (w, m, v))
        dh = torch.zeros(n, dtype=torch.half, device=DEV)
        for step in (1, 2, 3):
            g = (rng.standard_normal(n) * 1e-3).astype(np.float32)
            wd = 0.01 if step == 3 else 0.0
            assert oracle.adamw(w, g, m, v, step=step, lr=1e-3, wd=wd) == 0
            cfg = mgt.AdamWKernelConfig(n, step, 1e-3, weight_decay=wd)
            dg = torch.from_numpy(g).to(DEV)
            st = mgt.launch_adamw_kernel_with_half_mirror(cfg, dw, dh, dg, dm, dv) if mirror else mgt.launch_adamw_kernel(cfg, dw, dg, dm, dv)
            assert st == 0
            torch.cuda.synchronize()
            assert np.abs(dw.cpu().numpy() - w).max() <= 2e-6
            assert np.abs(dm.cpu().numpy() - m).max() <= 2e-8
            assert np.abs(dv.cpu().numpy() - v).max() <= 2e-10
            if mirror:
                assert torch.equal(dh, dw.half())
    assert mgt.validate_adamw_kernel_config(mgt.AdamWKernelConfig(0, 1, 1e-3)) == 1
    assert mgt.validate_adamw_kernel_config(mgt.AdamWKernelConfig(8, 0, 1e-3)) == 1
    assert mgt.validate_adamw_kernel_config(mgt.AdamWKernelConfig(8, 1, 0.0)) == 1
    assert mgt.validate_adamw_kernel_config(mgt.AdamWKernelConfig(8, 1, 1e-3, beta1=1.0)) == 1



def test_adamw_zero_and_denormal_gradients(oracle):
    """Exact zeros (dead units, padding columns) are the common case in a real gradient and the kernel treats them apart
    from the correctly rounded division and square root: a parameter whose gradient and moments are zero must not move,
    signed zeros and denormals must come out as the plain operations give them (the oracle's CpuAdamWStep restatement)."""
    rng = np.random.default_rng(11)
    n = 100003
    kinds = rng.integers(0, 6, n)
    g0 = (rng.standard_normal(n) * 1e-3).astype(np.float32)
    special = np.array([0.0, -0.0, 1e-41, -3e-39, 1e-20], np.float32)
    g = np.where(kinds < 5, special[np.minimum(kinds, 4)], g0).astype(np.float32)
    w = (rng.standard_normal(n) * 0.1).astype(np.float32)
    w0 = w.copy()
    m = np.zeros(n, np.float32)
    v = np.zeros(n, np.float32)
    dw, dm, dv, dg = (torch.from_numpy(x.copy()).to(DEV) for x in (w, m, v, g))
    dh = torch.zeros(n, dtype=torch.half, device=DEV)
    for step in (1, 2, 3):
        assert oracle.adamw(w, g, m, v, step=step, lr=1e-3, wd=0.0) == 0
        assert mgt.launch_adamw_kernel_with_half_mirror(mgt.AdamWKernelConfig(n, step, 1e-3), dw, dh, dg, dm, dv) == 0
        torch.cuda.synchronize()
        gw, gm, gv = dw.cpu().numpy(), dm.cpu().numpy(), dv.cpu().numpy()
        assert np.isfinite(gw).all() and np.isfinite(gm).all() and np.isfinite(gv).all()
        assert np.abs(gw - w).max() <= 2e-6
        assert np.abs(gm - m).max() <= 2e-8
        assert np.abs(gv - v).max() <= 2e-10
        zero = kinds < 2
        assert np.array_equal(gw[zero].view(np.uint32), w0[zero].view(np.uint32))
        assert not gm[zero].any() and not gv[zero].any()
        assert torch.equal(dh, dw.half())
