"""Two-rank tests of the NVLink peer gradient exchange (one process per GPU), through the C ABI.
Skipped when fewer than two GPUs are visible."""
import os
import socket

import numpy as np
import pytest

torch = pytest.importorskip("torch")
pytestmark = pytest.mark.gpu

if not torch.cuda.is_available() or torch.cuda.device_count() < 2:
    pytest.skip("needs two CUDA devices", allow_module_level=True)


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    return port


def _worker(rank, world, port, n, out_dir):
    import torch.distributed as dist
    import multigputrainmlp_b200 as mgt
    from multigputrainmlp_b200.comm import PeerBackend
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    os.environ["NCCL_NVLS_ENABLE"] = "0"
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("gloo", rank=rank, world_size=world)  # host rendezvous only
    id_file = os.path.join(out_dir, "peer.id")
    backend = PeerBackend(rank, world, rank, id_file, n)
    grad = backend.gradient_tensor(dev)
    rng = np.random.default_rng(7 + rank)
    w = torch.linspace(-0.1, 0.1, n, device=dev)
    wh = w.half()
    m = torch.zeros(n, device=dev)
    v = torch.zeros(n, device=dev)
    results = {}
    # (offset, count): three tiny vectors in a row (push protocol, both inbox slots, the first unaligned), a small range
    # (handshaken one-shot), a large range (two-shot), everything
    cases = [(3, 225), (7, 1024), (4096, 448), (1000, 50400), (70001, 300007), (0, n)]
    for idx, (off, cnt) in enumerate(cases):
        g = (rng.standard_normal(n) * 1e-3).astype(np.float32)
        grad.copy_(torch.from_numpy(g))
        torch.cuda.synchronize()
        dist.barrier()
        assert backend.allreduce_average(off, cnt) == 0
        st, code = backend.check()
        assert st == 0, code
        results[f"avg_{idx}"] = grad.cpu().numpy().copy()
        results[f"raw_{idx}"] = g
        dist.barrier()
    for step in (1, 2):
        g = (rng.standard_normal(n) * 1e-3).astype(np.float32)
        grad.copy_(torch.from_numpy(g))
        torch.cuda.synchronize()
        dist.barrier()
        cfg = mgt.AdamWKernelConfig(n, step, 1e-3, weight_decay=0.01)
        for off, cnt in ((n - 225, 225), (n // 2, n - 225 - n // 2), (0, n // 2)):
            assert backend.allreduce_average_adamw(off, cnt, cfg, w, wh, m, v) == 0
        st, code = backend.check()
        assert st == 0, code
        results[f"adam_raw_{step}"] = g
        dist.barrier()
    results["w"] = w.cpu().numpy()
    results["wh"] = wh.cpu().numpy()
    results["m"] = m.cpu().numpy()
    results["v"] = v.cpu().numpy()
    np.savez(os.path.join(out_dir, f"rank{rank}.npz"), **results)
    dist.barrier()
    backend.close()
    dist.destroy_process_group()


def test_two_rank_peer_allreduce_and_fused_adamw(tmp_path, oracle):
    import torch.multiprocessing as mp
    n = 1_000_003
    mp.spawn(_worker, args=(2, _free_port(), n, str(tmp_path)), nprocs=2, join=True)
    r = [np.load(tmp_path / f"rank{i}.npz") for i in range(2)]
    cases = [(3, 225), (7, 1024), (4096, 448), (1000, 50400), (70001, 300007), (0, n)]
    for idx, (off, cnt) in enumerate(cases):
        want = oracle.allreduce_average([r[0][f"raw_{idx}"], r[1][f"raw_{idx}"]])
        for rank in range(2):
            got = r[rank][f"avg_{idx}"]
            assert np.array_equal(got[off:off + cnt], want[off:off + cnt])  # same order of additions: bit-exact
            raw = r[rank][f"raw_{idx}"]
            assert np.array_equal(got[:off], raw[:off]) and np.array_equal(got[off + cnt:], raw[off + cnt:])  # untouched outside the range
    w = np.linspace(-0.1, 0.1, n).astype(np.float32)
    w = torch.linspace(-0.1, 0.1, n).numpy().copy()
    m = np.zeros(n, np.float32)
    v = np.zeros(n, np.float32)
    for step in (1, 2):
        avg = oracle.allreduce_average([r[0][f"adam_raw_{step}"], r[1][f"adam_raw_{step}"]])
        assert oracle.adamw(w, avg, m, v, step=step, lr=1e-3, wd=0.01) == 0
    for rank in range(2):
        assert np.abs(r[rank]["w"] - w).max() <= 2e-6      # tolerances of native/tests/cuda/test_cuda_adamw_smoke.cu
        assert np.abs(r[rank]["m"] - m).max() <= 2e-8
        assert np.abs(r[rank]["v"] - v).max() <= 2e-10
        assert np.array_equal(r[rank]["wh"], r[rank]["w"].astype(np.float16))
    assert np.array_equal(r[0]["w"], r[1]["w"])  # replicas stay bit-identical
