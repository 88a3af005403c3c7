"""What a rank sees when a peer does not show up for a gradient exchange: the kernel's bounded wait runs
out, the call chain stays alive, the status says so, and the communicator refuses further work.

The failure is made on the host: rank 1 simply does not launch the collective that rank 0 launches, so the
flag rank 0's kernel polls is one that nothing sets. No kernel faults, traps or spins without a limit; the
absent rank leaves between collectives with nothing in flight. Works on one GPU as well (both processes then
use device 0: only ONE of them ever has a waiting kernel on it)."""
import os
import socket

import numpy as np
import pytest

torch = pytest.importorskip("torch")
pytestmark = pytest.mark.gpu

if not torch.cuda.is_available():
    pytest.skip("needs a CUDA device", allow_module_level=True)


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    return port


def _worker(rank, world, port, out_dir, lonely_count):
    import torch.distributed as dist
    from multigputrainmlp_b200.comm import PeerBackend
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    os.environ["NCCL_NVLS_ENABLE"] = "0"
    device = rank if torch.cuda.device_count() >= world else 0
    torch.cuda.set_device(device)
    dev = torch.device("cuda", device)
    dist.init_process_group("gloo", rank=rank, world_size=world)  # host rendezvous only
    n = 100_000
    backend = PeerBackend(device, world, rank, os.path.join(out_dir, "peer.id"), n)
    grad = backend.gradient_tensor(dev)
    assert backend.set_wait_limit_ms(0) == 1 and backend.set_wait_limit_ms(200) == 0
    # the file rendezvous of the library itself: twice, so that a second round reuses nothing of the first
    assert backend.host_barrier(30000) == 0
    assert backend.host_barrier(30000) == 0
    result = {}
    two_devices = torch.cuda.device_count() >= world
    if two_devices:
        # a complete collective first: both ranks take part, nothing times out
        grad.fill_(float(rank + 1))
        torch.cuda.synchronize()
        dist.barrier()
        assert backend.allreduce_average(0, n) == 0
        st, code = backend.check()
        assert (st, code) == (0, 0)
        result["avg"] = float(grad[17].item())
    dist.barrier()
    if rank == 0:
        grad.fill_(1.0)
        torch.cuda.synchronize()
        t0 = torch.cuda.Event(enable_timing=True)
        t1 = torch.cuda.Event(enable_timing=True)
        t0.record()
        assert backend.allreduce_average(0, lonely_count) == 0   # the launch itself succeeds; the peer never joins
        t1.record()
        st, code = backend.check()
        result["status"], result["code"] = st, code
        result["wait_ms"] = t0.elapsed_time(t1)
        # the context is alive: plain work on the same device still runs
        result["alive"] = float((torch.ones(8, device=dev) * 2).sum().item())
        # ... but this communicator is finished: no launch, same status, also from check()
        result["next_launch"] = backend.allreduce_average(0, lonely_count)
        result["next_check"] = backend.check()[0]
    dist.barrier()  # rank 1 stays (idle, nothing in flight) until rank 0 has seen its status
    np.save(os.path.join(out_dir, f"rank{rank}.npy"), result, allow_pickle=True)
    backend.close()
    dist.destroy_process_group()


# 5000 floats: the handshaken kernels, which give up in their ready wait (code 1); 1000 floats: the push protocol of tiny
# vectors, whose only wait is the one for the peers' vectors (code 3)
@pytest.mark.parametrize("lonely_count,code", [(5000, 1), (1000, 3)])
def test_absent_peer_times_out_into_a_status(tmp_path, lonely_count, code):
    import torch.multiprocessing as mp
    mp.spawn(_worker, args=(2, _free_port(), str(tmp_path), lonely_count), nprocs=2, join=True)
    r0 = np.load(tmp_path / "rank0.npy", allow_pickle=True).item()
    assert r0["status"] == 7 and r0["code"] == code       # MGT_DEVICE_TIMEOUT and the wait that gave up
    assert 150.0 <= r0["wait_ms"] <= 2000.0               # the 200 ms limit, not the 1 s default and not forever
    assert r0["alive"] == 16.0
    assert r0["next_launch"] == 7 and r0["next_check"] == 7
    if "avg" in r0:
        assert r0["avg"] == 1.5
