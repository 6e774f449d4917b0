"""Expert parallelism on 2 GPUs (NCCL): every rank's output must equal what the single-GPU prefill layer computes
for that rank's tokens with the full pool.  Skipped when fewer than two GPUs are visible."""
import copy
import os
import socket

import pytest
import torch

pytestmark = pytest.mark.gpu

D, F, E, K = 1024, 512, 16, 4
ROOT = 0xB2000001


def _worker(rank, world, port, tokens, q):
    import torch.distributed as dist
    from mference_b200 import _lib as L
    from mference_b200.ep import DeviceOps, ExpertParallelLayer
    from mference_b200.moe import MoE, synth_layer, synth_normal
    os.environ["MASTER_ADDR"], os.environ["MASTER_PORT"] = "127.0.0.1", str(port)
    os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
    torch.cuda.set_device(rank)
    import datetime
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank),
                            timeout=datetime.timedelta(seconds=90))
    try:
        T = tokens[rank]
        full = synth_layer(ROOT, 0, D, F, E)
        local_E = E // world
        local = copy.copy(full)
        local.pool = full.pool[rank * local_E * full.slot_stride:(rank + 1) * local_E * full.slot_stride]
        local.shared_blob = None
        shared = copy.copy(full)
        shared.pool, shared.slot_stride, shared.routed_off = full.shared_blob, full.shared_blob.numel(), full.shared_off
        shared.shared_blob = None
        x = synth_normal(ROOT + rank, "x.ep", T * D, dtype=L.DT_BF16).view(T, D)
        ops = DeviceOps(D, F, E, K, world, max_tokens=T, max_recv_rows=sum(tokens) * K)
        layer = ExpertParallelLayer(ops, world)
        y = torch.empty_like(x)
        layer.forward(full, local, shared, x, y)
        ref_moe = MoE(D, F, E, K, max_tokens=T, tensor_core_prefill=True)
        y_ref = torch.empty_like(x)
        ref_moe.encode_layer_prefill(full, x, y_ref)
        torch.cuda.synchronize()
        exact = bool(torch.equal(y, y_ref))
        err = float((y.float() - y_ref.float()).norm() / y_ref.float().norm())
        q.put((rank, exact, err, layer.last_send_counts))
    except Exception as exc:   # report instead of leaving the peer waiting in a collective
        q.put((rank, False, float("inf"), [repr(exc)]))
        os._exit(1)
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("tokens", [(96, 160)])
def test_two_gpu_expert_parallel_layer_equals_single_gpu_layer(tokens):
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    import torch.multiprocessing as mp
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, tokens, q)) for r in range(2)]
    for p in procs:
        p.start()
    results = []
    try:
        for _ in range(2):
            results.append(q.get(timeout=240))
            if results[-1][2] == float("inf"):
                break
    finally:
        if len(results) < 2 or any(r[2] == float("inf") for r in results):
            for p in procs:
                if p.is_alive():
                    p.terminate()
    for p in procs:
        p.join(timeout=60)
    assert len(results) == 2 and all(r[2] != float("inf") for r in results), results
    results.sort()
    for rank, exact, err, send in results:
        assert err <= 1e-6, (rank, err)
        assert exact, rank
        assert sum(send) == tokens[rank] * K
