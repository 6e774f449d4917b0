"""Expert parallelism (2, 4 or 8 GPUs; both forms of the exchange): every rank's output must equal what the single-GPU
prefill layer computes for that rank's tokens with the full pool.  Multi-rank cases are skipped when too few GPUs are
visible; the one-rank case of the peer-memory exchange (a rank storing into its own buffers) runs on one GPU."""
import copy
import os
import socket

import pytest
import torch

pytestmark = pytest.mark.gpu

D, F, E, K = 1024, 512, 16, 4
ROOT = 0xB2000001


def _worker(rank, world, port, tokens, q, kind="nccl"):
    import torch.distributed as dist
    from mference_b200 import _lib as L
    from mference_b200.ep import DeviceOps, ExpertParallelLayer, PeerExpertParallelLayer
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
        if kind == "peer":
            ops = DeviceOps(D, F, E, K, world, max_tokens=T, max_recv_rows=world * max(tokens) * K)
            layer = PeerExpertParallelLayer(ops, rank, world, max(tokens))
        else:
            ops = DeviceOps(D, F, E, K, world, max_tokens=T, max_recv_rows=sum(tokens) * K)
            layer = ExpertParallelLayer(ops, world)
        y = torch.empty_like(x)
        layer.forward(full, local, shared, x, y)
        if kind == "peer":   # a second layer call through the same buffers, as a stack of layers would make
            y2 = torch.empty_like(x)
            layer.forward(full, local, shared, x, y2)
            torch.cuda.synchronize()
            assert torch.equal(y, y2)
            # and as a CUDA graph, replayed twice (every rank replays the same number of times)
            xg, yg = torch.empty_like(x), torch.empty_like(x)
            layer.capture(full, local, shared, xg, yg)
            for _ in range(2):
                xg.copy_(x)
                layer.replay()
                torch.cuda.synchronize()
                assert torch.equal(y, yg)
            st, counts = layer.ex.status(with_counts=True)
            assert st == 0, st
        ref_moe = MoE(D, F, E, K, max_tokens=T, tensor_core_prefill=True)
        y_ref = torch.empty_like(x)
        ref_moe.encode_layer_prefill(full, x, y_ref)
        torch.cuda.synchronize()
        exact = bool(torch.equal(y, y_ref))
        err = float((y.float() - y_ref.float()).norm() / y_ref.float().norm())
        q.put((rank, exact, err, layer.last_send_counts if kind == "nccl" else [T * K]))
    except Exception as exc:   # report instead of leaving the peer waiting in a collective
        q.put((rank, False, float("inf"), [repr(exc)]))
        os._exit(1)
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("kind,tokens", [("nccl", (96, 160)), ("peer", (96, 160)), ("peer", (64, 40, 96, 8)),
                                         ("nccl", (64, 40, 96, 8)), ("peer", (24, 48, 8, 40, 16, 56, 32, 64))])
def test_expert_parallel_layer_equals_single_gpu_layer(kind, tokens):
    world = len(tokens)
    if torch.cuda.device_count() < world:
        pytest.skip(f"needs {world} GPUs")
    import torch.multiprocessing as mp
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=_worker, args=(r, world, port, tokens, q, kind)) for r in range(world)]
    for p in procs:
        p.start()
    results = []
    try:
        for _ in range(world):
            results.append(q.get(timeout=240))
            if results[-1][2] == float("inf"):
                break
    finally:
        if len(results) < world or any(r[2] == float("inf") for r in results):
            for p in procs:
                if p.is_alive():
                    p.terminate()
    for p in procs:
        p.join(timeout=60)
    assert len(results) == world and all(r[2] != float("inf") for r in results), results
    results.sort()
    for rank, exact, err, send in results:
        assert err <= 1e-6, (rank, err)
        assert exact, rank
        assert sum(send) == tokens[rank] * K


def test_peer_exchange_with_one_rank_equals_the_prefill_layer():
    """The one-sided exchange with a single rank (it stores into its own buffers): dispatch, receive, grouped FFN with a
    destination address per row, return, results and combine give the single-GPU prefill layer bit for bit - twice in a
    row through the same buffers, with a 2-bit expert pool and a 4-bit shared expert the second time."""
    import copy
    from mference_b200 import _lib as L
    from mference_b200.ep import DeviceOps, PeerExpertParallelLayer
    from mference_b200.moe import MoE, synth_layer, synth_normal
    for bits, d, f, e, k, T in ((4, D, F, E, K, 72), (2, 1024, 1024, 8, 3, 50)):
        full = synth_layer(ROOT, 0, d, f, e, bits=bits, shared_bits=4)
        local = copy.copy(full)
        local.shared_blob = None
        shared = copy.copy(full)
        shared.pool, shared.slot_stride, shared.routed_off = full.shared_blob, full.shared_blob.numel(), full.shared_off
        shared.shared_blob = None
        x = synth_normal(ROOT, "x.ep1", T * d, dtype=L.DT_BF16).view(T, d)
        ops = DeviceOps(d, f, e, k, 1, max_tokens=T, max_recv_rows=T * k, bits=bits, shared_bits=4)
        layer = PeerExpertParallelLayer(ops, 0, 1, T)
        ref_moe = MoE(d, f, e, k, bits=bits, shared_bits=4, max_tokens=T, tensor_core_prefill=True)
        y_ref = torch.empty_like(x)
        ref_moe.encode_layer_prefill(full, x, y_ref)
        for _ in range(2):
            y = torch.empty_like(x)
            layer.forward(full, local, shared, x, y)
            torch.cuda.synchronize()
            assert torch.equal(y, y_ref)
        # the same layer recorded into a CUDA graph and replayed on other rows (the epoch advances on the device)
        xg, yg = torch.empty_like(x), torch.empty_like(x)
        layer.capture(full, local, shared, xg, yg)
        for seed in (1, 2):
            x2 = synth_normal(ROOT + seed, "x.ep1", T * d, dtype=L.DT_BF16).view(T, d)
            xg.copy_(x2)
            layer.replay()
            ref_moe.encode_layer_prefill(full, x2, y_ref)
            torch.cuda.synchronize()
            assert torch.equal(yg, y_ref)
        st, counts = layer.ex.status(with_counts=True)
        assert st == 0 and counts == [T * k]
        assert ref_moe.device_status() == 0 and ops.expert.device_status() == 0
