"""Host logic of the expert-parallel layer on CPU: two `gloo` ranks run ExpertParallelLayer.forward with stand-in
compute steps (plain torch on CPU, defined here - the product only ever uses the CUDA ones) and the result must
equal a direct evaluation; this pins the send order, the split sizes and the reversed exchange."""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from mference_b200.ep import ExpertParallelLayer

E, K, D, WORLD = 8, 2, 16, 2


class FakeOps:
    """Expert e multiplies a row by (e + 1); routing and weights are fixed functions of the token index."""

    def __init__(self, rank, world):
        self.rank, self.world, self.local_E = rank, world, E // world

    def route(self, weights, h):
        T = h.shape[0]
        t = torch.arange(T) + 100 * self.rank
        idx = torch.stack([(t * 3 + 1) % E, (t * 5 + 2) % E], dim=1).to(torch.int32)
        w = torch.stack([torch.full((T,), 0.75), torch.full((T,), 0.25)], dim=1).to(torch.float16)
        return h, idx, w

    def plan(self, idx):
        flat = idx.reshape(-1).to(torch.int64)
        dest = flat // self.local_E
        perm = torch.sort(dest, stable=True).indices
        inv = torch.empty_like(perm)
        inv[perm] = torch.arange(perm.numel())
        counts = torch.bincount(dest, minlength=self.world).to(torch.int32)
        local_expert = (flat[perm] - dest[perm] * self.local_E).to(torch.int32)
        return perm.to(torch.int32), inv.to(torch.int32), counts, local_expert

    def pack(self, xn, perm):
        return xn[(perm.to(torch.int64) // K)]

    def expert_ffn(self, local_weights, rows, local_expert):
        scale = (local_expert.to(torch.float32) + self.rank * self.local_E + 1.0).unsqueeze(1)
        return rows.to(torch.float32) * scale

    def shared_ffn(self, shared_weights, xn):
        return xn.to(torch.float32) * 0.5

    def combine(self, recv, inv, w, shared_partial, residual, y):
        T = w.shape[0]
        acc = residual.to(torch.float32).clone()
        if shared_partial is not None:
            acc += shared_partial
        for k in range(K):
            acc += w[:, k].to(torch.float32).unsqueeze(1) * recv[inv.to(torch.int64)[torch.arange(T) * K + k]]
        y.copy_(acc.to(y.dtype))


def _worker(rank, port, tokens, out_queue):
    os.environ["MASTER_ADDR"], os.environ["MASTER_PORT"] = "127.0.0.1", str(port)
    dist.init_process_group("gloo", rank=rank, world_size=WORLD)
    try:
        T = tokens[rank]
        h = (torch.arange(T * D, dtype=torch.float32).view(T, D) / 64.0 + rank).to(torch.bfloat16)
        layer = ExpertParallelLayer(FakeOps(rank, WORLD), WORLD)
        y = torch.empty_like(h)
        layer.forward(None, None, object(), h, y)
        # direct evaluation
        _, idx, w = FakeOps(rank, WORLD).route(None, h)
        ref = h.to(torch.float32) * 1.5
        for k in range(K):
            ref += w[:, k].to(torch.float32).unsqueeze(1) * h.to(torch.float32) * (idx[:, k].to(torch.float32) + 1.0).unsqueeze(1)
        ok = torch.equal(y, ref.to(torch.bfloat16))
        out_queue.put((rank, ok, layer.last_send_counts, layer.last_recv_counts))
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("tokens", [(5, 9), (0, 7)])
def test_two_rank_exchange_matches_direct_evaluation(tokens):
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=_worker, args=(r, port, tokens, q)) for r in range(WORLD)]
    for p in procs:
        p.start()
    results = sorted(q.get(timeout=120) for _ in range(WORLD))
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    assert all(ok for _, ok, _, _ in results)
    # what rank 0 sends to rank 1 is what rank 1 receives from rank 0, and vice versa
    (_, _, send0, recv0), (_, _, send1, recv1) = results
    assert send0[1] == recv1[0] and send1[0] == recv0[1]
    assert sum(send0) == tokens[0] * K and sum(send1) == tokens[1] * K
