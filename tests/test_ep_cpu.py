"""Expert-parallel exchange logic on CPU: two gloo ranks, a stand-in local layer, results equal to the one-rank layer."""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

E, H, TOPK = 8, 16, 3


class ToyLayer:
    """out[t] = sum over resident picks of rw * (x[t] * (e + 1) + e); non-resident experts (level 0) add nothing"""

    def __init__(self, resident):
        self.E, self.H, self.resident = E, H, set(resident)

    def _run(self, x, sel, rw):
        out = torch.zeros(x.shape[0], H, dtype=torch.float32)
        for t in range(x.shape[0]):
            for k in range(sel.shape[1]):
                e, w = int(sel[t, k]), float(rw[t, k])
                if e in self.resident and w != 0:
                    out[t] += w * (x[t].float() * (e + 1) + e)
        return out

    __call__ = _run
    prefill = _run


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, q):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from nestquant_b200.ep import EPLayer, owned_experts
    g = torch.Generator().manual_seed(5)
    T = 10
    x_all = torch.randn(world, T, H, generator=g).half()
    sel_all = torch.stack([torch.stack([torch.randperm(E, generator=g)[:TOPK] for _ in range(T)]) for _ in range(world)])
    rw_all = torch.softmax(torch.randn(world, T, TOPK, generator=g), -1).half()
    rw_all[0, 3, 1] = 0
    ep = EPLayer(ToyLayer(owned_experts(E, world, rank)), rank, world)
    full = ToyLayer(range(E))
    got = ep.prefill(x_all[rank], sel_all[rank], rw_all[rank])
    want = full.prefill(x_all[rank], sel_all[rank], rw_all[rank])
    ok_prefill = torch.allclose(got, want, rtol=1e-5, atol=1e-4)
    # every token row travels at most once per destination rank
    ok_stats = ep.last_stats["sent_rows"] <= T * min(TOPK, world)
    # decode: replicated tokens, all-reduced partial outputs
    y = ep.decode(x_all[0, :4], sel_all[0, :4], rw_all[0, :4])
    ok_decode = torch.allclose(y, full(x_all[0, :4], sel_all[0, :4], rw_all[0, :4]), rtol=1e-5, atol=1e-4)
    q.put((rank, ok_prefill, ok_stats, ok_decode))
    dist.barrier()
    dist.destroy_process_group()


@pytest.mark.parametrize("world", [2, 4])
def test_dispatch_and_combine_match_single_rank(world):
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, world, port, q)) for r in range(world)]
    for p in procs:
        p.start()
    res = [q.get(timeout=120) for _ in procs]
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    assert all(r[1] and r[2] and r[3] for r in res), res


def test_owned_experts_partition():
    from nestquant_b200.ep import owned_experts
    for world in (1, 2, 4, 8):
        got = [e for r in range(world) for e in owned_experts(256, world, r)]
        assert got == list(range(256))
