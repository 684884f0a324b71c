"""ZeRO unit state machine in one process: R units on threads, collectives replaced by an in-process
stand-in (lists standing in for the ranks).  Checks lifetimes and counts (one all-gather per pass that
needs the parameters, one reduce-scatter per step) and that R sharded units end where one unsharded unit
ends when it is fed the summed gradients."""
import threading

import pytest
import torch

from zorse_b200.engine import zero
from zorse_b200.engine.zero import EngineConfig, Streams, ZeroUnit
from zorse_b200.models import registry
from zorse_b200.ops.api import get_ops
from zorse_b200.parallel.groups import Group


class FakeDist:
    """all_gather_into_tensor / reduce_scatter_tensor / all_reduce / broadcast / reduce over threads."""

    def __init__(self, R):
        self.R = R
        self.slots = [None] * R
        self.bar = threading.Barrier(R)
        self.local = threading.local()

    def _exchange(self, t):
        self.slots[self.local.rank] = t
        self.bar.wait()
        got = list(self.slots)
        self.bar.wait()
        return got

    def all_gather_into_tensor(self, out, inp, group=None):
        out.copy_(torch.cat(self._exchange(inp.clone())))

    def reduce_scatter_tensor(self, out, inp, group=None):
        got = self._exchange(inp.clone())
        n = out.numel()
        r = self.local.rank
        out.copy_(sum(g[r * n:(r + 1) * n] for g in got))

    def all_reduce(self, t, group=None):
        t.copy_(sum(self._exchange(t.clone())))

    def broadcast(self, t, src=0, group=None):
        t.copy_(self._exchange(t.clone())[src])

    def reduce(self, t, dst=0, group=None):
        got = self._exchange(t.clone())
        if self.local.rank == dst:
            t.copy_(sum(got))


@pytest.mark.parametrize("R,level,ratios", [(4, 3, None), (2, 2, None), (3, 3, (3, 1, 2))])
def test_sharded_units_follow_the_unsharded_one(monkeypatch, R, level, ratios):
    spec = registry.get_spec("tiny_llama", vocab=512)
    fake = FakeDist(R)
    monkeypatch.setattr(zero, "dist", fake)
    results, errors = [None] * R, []

    def grads_for(rank, n, step):
        g = torch.Generator().manual_seed(100 * step + rank)
        return torch.randn(n, generator=g)

    def run(rank):
        try:
            fake.local.rank = rank
            u = ZeroUnit(registry.make_block(spec), 1, device=torch.device("cpu"),
                         cfg=EngineConfig(compute_dtype=torch.float32, reduce_dtype=torch.float32),
                         ops=get_ops("ref"), shard=Group(tuple(range(R)), pg=object()), replicate=Group((rank,)),
                         rank=rank, streams=Streams(torch.device("cpu")), zero_level=level, shard_ratios=ratios)
            seen = []
            for step in range(2):
                u.acquire()                                   # forward
                seen.append(u.full.clone())
                u.release()
                assert (u.full is None) == (level == 3)
                u.acquire()                                   # backward
                u.grad_views()
                u.grad.copy_(grads_for(rank, u.n, step))
                u.release()
                u.reduce_grads()
                assert u.grad is None and u.grad_shard is not None
                u.optimizer_step()
                u.finish_step()
                assert u.full is None
            results[rank] = (seen, u.full_master(), u.counters, u.n, u.shard_n)
        except Exception as e:      # noqa: BLE001
            errors.append((rank, repr(e)))
            fake.bar.abort()

    ths = [threading.Thread(target=run, args=(r,)) for r in range(R)]
    for t in ths:
        t.start()
    for t in ths:
        t.join(120)
    assert not errors, errors
    n = results[0][3]
    # one unsharded unit fed with the summed gradients
    monkeypatch.undo()
    ref = ZeroUnit(registry.make_block(spec), 1, device=torch.device("cpu"),
                   cfg=EngineConfig(compute_dtype=torch.float32, reduce_dtype=torch.float32), ops=get_ops("ref"),
                   shard=Group((0,)), replicate=Group((0,)), rank=0, streams=Streams(torch.device("cpu")))
    ref_seen = []
    for step in range(2):
        ref.acquire()
        ref_seen.append(ref.full.clone())
        ref.grad_views()
        ref.grad[:] = 0
        total = sum(grads_for(r, n, step) for r in range(R))
        ref.grad[: min(n, ref.n)].copy_(total[: min(n, ref.n)])
        ref.reduce_grads()
        ref.optimizer_step()
        ref.finish_step()
    raw = ref.layer.layout()[1]
    for rank in range(R):
        seen, master, counters, _, shard_n = results[rank]
        for a, b in zip(seen, ref_seen):
            assert torch.allclose(a[:raw], b[:raw], atol=1e-6)            # same parameters gathered on every rank
        assert torch.allclose(master[:raw], ref.full_master()[:raw], atol=1e-6)
        assert counters.reduce_scatters == 2 and counters.adam_steps == 2
        # ZeRO-3 gathers for the forward and again for the backward; ZeRO-2 keeps the forward's copy
        assert counters.all_gathers == (4 if level == 3 else 2)
    assert sum(r[4] for r in results) == n
    if ratios:
        assert results[0][4] > results[1][4]
