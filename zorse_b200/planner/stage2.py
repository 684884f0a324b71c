"""Stage-2 optimizer: given GPU groups in pipeline order, choose microbatches per rank, layers
per group (uneven splits), the interleaving degree, and predict the iteration latency.

Arithmetic (all times in ms), after reference zorse_optimizer/optimizer.py:67-505:
* microbatches per rank of a group: share w_i = (1/t_i) / sum_j (1/t_j) of the M microbatches,
  floor, leftovers one each to the ranks with the largest share;
* layers per group: time per layer T_g = max_i (t_i * m_i); share c_g = (1/T_g) / sum_h (1/T_h);
  floor + largest remainder; groups left with no layer are dropped;
* interleaving with degree d: every group's layers are cut into d chunks and stages are
  emitted chunk-major (chunk 0 of every group, chunk 1, ...), so a group owns d stages;
* latency = start-up + steady state + drain, with all-gather / reduce-scatter / send-recv
  overlapped against compute by max(), plus the optimizer update that the reference leaves out.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Optional

from .cluster import GPUGroup, ModelConfig, ModelLatencies, StagePlan
from .memory import validate_memory


def distribute_microbatches(total: int, lat: list[float]) -> list[int]:
    inv = [1.0 / max(t, 1e-9) for t in lat]
    s = sum(inv)
    w = [x / s for x in inv]
    m = [int(total * x) for x in w]
    left = total - sum(m)
    order = sorted(range(len(w)), key=lambda i: -w[i])
    k = 0
    while left > 0:
        m[order[k % len(order)]] += 1
        left -= 1
        k += 1
    return m


def distribute_layers(total_layers: int, group_time: list[float], rule: str = "ratio") -> list[int]:
    """Whole layers per group in proportion to the groups' speed (1 / time per layer).  Layers left
    after rounding down go, one each, to the groups with the largest share (`rule="ratio"`, the
    reference's rule, zorse_optimizer/optimizer.py:138-156: shares 0.5/0.3/0.2 of 32 layers give
    17/9/6) or to the groups with the largest fractional remainder (`rule="remainder"`: 16/10/6)."""
    inv = [1.0 / max(t, 1e-9) for t in group_time]
    s = sum(inv)
    c = [x / s for x in inv]
    exact = [total_layers * x for x in c]
    L = [int(e) for e in exact]
    left = total_layers - sum(L)
    if rule == "remainder":
        order = sorted(range(len(c)), key=lambda i: -(exact[i] - L[i]))
    else:
        order = sorted(range(len(c)), key=lambda i: -c[i])
    for i in range(left):
        L[order[i % len(order)]] += 1
    return L


@dataclass
class PlanResult:
    stages: list[StagePlan]
    latency_ms: float
    interleave_degree: int
    microbatch_size: int
    memory_gb: dict = field(default_factory=dict)
    breakdown: dict = field(default_factory=dict)


class PipelineOptimizer:
    def __init__(self, groups: list[GPUGroup], model: ModelConfig, latencies: dict[str, ModelLatencies], microbatch_size: int,
                 *, dtype_multiplier: float = 2.0, optimizer_multiplier: float = 12.0, reserved_memory_gb: float = 2.0,
                 recompute: bool = True, optimizer_ms_per_layer: float = 0.0, max_interleave: Optional[int] = None,
                 head_ms: tuple = (0.0, 0.0), embedding_ms: tuple = (0.0, 0.0),
                 activation_table: Optional[dict] = None, dtype: str = "bfloat16"):
        self.groups = list(groups)
        self.model = model
        self.lat = latencies
        self.mbs = microbatch_size
        self.M = model.global_batch_size // microbatch_size
        self.dm, self.om, self.reserved = dtype_multiplier, optimizer_multiplier, reserved_memory_gb
        self.recompute = recompute
        self.opt_ms = optimizer_ms_per_layer
        self.max_interleave = max_interleave
        # (forward, backward) time per microbatch of the output head (final norm + vocabulary
        # projection + loss) on the last stage and of the embedding on the first one; the
        # reference's model treats the network as L identical blocks and leaves both out
        self.head_ms = head_ms
        # profile table with measured activation bytes per block (memory model); None: closed formula
        self.act_table, self.dtype = activation_table, dtype
        self.embedding_ms = embedding_ms

    # ---- work split ------------------------------------------------------------------
    def microbatches_for_group(self, g: GPUGroup) -> list[int]:
        return distribute_microbatches(self.M, [self.lat[x.identifier].total for x in g.gpus])

    def generate_stage_configs(self) -> tuple[list[StagePlan], dict[int, list[int]]]:
        mb = {g.group_id: self.microbatches_for_group(g) for g in self.groups}
        gtime = [max(self.lat[x.identifier].total * m for x, m in zip(g.gpus, mb[g.group_id])) for g in self.groups]
        layers = distribute_layers(self.model.num_layers, gtime)
        stages, start = [], 0
        for g, n in zip(self.groups, layers):
            if n == 0:
                continue
            stages.append(StagePlan(g.group_id, g.ranks, mb[g.group_id], (start, start + n)))
            start += n
        return stages, mb

    def interleave(self, stages: list[StagePlan], degree: int) -> Optional[list[StagePlan]]:
        if degree == 1:
            return stages
        if any(s.num_layers < degree for s in stages):
            return None
        chunks = []
        for s in stages:
            base, rem = divmod(s.num_layers, degree)
            chunks.append([base + (1 if c < rem else 0) for c in range(degree)])
        out, start = [], 0
        for c in range(degree):
            for s, ch in zip(stages, chunks):
                out.append(StagePlan(s.group_id, s.gpu_ranks, s.num_microbatches_per_rank, (start, start + ch[c])))
                start += ch[c]
        return out

    # ---- latency -----------------------------------------------------------------------
    def pipeline_latency(self, stages: list[StagePlan]) -> tuple[float, dict]:
        by_id = {g.group_id: g for g in self.groups}
        first_of_group = {}
        for i, s in enumerate(stages):
            first_of_group.setdefault(s.group_id, i)

        def f(g):
            return [self.lat[x.identifier].forward for x in by_id[g].gpus]

        def b(g):
            return [self.lat[x.identifier].backward for x in by_id[g].gpus]

        startup = 0.0
        for i, s in enumerate(stages[:-1]):
            g = by_id[s.group_id]
            per_layer = max(f(s.group_id))
            if i == 0:
                per_layer = max(per_layer, g.all_gather_latency)
            startup += s.num_layers * per_layer + g.send_recv_latency_next
        steady = 0.0
        for g in self.groups:
            tot = 0.0
            for i, s in enumerate(stages):
                if s.group_id != g.group_id:
                    continue
                n = s.num_layers
                sr = max(g.send_recv_latency_next, g.send_recv_latency_prev)
                ff, bb = f(g.group_id), b(g.group_id)
                first = 1 if first_of_group[g.group_id] == i else 0
                fwd = max(max(max(fi * n, sr) * max(m - first, 0) for fi, m in zip(ff, s.num_microbatches_per_rank)),
                          g.all_gather_latency * n)
                bk = [(fi + bi) if self.recompute else bi for fi, bi in zip(ff, bb)]
                bwd = max(max(max(x * n, sr) * m for x, m in zip(bk, s.num_microbatches_per_rank)),
                          (g.all_gather_latency + g.reduce_scatter_latency) * n)
                extra = 0.0
                m_max = max(s.num_microbatches_per_rank)
                if i == len(stages) - 1:
                    hf, hb = self.head_ms
                    extra += m_max * (hf + hb + (hf if self.recompute else 0.0))
                if i == 0:
                    ef, eb = self.embedding_ms
                    extra += m_max * (ef + eb)
                tot += fwd + bwd + self.opt_ms * n + extra
            steady = max(steady, tot)
        drain = 0.0
        for i, s in enumerate(reversed(stages[1:])):
            g = by_id[s.group_id]
            per_layer = max(self.lat[x.identifier].total for x in g.gpus)
            if i == 0:
                per_layer = max(per_layer, g.reduce_scatter_latency)
            drain += s.num_layers * per_layer + g.send_recv_latency_prev
        return startup + steady + drain, {"startup_ms": startup, "steady_ms": steady, "drain_ms": drain}

    # ---- search ------------------------------------------------------------------------
    def optimize(self) -> Optional[PlanResult]:
        stages, _ = self.generate_stage_configs()
        groups = {g.group_id: g for g in self.groups}
        ok, mem = validate_memory(stages, groups, self.model, self.mbs, self.dm, self.om, self.reserved,
                                   table=self.act_table, dtype=self.dtype)
        if not ok:
            return None
        best = None
        max_d = min(self.model.num_layers // 2, len(stages)) + 2
        if len(self.groups) == 1:
            max_d = 1
        if self.max_interleave is not None:
            max_d = min(max_d, self.max_interleave)
        for d in range(1, max(max_d, 1) + 1):
            st = self.interleave(stages, d)
            if st is None:
                continue
            ok, mem_d = validate_memory(st, groups, self.model, self.mbs, self.dm, self.om, self.reserved,
                                         table=self.act_table, dtype=self.dtype)
            if not ok:
                continue
            lat, br = self.pipeline_latency(st)
            if best is None or lat < best.latency_ms:
                best = PlanResult(st, lat, d, self.mbs, mem_d, br)
        return best
