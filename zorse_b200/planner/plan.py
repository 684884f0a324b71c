"""Two-stage search that turns a cluster description into a training config.

For k = number of machines ... 1 (and, on a single machine, every k that divides the GPU
count): partition the GPU graph into k groups, cost each group's all-gather / reduce-scatter
of one layer and the send/recv between consecutive groups, order the groups (fastest
all-gather first, then greedily by bandwidth to the previous group), sweep the microbatch
size 1, 2, 4, ... and let the stage-2 optimizer pick microbatch counts, uneven layer splits
and the interleaving degree; keep the plan with the lowest predicted iteration latency that
passes the memory model.  Reference: zorse_planner.py:355-647, 811-902.
"""
from __future__ import annotations

import json
from typing import Optional

from ..models import registry
from ..utils.metrics import clean_gpu_name
from . import comm_model
from .cluster import GPU, GPUGroup, ModelConfig, link_bandwidth, link_latency
from .latency import head_and_embedding_ms, load_model_compute_latencies_per_gpu, load_table
from .partition import build_gpu_graph, partition
from .stage2 import PipelineOptimizer, PlanResult


def groups_from_partition(data: dict, pmap: dict) -> list[GPUGroup]:
    by_id = {g["id"]: g for g in data["gpu_list"]}
    parts: dict[int, list] = {}
    for node, p in pmap.items():
        parts.setdefault(p, []).append(by_id[node])
    groups = []
    for gid, members in sorted(parts.items()):
        members.sort(key=lambda g: g["global_rank"])
        gpus = [GPU(clean_gpu_name(g["name"]), int(g["global_rank"]), g["machine"], int(g.get("memory_total_mib", 0)))
                for g in members]
        groups.append(GPUGroup(gid, gpus, machines=tuple(sorted({g["machine"] for g in members}))))
    return groups


def inter_group_bandwidth(data: dict, a: GPUGroup, b: GPUGroup) -> tuple[float, float]:
    """(slowest link GB/s, its reference-message latency s) between two groups."""
    by_rank = {g["global_rank"]: g for g in data["gpu_list"]}
    best = None
    for x in a.gpus:
        for y in b.gpus:
            bw = link_bandwidth(data, by_rank[x.rank], by_rank[y.rank])
            lat = link_latency(data, by_rank[x.rank], by_rank[y.rank])
            if best is None or bw < best[0]:
                best = (bw, lat)
    return best


def order_groups(data: dict, groups: list[GPUGroup]) -> list[GPUGroup]:
    if len(groups) <= 1:
        return groups
    rest = sorted(groups, key=lambda g: (g.all_gather_latency, g.group_id))
    out = [rest.pop(0)]
    while rest:
        prev = out[-1]
        rest.sort(key=lambda g: (-inter_group_bandwidth(data, prev, g)[0], g.group_id))
        out.append(rest.pop(0))
    return out


def microbatch_sizes(gbs: int) -> list[int]:
    out, m = [], 1
    while m <= max(gbs // 2, 1):
        if gbs % m == 0:
            out.append(m)
        m *= 2
    return out


def plan_partition(data: dict, pmap: dict, model_name: str, *, global_batch_size: int, sequence_length: int,
                   autocast_dtype: str, vocab_size: int, dtype_multiplier: float, optimizer_multiplier: float,
                   reserved_memory_gb: float, recompute: bool = True, measured_agrs: Optional[dict] = None,
                   table: Optional[dict] = None, optimizer_gbs: float = 6000.0,
                   microbatch_size: Optional[int] = None, compute_overhead: float = 1.075,
                   tensor_parallel_size: int = 1, lane_members: Optional[dict] = None,
                   full_data: Optional[dict] = None) -> Optional[PlanResult]:
    """With tensor_parallel_size t > 1, `data` describes lanes (planner/tensor_parallel.coarsen), `lane_members` maps
    a lane to the GPUs of `full_data` it is made of, parameters per layer and block latencies are per lane."""
    stats = registry.get_model_stats(model_name, vocab=vocab_size)
    tp = max(int(tensor_parallel_size), 1)
    model = ModelConfig(model_name, stats["num_layers"], stats["hidden_size"], stats["parameters_per_layer"] // tp,
                        stats["total_parameters"] // tp, sequence_length, global_batch_size, vocab_size)
    groups = groups_from_partition(data, pmap)
    size = comm_model.tensor_size_bytes(model.parameters_per_layer, autocast_dtype)
    for g in groups:
        key = ",".join(map(str, g.ranks))
        if measured_agrs and key in measured_agrs:
            g.all_gather_latency = measured_agrs[key]["all_gather_ms"]
            g.reduce_scatter_latency = measured_agrs[key]["reduce_scatter_ms"]
        else:
            g.all_gather_latency = comm_model.collective_ms(data, g.ranks, size, "all_gather")
            g.reduce_scatter_latency = comm_model.collective_ms(data, g.ranks, size, "reduce_scatter")
    groups = order_groups(data, groups)
    best = None
    for mbs in ([microbatch_size] if microbatch_size else microbatch_sizes(global_batch_size)):
        act_bytes = mbs * sequence_length * model.hidden_size * comm_model.DTYPE_BYTES[autocast_dtype]
        for a, b in zip(groups, groups[1:]):
            bw, lat = inter_group_bandwidth(data, a, b)
            t = comm_model.p2p_ms(act_bytes, bw, lat)
            a.send_recv_latency_next = t
            b.send_recv_latency_prev = t
        gpus = [x.identifier for g in groups for x in g.gpus]
        lat_tbl = load_model_compute_latencies_per_gpu(model_name, gpus, sequence_length, autocast_dtype, mbs, table)
        # the layer profile times one block in a tight loop; a whole stage also pays for launch gaps and allocator
        # traffic between blocks: the profiler measures that ratio on a chain of blocks (`_chain_overhead`)
        full_table = table if table is not None else load_table()
        lat_tbl = {g: type(v)(v.forward * _overhead(full_table, model_name, g, compute_overhead),
                              v.backward * _overhead(full_table, model_name, g, compute_overhead))
                   for g, v in lat_tbl.items()}
        if tp > 1:
            from .tensor_parallel import lane_collective_ms, lane_latencies

            cf, cb = lane_collective_ms(full_data, next(iter(lane_members.values())), mbs * sequence_length,
                                        model.hidden_size, comm_model.DTYPE_BYTES[autocast_dtype])
            lat_tbl = lane_latencies(lat_tbl, tp, cf, cb)
        # optimizer: 28 bytes per parameter of HBM traffic on each rank's shard
        opt_ms = model.parameters_per_layer / max(min(len(g.gpus) for g in groups), 1) * 28 / (optimizer_gbs * 1e9) * 1e3
        slowest = max(gpus, key=lambda g: lat_tbl[g].total)
        head_ms, emb_ms = head_and_embedding_ms(model_name, slowest, sequence_length, mbs, vocab_size)
        res = PipelineOptimizer(groups, model, lat_tbl, mbs, dtype_multiplier=dtype_multiplier,
                                optimizer_multiplier=optimizer_multiplier, reserved_memory_gb=reserved_memory_gb,
                                recompute=recompute, optimizer_ms_per_layer=opt_ms, head_ms=head_ms,
                                embedding_ms=emb_ms, activation_table=table if table is not None else load_table(),
                                dtype=autocast_dtype).optimize()
        if res is None:
            if best is not None:
                break   # larger microbatches only need more memory
            continue
        if best is None or res.latency_ms < best.latency_ms:
            best = res
    return best


def _overhead(table: dict, model: str, gpu: str, fallback: float) -> float:
    """Whole-stage time over the sum of single-block times: the layer profiler's measured chain overhead for this
    model and GPU when the table has one, else the caller's constant."""
    try:
        return float(table["_chain_overhead"][model][gpu])
    except (KeyError, TypeError, ValueError):
        return fallback


def candidate_ks(data: dict) -> list[int]:
    n_machines = len(data["machines"])
    n_gpus = len(data["gpu_list"])
    if n_machines > 1:
        return list(range(n_machines, 0, -1))
    return [k for k in range(n_gpus, 0, -1) if n_gpus % k == 0]


def plan(data: dict, model_name: str, *, global_batch_size: int, sequence_length: int, autocast_dtype: str = "bfloat16",
         reduce_dtype: str = "float32", vocab_size: int = 32000, partition_algorithm: str = "min_k_cut_split",
         dtype_multiplier: float = 2.0, optimizer_multiplier: float = 12.0, reserved_memory_gb: float = 2.0,
         recompute: bool = True, measured_agrs: Optional[dict] = None, table: Optional[dict] = None,
         ks: Optional[list[int]] = None, microbatch_size: Optional[int] = None,
         compute_overhead: float = 1.075, tensor_parallel_size: int = 1,
         schedule: Optional[str] = None, graph_weighting: str = "bandwidth") -> tuple[Optional[PlanResult], list[dict]]:
    """tensor_parallel_size t > 1 plans for lanes of t GPUs; the ranks of the result are lane numbers, which is
    what the trainer's config means when it carries `tensor_parallel_size` (export_config writes it).

    `schedule`: the schedule the trainer will run.  The stage-2 optimizer costs every candidate with the reference's
    all-forward-then-all-backward model; with a schedule name the candidates (one per number of groups) are ranked by
    `predict.predict_step_ms` for that schedule instead (1F1B ramps, layer-major replay, tail deferral; every rank
    with its own GPU model's times), and each entry of the returned list carries both figures."""
    full_data, lane_members = data, None
    if tensor_parallel_size > 1:
        from .tensor_parallel import coarsen

        data, lane_members = coarsen(data, tensor_parallel_size)
    gpu_ms = None
    if graph_weighting == "mixed":
        # compute similarity of two GPUs = how alike their block latencies for this model are
        names = sorted({str(g.get("name", "")).lower() for g in data["gpu_list"]})
        try:
            lat = load_model_compute_latencies_per_gpu(model_name, names, sequence_length, autocast_dtype, 1, table)
            gpu_ms = {n: v.total for n, v in lat.items()}
        except Exception:      # noqa: BLE001 - no profile for some GPU model: that term stays neutral
            gpu_ms = None
    G = build_gpu_graph(data, weighting=graph_weighting, gpu_latency_ms=gpu_ms)
    best, best_score, tried = None, None, []
    for k in (ks or candidate_ks(data)):
        pmap = partition(G, k, partition_algorithm)
        res = plan_partition(data, pmap, model_name, global_batch_size=global_batch_size,
                             sequence_length=sequence_length, autocast_dtype=autocast_dtype, vocab_size=vocab_size,
                             dtype_multiplier=dtype_multiplier, optimizer_multiplier=optimizer_multiplier,
                             reserved_memory_gb=reserved_memory_gb, recompute=recompute, measured_agrs=measured_agrs,
                             table=table, microbatch_size=microbatch_size, compute_overhead=compute_overhead,
                             tensor_parallel_size=tensor_parallel_size, lane_members=lane_members, full_data=full_data)
        entry = {"k": k, "latency_ms": None if res is None else res.latency_ms,
                 "microbatch_size": None if res is None else res.microbatch_size,
                 "interleave_degree": None if res is None else res.interleave_degree}
        score = None if res is None else res.latency_ms
        if res is not None and schedule and tensor_parallel_size == 1:
            ms = _schedule_ms(res, data, model_name, global_batch_size, sequence_length, vocab_size, autocast_dtype,
                              reduce_dtype, schedule, recompute, table)
            if ms is not None:
                entry["schedule_ms"] = score = ms
        tried.append(entry)
        if res is not None and (best is None or score < best_score):
            best, best_score = res, score
    return best, tried


def _schedule_ms(res: PlanResult, data: dict, model_name: str, gbs: int, seq: int, vocab: int, autocast_dtype: str,
                 reduce_dtype: str, schedule: str, recompute: bool, table: Optional[dict]) -> Optional[float]:
    """Predicted step of a candidate plan under `schedule` (every rank costed with its own GPU model's profile, or
    the analytic estimate where the table has none), or None when the predictor fails."""
    from .predict import best_tail_deferral, predict_step_ms

    gpu = {int(g["global_rank"]): clean_gpu_name(g["name"]) for g in data.get("gpu_list", []) if isinstance(g, dict)}
    if not gpu:
        return None
    if len(set(gpu.values())) == 1:
        gpu = next(iter(gpu.values()))
    cfg = export_config(res, model_name, gbs, seq, vocab, autocast_dtype, reduce_dtype)
    rc = None if recompute else False
    try:
        k = best_tail_deferral(cfg, schedule, recompute=rc, table=table, gpu=gpu) if schedule == "1f1b" else 0
        return float(predict_step_ms(cfg, schedule, recompute=rc, table=table, gpu=gpu, defer_tail_wgrad=k)["ms"])
    except Exception:      # noqa: BLE001 - no rows for this model / GPU / sequence length
        return None


def export_config(res: PlanResult, model_name: str, global_batch_size: int, sequence_length: int, vocab_size: int,
                  autocast_dtype: str, reduce_dtype: str, path: Optional[str] = None,
                  total_ranks: Optional[int] = None, tensor_parallel_size: int = 1) -> dict:
    """The training_config.json the trainer reads (reference zorse_planner.py:616-647).  A group of
    GPUs that is too slow to be given a single layer owns no stage; with `total_ranks` such ranks are
    listed under `unused_ranks` so that a job launched on every GPU of the cluster file still starts
    (the reference drops them silently, zorse_optimizer/optimizer.py:153-170, and its trainer then
    cannot match the launched world size)."""
    d = {
        "model_name": model_name, "global_batch_size": global_batch_size, "microbatch_size": res.microbatch_size,
        "sequence_length": sequence_length, "vocab_size": vocab_size, "fused_optimizer": True,
        "interleave_degree": res.interleave_degree, "latency": res.latency_ms, "autocast_dtype": autocast_dtype,
        "reduce_dtype": reduce_dtype,
        "pipeline_config": [{"gpu_ranks": list(s.gpu_ranks), "num_microbatches_per_rank": list(s.num_microbatches_per_rank),
                             "layer_partition": list(s.layer_partition), "zero_config": [list(s.gpu_ranks)]}
                            for s in res.stages],
    }
    if tensor_parallel_size > 1:
        d["tensor_parallel_size"] = tensor_parallel_size      # rank numbers above are lanes; total_ranks counts lanes
    if total_ranks is not None:
        used = {r for s in res.stages for r in s.gpu_ranks}
        idle = [r for r in range(total_ranks) if r not in used]
        if idle:
            d["unused_ranks"] = idle
    if path:
        with open(path, "w") as f:
            json.dump(d, f, indent=4)
    return d
