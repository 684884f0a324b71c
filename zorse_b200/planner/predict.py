"""Predicted iteration time of a GIVEN training config (stages, ranks, layer ranges, microbatch
counts) under a named schedule — what the trainer and `bench.py` print next to the measured time.

The stage-2 optimizer's `pipeline_latency` models the reference's schedules: every stage runs all
its forwards, then all its backwards (reference zorse_optimizer/optimizer.py:215-505).  The true
1F1B schedules of this repository have another shape, so this module adds their closed form:

    per stage s:  F_s = n_s * f + [last] head_f + [first] emb_f        (one microbatch, forward)
                  B_s = n_s * b + [last] head_b + [first] emb_b  (+ F_s when layers are recomputed)
    1F1B:         T = (m - 1) * max_s (F_s + B_s) + sum_s (F_s + B_s) + 2 (P - 1) * p2p
    deferred weight gradients shorten the ramps by the weight-gradient time W_s of every stage that
    is not the bottleneck; v-way interleaving divides the ramps by v.
    layer-major schedules on several stages: a replay of the loop (a stage passes microbatches on only from its last
    layer, so the stages run almost one after the other).

On top: the all-gather of the first layer (nothing to hide it behind), the reduce-scatter of the
layer that finishes last, and the optimizer pass over each rank's shard (HBM-bound, 28 bytes per
parameter: fp32 master + two moments read and written, bf16 copy written).

Block times come from the layer-profile table (`data/model_latencies.json`, one block timed in a
loop); `chain_overhead` (the ratio of a chain of consecutive blocks to the same number of single
blocks, stored by the layer profiler under `_chain_overhead`) scales them when it was measured.
"""
from __future__ import annotations

from typing import Optional

from ..models import registry
from . import comm_model
from .latency import activation_bytes, head_and_embedding_ms, load_model_compute_latencies_per_gpu, load_table

# "for layer: for microbatch" on every stage: a stage hands its first microbatch downstream only while it runs its LAST
# layer, so consecutive stages overlap by one layer's pass at most (see `_layer_major_ms`)
LAYER_MAJOR_SHAPED = ("layer_major", "default", "no_overlap", "two_stage_sync")
GPIPE_SHAPED = ("layer_major", "default", "no_overlap", "two_stage_sync", "zero2", "flashflex", "gpipe")
WGRAD_SHARE_OF_FORWARD = 0.75      # weight-gradient GEMMs ~ the forward GEMMs; the rest of a forward block is attention


def chain_overhead(table: dict, model: str, gpu: str) -> float:
    try:
        return float(table["_chain_overhead"][model][gpu])
    except (KeyError, TypeError, ValueError):
        return 1.0


def _layer_major_ms(G, p2p, recompute) -> float:
    """Replays the layer-major loop of every stage under the block-time model: stage s runs layer 0 on microbatch j
    once stage s-1 has finished its last layer on that microbatch (plus the transfer), then every further layer on all
    microbatches; backward mirrors it from the last stage (which turns around at once).  Returns the time at which
    the first stage finishes its backward (reference loop: zorse_utils/pipeline_schedule_v2.py:202-374).  Every
    group entry carries its own block, head and embedding times (those of its slowest GPU)."""

    def feed(up_out, m):
        if up_out is None:
            return [0.0] * m
        mu = len(up_out)
        return [up_out[min(mu - 1, ((j + 1) * mu + m - 1) // m - 1)] + p2p for j in range(m)]

    fwd_end, out = [], None
    for g in G:
        arr, t = feed(out, g["m"]), 0.0
        for l in range(g["n"]):
            c = g["f"] + (g["ef"] if g["first"] and l == 0 else 0.0) + (g["hf"] if g["last"] and l == g["n"] - 1 else 0.0)
            out = []
            for j in range(g["m"]):
                t = max(t, arr[j]) if l == 0 else t
                t += c
                out.append(t)
        fwd_end.append(t)
    out = None
    for g, t0 in zip(reversed(G), reversed(fwd_end)):
        arr, t = feed(out, g["m"]), t0
        for l in reversed(range(g["n"])):
            c = g["b"] + (g["f"] if recompute else 0.0)
            if g["last"] and l == g["n"] - 1:
                c += g["hb"] + (g["hf"] if recompute else 0.0)
            if g["first"] and l == 0:
                c += g["eb"] + (g["ef"] if recompute else 0.0)
            out = []
            for j in range(g["m"]):
                t = max(t, arr[j]) if l == g["n"] - 1 else t
                t += c
                out.append(t)
    return t


def predict_step_ms(cfg: dict, schedule: str, *, recompute: Optional[bool] = None, gpu="b200",
                    table: Optional[dict] = None, defer_wgrad: bool = False, defer_tail_wgrad: int = 0,
                    optimizer_gbs: float = 6000.0,
                    p2p_gbs: float = 700.0, p2p_latency_ms: float = 0.02, collective_gbs: float = 600.0,
                    collective_latency_ms: float = 0.03) -> dict:
    """`cfg` is a training_config dict.  `gpu`: the GPU model every rank runs on, or a mapping rank -> GPU model for
    a mixed cluster (a rank's block, head and embedding times are those of its own model; a stage's single-microbatch
    time is its slowest rank's, its share of the steady state the largest `microbatches x time` over its ranks, which
    is what unequal microbatch counts per rank are there to balance).  Returns {"ms": total, ...terms}."""
    table = load_table() if table is None else table
    model = cfg["model_name"]
    seq, mbs, vocab = int(cfg["sequence_length"]), int(cfg["microbatch_size"]), int(cfg.get("vocab_size", 32000))
    dtype = cfg.get("autocast_dtype", "bfloat16")
    stats = registry.get_model_stats(model, vocab=vocab)
    name_of = (lambda r: str(gpu[r]).lower()) if isinstance(gpu, dict) else (lambda r: gpu)
    cache: dict = {}

    def times(name):
        if name not in cache:
            lat = load_model_compute_latencies_per_gpu(model, [name], seq, dtype, mbs, table)[name]
            oh = chain_overhead(table, model, name)
            (hf, hb), (ef, eb) = head_and_embedding_ms(model, name, seq, mbs, vocab)
            cache[name] = {"f": lat.forward * oh, "b": lat.backward * oh, "hf": hf, "hb": hb, "ef": ef, "eb": eb, "oh": oh}
        return cache[name]

    sched = (schedule or "layer_major").lower()
    gpipe = sched in GPIPE_SHAPED
    if recompute is None:
        recompute = gpipe
    stages = sorted(cfg["pipeline_config"], key=lambda s: s["layer_partition"][0])
    # interleaved plans list v chunks per rank group: fold them into one entry per group for the stage sums
    groups: dict = {}
    for i, s in enumerate(stages):
        key = tuple(s["gpu_ranks"])
        g = groups.setdefault(key, {"n": 0, "first": False, "last": False, "m": max(s["num_microbatches_per_rank"]),
                                    "R": len(s["gpu_ranks"]), "chunks": 0, "ranks": list(s["gpu_ranks"]),
                                    "counts": list(s["num_microbatches_per_rank"])})
        g["n"] += s["layer_partition"][1] - s["layer_partition"][0]
        g["first"] |= i == 0
        g["last"] |= i == len(stages) - 1
        g["chunks"] += 1
    G = list(groups.values())
    v = max(g["chunks"] for g in G)
    P = len(G)
    bytes_per = comm_model.DTYPE_BYTES.get(dtype, 2)
    p2p = p2p_latency_ms + mbs * seq * stats["hidden_size"] * bytes_per / (p2p_gbs * 1e9) * 1e3
    layer_bytes = stats["parameters_per_layer"] * bytes_per

    def coll(R):
        return 0.0 if R <= 1 else collective_latency_ms + layer_bytes * (R - 1) / R / (collective_gbs * 1e9) * 1e3

    def one_microbatch(g, t, less=0.0):
        F = g["n"] * t["f"] + (t["hf"] if g["last"] else 0.0) + (t["ef"] if g["first"] else 0.0)
        B = g["n"] * t["b"] + (t["hb"] if g["last"] else 0.0) + (t["eb"] if g["first"] else 0.0) + (F if recompute else 0.0)
        return F + B - less

    tail_on = defer_tail_wgrad > 0 and not gpipe and P > 1 and v == 1
    T, W, S = [], [], []
    for g in G:
        per_rank = [times(name_of(r)) for r in g["ranks"]]
        slow = max(per_rank, key=lambda t: one_microbatch(g, t))
        g.update(slow)                      # the stage's own block / head / embedding times: its slowest GPU's
        # the last stage's head (+ blocks) weight gradients leave every microbatch's backward and run after its last
        # one, inside the time the stages before it need to finish (see `best_tail_deferral`)
        held = [(max(t["hb"] - t["hf"], 0.0) + (min(defer_tail_wgrad, g["n"] + 1) - 1) * t["f"] * WGRAD_SHARE_OF_FORWARD)
                if tail_on and g is G[-1] else 0.0 for t in per_rank]
        per_mb = [one_microbatch(g, t, w) for t, w in zip(per_rank, held)]
        T.append(max(per_mb))
        S.append(max(c * x for c, x in zip(g["counts"], per_mb)))
        W.append(g["n"] * slow["f"] * WGRAD_SHARE_OF_FORWARD)
        g["held"] = max(c * w for c, w in zip(g["counts"], held))
    tail = max(0.0, G[-1]["held"] - sum(g["n"] * g["b"] for g in G[:-1])) if tail_on else 0.0
    k = max(range(P), key=lambda i: S[i])
    steady = S[k]
    layer_major = sched in LAYER_MAJOR_SHAPED and v == 1 and P > 1
    if layer_major:
        ramp = _layer_major_ms(G, p2p, recompute) - steady
    elif gpipe:
        # all forwards, then all backwards: the ramps are the other stages' single-microbatch passes too
        ramp = sum(T[i] for i in range(P) if i != k)
    else:
        ramp = sum(T[i] - (W[i] if defer_wgrad else 0.0) for i in range(P) if i != k) / v
    opt = max(g["n"] * stats["parameters_per_layer"] / g["R"] for g in G) * 28 / (optimizer_gbs * 1e9) * 1e3
    if G[0]["first"]:
        opt_emb = stats["total_parameters"] - stats["num_layers"] * stats["parameters_per_layer"]
        opt += opt_emb / max(G[0]["R"], 1) * 28 / (optimizer_gbs * 1e9) * 1e3 * (0.5 if P > 1 else 1.0)
    zero = max(coll(g["R"]) for g in G) * 2.0          # first gather + last reduction are exposed
    if gpipe and any(g["R"] > 1 for g in G):
        # layer-major / ZeRO-2 pipeline shapes re-gather in backward; the gathers overlap unless they are longer
        # than the compute they hide behind
        per_layer_compute = min(gg["m"] * gg["f"] for gg in G)
        zero += max(0.0, max(coll(g["R"]) for g in G) - per_layer_compute) * max(g["n"] for g in G)
    comm = 0.0 if layer_major else 2.0 * (P - 1) * p2p * (v if not gpipe else 1)     # layer-major: inside the replay
    total = steady + ramp + opt + zero + comm + tail
    slowest = max(G, key=lambda g: g["f"] + g["b"])
    return {"ms": total, "steady_ms": steady, "ramp_ms": ramp, "optimizer_ms": opt, "zero_exposed_ms": zero,
            "p2p_ms": comm, "tail_wgrad_ms": tail, "block_fwd_ms": slowest["f"], "block_bwd_ms": slowest["b"],
            "chain_overhead": slowest["oh"], "recompute": bool(recompute),
            "form": "layer_major" if layer_major else "gpipe" if gpipe else "1f1b",
            "stage_ms": T, "stage_layers": [g["n"] for g in G], "stage_microbatches": [g["m"] for g in G],
            "stage_block_bwd_ms": [g["b"] for g in G], "interleave": v,
            "head_wgrad_ms": max(G[-1]["hb"] - G[-1]["hf"], 0.0), "block_wgrad_ms": G[-1]["f"] * WGRAD_SHARE_OF_FORWARD}


def best_tail_deferral(cfg: dict, schedule: str, *, recompute: Optional[bool] = None, table: Optional[dict] = None,
                       max_layers: int = 2, min_gain: float = 0.015, window_share: float = 0.8,
                       max_hold_gib: float = 32.0, **kw) -> int:
    """How many layers of the last stage (the head first) should hold their weight-gradient GEMMs back until the
    stage's last backward (`defer_tail_wgrad` of the 1F1B schedule); 0 = none.

    The last stage carries the head on top of its blocks and so sets the period of a balanced 1F1B pipeline; it is also
    the stage that idles longest at the end of a step, while the stages before it finish their last backward one after
    the other.  Holding back w ms of weight gradients per microbatch shortens the period to max(T_last - w, T_others)
    and moves m * w ms into that idle window.  Chosen: the deepest k <= max_layers whose held-back work fits into
    `window_share` of the window, if the predicted gain is at least `min_gain` of the step.  (Measured on 4 stages
    of 8 Llama-2-7B blocks, 32 microbatches: k = 2 -> 1548 to 1484 ms, k = 3 -> 1511 ms; at 2 stages with 64
    microbatches k = 2 does not fit the window and costs 0.6 %.)  The operands of the held-back GEMMs stay alive for
    every microbatch (the logits' gradient, and per block about 1.8x its stored activations): at most
    `max_hold_gib` of them."""
    p = predict_step_ms(cfg, schedule, recompute=recompute, table=table, **kw)
    T, P = p["stage_ms"], len(p["stage_ms"])
    if p["form"] != "1f1b" or p["interleave"] > 1 or P < 2 or p["recompute"]:
        return 0
    m = p["stage_microbatches"][-1]
    others = max(T[:-1])
    if T[-1] <= others:
        return 0
    window = window_share * sum(n * b for n, b in zip(p["stage_layers"][:-1], p["stage_block_bwd_ms"][:-1]))
    seq, mbs, vocab = int(cfg["sequence_length"]), int(cfg["microbatch_size"]), int(cfg.get("vocab_size", 32000))
    stats = registry.get_model_stats(cfg["model_name"], vocab=vocab)
    tokens = seq * mbs
    head_bytes = tokens * (vocab + stats["hidden_size"]) * 2
    act = activation_bytes(load_table() if table is None else table, cfg["model_name"], kw.get("gpu", "b200"), seq,
                           cfg.get("autocast_dtype", "bfloat16"), mbs)
    block_bytes = 1.8 * (act if act else 34 * tokens * stats["hidden_size"])
    best, best_gain = 0, 0.0
    for k in range(1, min(max_layers, p["stage_layers"][-1] + 1) + 1):
        w = p["head_wgrad_ms"] + (k - 1) * p["block_wgrad_ms"]
        if m * w > window or m * (head_bytes + (k - 1) * block_bytes) > max_hold_gib * 2 ** 30:
            break
        gain = m * (T[-1] - max(T[-1] - w, others))
        if gain > best_gain:
            best, best_gain = k, gain
    return best if best_gain >= min_gain * p["ms"] else 0
