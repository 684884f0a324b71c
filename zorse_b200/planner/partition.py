"""Stage 1 of the planner: the GPU graph and its partition into k groups.

Nodes are GPUs, edges carry the link bandwidth (GB/s) between every pair
(reference zorse_planner.py:86-147).  Four partitioners, as in the reference
(:150-190, :650-808): greedy SPLIT of repeated Stoer-Wagner minimum cuts
(`min_k_cut_split`, default), a cheaper variant that only ever splits the largest component
(`min_k_cut_efficient`), METIS when `pymetis` is importable, and spectral clustering.  On a
single NVSwitch domain every edge has the same weight, all cuts tie, and the partition falls
back to contiguous blocks of equal size in rank order.
"""
from __future__ import annotations

import networkx as nx

from .cluster import link_bandwidth


def build_gpu_graph(data: dict, weighting: str = "bandwidth", gpu_latency_ms: dict | None = None) -> nx.Graph:
    """`weighting="bandwidth"` (default, the reference's live path): an edge weighs its link bandwidth in GB/s.
    `weighting="mixed"`: 0.7 x bandwidth (min-max normalised over the cluster's links) + 0.2 x memory similarity
    (1 - difference over the cluster's range) + 0.1 x compute similarity (square root of the ratio of the two GPUs'
    block latencies, from `gpu_latency_ms`: GPU name -> ms), scaled to 1..100 — the combination the reference carries
    switched off (zorse_planner.py:44-71, 136-141).  It keeps alike GPUs together where bandwidth alone ties, which
    is the case inside one NVSwitch domain that mixes GPU generations."""
    if weighting not in ("bandwidth", "mixed"):
        raise ValueError(f"weighting must be bandwidth or mixed, not {weighting!r}")
    G = nx.Graph()
    for g in data["gpu_list"]:
        G.add_node(g["id"], **{k: g[k] for k in ("id", "name", "memory_total_mib", "machine", "global_rank") if k in g})
    gl = data["gpu_list"]
    pairs = [(i, j) for i in range(len(gl)) for j in range(i + 1, len(gl))]
    bw = {p: link_bandwidth(data, gl[p[0]], gl[p[1]]) for p in pairs}
    if weighting == "bandwidth":
        for (i, j), b in bw.items():
            G.add_edge(gl[i]["id"], gl[j]["id"], weight=int(max(b, 1)))
        return G
    lo_b, hi_b = (min(bw.values()), max(bw.values())) if bw else (0.0, 0.0)
    mem = [float(g.get("memory_total_mib", 0)) for g in gl]
    lo_m, hi_m = min(mem), max(mem)
    lat = {str(k).lower(): float(v) for k, v in (gpu_latency_ms or {}).items()}
    for i, j in pairs:
        b = 1.0 if hi_b == lo_b else (bw[(i, j)] - lo_b) / (hi_b - lo_b)
        m = 1.0 if hi_m == lo_m else 1.0 - abs(mem[i] - mem[j]) / (hi_m - lo_m)
        a, c = lat.get(str(gl[i].get("name", "")).lower()), lat.get(str(gl[j].get("name", "")).lower())
        sim = 1.0 if not a or not c else (min(a, c) / max(a, c)) ** 0.5
        G.add_edge(gl[i]["id"], gl[j]["id"], weight=int(max(round(100 * (0.7 * b + 0.2 * m + 0.1 * sim)), 1)))
    return G


def _uniform(G: nx.Graph) -> bool:
    w = {d["weight"] for _, _, d in G.edges(data=True)}
    return len(w) <= 1


def _rank_order(G: nx.Graph, nodes) -> list:
    return sorted(nodes, key=lambda n: G.nodes[n].get("global_rank", 0))


def contiguous_blocks(G: nx.Graph, k: int) -> dict:
    nodes = _rank_order(G, G.nodes)
    n = len(nodes)
    out = {}
    for p in range(k):
        for nd in nodes[p * n // k:(p + 1) * n // k]:
            out[nd] = p
    return out


def _to_map(parts: list) -> dict:
    return {n: i for i, part in enumerate(parts) for n in part}


def min_k_cut_split(G: nx.Graph, k: int) -> dict:
    """SPLIT: start with one component; k-1 times, cut the component whose Stoer-Wagner
    minimum cut is the lightest."""
    if k <= 1:
        return {n: 0 for n in G.nodes}
    if _uniform(G):
        return contiguous_blocks(G, k)
    parts = [set(G.nodes)]
    while len(parts) < k:
        best = None
        for idx, part in enumerate(parts):
            if len(part) < 2:
                continue
            cut, (a, b) = nx.stoer_wagner(G.subgraph(part))
            if best is None or cut < best[0]:
                best = (cut, idx, set(a), set(b))
        if best is None:
            break
        _, idx, a, b = best
        parts[idx:idx + 1] = [a, b]
    return _to_map([_rank_order(G, p) for p in parts])


def min_k_cut_efficient(G: nx.Graph, k: int) -> dict:
    """Cheaper heuristic: always split the largest remaining component by its minimum cut."""
    if k <= 1:
        return {n: 0 for n in G.nodes}
    if _uniform(G):
        return contiguous_blocks(G, k)
    parts = [set(G.nodes)]
    while len(parts) < k:
        parts.sort(key=len, reverse=True)
        big = parts[0]
        if len(big) < 2:
            break
        _, (a, b) = nx.stoer_wagner(G.subgraph(big))
        parts[0:1] = [set(a), set(b)]
    return _to_map([_rank_order(G, p) for p in parts])


def partition_with_metis(G: nx.Graph, k: int) -> dict:
    try:
        import pymetis
    except ImportError as e:
        raise RuntimeError("the metis partitioner needs the optional package pymetis") from e
    nodes = list(G.nodes)
    idx = {n: i for i, n in enumerate(nodes)}
    adj = [[idx[m] for m in G.neighbors(n)] for n in nodes]
    ew = [[int(G[n][m]["weight"]) for m in G.neighbors(n)] for n in nodes]
    xadj, adjncy, w = [0], [], []
    for a, b in zip(adj, ew):
        adjncy += a
        w += b
        xadj.append(len(adjncy))
    _, membership = pymetis.part_graph(k, xadj=xadj, adjncy=adjncy, eweights=w)
    return {n: membership[i] for i, n in enumerate(nodes)}


def spectral_partition(G: nx.Graph, k: int, seed: int = 0) -> dict:
    if k <= 1:
        return {n: 0 for n in G.nodes}
    if _uniform(G):
        return contiguous_blocks(G, k)
    from sklearn.cluster import SpectralClustering

    nodes = list(G.nodes)
    A = nx.to_numpy_array(G, nodelist=nodes, weight="weight")
    labels = SpectralClustering(n_clusters=k, affinity="precomputed", random_state=seed, assign_labels="kmeans").fit_predict(A)
    return {n: int(l) for n, l in zip(nodes, labels)}


PARTITIONERS = {"min_k_cut_split": min_k_cut_split, "min_k_cut_efficient": min_k_cut_efficient,
                "metis": partition_with_metis, "clustering": spectral_partition}


def partition(G: nx.Graph, k: int, algorithm: str = "min_k_cut_split") -> dict:
    if algorithm not in PARTITIONERS:
        raise ValueError(f"unknown partition algorithm {algorithm!r}; known: {sorted(PARTITIONERS)}")
    return PARTITIONERS[algorithm](G, k)
