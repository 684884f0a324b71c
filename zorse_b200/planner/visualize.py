"""Optional PNG drawings of the GPU graph and its partition (CPU rasterisation to a file with
matplotlib's Agg backend; skipped silently when matplotlib is not installed).
Reference: zorse_optimizer/visualize.py:26-306."""
from __future__ import annotations


def visualize_partition(G, partition_map=None, path="gpu_graph.png") -> bool:
    try:
        import matplotlib

        matplotlib.use("Agg")
        import matplotlib.pyplot as plt
        import networkx as nx
    except ImportError:
        return False
    pos = nx.spring_layout(G, seed=0, weight="weight")
    colors = [partition_map.get(n, 0) for n in G.nodes] if partition_map else "tab:blue"
    plt.figure(figsize=(8, 6))
    nx.draw_networkx(G, pos, node_color=colors, cmap="tab10", labels={n: f"{G.nodes[n].get('name','')}\n{n}" for n in G.nodes},
                     font_size=7)
    nx.draw_networkx_edge_labels(G, pos, edge_labels={(a, b): d["weight"] for a, b, d in G.edges(data=True)}, font_size=6)
    plt.axis("off")
    plt.savefig(path, dpi=120, bbox_inches="tight")
    plt.close()
    return True
