"""Drawings of the GPU graph and of its partition into pipeline stages.

Three pictures, as in the reference (zorse_optimizer/visualize.py): the GPU graph with nodes coloured
by machine and edges weighted by bandwidth (`visualize_graph`, :26-90), the partitioned graph with
cut edges dashed in red (`visualize_partitioned_graph`, :93-189), and the partitioned graph next to a
panel of partition metrics (`visualize_partitions_with_metrics`, :192-306).

Each picture is first built as a renderer-independent scene (node positions from a seeded spring
layout, colours, labels, edge classes, legend, side text) and then written by one of two back ends:
matplotlib's Agg rasteriser when matplotlib is installed and the file name does not end in `.svg`
(PNG, like the reference), otherwise a dependency-free SVG writer.  Everything runs on the CPU and
ends in a file; no window or graphics API is involved.
"""
from __future__ import annotations

import colorsys
from dataclasses import dataclass, field
from typing import Optional
from xml.sax.saxutils import escape

import networkx as nx


# ---- metrics -----------------------------------------------------------------------------------
def partition_metrics(G: nx.Graph, partitions: dict) -> dict:
    """Cut weight, weight inside the parts, their ratio to the total, balance (smallest part over the
    largest) and part sizes."""
    cut = inside = 0.0
    for u, v, d in G.edges(data=True):
        w = float(d.get("weight", 1.0))
        if partitions[u] != partitions[v]:
            cut += w
        else:
            inside += w
    sizes: dict = {}
    for p in partitions.values():
        sizes[p] = sizes.get(p, 0) + 1
    total = cut + inside
    return {"cut_weight": cut, "internal_weight": inside, "ratio_cut_to_total": cut / total if total else 0.0,
            "balance": (min(sizes.values()) / max(sizes.values())) if sizes else 1.0,
            "partition_sizes": dict(sorted(sizes.items()))}


# ---- scene -------------------------------------------------------------------------------------
@dataclass
class Scene:
    title: str
    nodes: list = field(default_factory=list)     # dicts: id, x, y (0..1), color "#rrggbb", label
    edges: list = field(default_factory=list)     # dicts: u, v, width, color, dashed, label
    legend: list = field(default_factory=list)    # (color, text)
    legend_title: str = ""
    side_text: list = field(default_factory=list)  # lines of the metrics panel


def _hex(r, g, b):
    return f"#{int(r * 255):02x}{int(g * 255):02x}{int(b * 255):02x}"


def palette(n: int) -> list:
    """n distinct colours (evenly spaced hues, two lightness levels)."""
    return [_hex(*colorsys.hls_to_rgb(i / max(n, 1), 0.55 if i % 2 == 0 else 0.42, 0.75)) for i in range(n)]


def _layout(G: nx.Graph, seed: int = 42) -> dict:
    if G.number_of_nodes() == 1:
        return {next(iter(G.nodes)): (0.5, 0.5)}
    pos = nx.spring_layout(G, seed=seed)
    xs, ys = [p[0] for p in pos.values()], [p[1] for p in pos.values()]
    sx, sy = (max(xs) - min(xs)) or 1.0, (max(ys) - min(ys)) or 1.0
    return {n: (0.08 + 0.84 * (p[0] - min(xs)) / sx, 0.08 + 0.84 * (p[1] - min(ys)) / sy) for n, p in pos.items()}


def _short_name(G, n):
    return str(G.nodes[n].get("name", "GPU")).split()[-1]


def _edge_widths(G):
    w = {(u, v): float(d.get("weight", 0.5)) for u, v, d in G.edges(data=True)}
    mx = max(w.values(), default=1.0) or 1.0
    return {e: max(0.5, 5.0 * x / mx) for e, x in w.items()}, w


def scene_graph(G: nx.Graph, data: Optional[dict] = None, title: str = "GPU Graph") -> Scene:
    pos = _layout(G)
    machines = sorted({str(G.nodes[n].get("machine", "Unknown")) for n in G.nodes})
    colour = dict(zip(machines, palette(len(machines))))
    sc = Scene(title, legend=[(colour[m], m) for m in machines], legend_title="Machines")
    for n in G.nodes:
        mem = float(G.nodes[n].get("memory_total_mib", 0)) / 1024
        sc.nodes.append({"id": n, "x": pos[n][0], "y": pos[n][1], "color": colour[str(G.nodes[n].get("machine", "Unknown"))],
                         "label": f"{_short_name(G, n)}\n{mem:.1f}GB"})
    widths, weights = _edge_widths(G)
    for (u, v), wd in widths.items():
        sc.edges.append({"u": u, "v": v, "width": wd, "color": "#000000", "dashed": False, "label": f"{weights[(u, v)]:.2f}"})
    return sc


def scene_partitioned(G: nx.Graph, partitions: dict, data: Optional[dict] = None,
                      title: str = "Partitioned GPU Graph", uniform_edges: bool = False) -> Scene:
    pos = _layout(G)
    parts = sorted(set(partitions.values()))
    colour = dict(zip(parts, palette(len(parts))))
    sc = Scene(title, legend=[(colour[p], f"Partition {p}") for p in parts], legend_title="Partitions")
    for n in G.nodes:
        mem = float(G.nodes[n].get("memory_total_mib", 0)) / 1024
        mach = str(G.nodes[n].get("machine", "Unknown"))
        label = f"{_short_name(G, n)}\nP{partitions[n]}" if uniform_edges else f"{_short_name(G, n)}\n{mem:.1f}GB\n{mach[-3:]}"
        sc.nodes.append({"id": n, "x": pos[n][0], "y": pos[n][1], "color": colour[partitions[n]], "label": label})
    widths, _ = _edge_widths(G)
    for (u, v), wd in widths.items():
        cut = partitions[u] != partitions[v]
        sc.edges.append({"u": u, "v": v, "width": (2.0 if cut else 1.0) if uniform_edges else wd,
                         "color": "#d62728" if cut else "#808080", "dashed": cut, "label": ""})
    return sc


def scene_with_metrics(G: nx.Graph, partitions: dict, metrics: Optional[dict] = None, data: Optional[dict] = None,
                       title: str = "GPU Partitions with Metrics") -> Scene:
    m = metrics if metrics is not None else partition_metrics(G, partitions)
    sc = scene_partitioned(G, partitions, data, title, uniform_edges=True)

    def num(key):
        v = m.get(key)
        return f"{v:.2f}" if isinstance(v, (int, float)) else "N/A"

    sc.side_text = ["Partitioning Metrics:", "", f"Number of partitions: {len(set(partitions.values()))}", "",
                    f"Cut value: {num('cut_weight')}", "", f"Internal weight: {num('internal_weight')}", "",
                    f"Cut ratio: {num('ratio_cut_to_total')}", "", f"Balance: {num('balance')}", "", "Partition sizes:"]
    sc.side_text += [f"   P{p}: {s} nodes" for p, s in (m.get("partition_sizes") or {}).items()]
    return sc


# ---- back ends ---------------------------------------------------------------------------------
def render_svg(sc: Scene, path: str, width: int = 1200, height: int = 900) -> str:
    side = 260 if sc.side_text else 0
    gw, gh = width - side, height - 40
    P = lambda x, y: (x * gw, 40 + (1.0 - y) * gh)
    xy = {n["id"]: P(n["x"], n["y"]) for n in sc.nodes}
    out = [f'<svg xmlns="http://www.w3.org/2000/svg" width="{width}" height="{height}" font-family="sans-serif">',
           f'<rect width="{width}" height="{height}" fill="white"/>',
           f'<text x="{gw / 2:.0f}" y="26" text-anchor="middle" font-size="20">{escape(sc.title)}</text>']
    for e in sc.edges:
        (x1, y1), (x2, y2) = xy[e["u"]], xy[e["v"]]
        dash = ' stroke-dasharray="8,5"' if e["dashed"] else ""
        out.append(f'<line x1="{x1:.1f}" y1="{y1:.1f}" x2="{x2:.1f}" y2="{y2:.1f}" stroke="{e["color"]}" '
                   f'stroke-width="{e["width"]:.2f}" stroke-opacity="0.7"{dash}/>')
        if e["label"]:
            out.append(f'<text x="{(x1 + x2) / 2:.1f}" y="{(y1 + y2) / 2:.1f}" font-size="10" text-anchor="middle" '
                       f'fill="#333">{escape(e["label"])}</text>')
    for n in sc.nodes:
        x, y = xy[n["id"]]
        out.append(f'<circle cx="{x:.1f}" cy="{y:.1f}" r="22" fill="{n["color"]}" stroke="#222"/>')
        lines = n["label"].split("\n")
        for i, ln in enumerate(lines):
            out.append(f'<text x="{x:.1f}" y="{y + 11 * (i - (len(lines) - 1) / 2) + 3:.1f}" font-size="10" '
                       f'text-anchor="middle">{escape(ln)}</text>')
    if sc.legend:
        out.append(f'<text x="12" y="56" font-size="12" font-weight="bold">{escape(sc.legend_title)}</text>')
        for i, (c, t) in enumerate(sc.legend):
            out.append(f'<rect x="12" y="{64 + 18 * i}" width="14" height="12" fill="{c}"/>')
            out.append(f'<text x="32" y="{75 + 18 * i}" font-size="11">{escape(str(t))}</text>')
    for i, ln in enumerate(sc.side_text):
        out.append(f'<text x="{gw + 10}" y="{height / 2 - 9 * len(sc.side_text) + 18 * i:.0f}" font-size="13" '
                   f'xml:space="preserve">{escape(ln)}</text>')
    out.append("</svg>")
    with open(path, "w") as f:
        f.write("\n".join(out))
    return path


def render_matplotlib(sc: Scene, path: str) -> Optional[str]:
    try:
        import matplotlib

        matplotlib.use("Agg")
        import matplotlib.pyplot as plt
        from matplotlib.patches import Patch
    except ImportError:
        return None
    fig = plt.figure(figsize=(16, 10) if sc.side_text else (14, 12))
    ax = plt.subplot2grid((1, 5), (0, 0), colspan=4) if sc.side_text else fig.add_subplot(111)
    xy = {n["id"]: (n["x"], n["y"]) for n in sc.nodes}
    for e in sc.edges:
        (x1, y1), (x2, y2) = xy[e["u"]], xy[e["v"]]
        ax.plot([x1, x2], [y1, y2], color=e["color"], linewidth=e["width"], linestyle="--" if e["dashed"] else "-",
                alpha=0.7, zorder=1)
        if e["label"]:
            ax.text((x1 + x2) / 2, (y1 + y2) / 2, e["label"], fontsize=7, ha="center", zorder=3)
    ax.scatter([n["x"] for n in sc.nodes], [n["y"] for n in sc.nodes], s=700, c=[n["color"] for n in sc.nodes], zorder=2)
    for n in sc.nodes:
        ax.text(n["x"], n["y"], n["label"], fontsize=8, ha="center", va="center", zorder=4)
    if sc.legend:
        ax.legend(handles=[Patch(facecolor=c, label=t) for c, t in sc.legend], title=sc.legend_title, loc="upper right")
    ax.set_title(sc.title)
    ax.axis("off")
    if sc.side_text:
        ax2 = plt.subplot2grid((1, 5), (0, 4), colspan=1)
        ax2.axis("off")
        ax2.text(0, 0.5, "\n".join(sc.side_text), fontsize=10, va="center")
    plt.tight_layout()
    plt.savefig(path, dpi=300)
    plt.close(fig)
    return path


def render(sc: Scene, output_file: Optional[str]) -> str:
    """PNG through matplotlib when it is installed (and the name does not ask for SVG), else SVG;
    returns the path written.  Default name: the title with underscores, as in the reference."""
    path = output_file or f"{sc.title.replace(' ', '_')}.png"
    if not path.lower().endswith(".svg"):
        done = render_matplotlib(sc, path)
        if done:
            return done
        path = path.rsplit(".", 1)[0] + ".svg"
    return render_svg(sc, path)


# ---- public functions (reference names) ----------------------------------------------------------
def visualize_graph(G, data=None, title="GPU Graph", output_file=None) -> Optional[str]:
    if G.number_of_nodes() == 0:
        print("Error: Graph has no nodes to visualize.")
        return None
    return render(scene_graph(G, data, title), output_file)


def visualize_partitioned_graph(G, partitions, data=None, title="Partitioned GPU Graph", output_file=None) -> Optional[str]:
    if G.number_of_nodes() == 0:
        print("Error: Graph has no nodes to visualize.")
        return None
    return render(scene_partitioned(G, partitions, data, title), output_file)


def visualize_partitions_with_metrics(G, partitions, metrics=None, data=None, title="GPU Partitions with Metrics",
                                      output_file=None) -> Optional[str]:
    if G.number_of_nodes() == 0:
        print("Error: Graph has no nodes to visualize.")
        return None
    return render(scene_with_metrics(G, partitions, metrics, data, title), output_file)


def visualize_partition(G, partition_map=None, path="gpu_graph.png") -> bool:
    """The planner's `--draw FILE`: the partitioned graph with its metrics panel (the plain graph when
    no partition is given).  Also writes `<stem>_graph.<ext>` and `<stem>_partitioned.<ext>`."""
    if G.number_of_nodes() == 0:
        return False
    if not partition_map:
        visualize_graph(G, output_file=path)
        return True
    stem, ext = path.rsplit(".", 1) if "." in path else (path, "png")
    visualize_graph(G, output_file=f"{stem}_graph.{ext}")
    visualize_partitioned_graph(G, partition_map, output_file=f"{stem}_partitioned.{ext}")
    visualize_partitions_with_metrics(G, partition_map, output_file=path)
    return True
