"""Charts of benchmark results as standalone SVG files, written as text (no plotting library, no display).

Reads JSON lines (what `tools/sweep.py`, `tools/quickbench.py` or `bench.py` print), picks an x and a y key, and writes a
line chart with one series per input file. The role of the reference's chart scripts (`tools/gfx/bench.py`,
`tools/gfx/gfxlib.py`), reduced to what the sweep output needs.

    python -m ferrite_b200.tools.sweep --streams 1,2,4,8 > sweep.jsonl
    python -m ferrite_b200.tools.chart --x streams --y aggregate_tok_s --title "decode throughput" -o sweep.svg sweep.jsonl
"""
from __future__ import annotations

import argparse
import json
import math
from typing import Dict, List, Sequence, Tuple

COLORS = ["#1f77b4", "#d62728", "#2ca02c", "#ff7f0e", "#9467bd", "#8c564b"]


def read_points(path: str, x: str, y: str) -> List[Tuple[float, float]]:
    """(x, y) pairs of every JSON line of the file that has both keys (dotted keys reach into nested objects)."""
    def get(d, key):
        for part in key.split("."):
            if not isinstance(d, dict) or part not in d:
                return None
            d = d[part]
        return d
    pts = []
    with open(path) as f:
        for line in f:
            line = line.strip()
            if not line.startswith("{"):
                continue
            try:
                d = json.loads(line)
            except ValueError:
                continue
            a, b = get(d, x), get(d, y)
            if isinstance(a, (int, float)) and isinstance(b, (int, float)):
                pts.append((float(a), float(b)))
    return sorted(pts)


def _ticks(lo: float, hi: float, n: int = 5) -> List[float]:
    if hi <= lo:
        hi = lo + 1.0
    step = 10 ** math.floor(math.log10((hi - lo) / n))
    for m in (1, 2, 5, 10):
        if (hi - lo) / (step * m) <= n:
            step *= m
            break
    t0 = math.ceil(lo / step) * step
    out = []
    while t0 <= hi + 1e-9:
        out.append(round(t0, 10))
        t0 += step
    return out


def render(series: Dict[str, Sequence[Tuple[float, float]]], title: str, xlabel: str, ylabel: str, width: int = 720,
           height: int = 420) -> str:
    """SVG text of a line chart; the y axis starts at zero."""
    allp = [p for pts in series.values() for p in pts]
    if not allp:
        raise ValueError("no points to draw")
    x0, x1 = min(p[0] for p in allp), max(p[0] for p in allp)
    y0, y1 = 0.0, max(p[1] for p in allp) * 1.08 or 1.0
    if x1 == x0:
        x1 = x0 + 1.0
    L, R, T, B = 70, 20, 40, 50
    sx = lambda v: L + (v - x0) / (x1 - x0) * (width - L - R)      # noqa: E731
    sy = lambda v: height - B - (v - y0) / (y1 - y0) * (height - T - B)   # noqa: E731
    o = [f'<svg xmlns="http://www.w3.org/2000/svg" width="{width}" height="{height}" font-family="sans-serif" font-size="12">',
         f'<rect width="{width}" height="{height}" fill="white"/>',
         f'<text x="{width / 2}" y="22" text-anchor="middle" font-size="15">{title}</text>']
    for t in _ticks(y0, y1):
        o.append(f'<line x1="{L}" y1="{sy(t):.1f}" x2="{width - R}" y2="{sy(t):.1f}" stroke="#ddd"/>')
        o.append(f'<text x="{L - 6}" y="{sy(t) + 4:.1f}" text-anchor="end">{t:g}</text>')
    for t in sorted({p[0] for p in allp}) if len({p[0] for p in allp}) <= 12 else _ticks(x0, x1, 8):
        o.append(f'<text x="{sx(t):.1f}" y="{height - B + 16}" text-anchor="middle">{t:g}</text>')
    o.append(f'<line x1="{L}" y1="{height - B}" x2="{width - R}" y2="{height - B}" stroke="black"/>')
    o.append(f'<line x1="{L}" y1="{T}" x2="{L}" y2="{height - B}" stroke="black"/>')
    o.append(f'<text x="{(L + width - R) / 2}" y="{height - 10}" text-anchor="middle">{xlabel}</text>')
    o.append(f'<text x="16" y="{(T + height - B) / 2}" text-anchor="middle" transform="rotate(-90 16 {(T + height - B) / 2})">{ylabel}</text>')
    for i, (name, pts) in enumerate(series.items()):
        c = COLORS[i % len(COLORS)]
        path = " ".join(f"{sx(x):.1f},{sy(y):.1f}" for x, y in pts)
        o.append(f'<polyline fill="none" stroke="{c}" stroke-width="2" points="{path}"/>')
        for x, y in pts:
            o.append(f'<circle cx="{sx(x):.1f}" cy="{sy(y):.1f}" r="3" fill="{c}"/>')
        o.append(f'<rect x="{width - R - 150}" y="{T + 4 + 16 * i}" width="10" height="10" fill="{c}"/>')
        o.append(f'<text x="{width - R - 136}" y="{T + 13 + 16 * i}">{name}</text>')
    o.append("</svg>")
    return "\n".join(o)


def main(argv=None) -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("files", nargs="+", help="JSON-lines files, one series each")
    ap.add_argument("--x", default="streams")
    ap.add_argument("--y", default="aggregate_tok_s")
    ap.add_argument("--title", default="")
    ap.add_argument("-o", "--out", default="chart.svg")
    a = ap.parse_args(argv)
    series = {f.rsplit("/", 1)[-1]: read_points(f, a.x, a.y) for f in a.files}
    series = {k: v for k, v in series.items() if v}
    with open(a.out, "w") as f:
        f.write(render(series, a.title or f"{a.y} vs {a.x}", a.x, a.y))
    print(f"wrote {a.out}: {sum(len(v) for v in series.values())} points in {len(series)} series")
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
