"""Dependency-free SVG charts for benchmark results: grouped bars, stacked bars, multi-line
plots and a pipeline Gantt chart.

The reference draws its paper figures with three matplotlib chart classes
(``lorafusion/utils/grouped_bar_chart.py``, ``stacked_bar_chart.py``, ``multi_line_plot.py``)
and a Gantt plot of simulated pipelines
(``benchmarks_paper/imbalance_simulator/main_random_data.py:467-606``).  matplotlib is not a
dependency here; the same four figure kinds are written as plain SVG text, which every browser
and paper toolchain reads.  All classes share: ``title``, axis labels, a categorical palette,
a legend, and ``save(path)`` / ``to_svg()``.
"""

from __future__ import annotations

import math
from pathlib import Path
from typing import Optional, Sequence
from xml.sax.saxutils import escape

PALETTE = ["#4C72B0", "#DD8452", "#55A868", "#C44E52", "#8172B3", "#937860", "#DA8BC3", "#8C8C8C",
           "#CCB974", "#64B5CD"]


def _nice_ticks(lo: float, hi: float, n: int = 5) -> list:
    if hi <= lo:
        hi = lo + 1.0
    raw = (hi - lo) / max(n, 1)
    mag = 10 ** math.floor(math.log10(raw))
    step = min((m for m in (1, 2, 2.5, 5, 10) if m * mag >= raw), default=10) * mag
    start = math.floor(lo / step) * step
    ticks, v = [], start
    while v <= hi + 1e-9 * step:
        if v >= lo - 1e-9 * step:
            ticks.append(round(v, 10))
        v += step
    return ticks


def _fmt(v: float) -> str:
    if abs(v) >= 1000:
        return f"{v:,.0f}"
    if abs(v) >= 10 or float(v).is_integer():
        return f"{v:.0f}" if float(v).is_integer() else f"{v:.1f}"
    return f"{v:.2f}"


class _Chart:
    def __init__(self, title: str = "", xlabel: str = "", ylabel: str = "", width: int = 760, height: int = 420,
                 colors: Optional[Sequence[str]] = None):
        self.title, self.xlabel, self.ylabel = title, xlabel, ylabel
        self.width, self.height = width, height
        self.colors = list(colors or PALETTE)
        self.left, self.right, self.top, self.bottom = 70, 20, 46, 64

    # plot-area geometry
    @property
    def pw(self) -> float:
        return self.width - self.left - self.right

    @property
    def ph(self) -> float:
        return self.height - self.top - self.bottom

    def _y(self, v: float, lo: float, hi: float) -> float:
        return self.top + self.ph * (1.0 - (v - lo) / (hi - lo))

    def _frame(self, lo: float, hi: float, legend: Sequence[str]) -> list:
        out = [f'<svg xmlns="http://www.w3.org/2000/svg" width="{self.width}" height="{self.height}" '
               f'viewBox="0 0 {self.width} {self.height}" font-family="Helvetica,Arial,sans-serif" font-size="12">',
               f'<rect width="{self.width}" height="{self.height}" fill="white"/>']
        if self.title:
            out.append(f'<text x="{self.width / 2}" y="18" text-anchor="middle" font-size="14" '
                       f'font-weight="bold">{escape(self.title)}</text>')
        for t in _nice_ticks(lo, hi):
            y = self._y(t, lo, hi)
            out.append(f'<line x1="{self.left}" y1="{y:.1f}" x2="{self.left + self.pw}" y2="{y:.1f}" stroke="#ddd"/>')
            out.append(f'<text x="{self.left - 6}" y="{y + 4:.1f}" text-anchor="end">{_fmt(t)}</text>')
        out.append(f'<line x1="{self.left}" y1="{self.top}" x2="{self.left}" y2="{self.top + self.ph}" stroke="black"/>')
        out.append(f'<line x1="{self.left}" y1="{self.top + self.ph}" x2="{self.left + self.pw}" '
                   f'y2="{self.top + self.ph}" stroke="black"/>')
        if self.ylabel:
            cy = self.top + self.ph / 2
            out.append(f'<text x="16" y="{cy}" text-anchor="middle" transform="rotate(-90 16 {cy})">'
                       f'{escape(self.ylabel)}</text>')
        if self.xlabel:
            out.append(f'<text x="{self.left + self.pw / 2}" y="{self.height - 8}" text-anchor="middle">'
                       f'{escape(self.xlabel)}</text>')
        x = self.left
        for i, name in enumerate(legend):
            out.append(f'<rect x="{x}" y="26" width="12" height="12" fill="{self.colors[i % len(self.colors)]}"/>')
            out.append(f'<text x="{x + 16}" y="36">{escape(str(name))}</text>')
            x += 28 + 7 * len(str(name))
        return out

    def to_svg(self) -> str:  # pragma: no cover - overridden
        raise NotImplementedError

    def save(self, path) -> Path:
        path = Path(path)
        path.parent.mkdir(parents=True, exist_ok=True)
        path.write_text(self.to_svg())
        return path


class GroupedBarChart(_Chart):
    """``values[series][group]`` drawn as side-by-side bars per group, optional value labels
    and an optional per-group normalisation to one series (speed-up plots)."""

    def __init__(self, groups: Sequence[str], series: Sequence[str], values, *, normalize_to: Optional[str] = None,
                 annotate: bool = True, **kw):
        super().__init__(**kw)
        self.groups, self.series = list(groups), list(series)
        self.values = [list(map(float, row)) for row in values]
        if normalize_to is not None:
            base = self.values[self.series.index(normalize_to)]
            self.values = [[v / b if b else 0.0 for v, b in zip(row, base)] for row in self.values]
        self.annotate = annotate

    def to_svg(self) -> str:
        hi = max(max(r) for r in self.values) * 1.12
        out = self._frame(0.0, hi, self.series)
        gw = self.pw / len(self.groups)
        bw = gw * 0.8 / len(self.series)
        for g, gname in enumerate(self.groups):
            x0 = self.left + g * gw + gw * 0.1
            for s in range(len(self.series)):
                v = self.values[s][g]
                y = self._y(v, 0.0, hi)
                out.append(f'<rect x="{x0 + s * bw:.1f}" y="{y:.1f}" width="{bw * 0.92:.1f}" '
                           f'height="{self.top + self.ph - y:.1f}" fill="{self.colors[s % len(self.colors)]}"/>')
                if self.annotate:
                    out.append(f'<text x="{x0 + s * bw + bw * 0.46:.1f}" y="{y - 3:.1f}" text-anchor="middle" '
                               f'font-size="9">{_fmt(v)}</text>')
            out.append(f'<text x="{self.left + g * gw + gw / 2:.1f}" y="{self.top + self.ph + 16}" '
                       f'text-anchor="middle">{escape(str(gname))}</text>')
        out.append("</svg>")
        return "\n".join(out)


class StackedBarChart(_Chart):
    """``values[component][bar]`` stacked bottom-up per bar (time or memory breakdowns)."""

    def __init__(self, bars: Sequence[str], components: Sequence[str], values, **kw):
        super().__init__(**kw)
        self.bars, self.components = list(bars), list(components)
        self.values = [list(map(float, row)) for row in values]

    def to_svg(self) -> str:
        totals = [sum(self.values[c][b] for c in range(len(self.components))) for b in range(len(self.bars))]
        hi = max(totals) * 1.1
        out = self._frame(0.0, hi, self.components)
        gw = self.pw / len(self.bars)
        for b, name in enumerate(self.bars):
            x = self.left + b * gw + gw * 0.2
            acc = 0.0
            for c in range(len(self.components)):
                v = self.values[c][b]
                y1, y0 = self._y(acc + v, 0.0, hi), self._y(acc, 0.0, hi)
                out.append(f'<rect x="{x:.1f}" y="{y1:.1f}" width="{gw * 0.6:.1f}" height="{y0 - y1:.1f}" '
                           f'fill="{self.colors[c % len(self.colors)]}"/>')
                acc += v
            out.append(f'<text x="{x + gw * 0.3:.1f}" y="{self._y(acc, 0.0, hi) - 3:.1f}" text-anchor="middle" '
                       f'font-size="9">{_fmt(acc)}</text>')
            out.append(f'<text x="{x + gw * 0.3:.1f}" y="{self.top + self.ph + 16}" text-anchor="middle">'
                       f'{escape(str(name))}</text>')
        out.append("</svg>")
        return "\n".join(out)


class MultiLinePlot(_Chart):
    """Several ``(xs, ys)`` series over a numeric x axis (scaling curves), with markers."""

    def __init__(self, series: Sequence[str], xs: Sequence[Sequence[float]], ys: Sequence[Sequence[float]], *,
                 logx: bool = False, **kw):
        super().__init__(**kw)
        self.series = list(series)
        self.xs = [list(map(float, x)) for x in xs]
        self.ys = [list(map(float, y)) for y in ys]
        self.logx = logx

    def to_svg(self) -> str:
        tx = (lambda v: math.log2(v)) if self.logx else (lambda v: v)
        all_x = [tx(v) for x in self.xs for v in x]
        xlo, xhi = min(all_x), max(all_x)
        if xhi == xlo:
            xhi = xlo + 1.0
        hi = max(v for y in self.ys for v in y) * 1.1
        out = self._frame(0.0, hi, self.series)
        px = lambda v: self.left + self.pw * (0.04 + 0.92 * (tx(v) - xlo) / (xhi - xlo))  # noqa: E731
        for v in sorted({v for x in self.xs for v in x}):
            out.append(f'<text x="{px(v):.1f}" y="{self.top + self.ph + 16}" text-anchor="middle">{_fmt(v)}</text>')
        for s in range(len(self.series)):
            col = self.colors[s % len(self.colors)]
            pts = " ".join(f"{px(x):.1f},{self._y(y, 0.0, hi):.1f}" for x, y in zip(self.xs[s], self.ys[s]))
            out.append(f'<polyline points="{pts}" fill="none" stroke="{col}" stroke-width="2"/>')
            for x, y in zip(self.xs[s], self.ys[s]):
                out.append(f'<circle cx="{px(x):.1f}" cy="{self._y(y, 0.0, hi):.1f}" r="3" fill="{col}"/>')
        out.append("</svg>")
        return "\n".join(out)


class PipelineGantt(_Chart):
    """Forward / backward boxes of every (stage, microbatch) of a simulated or measured 1F1B
    run.  ``fwd`` / ``bwd`` are ``[stages][microbatches]`` lists of ``(start, end)``."""

    def __init__(self, fwd, bwd, **kw):
        kw.setdefault("xlabel", "time")
        kw.setdefault("height", 80 + 36 * len(fwd))
        super().__init__(**kw)
        self.fwd, self.bwd = fwd, bwd

    def to_svg(self) -> str:
        stages = len(self.fwd)
        t_end = max(e for row in list(self.fwd) + list(self.bwd) for _, e in row) or 1.0
        out = [f'<svg xmlns="http://www.w3.org/2000/svg" width="{self.width}" height="{self.height}" '
               f'viewBox="0 0 {self.width} {self.height}" font-family="Helvetica,Arial,sans-serif" font-size="11">',
               f'<rect width="{self.width}" height="{self.height}" fill="white"/>']
        if self.title:
            out.append(f'<text x="{self.width / 2}" y="18" text-anchor="middle" font-size="14" '
                       f'font-weight="bold">{escape(self.title)}</text>')
        row_h = self.ph / stages
        for s in range(stages):
            y = self.top + s * row_h
            out.append(f'<text x="{self.left - 6}" y="{y + row_h / 2 + 4:.1f}" text-anchor="end">stage {s}</text>')
            for kind, rows, shade in (("F", self.fwd, 0), ("B", self.bwd, 1)):
                for m, (t0, t1) in enumerate(rows[s]):
                    if t1 <= t0:
                        continue
                    x0 = self.left + self.pw * t0 / t_end
                    w = self.pw * (t1 - t0) / t_end
                    col = self.colors[m % len(self.colors)]
                    out.append(f'<rect x="{x0:.1f}" y="{y + 2:.1f}" width="{max(w, 0.5):.1f}" height="{row_h - 4:.1f}" '
                               f'fill="{col}" fill-opacity="{0.55 if shade == 0 else 1.0}" stroke="#333" '
                               f'stroke-width="0.3"><title>{kind}{m} stage {s}: {t0:.3f}-{t1:.3f}</title></rect>')
        out.append(f'<text x="{self.left + self.pw / 2}" y="{self.height - 8}" text-anchor="middle">'
                   f'{escape(self.xlabel)} (0 .. {_fmt(t_end)}); light = forward, solid = backward</text>')
        out.append("</svg>")
        return "\n".join(out)
