"""Metric history, optional plots and a small HTML report.

Same role and method names as the reference (chronicals/utils/
visual_reporter.py:19-29 ``TrainingMetrics``, :32-388 ``VisualReporter``,
:391-397 ``create_progress_bar``).  matplotlib is optional; without it the
report embeds inline SVG polylines instead of PNGs.
"""
from __future__ import annotations

import json
import os
import time
from dataclasses import asdict, dataclass, field
from typing import Any, Dict, List, Optional


@dataclass
class TrainingMetrics:
    steps: List[int] = field(default_factory=list)
    losses: List[float] = field(default_factory=list)
    learning_rates: List[float] = field(default_factory=list)
    throughputs: List[float] = field(default_factory=list)
    memory_gb: List[float] = field(default_factory=list)
    timestamps: List[float] = field(default_factory=list)
    checkpoints: List[Dict[str, Any]] = field(default_factory=list)


def _svg_polyline(xs: List[float], ys: List[float], w: int = 640, h: int = 220, color: str = "#1f77b4") -> str:
    if len(xs) < 2:
        return "<svg/>"
    x0, x1 = min(xs), max(xs)
    y0, y1 = min(ys), max(ys)
    sx = (w - 20) / (x1 - x0 or 1.0)
    sy = (h - 20) / (y1 - y0 or 1.0)
    pts = " ".join(f"{10 + (x - x0) * sx:.1f},{h - 10 - (y - y0) * sy:.1f}" for x, y in zip(xs, ys))
    return (f'<svg width="{w}" height="{h}" xmlns="http://www.w3.org/2000/svg">'
            f'<rect width="{w}" height="{h}" fill="#fafafa" stroke="#ccc"/>'
            f'<polyline fill="none" stroke="{color}" stroke-width="1.5" points="{pts}"/></svg>')


class VisualReporter:
    def __init__(self, output_dir: str = "./reports", experiment_name: str = "chronicals"):
        self.output_dir = output_dir
        self.experiment_name = experiment_name
        self.metrics = TrainingMetrics()
        self.start_time = time.time()
        os.makedirs(output_dir, exist_ok=True)

    def log_step(self, step: int, loss: float, lr: float = 0.0, throughput: float = 0.0, memory_gb: float = 0.0) -> None:
        m = self.metrics
        m.steps.append(int(step))
        m.losses.append(float(loss))
        m.learning_rates.append(float(lr))
        m.throughputs.append(float(throughput))
        m.memory_gb.append(float(memory_gb))
        m.timestamps.append(time.time() - self.start_time)

    def log_checkpoint(self, step: int, path: str, extra: Optional[Dict[str, Any]] = None) -> str:
        rec = {"step": int(step), "path": path, "time": time.time() - self.start_time,
               "loss": self.metrics.losses[-1] if self.metrics.losses else None}
        rec.update(extra or {})
        self.metrics.checkpoints.append(rec)
        out = os.path.join(self.output_dir, f"checkpoint_{step}.json")
        with open(out, "w") as f:
            json.dump(rec, f, indent=2)
        return out

    def save_metrics_json(self, name: str = "metrics.json") -> str:
        out = os.path.join(self.output_dir, name)
        with open(out, "w") as f:
            json.dump(asdict(self.metrics), f)
        return out

    def plot_curves(self) -> List[str]:
        """PNG curves when matplotlib is installed, otherwise nothing (the HTML report has SVGs)."""
        try:
            import matplotlib
            matplotlib.use("Agg")
            import matplotlib.pyplot as plt
        except Exception:
            return []
        files = []
        for name, ys in (("loss", self.metrics.losses), ("throughput", self.metrics.throughputs)):
            if not ys:
                continue
            fig, ax = plt.subplots(figsize=(7, 3))
            ax.plot(self.metrics.steps, ys)
            ax.set_xlabel("step")
            ax.set_ylabel(name)
            path = os.path.join(self.output_dir, f"{name}.png")
            fig.savefig(path, dpi=100, bbox_inches="tight")
            plt.close(fig)
            files.append(path)
        return files

    def generate_html_report(self, name: str = "report.html") -> str:
        m = self.metrics
        self.plot_curves()
        rows = "".join(f"<tr><td>{c['step']}</td><td>{c['path']}</td><td>{c.get('loss')}</td></tr>" for c in m.checkpoints)
        summary = {
            "steps": m.steps[-1] if m.steps else 0,
            "final loss": f"{m.losses[-1]:.4f}" if m.losses else "-",
            "best loss": f"{min(m.losses):.4f}" if m.losses else "-",
            "mean tokens/s": f"{sum(m.throughputs) / len(m.throughputs):,.0f}" if m.throughputs else "-",
            "peak memory (GB)": f"{max(m.memory_gb):.2f}" if m.memory_gb else "-",
            "wall time (s)": f"{time.time() - self.start_time:.1f}",
        }
        html = ["<html><head><meta charset='utf-8'><title>", self.experiment_name, "</title></head><body>",
                f"<h1>{self.experiment_name}</h1><table border='1' cellpadding='4'>"]
        html += [f"<tr><th align='left'>{k}</th><td>{v}</td></tr>" for k, v in summary.items()]
        html.append("</table><h2>loss</h2>")
        html.append(_svg_polyline([float(s) for s in m.steps], m.losses))
        html.append("<h2>tokens/s</h2>")
        html.append(_svg_polyline([float(s) for s in m.steps], m.throughputs, color="#2ca02c"))
        html.append(f"<h2>checkpoints</h2><table border='1' cellpadding='4'><tr><th>step</th><th>path</th><th>loss</th></tr>{rows}</table>")
        html.append("</body></html>")
        out = os.path.join(self.output_dir, name)
        with open(out, "w") as f:
            f.write("".join(html))
        return out


def create_progress_bar(total: int, desc: str = "training"):
    try:
        from tqdm import tqdm
        return tqdm(total=total, desc=desc)
    except Exception:
        return None
