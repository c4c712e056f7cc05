"""TEST-ONLY stand-in for matplotlib.pyplot: figures and axes that record what is plotted."""
from pathlib import Path


class _Axes:
    def __init__(self):
        self.series = []

    def plot(self, x, y, *args, **kwargs):
        self.series.append((kwargs.get("label", ""), list(x), list(y)))
        return [object()]

    def __getattr__(self, name):  # set_xlabel, set_title, grid, legend, axhline, ...
        return lambda *args, **kwargs: None


class _Figure:
    def __init__(self, axes):
        self.axes = axes

    def savefig(self, path, *args, **kwargs):
        lines = [f"{label}: x={x} y={y}" for ax in self.axes for label, x, y in ax.series]
        Path(path).write_text("placeholder figure (matplotlib stand-in)\n" + "\n".join(lines) + "\n")

    def __getattr__(self, name):  # tight_layout, suptitle, ...
        return lambda *args, **kwargs: None


_current = None


def subplots(nrows=1, ncols=1, **kwargs):
    global _current
    n = nrows * ncols
    axes = [_Axes() for _ in range(n)]
    _current = _Figure(axes)
    if n == 1:
        return _current, axes[0]
    return _current, axes


def figure(*args, **kwargs):
    return subplots()[0]


def close(*args, **kwargs):
    return None


def savefig(path, *args, **kwargs):
    if _current is not None:
        _current.savefig(path)


def __getattr__(name):
    return lambda *args, **kwargs: None
