"""Figure rendering without a plotting library: heat maps and histograms as PNG bytes.

The reference renders its evaluation figures with matplotlib (Agg, CPU) and logs PNG bytes
(param_decomp/core/slow_eval.py:635-1045). Here a figure is a raster drawn directly into a uint8
array and encoded with zlib + the PNG chunk layout; the underlying arrays are saved next to it
(`.npy`) so any plotting tool can redo the picture.
"""

from __future__ import annotations

import struct
import zlib
from pathlib import Path

import numpy as np

# a compact perceptual ramp (dark blue -> green -> yellow), 9 knots, linearly interpolated
_RAMP = np.array([[68, 1, 84], [71, 44, 122], [59, 81, 139], [44, 113, 142], [33, 144, 141], [39, 173, 129],
                  [92, 200, 99], [170, 220, 50], [253, 231, 37]], dtype=np.float64)


def colormap(unit: np.ndarray) -> np.ndarray:
    """Values in [0, 1] -> RGB uint8."""
    x = np.clip(np.nan_to_num(unit, nan=0.0), 0.0, 1.0) * (len(_RAMP) - 1)
    lo = np.floor(x).astype(int).clip(0, len(_RAMP) - 2)
    t = (x - lo)[..., None]
    return (_RAMP[lo] * (1 - t) + _RAMP[lo + 1] * t).round().astype(np.uint8)


def png_bytes(rgb: np.ndarray) -> bytes:
    """Encode `[H, W, 3]` uint8 as a PNG."""
    assert rgb.ndim == 3 and rgb.shape[2] == 3 and rgb.dtype == np.uint8
    h, w, _ = rgb.shape
    raw = b"".join(b"\x00" + rgb[r].tobytes() for r in range(h))  # filter type 0 per scan line

    def chunk(tag: bytes, data: bytes) -> bytes:
        return struct.pack(">I", len(data)) + tag + data + struct.pack(">I", zlib.crc32(tag + data) & 0xFFFFFFFF)

    return (b"\x89PNG\r\n\x1a\n" + chunk(b"IHDR", struct.pack(">IIBBBBB", w, h, 8, 2, 0, 0, 0))
            + chunk(b"IDAT", zlib.compress(raw, 6)) + chunk(b"IEND", b""))


def heatmap(values: np.ndarray, cell: int = 4, vmin: float | None = None, vmax: float | None = None) -> bytes:
    """A matrix as a colour raster, each entry a `cell x cell` square."""
    v = np.asarray(values, dtype=np.float64)
    lo = np.nanmin(v) if vmin is None else vmin
    hi = np.nanmax(v) if vmax is None else vmax
    unit = (v - lo) / (hi - lo) if hi > lo else np.zeros_like(v)
    rgb = colormap(unit)
    return png_bytes(np.repeat(np.repeat(rgb, cell, axis=0), cell, axis=1))


def grid_of_heatmaps(mats: list[np.ndarray], cols: int = 6, cell: int = 3, gap: int = 2) -> bytes:
    """Several equally shaped matrices tiled into one image (shared colour scale per tile)."""
    assert mats
    h, w = mats[0].shape
    rows = -(-len(mats) // cols)
    canvas = np.full((rows * (h * cell + gap) + gap, cols * (w * cell + gap) + gap, 3), 255, dtype=np.uint8)
    for i, m in enumerate(mats):
        r, c = divmod(i, cols)
        lo, hi = float(np.nanmin(m)), float(np.nanmax(m))
        unit = (m - lo) / (hi - lo) if hi > lo else np.zeros_like(m, dtype=np.float64)
        tile = np.repeat(np.repeat(colormap(unit), cell, axis=0), cell, axis=1)
        y0, x0 = gap + r * (h * cell + gap), gap + c * (w * cell + gap)
        canvas[y0:y0 + h * cell, x0:x0 + w * cell] = tile
    return png_bytes(canvas)


def histogram(counts: np.ndarray, height: int = 120, bar: int = 4, log: bool = True) -> bytes:
    """Bar chart of bin counts (log-scaled heights by default)."""
    c = np.asarray(counts, dtype=np.float64)
    y = np.log1p(c) if log else c
    top = y.max() if y.max() > 0 else 1.0
    bars = (y / top * (height - 1)).round().astype(int)
    img = np.full((height, len(c) * bar, 3), 255, dtype=np.uint8)
    for i, b in enumerate(bars):
        img[height - 1 - b:, i * bar:(i + 1) * bar - 1] = (59, 81, 139)
    return png_bytes(img)


def scatter(x: np.ndarray, y: np.ndarray, size: int = 240) -> bytes:
    """Point cloud on a square canvas (axes scaled to the data range)."""
    img = np.full((size, size, 3), 255, dtype=np.uint8)
    x, y = np.asarray(x, dtype=np.float64), np.asarray(y, dtype=np.float64)
    ok = np.isfinite(x) & np.isfinite(y)
    if ok.any():
        x, y = x[ok], y[ok]
        sx = (x - x.min()) / (np.ptp(x) or 1.0)
        sy = (y - y.min()) / (np.ptp(y) or 1.0)
        px = (sx * (size - 3)).astype(int) + 1
        py = size - 2 - (sy * (size - 3)).astype(int)
        for dx in (-1, 0, 1):
            for dy in (-1, 0, 1):
                img[(py + dy).clip(0, size - 1), (px + dx).clip(0, size - 1)] = (33, 144, 141)
    return png_bytes(img)


def save_figure(run_dir: Path | str | None, name: str, png: bytes, arrays: dict[str, np.ndarray] | None = None) -> Path | None:
    """Write `<run_dir>/figures/<name>.png` (+ `<name>.npz` with the data); no-op without a run dir."""
    if run_dir is None:
        return None
    d = Path(run_dir) / "figures"
    d.mkdir(parents=True, exist_ok=True)
    path = d / f"{name.replace('/', '_')}.png"
    path.write_bytes(png)
    if arrays:
        np.savez_compressed(path.with_suffix(".npz"), **arrays)
    return path
