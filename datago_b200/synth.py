"""Seeded synthetic inputs with the shapes, sizes and value distributions of the five benchmark workloads.

They stand in for the ImageNet / PD12M style data datago's own benchmarks read
(python/benchmark_filesystem.py, python/benchmark_webdataset.py in the datago tree), which need a network.

Image i of workload k is a pure function of (k, i): numpy.random.default_rng(k * 1_000_003 + i).
JPEGs are written by Pillow/libjpeg-turbo as baseline (SOF0), standard Huffman tables.

  c0  1024 JPEG files, W,H uniform over {256,264..2048}, 4:2:0, q=90, no restart markers
  c1  256 raw RGB buffers, W,H uniform in [512,4096], iid uniform pixels
  c2  8192 JPEGs, W,H uniform over {512,528..1536}, 4:2:0, q uniform in [75,95], odd i: restart interval 4
  c3  tar shards of (.jpg as c2 but sides up to 2048, .json caption) samples
  c4  512 (4:4:4 JPEG up to 4096 on the long side, aspect uniform in [0.33,3], same-size L8 ellipse mask) pairs
"""
import io
import json
import tarfile

import numpy as np
from PIL import Image

try:
    import cv2
    cv2.setNumThreads(1)  # generation is parallelised over processes
except ImportError:
    cv2 = None

IMAGE_CONFIGS = {
    "c0": dict(crop_and_resize=True, default_image_size=1024, downsampling_ratio=32, min_aspect_ratio=0.5, max_aspect_ratio=2.0),
    "c1": dict(crop_and_resize=True, default_image_size=512, downsampling_ratio=16, min_aspect_ratio=0.5, max_aspect_ratio=2.0),
    "c2": None,
    "c3": dict(crop_and_resize=True, default_image_size=1024, downsampling_ratio=32, min_aspect_ratio=0.5, max_aspect_ratio=2.0),
    "c4": dict(crop_and_resize=True, default_image_size=2048, downsampling_ratio=64, min_aspect_ratio=0.5, max_aspect_ratio=2.0),
}
COUNTS = {"c0": 1024, "c1": 256, "c2": 8192, "c3": 64000, "c4": 512}
_BASE = {"c0": 0, "c1": 1, "c2": 2, "c3": 3, "c4": 4}


def _rng(workload, i):
    return np.random.default_rng(_BASE[workload] * 1_000_003 + i)


def _upsample(grid, w, h):
    """Smooth interpolation of a small (gh, gw, 3) float32 grid to (h, w, 3)."""
    if cv2 is not None:
        return cv2.resize(grid, (w, h), interpolation=cv2.INTER_CUBIC)
    else:  # numpy only: separable smoothstep interpolation
        gh, gw = grid.shape[:2]
        ys = np.linspace(0, gh - 1, h, dtype=np.float32)
        xs = np.linspace(0, gw - 1, w, dtype=np.float32)
        y0 = np.clip(np.floor(ys).astype(int), 0, gh - 2)
        x0 = np.clip(np.floor(xs).astype(int), 0, gw - 2)
        ty = ys - y0
        tx = xs - x0
        ty = ty * ty * (3 - 2 * ty)
        tx = tx * tx * (3 - 2 * tx)
        rows = grid[y0] * (1 - ty)[:, None, None] + grid[y0 + 1] * ty[:, None, None]
        return rows[:, x0] * (1 - tx)[None, :, None] + rows[:, x0 + 1] * tx[None, :, None]


def gradient_noise(rng, w, h, octaves=8):
    """Multi-octave smooth noise in [0,1], 3 channels (a Perlin-style stand-in for natural image content).
    The coarse octaves are summed on a quarter-size canvas and interpolated once."""
    qw, qh = max(8, w // 4), max(8, h // 4)
    coarse = np.zeros((qh, qw, 3), np.float32)
    acc = None
    amp, total = 1.0, 0.0
    for o in range(octaves):
        cells = 2 ** (o + 1)
        gw = max(2, int(round(cells * w / max(w, h))) + 1)
        gh = max(2, int(round(cells * h / max(w, h))) + 1)
        if gw >= w or gh >= h:
            break
        grid = rng.random((gh, gw, 3), dtype=np.float32)
        if gw * 2 <= qw and gh * 2 <= qh:
            up = _upsample(grid, qw, qh)
            up *= np.float32(amp)
            coarse += up
        else:
            if acc is None:
                acc = _upsample(coarse, w, h)
            up = _upsample(grid, w, h)
            up *= np.float32(amp)
            acc += up
        total += amp
        amp *= 0.6
    if total == 0.0:  # too small for any octave
        return rng.random((h, w, 3), dtype=np.float32)
    if acc is None:
        acc = _upsample(coarse, w, h)
    acc *= np.float32(1.0 / total)
    return acc


def natural_image(rng, w, h, noise_sigma=8.0, edges=False):
    img = gradient_noise(rng, w, h)
    img *= np.float32(255.0)
    # linear gradients
    a = rng.uniform(-60, 60, 3).astype(np.float32)
    b = rng.uniform(-60, 60, 3).astype(np.float32)
    img += np.linspace(0, 1, w, dtype=np.float32)[None, :, None] * a
    img += np.linspace(0, 1, h, dtype=np.float32)[:, None, None] * b
    if edges:  # hard-edged rectangles and lines
        for _ in range(int(rng.integers(4, 12))):
            x0, x1 = np.sort(rng.integers(0, w, 2))
            y0, y1 = np.sort(rng.integers(0, h, 2))
            if rng.random() < 0.3:
                y1 = min(h, y0 + int(rng.integers(1, 4)))
            img[y0:y1 + 1, x0:x1 + 1] = rng.integers(0, 256, 3)
    if noise_sigma > 0:
        img += rng.standard_normal(img.shape, dtype=np.float32) * np.float32(noise_sigma)
    np.clip(img, 0, 255, out=img)
    return img.astype(np.uint8)


def encode_jpeg(arr, quality, subsampling, restart_blocks=0):
    b = io.BytesIO()
    kw = dict(quality=int(quality), subsampling=subsampling, progressive=False, optimize=False)
    if restart_blocks:
        kw["restart_marker_blocks"] = int(restart_blocks)
    Image.fromarray(arr).save(b, "JPEG", **kw)
    return b.getvalue()


def ellipse_mask(rng, w, h):
    m = np.zeros((h, w), np.uint8)
    yy, xx = np.ogrid[0:h, 0:w]
    for _ in range(int(rng.integers(8, 33))):
        cx, cy = rng.uniform(0, w), rng.uniform(0, h)
        rx, ry = rng.uniform(0.02, 0.25) * w, rng.uniform(0.02, 0.25) * h
        x0, x1 = max(0, int(cx - rx)), min(w, int(cx + rx) + 1)
        y0, y1 = max(0, int(cy - ry)), min(h, int(cy + ry) + 1)
        sub = ((xx[:, x0:x1] - cx) / rx) ** 2 + ((yy[y0:y1] - cy) / ry) ** 2 <= 1.0
        m[y0:y1, x0:x1][sub] = 255
    return m


def c0_item(i):
    rng = _rng("c0", i)
    w, h = (int(rng.integers(32, 257)) * 8 for _ in range(2))
    return encode_jpeg(natural_image(rng, w, h, 8.0), 90, "4:2:0")


def c1_item(i):
    rng = _rng("c1", i)
    w, h = (int(rng.integers(512, 4097)) for _ in range(2))
    return rng.integers(0, 256, (h, w, 3), dtype=np.uint8)


def c2_item(i, max_side=1536):
    rng = _rng("c2" if max_side == 1536 else "c3", i)
    w, h = (int(rng.integers(32, max_side // 16 + 1)) * 16 for _ in range(2))
    q = int(rng.integers(75, 96))
    return encode_jpeg(natural_image(rng, w, h, 0.0, edges=True), q, "4:2:0", 4 if i % 2 else 0)


def c3_item(i):
    """(key, jpeg bytes, json bytes) of global sample i; shard = i // 1000."""
    jpg = c2_item(i, max_side=2048)
    rng = _rng("c3", 10_000_000 + i)
    toks = ["".join(chr(int(c)) for c in rng.integers(97, 123, int(rng.integers(2, 9)))) for _ in range(20)]
    return "%06d_%04d" % (i // 1000, i % 1000), jpg, json.dumps({"caption": " ".join(toks)}).encode()


def c4_item(i):
    """(jpeg 4:4:4, mask L8 array) of the same size."""
    rng = _rng("c4", i)
    aspect = rng.uniform(0.33, 3.0)
    long_side = int(rng.integers(1024, 4097))
    w, h = (long_side, max(8, int(round(long_side / aspect)))) if aspect >= 1 else (max(8, int(round(long_side * aspect))), long_side)
    return encode_jpeg(natural_image(rng, w, h, 4.0), 90, "4:4:4"), ellipse_mask(rng, w, h)


def write_shard(path, first, count):
    """One webdataset-shaped tar: <key>.jpg then <key>.json per sample."""
    with tarfile.open(path, "w") as tf:
        for i in range(first, first + count):
            key, jpg, js = c3_item(i)
            for name, payload in ((key + ".jpg", jpg), (key + ".json", js)):
                ti = tarfile.TarInfo(name)
                ti.size = len(payload)
                tf.addfile(ti, io.BytesIO(payload))


_MAKERS = {"c0": c0_item, "c1": c1_item, "c2": c2_item, "c3": c3_item, "c4": c4_item}


def make(workload, indices, processes=0):
    """Items of `workload` for `indices`, optionally over a process pool (the encode is the slow part)."""
    fn = _MAKERS[workload]
    indices = list(indices)
    if processes and len(indices) > 8:
        import multiprocessing as mp
        with mp.get_context("fork").Pool(processes) as pool:
            return pool.map(fn, indices, chunksize=max(1, len(indices) // (processes * 8)))
    return [fn(i) for i in indices]
