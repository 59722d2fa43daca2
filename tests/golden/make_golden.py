"""Regenerates the golden fixtures in this folder.  Run from the repository root: python tests/golden/make_golden.py

The reference (datago) cannot be built or imported here, and its own tests hold no pixel values, so the fixtures pin
the oracle against the independent implementations that ARE available:
  * jpeg_*.jpg + decode.npz : baseline JPEGs written by Pillow/libjpeg-turbo and the pixels Pillow decodes from them
                              (libjpeg-turbo: islow IDCT, fancy upsampling) -- pins oracle.jpeg_decode bit-exactly;
  * resize.npz              : random images and what PIL.Image.resize(LANCZOS, box=...) returns for them -- pins the
                              oracle's Pillow-coefficient mode bit-exactly (same convolution code as the default mode,
                              which differs only in how the f64 weights are quantised);
  * buckets.json            : bucket tables and geometry known answers; the 224/16 rows are the asserts of datago's
                              src/image_processing.rs:441-478, the rest is derived with oracle.plan_geometry and kept as a
                              regression anchor.
"""
import io
import json
import os
import sys

import numpy as np
from PIL import Image

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.join(HERE, "..", ".."))
import oracle  # noqa: E402
from datago_b200 import synth  # noqa: E402

JPEG_CASES = [  # name, w, h, subsampling, quality, restart blocks, gray
    ("420_q90", 64, 48, "4:2:0", 90, 0, False),
    ("420_q75_rst2", 80, 64, "4:2:0", 75, 2, False),
    ("420_odd", 37, 53, "4:2:0", 85, 0, False),
    ("420_odd_rst4", 129, 67, "4:2:0", 95, 4, False),
    ("444_q90", 56, 40, "4:4:4", 90, 0, False),
    ("444_odd_rst1", 33, 17, "4:4:4", 50, 1, False),
    ("422_q85", 72, 40, "4:2:2", 85, 0, False),
    ("gray_q80", 90, 70, None, 80, 0, True),
    ("gray_rst3", 50, 60, None, 60, 3, True),
    ("tiny_3x3", 3, 3, "4:2:0", 90, 0, False),
    ("tiny_1x1", 1, 1, "4:2:0", 90, 0, False),
]

RESIZE_CASES = [  # src w, h, channels, out w, h, box (left, top, right, bottom) or None
    (60, 40, 3, 67, 45, None),
    (200, 140, 3, 64, 45, None),
    (97, 131, 1, 40, 54, None),
    (70, 64, 3, 64, 64, (3.0, 0.0, 67.0, 64.0)),
    (71, 64, 3, 64, 64, (3.5, 0.0, 67.5, 64.0)),
    (64, 75, 1, 64, 64, (0.0, 5.5, 64.0, 69.5)),
    (120, 90, 3, 33, 29, (2.25, 7.5, 100.75, 80.0)),
]


def main():
    rng = np.random.default_rng(20240607)
    decoded = {}
    for name, w, h, sub, q, rst, gray in JPEG_CASES:
        a = synth.natural_image(rng, w, h, 6.0, edges=True)
        if gray:
            a = a[:, :, 0]
        kw = dict(quality=q, progressive=False, optimize=False)
        if sub:
            kw["subsampling"] = sub
        if rst:
            kw["restart_marker_blocks"] = rst
        b = io.BytesIO()
        Image.fromarray(a).save(b, "JPEG", **kw)
        data = b.getvalue()
        with open(os.path.join(HERE, f"jpeg_{name}.jpg"), "wb") as f:
            f.write(data)
        im = Image.open(io.BytesIO(data))
        decoded[name] = np.asarray(im if gray else im.convert("RGB"))
    np.savez_compressed(os.path.join(HERE, "decode.npz"), **decoded)

    rs = {}
    for i, (w, h, c, dw, dh, box) in enumerate(RESIZE_CASES):
        a = rng.integers(0, 256, (h, w, c) if c == 3 else (h, w), dtype=np.uint8)
        bx = box or (0.0, 0.0, float(w), float(h))
        out = np.asarray(Image.fromarray(a).resize((dw, dh), Image.LANCZOS, box=bx))
        rs[f"src{i}"] = a
        rs[f"box{i}"] = np.array(bx, np.float64)
        rs[f"pil{i}"] = out
        rs[f"fir{i}"] = oracle.resample(a, (bx[0], bx[1], bx[2] - bx[0], bx[3] - bx[1]), (dw, dh), oracle.MODE_FIR)
    np.savez_compressed(os.path.join(HERE, "resize.npz"), **rs)

    kat = {"tables": {}, "plans": []}
    for size, ratio in ((224, 16), (1024, 32), (512, 16), (2048, 64)):
        cfg = dict(default_image_size=size, downsampling_ratio=ratio, min_aspect_ratio=0.5, max_aspect_ratio=2.0)
        kat["tables"][f"{size}/{ratio}"] = [[k, w, h] for k, _, w, h in oracle.bucket_table(cfg)]
        for (w, h, key) in [(100, 100, None), (200, 100, None), (100, 200, None), (400, 200, None), (300, 200, None),
                            (300, 200, "1.000"), (1784, 1000, None), (999, 1501, None), (2048, 2048, None),
                            (4096, 512, None), (640, 481, None), (513, 777, None)]:
            p = oracle.plan_geometry(cfg, w, h, key)
            kat["plans"].append(dict(size=size, ratio=ratio, w=w, h=h, forced=key, plan=list(p.as_tuple())))
    with open(os.path.join(HERE, "buckets.json"), "w") as f:
        json.dump(kat, f, indent=1)


if __name__ == "__main__":
    main()
