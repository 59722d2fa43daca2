"""Shared helpers of the GPU parity tests (the oracle is the checker, the C-ABI library is the thing checked)."""
import io

import numpy as np

import datago_b200 as dg
import oracle
from datago_b200 import synth

_CTX = {}


def ctx(image_config=None):
    key = None if image_config is None else tuple(sorted(image_config.items()))
    if key not in _CTX:
        _CTX[key] = dg.Context(0, image_config)
    return _CTX[key]


def jpeg(rng, w, h, sub="4:2:0", q=90, rst=0, gray=False, noise=5.0):
    a = synth.natural_image(rng, w, h, noise, edges=True)
    if gray:
        from PIL import Image
        b = io.BytesIO()
        kw = dict(quality=q)
        if rst:
            kw["restart_marker_blocks"] = rst
        Image.fromarray(a[:, :, 0]).save(b, "JPEG", **kw)
        return b.getvalue()
    return synth.encode_jpeg(a, q, sub, rst)


def scan_order(coefs, info):
    """Oracle coefficients (raster order per component) rearranged into MCU scan order."""
    if info.channels == 1:
        return coefs[0]
    hs, vs, mx, my = info.hsamp, info.vsamp, info.mcux, info.mcuy
    y = coefs[0].reshape(my, vs, mx, hs, 64).transpose(0, 2, 1, 3, 4).reshape(my * mx, vs * hs, 64)
    cb = coefs[1].reshape(my * mx, 1, 64)
    cr = coefs[2].reshape(my * mx, 1, 64)
    return np.concatenate([y, cb, cr], axis=1).reshape(-1, 64)


def assert_same(got, want, what=""):
    assert got is not None, what
    assert got.shape == want.shape, (what, got.shape, want.shape)
    if not np.array_equal(got, want):
        d = np.abs(got.astype(int) - want.astype(int))
        raise AssertionError(f"{what}: {int((d > 0).sum())} of {d.size} bytes differ, max |d| = {int(d.max())}")
