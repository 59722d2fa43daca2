"""Pins the oracle's pixel arithmetic against golden fixtures made with libjpeg-turbo / Pillow."""
import glob
import io
import os

import numpy as np
import pytest

import oracle


def _golden_jpegs(golden_dir):
    dec = np.load(os.path.join(golden_dir, "decode.npz"))
    for path in sorted(glob.glob(os.path.join(golden_dir, "jpeg_*.jpg"))):
        name = os.path.basename(path)[5:-4]
        yield name, open(path, "rb").read(), dec[name]


def test_decode_matches_libjpeg_turbo_golden(golden_dir):
    n = 0
    for name, data, want in _golden_jpegs(golden_dir):
        got = oracle.jpeg_decode(data)
        assert got.shape == want.shape, name
        assert np.array_equal(got, want), name  # bit-exact
        n += 1
    assert n >= 11


def test_decode_matches_live_pillow():
    PIL = pytest.importorskip("PIL.Image")
    from datago_b200 import synth
    rng = np.random.default_rng(7)
    for (w, h, sub, q, rst) in [(160, 120, "4:2:0", 90, 0), (123, 77, "4:2:0", 76, 4), (96, 96, "4:4:4", 95, 0),
                                (200, 64, "4:2:2", 80, 3), (41, 203, "4:2:0", 88, 1)]:
        data = synth.encode_jpeg(synth.natural_image(rng, w, h, 5.0, True), q, sub, rst)
        want = np.asarray(PIL.open(io.BytesIO(data)).convert("RGB"))
        assert np.array_equal(oracle.jpeg_decode(data), want)


def test_decode_stage_outputs_are_consistent(golden_dir):
    data = open(os.path.join(golden_dir, "jpeg_420_q90.jpg"), "rb").read()
    coefs, planes, out = oracle.jpeg_decode_stages(data)
    info = oracle.jpeg_info(data)
    assert coefs[0].shape == (info.mcux * info.mcuy * 4, 64) and coefs[1].shape == (info.mcux * info.mcuy, 64)
    assert planes[0].shape == (info.mcuy * 16, info.mcux * 16)
    assert np.array_equal(out, oracle.jpeg_decode(data))


def test_decode_errors():
    with pytest.raises(oracle.OracleError):
        oracle.jpeg_decode(b"")
    with pytest.raises(oracle.OracleError):
        oracle.jpeg_decode(b"\x89PNG\r\n\x1a\n" + b"\0" * 64)


def test_resize_pillow_mode_matches_pillow_golden(golden_dir):
    z = np.load(os.path.join(golden_dir, "resize.npz"))
    i = 0
    while f"src{i}" in z:
        src, box, want = z[f"src{i}"], z[f"box{i}"], z[f"pil{i}"]
        dw, dh = want.shape[1], want.shape[0]
        got = oracle.resample(src, (box[0], box[1], box[2] - box[0], box[3] - box[1]), (dw, dh), oracle.MODE_PILLOW)
        assert np.array_equal(got, want), i  # bit-exact
        i += 1
    assert i >= 7


def test_resize_default_mode_regression_and_closeness(golden_dir):
    z = np.load(os.path.join(golden_dir, "resize.npz"))
    i = 0
    while f"src{i}" in z:
        src, box, pil, fir = z[f"src{i}"], z[f"box{i}"], z[f"pil{i}"], z[f"fir{i}"]
        dw, dh = pil.shape[1], pil.shape[0]
        got = oracle.resample(src, (box[0], box[1], box[2] - box[0], box[3] - box[1]), (dw, dh), oracle.MODE_FIR)
        assert np.array_equal(got, fir), i
        # 16-bit vs 22-bit coefficients: the same filter, a couple of LSB apart at most
        assert np.abs(got.astype(int) - pil.astype(int)).max() <= 2
        i += 1


def test_resize_integral_crop_is_a_copy():
    rng = np.random.default_rng(3)
    a = rng.integers(0, 256, (50, 80, 3), dtype=np.uint8)
    got = oracle.resample(a, (8.0, 0.0, 64.0, 50.0), (64, 50))
    assert np.array_equal(got, a[:, 8:72])


def test_resize_constant_image_stays_constant():
    a = np.full((90, 130, 3), 77, np.uint8)
    for mode in (oracle.MODE_FIR, oracle.MODE_PILLOW):
        assert (oracle.resample(a, (0, 0, 130, 90), (47, 33), mode) == 77).all()
        assert (oracle.resample(a, (0, 0, 130, 90), (200, 150), mode) == 77).all()


def test_coefficients_sum_to_one():
    start, size, k, prec = oracle.coeffs(1000, 0.0, 1000.0, 320)
    assert prec >= 4
    sums = k.sum(axis=1)
    assert np.abs(sums - (1 << prec)).max() <= 8  # rounding of ~20 taps
    assert (start >= 0).all() and (start + size <= 1000).all()


def test_crop_and_resize_half_pixel_crop():
    # 300x200 into the 272x176 bucket: height 181 -> crop top 2.5, a 6-tap vertical shift
    cfg = dict(default_image_size=224, downsampling_ratio=16, min_aspect_ratio=0.5, max_aspect_ratio=2.0)
    rng = np.random.default_rng(11)
    a = rng.integers(0, 256, (200, 300, 3), dtype=np.uint8)
    out, p = oracle.crop_and_resize(cfg, a)
    assert (p.target_w, p.target_h, p.new_w, p.new_h, p.crop_top) == (272, 176, 272, 181, 2.5)
    mid = oracle.resample(a, (0, 0, 300, 200), (272, 181))
    want = oracle.resample(mid, (0.0, 2.5, 272.0, 176.0), (272, 176))
    assert np.array_equal(out, want)


def test_to_rgb8_reference_known_answers():
    # datago src/image_processing.rs:847-920: opaque kept, transparent -> (128,128,128), (200,100,50,128) within 2 of
    # (164,114,89); gray repeated; RGB unchanged
    rgba = np.array([[[255, 100, 50, 255], [200, 100, 50, 128], [255, 0, 0, 0]]], np.uint8)
    out = oracle.to_rgb8(rgba)
    assert out[0, 0].tolist() == [255, 100, 50] and out[0, 2].tolist() == [128, 128, 128]
    assert np.all(np.abs(out[0, 1].astype(int) - [164, 114, 89]) <= 2)
    assert oracle.to_rgb8(np.array([[100]], np.uint8))[0, 0].tolist() == [100, 100, 100]
    assert oracle.to_rgb8(np.array([[[255, 100, 50]]], np.uint8))[0, 0].tolist() == [255, 100, 50]
    # against exact rational source-over: never more than one step away (f32 rounding + truncation)
    rng = np.random.default_rng(5)
    a = rng.integers(0, 256, (64, 64, 4), dtype=np.uint8)
    al = a[:, :, 3:4].astype(np.float64) / 255.0
    exact = a[:, :, :3] * al + 128.0 * (1.0 - al)
    d = oracle.to_rgb8(a).astype(np.float64) - exact
    assert d.max() <= 0.01 and d.min() > -1.01
