"""`image_to_rgb8` (datago's ImageEncoding.img_to_rgb8): payloads that are not RGB8 are converted after crop_and_resize.
Known answers are the reference's own (src/image_processing.rs:847-920, src/worker_files.rs:323-447); everything else
is compared with the oracle's restatement, bit for bit."""
import numpy as np
import pytest

import datago_b200 as dg
import oracle
from gpu_common import assert_same, ctx, jpeg

pytestmark = pytest.mark.gpu

CFG224 = dict(crop_and_resize=True, default_image_size=224, downsampling_ratio=16, min_aspect_ratio=0.5, max_aspect_ratio=2.0)


def test_reference_known_answers():
    rgba = np.array([[[255, 100, 50, 255], [200, 100, 50, 128], [255, 0, 0, 0]]], np.uint8)
    gray = np.array([[100]], np.uint8)
    rgb = np.array([[[255, 100, 50]]], np.uint8)
    res = ctx(None).process([rgba, gray, rgb], None, 0, to_rgb8=True)
    (s0, o0, r0), (s1, o1, r1), (s2, o2, r2) = res
    assert (s0, s1, s2) == (0, 0, 0)
    assert (r0.channels, r0.bit_depth, r0.width, r0.height) == (3, 8, 3, 1)
    assert o0[0, 0].tolist() == [255, 100, 50]                 # fully opaque: unchanged
    assert np.all(np.abs(o0[0, 1].astype(int) - [164, 114, 89]) <= 2)   # the tolerance the reference's test states
    assert o0[0, 2].tolist() == [128, 128, 128]                # fully transparent: the gray background
    assert r1.channels == 3 and o1[0, 0].tolist() == [100, 100, 100]
    assert r2.channels == 3 and o2[0, 0].tolist() == [255, 100, 50]


def test_every_alpha_and_value_matches_the_oracle():
    # all 256 alphas x a spread of foreground values: the f32 blend must agree with the CPU evaluation bit for bit
    rng = np.random.default_rng(91)
    a = np.zeros((256, 384, 4), np.uint8)
    a[:, :, 3] = np.arange(256, dtype=np.uint8)[:, None]
    a[:, :, :3] = rng.integers(0, 256, (256, 384, 3), dtype=np.uint8)
    a[:, :256, 0] = np.arange(256, dtype=np.uint8)[None, :]
    la = rng.integers(0, 256, (37, 53, 2), dtype=np.uint8)
    res = ctx(None).process([a, la], None, 0, to_rgb8=True)
    assert_same(res[0][1], oracle.to_rgb8(a), "rgba")
    assert_same(res[1][1], oracle.to_rgb8(la), "luma + alpha")


def test_gray_sources_are_resized_in_one_channel_then_expanded():
    rng = np.random.default_rng(92)
    gj = jpeg(rng, 333, 222, gray=True)
    raw = rng.integers(0, 256, (301, 457), dtype=np.uint8)
    cj = jpeg(rng, 200, 300)
    inputs = [gj, raw, cj, gj]
    flags = [True, True, True, False]                          # a mask beside them keeps its single channel
    c = ctx(CFG224)
    res = c.process(inputs, None, 0, to_rgb8=flags)
    for i, x in enumerate(inputs):
        st, out, r = res[i]
        assert st == 0, i
        dec = oracle.jpeg_decode(x) if isinstance(x, bytes) else x
        want, p = oracle.crop_and_resize(CFG224, dec)
        if flags[i]:
            want = oracle.to_rgb8(want) if want.ndim == 2 else want
            assert r.channels == 3
        else:
            assert r.channels == 1
        assert (r.original_width, r.original_height) == (dec.shape[1], dec.shape[0])
        assert r.plan.key.decode() == p.key.decode()
        assert_same(out, want, f"item {i}")
    # decode-only: gray JPEG -> RGB without any resize
    st, out, r = ctx(None).process([gj], None, dg.BATCH_DECODE_ONLY, to_rgb8=True)[0]
    assert st == 0 and r.channels == 3
    assert_same(out, oracle.to_rgb8(oracle.jpeg_decode(gj)), "decode-only gray")


def test_alpha_images_are_resized_with_premultiplied_colour():
    # RGBA and LA inputs: colour multiplied by alpha before each convolution resize and divided afterwards, as
    # fast_image_resize does for U8x4 / U8x2; with image_to_rgb8 the result is then composited over gray
    rng = np.random.default_rng(93)
    shapes = [(100, 150, 4), (224, 224, 4), (300, 777, 4), (640, 481, 2), (224, 229, 4), (231, 224, 2), (1500, 2200, 4)]
    raws = [rng.integers(0, 256, s, dtype=np.uint8) for s in shapes]
    raws[2][:, :, 3] = 255                                       # opaque: must equal the three-channel result
    raws[0][:40, :, 3] = 0                                       # a fully transparent band
    c = ctx(CFG224)
    plain = c.process(raws, None, 0)
    for a, (st, out, r) in zip(raws, plain):
        want, p = oracle.crop_and_resize(CFG224, a)
        assert st == 0 and r.channels == a.shape[2] and r.plan.as_tuple() == p.as_tuple()
        assert_same(out, want, f"alpha payload {a.shape}")
    opaque_rgb = oracle.crop_and_resize(CFG224, np.ascontiguousarray(raws[2][:, :, :3]))[0]
    assert np.array_equal(plain[2][1][:, :, :3], opaque_rgb) and np.all(plain[2][1][:, :, 3] == 255)
    for a, (st, out, r) in zip(raws, c.process(raws, None, 0, to_rgb8=True)):
        assert st == 0 and r.channels == 3
        assert_same(out, oracle.to_rgb8(oracle.crop_and_resize(CFG224, a)[0]), f"alpha to rgb8 {a.shape}")
    # forced bucket far from the image's aspect ratio, and a four-channel image without any transform
    (st, out, r), = c.process([raws[0]], ["1.900"], 0)
    assert st == 0
    assert_same(out, oracle.crop_and_resize(CFG224, raws[0], "1.900")[0])
    (st, out, r), = ctx(None).process([raws[0]], None, 0)
    assert st == 0 and r.channels == 4
    assert_same(out, raws[0])


def test_collated_buckets_use_the_payload_channel_count():
    rng = np.random.default_rng(94)
    grays = [rng.integers(0, 256, (300, 300), dtype=np.uint8) for _ in range(3)]
    b = ctx(CFG224).batch(grays + grays[:1], None, dg.BATCH_COLLATE, to_rgb8=[True, True, True, False])
    b.upload(); b.run()
    host = np.empty(b.packed_bytes(), np.uint8)
    b.download_packed(host)
    b.sync()
    shapes = sorted(bk["shape"] for bk in b.buckets())
    assert shapes == [(1, 224, 224, 1), (3, 224, 224, 3)]
    for bk in b.buckets():
        n, h, w, ch = bk["shape"]
        dense = host[bk["packed_offset"]:bk["packed_offset"] + bk["nbytes"]].reshape(n, h, w, ch)
        for pos, i in enumerate(bk["items"]):
            want, _ = oracle.crop_and_resize(CFG224, (grays + grays[:1])[i])
            want = oracle.to_rgb8(want) if ch == 3 else want[:, :, None]
            assert_same(dense[pos], want, f"item {i}")
    b.close()


def test_feeder_passes_the_flag_through():
    rng = np.random.default_rng(95)
    gj = jpeg(rng, 120, 80, gray=True)
    with dg.Feeder(0, None, max_batch=4, max_wait_us=300) as f:
        st, out, r = f.process_one(gj, to_rgb8=True)
        assert st == 0 and r.channels == 3
        assert_same(out, oracle.to_rgb8(oracle.jpeg_decode(gj)), "feeder")
        st, out, r = f.process_one(gj)
        assert st == 0 and r.channels == 1
