"""CUDA crop_and_resize on raw pixels and on decoded JPEGs against the oracle: bucket and crop offsets bit-exact,
pixels bit-exact (tolerance 0 LSB; the north-star bar against the reference CPU resizer is max |d| <= 1)."""
import numpy as np
import pytest

import datago_b200 as dg
import oracle
from datago_b200 import synth
from gpu_common import assert_same, ctx, jpeg

pytestmark = pytest.mark.gpu

C0 = synth.IMAGE_CONFIGS["c0"]
C1 = synth.IMAGE_CONFIGS["c1"]
C4 = synth.IMAGE_CONFIGS["c4"]
CFG224 = dict(crop_and_resize=True, default_image_size=224, downsampling_ratio=16, min_aspect_ratio=0.5, max_aspect_ratio=2.0)


def _check_raw(cfg, raws, forced=None):
    res = ctx(cfg).process(raws, forced)
    for i, (a, (st, out, r)) in enumerate(zip(raws, res)):
        want, p = oracle.crop_and_resize(cfg, a, forced[i] if forced else None)
        assert st == 0, i
        assert r.plan.as_tuple() == p.as_tuple(), i   # bucket key, sizes, crop offsets: bit-exact
        assert (r.width, r.height) == (p.target_w, p.target_h)
        assert (r.original_width, r.original_height) == (a.shape[1], a.shape[0])
        assert_same(out, want, f"item {i} {a.shape}")


def test_raw_resize_matrix():
    rng = np.random.default_rng(21)
    sizes = [(640, 480), (513, 777), (1000, 1000), (512, 512), (2048, 1024), (1500, 701), (300, 200), (4096, 512),
             (512, 4096), (1023, 1025), (3000, 2000), (17, 900), (900, 17), (1, 1), (2, 3)]
    raws = [rng.integers(0, 256, (h, w, 3), dtype=np.uint8) for (w, h) in sizes]
    raws += [rng.integers(0, 256, (600, 900), dtype=np.uint8), rng.integers(0, 256, (1333, 777), dtype=np.uint8)]
    _check_raw(C1, raws)


def test_reference_dimension_asserts():
    # datago src/image_processing.rs:463-477
    rng = np.random.default_rng(22)
    a = rng.integers(0, 256, (200, 300, 3), dtype=np.uint8)
    b = rng.integers(0, 256, (200, 400, 3), dtype=np.uint8)
    res = ctx(CFG224).process([a, a, b], ["1.000", "1.900", None])
    assert [(r.width, r.height) for _, _, r in res] == [(224, 224), (304, 160), (304, 160)]
    _check_raw(CFG224, [a, a, b], ["1.000", "1.900", None])


def test_half_pixel_and_integral_crops_both_axes():
    rng = np.random.default_rng(23)
    raws, seen = [], set()
    for _ in range(400):
        w, h = int(rng.integers(100, 900)), int(rng.integers(100, 900))
        p = oracle.plan_geometry(CFG224, w, h)
        kind = (p.crop_left > 0, p.crop_top > 0, (p.crop_left % 1) != 0 or (p.crop_top % 1) != 0, p.new_w > w)
        if kind not in seen:
            seen.add(kind)
            raws.append(rng.integers(0, 256, (h, w, 3), dtype=np.uint8))
    assert len(raws) >= 6
    _check_raw(CFG224, raws)


def test_identity_and_same_scale_crop():
    rng = np.random.default_rng(24)
    raws = [rng.integers(0, 256, (224, 224, 3), dtype=np.uint8),   # identity
            rng.integers(0, 256, (224, 230, 3), dtype=np.uint8),   # scale 1, integral crop (left 3)
            rng.integers(0, 256, (224, 229, 3), dtype=np.uint8),   # scale 1, half-pixel crop (left 2.5)
            rng.integers(0, 256, (231, 224), dtype=np.uint8)]      # gray, half-pixel vertical crop
    _check_raw(CFG224, raws, ["1.000"] * 4)


def test_forced_key_far_from_own_aspect():
    rng = np.random.default_rng(25)
    raws = [rng.integers(0, 256, (300, 900, 3), dtype=np.uint8), rng.integers(0, 256, (900, 300), dtype=np.uint8)]
    _check_raw(C1, raws, ["0.489", "2.045"])
    res = ctx(C1).process(raws, ["7.777", None])
    assert res[0][0] == 8 and res[1][0] == 0   # unknown key: that item fails, the other is processed


def test_jpeg_to_payload_c0_style():
    rng = np.random.default_rng(26)
    datas = [jpeg(rng, w, h, "4:2:0", 90) for (w, h) in [(256, 2048), (2048, 256), (1024, 1024), (1032, 1024), (776, 1000), (1784, 1000), (264, 256)]]
    datas.append(jpeg(rng, 640, 800, None, 85, 0, True))
    res = ctx(C0).process(datas)
    for i, (data, (st, out, r)) in enumerate(zip(datas, res)):
        want, p = oracle.jpeg_to_payload(data, C0)
        assert st == 0
        assert r.plan.as_tuple() == p.as_tuple()
        assert_same(out, want, f"item {i}")


def test_decoded_intermediate_is_the_decoded_image():
    rng = np.random.default_rng(27)
    datas = [jpeg(rng, 500, 400), jpeg(rng, 300, 700, rst=4)]
    with ctx(C0).batch(datas) as b:
        b.upload(); b.run(); b.sync()
        for i, d in enumerate(datas):
            assert_same(b.debug_decoded(i), oracle.jpeg_decode(d))


def test_multi_payload_sample_shares_the_bucket():
    # src/worker_wds.rs:68-76: the first image fixes the key, later payloads (here an L8 mask) are forced into it
    rng = np.random.default_rng(28)
    img = jpeg(rng, 1500, 1100, "4:4:4", 90)
    mask = synth.ellipse_mask(rng, 1500, 1100)
    c = ctx(C4)
    first = c.plan_geometry(1500, 1100, 3)
    key = dg.aspect_ratio_to_str(first.target_w, first.target_h)
    assert key == first.key.decode()
    res = c.process([img, mask], [None, key])
    (st0, out0, r0), (st1, out1, r1) = res
    assert st0 == 0 and st1 == 0
    assert (r0.width, r0.height) == (r1.width, r1.height) and r1.channels == 1 and r0.channels == 3
    assert_same(out0, oracle.jpeg_to_payload(img, C4)[0])
    assert_same(out1, oracle.crop_and_resize(C4, mask, key)[0])


def test_decode_only_flag_ignores_the_transform():
    rng = np.random.default_rng(29)
    d = jpeg(rng, 333, 444)
    (st, out, r), = ctx(C0).process([d], None, dg.BATCH_DECODE_ONLY)
    assert st == 0 and (r.width, r.height) == (333, 444)
    assert_same(out, oracle.jpeg_decode(d))


def test_stage_timers_and_counters():
    rng = np.random.default_rng(30)
    datas = [jpeg(rng, 640, 480), jpeg(rng, 640, 480, rst=4)]
    with ctx(C0).batch(datas, None, dg.BATCH_TIMING) as b:
        b.upload(); b.run(); b.sync()
        ms = b.stage_ms()
        c = b.counters()
        assert c["kernel_launches"] >= 6 and c["h2d_bytes"] > sum(len(d) for d in datas) // 2
        assert ms["huff_spec"] > 0 and ms["huff_restart"] > 0 and ms["idct"] > 0 and ms["color"] > 0


def test_packed_download_matches_per_item_download():
    rng = np.random.default_rng(33)
    datas = [jpeg(rng, 300, 200), jpeg(rng, 640, 480, rst=4), b"junk", jpeg(rng, 100, 333, None, 80, 0, True)]
    c = ctx(C0)
    per_item = c.process(datas)
    with c.batch(datas) as b:
        b.upload(); b.run()
        buf = np.zeros(b.packed_bytes(), np.uint8)
        b.download_packed(buf)
        b.sync()
        for i, (st, want, _) in enumerate(per_item):
            r = b.result(i)
            assert r.status == st
            if st == 0:
                assert r.packed_offset % 256 == 0
                assert np.array_equal(buf[r.packed_offset:r.packed_offset + r.nbytes], want.reshape(-1))


def test_raw_input_without_transform_is_returned_unchanged():
    # image_to_payload with img_tfm None (src/image_processing.rs:354-361 skipped): the payload is the image itself
    rng = np.random.default_rng(29)
    raws = [rng.integers(0, 256, (33, 47, 3), dtype=np.uint8), rng.integers(0, 256, (200, 1000), dtype=np.uint8),
            rng.integers(0, 256, (1, 1, 3), dtype=np.uint8)]
    mixed = [raws[0], jpeg(rng, 120, 90), raws[1], raws[2]]
    for c in (ctx(None), ctx(C1)):
        res = c.process(mixed, None, dg.BATCH_DECODE_ONLY)
        for i, a in ((0, raws[0]), (2, raws[1]), (3, raws[2])):
            st, out, r = res[i]
            assert st == 0 and (r.width, r.height) == (a.shape[1], a.shape[0])
            assert_same(out, a, f"raw item {i}")
        assert_same(res[1][1], oracle.jpeg_decode(mixed[1]), "the JPEG beside them")


def test_filter_table_cache_can_be_dropped_at_any_time(monkeypatch):
    # a context keeps the Lanczos tables it has built; with a tiny cap the cache is emptied again and again, and a
    # batch must keep the tables it uses alive by itself
    monkeypatch.setenv("DATAGO_B200_TABLE_CACHE_MB", "0")
    small = dg.Context(0, C1)
    monkeypatch.delenv("DATAGO_B200_TABLE_CACHE_MB")
    rng = np.random.default_rng(31)
    raws = [rng.integers(0, 256, (int(rng.integers(300, 900)), int(rng.integers(300, 900)), 3), dtype=np.uint8) for _ in range(12)]
    for _ in range(2):   # second round: same sizes again (cache hits in a normal context, rebuilds here)
        for a, (st, out, r) in zip(raws, small.process(raws)):
            want, p = oracle.crop_and_resize(C1, a)
            assert st == 0 and r.plan.as_tuple() == p.as_tuple()
            assert_same(out, want, f"{a.shape}")
        for a, (st, out, r) in zip(raws, ctx(C1).process(raws)):
            assert_same(out, oracle.crop_and_resize(C1, a)[0], f"cached {a.shape}")
    small.close()


def test_both_horizontal_kernels_agree_with_the_oracle():
    # horizontal passes run on the tensor-core kernel where their geometry fits; DATAGO_B200_HMMA=0 keeps every pass on
    # the dp2a kernel.  Both must give the oracle's bytes: a mix of scales (up, slightly down, 8x down), channel counts,
    # odd widths, and a pass too wide for the tensor-core path (downscale beyond 10x) in the same batch.
    import os
    rng = np.random.default_rng(26)
    sizes = [(640, 480, 3), (4096, 4096, 3), (3000, 777, 3), (513, 1025, 1), (300, 200, 3), (4001, 1999, 1), (1201, 900, 3)]
    raws = [rng.integers(0, 256, (h, w, c) if c == 3 else (h, w), dtype=np.uint8) for (w, h, c) in sizes]
    wide = rng.integers(0, 256, (700, 9000, 3), dtype=np.uint8)   # 9000 -> 720: 12.5x, beyond what a CTA can stage
    raws.append(wide)
    wants = [oracle.crop_and_resize(C1, a)[0] for a in raws]
    old = os.environ.get("DATAGO_B200_HMMA")
    try:
        for flag in ("1", "0"):
            os.environ["DATAGO_B200_HMMA"] = flag
            c = dg.Context(0, C1)
            try:
                for i, (st, out, _) in enumerate(c.process(raws)):
                    assert st == 0
                    assert_same(out, wants[i], f"HMMA={flag} item {i} {raws[i].shape}")
            finally:
                c.close()
    finally:
        if old is None:
            os.environ.pop("DATAGO_B200_HMMA", None)
        else:
            os.environ["DATAGO_B200_HMMA"] = old


def test_tensor_core_passes_at_their_tile_edges():
    # outputs wider than one column range of the vertical tensor-core pass (4096 bytes) and taller than many row tiles,
    # strong enlargements (short bands), and reductions beyond what the tensor-core passes stage (> 9x: the dp2a kernels)
    rng = np.random.default_rng(27)
    big = [rng.integers(0, 256, (1500, 3000, 3), dtype=np.uint8),   # 2048/64 bucket about 2880 x 1472: three column ranges
           rng.integers(0, 256, (200, 300, 3), dtype=np.uint8),     # enlarged about 9x
           rng.integers(0, 256, (2900, 1400), dtype=np.uint8),      # gray, tall
           rng.integers(0, 256, (70, 4000, 3), dtype=np.uint8)]     # far from every bucket: heavy crop
    _check_raw(C4, big)
    small = [rng.integers(0, 256, (3000, 4000, 3), dtype=np.uint8),  # 224-bucket: about 13x reduction
             rng.integers(0, 256, (2300, 2300), dtype=np.uint8),    # gray, about 10x
             rng.integers(0, 256, (1900, 1700, 3), dtype=np.uint8)]  # about 8x: still on the tensor cores
    _check_raw(CFG224, small)
