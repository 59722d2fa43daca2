"""Parity of the code paths that only large batches reach: the narrow-CTA instantiation of the speculative entropy
decoder (picked when a launch holds at least 1024 restart-free images), batches of several waves (two stream lanes,
auxiliary streams, scratch blocks reused with a carried zero prefix, the IDCT's zero write-back) and the L2-sized
IDCT / colour launch groups.  Every payload is compared with the oracle, bit for bit."""
import os
from concurrent.futures import ThreadPoolExecutor

import numpy as np
import pytest

import datago_b200 as dg
import oracle
from datago_b200 import synth
from gpu_common import assert_same, ctx, jpeg, scan_order

pytestmark = pytest.mark.gpu


def _oracle_all(datas):
    with ThreadPoolExecutor(os.cpu_count() or 4) as ex:  # ctypes drops the GIL inside the oracle
        return list(ex.map(oracle.jpeg_decode, datas))


def test_many_restart_free_images_in_one_launch():
    # >= 1024 restart-free images in one wave select the 256-thread decoder CTA; a few long streams need more
    # than 256 subsequences, i.e. several chunks with the decoder state carried between them
    rng = np.random.default_rng(101)
    datas = []
    for i in range(1100):
        w, h = int(rng.integers(6, 13)) * 8, int(rng.integers(4, 9)) * 8
        datas.append(jpeg(rng, w, h, "4:2:0" if i % 3 else "4:4:4", int(rng.integers(60, 96)), 0, gray=(i % 17 == 0)))
    for _ in range(3):  # noisy and large: well over 256 subsequences of 2048 bits
        datas.append(synth.encode_jpeg(rng.integers(0, 256, (512, 640, 3), dtype=np.uint8), 95, "4:2:0", 0))
    assert min(len(d) for d in datas[-3:]) * 8 > 300 * 2048
    want = _oracle_all(datas)
    with ctx().batch(datas, None, dg.BATCH_KEEP_COEFFICIENTS) as b:
        b.upload(); b.run()
        outs = b.download(); b.sync()
        for i in range(len(datas)):
            assert b.result(i).status == 0, i
            assert_same(outs[i], want[i], f"image {i}")
        for i in (0, 1, 16, 17, 1099, 1100, 1102):  # coefficients of a sample, the long streams included
            coefs, _, _ = oracle.jpeg_decode_stages(datas[i])
            assert np.array_equal(b.debug_coefficients(i), scan_order(coefs, oracle.jpeg_info(datas[i]))), i
        st = b.huffman_stats()
        assert st["chunks"] >= 1100 + 3 * 2  # every image at least one chunk, the long ones several


def _with_env(name, value):
    class _Env:
        def __enter__(self):
            self.old = os.environ.get(name)
            os.environ[name] = value

        def __exit__(self, *a):
            if self.old is None:
                os.environ.pop(name, None)
            else:
                os.environ[name] = self.old
    return _Env()


def _multi_wave_case(extra_env=None):
    datas = synth.make("c2", range(100, 140), processes=4)  # even: restart-free, odd: restart interval 4
    datas.append(jpeg(np.random.default_rng(7), 200, 120, None, 80, 0, True))
    want = _oracle_all(datas)
    envs = [_with_env("DATAGO_B200_WAVE_MB", "16")] + ([_with_env(*extra_env)] if extra_env else [])
    for e in envs:
        e.__enter__()
    try:
        c = dg.Context(0, None)  # the limits are read when a context is created
    finally:
        for e in reversed(envs):
            e.__exit__()
    try:
        with c.batch(datas) as b:
            b.upload()
            for rerun in range(2):  # the second pass reuses both scratch blocks: they must have been left zeroed
                b.run()
                outs = b.download(); b.sync()
                for i in range(len(datas)):
                    assert b.result(i).status == 0, (rerun, i)
                    assert_same(outs[i], want[i], f"pass {rerun} image {i}")
            assert b.counters()["kernel_launches"] >= 3 * 4  # at least three waves
        # a second, different batch on the same context inherits the scratch blocks and their zero prefix
        other = [datas[i] for i in (5, 2, 40, 9, 12, 1)]
        with c.batch(other) as b:
            b.upload(); b.run()
            outs = b.download(); b.sync()
            for k, i in enumerate((5, 2, 40, 9, 12, 1)):
                assert_same(outs[k], want[i], f"follow-up batch image {i}")
    finally:
        c.close()


def test_multi_wave_batch_two_lanes_bit_exact():
    _multi_wave_case()


def test_multi_wave_batch_with_l2_groups_bit_exact():
    _multi_wave_case(("DATAGO_B200_L2_GROUP_MB", "8"))


def test_multi_wave_decode_and_resize_bit_exact():
    # decode + bucket crop/resize across several waves: the full-size decoded images live in the reused scratch blocks
    cfg = synth.IMAGE_CONFIGS["c0"]
    datas = synth.make("c0", range(8, 20), processes=4)
    with _with_env("DATAGO_B200_WAVE_MB", "16"):
        c = dg.Context(0, cfg)
    try:
        with c.batch(datas) as b:
            b.upload()
            for rerun in range(2):
                b.run()
                outs = b.download(); b.sync()
                for i, d in enumerate(datas):
                    want, p = oracle.jpeg_to_payload(d, cfg)
                    assert b.result(i).status == 0 and b.result(i).plan.as_tuple() == p.as_tuple()
                    assert_same(outs[i], want, f"pass {rerun} image {i}")
    finally:
        c.close()


def test_general_kernels_still_decode_420_images():
    # three-component 4:2:0 images normally take the fused kernels; with DATAGO_B200_FUSED=0 they go through the general
    # IDCT and colour kernels (the path of every other sampling), which must give the same bytes
    rng = np.random.default_rng(202)
    datas = [jpeg(rng, 640, 480), jpeg(rng, 257, 131, rst=4), jpeg(rng, 17, 33), jpeg(rng, 1024, 768, q=70),
             jpeg(rng, 100, 60, "4:4:4"), jpeg(rng, 90, 70, None, 80, 0, True)]
    want = _oracle_all(datas)
    with _with_env("DATAGO_B200_FUSED", "0"):
        c = dg.Context(0, None)
    try:
        for i, (st, out, _) in enumerate(c.process(datas)):
            assert st == 0
            assert_same(out, want[i], f"general path image {i}")
    finally:
        c.close()
    for i, (st, out, _) in enumerate(ctx().process(datas)):
        assert st == 0
        assert_same(out, want[i], f"fused path image {i}")


def test_longest_images_take_the_widest_decoder_beside_the_others():
    # images with more than 1024 subsequences are decoded by 1024-thread CTAs on the lane's auxiliary stream while the
    # rest of the wave goes through the ordinary variant; alone in a batch they run on the main stream
    rng = np.random.default_rng(303)
    big = [synth.encode_jpeg(rng.integers(0, 256, (1024, 1024, 3), dtype=np.uint8), 97, "4:4:4", 0),
           synth.encode_jpeg(rng.integers(0, 256, (1400, 900, 3), dtype=np.uint8), 95, "4:2:0", 0)]
    assert all(len(b) > 400_000 for b in big)
    small = [jpeg(rng, 320, 200), jpeg(rng, 200, 320, rst=3), jpeg(rng, 640, 480, q=95, noise=20.0)]
    datas = [small[0], big[0], small[1], big[1], small[2]]
    want = _oracle_all(datas)
    for batch in (datas, big, [big[1]]):
        for (st, out, _), d in zip(ctx().process(batch), batch):
            assert st == 0
            assert_same(out, want[datas.index(d)], f"{len(d)} bytes")
