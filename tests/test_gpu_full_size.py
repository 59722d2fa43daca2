"""Full-size workloads: samples drawn from the benchmark generators at their real sizes.  The oracle is too slow to
check thousands of images, so a slice is compared exactly and the rest through size-independent properties."""
import numpy as np
import pytest

import datago_b200 as dg
import oracle
from datago_b200 import synth
from gpu_common import assert_same, ctx

pytestmark = pytest.mark.gpu


def test_c2_slice_bit_exact():
    idx = [0, 1, 2, 3, 17, 18]
    datas = synth.make("c2", idx)
    res = ctx().process(datas)
    for i, d, (st, out, _) in zip(idx, datas, res):
        assert st == 0
        assert_same(out, oracle.jpeg_decode(d), f"c2[{i}]")


def test_c0_slice_bit_exact():
    cfg = synth.IMAGE_CONFIGS["c0"]
    datas = synth.make("c0", [0, 1, 2])
    for d, (st, out, r) in zip(datas, ctx(cfg).process(datas)):
        want, p = oracle.jpeg_to_payload(d, cfg)
        assert st == 0 and r.plan.as_tuple() == p.as_tuple()
        assert_same(out, want)


def test_c1_slice_bit_exact():
    cfg = synth.IMAGE_CONFIGS["c1"]
    raws = synth.make("c1", [0, 1, 2])
    for a, (st, out, r) in zip(raws, ctx(cfg).process(raws)):
        want, p = oracle.crop_and_resize(cfg, a)
        assert st == 0 and r.plan.as_tuple() == p.as_tuple()
        assert_same(out, want)


def test_c4_pair_bit_exact():
    cfg = synth.IMAGE_CONFIGS["c4"]
    jpg, mask = synth.c4_item(3)
    info = dg.jpeg_probe(jpg)
    key = ctx(cfg).plan_geometry(info.width, info.height, 3).key.decode()
    (s0, o0, r0), (s1, o1, r1) = ctx(cfg).process([jpg, mask], [None, key])
    assert s0 == 0 and s1 == 0 and (r0.width, r0.height) == (r1.width, r1.height)
    assert_same(o0, oracle.jpeg_to_payload(jpg, cfg)[0])
    assert_same(o1, oracle.crop_and_resize(cfg, mask, key)[0])


def test_batch_order_and_batching_do_not_change_results():
    # property: an image's payload does not depend on its neighbours, their order, or the wave it lands in
    datas = synth.make("c2", range(40, 72), processes=4)
    a = ctx().process(datas)
    perm = np.random.default_rng(0).permutation(len(datas))
    b = ctx().process([datas[i] for i in perm])
    for k, i in enumerate(perm):
        assert a[i][0] == 0 and b[k][0] == 0
        assert np.array_equal(a[i][1], b[k][1])
    singles = [ctx().process([datas[i]])[0] for i in (0, 5, 9)]
    for s, i in zip(singles, (0, 5, 9)):
        assert np.array_equal(s[1], a[i][1])


def test_restart_and_plain_encodings_of_one_image_decode_identically():
    # property: restart markers change the bitstream, not the pixels; the two entropy-decoder paths must agree
    rng = np.random.default_rng(31)
    img = synth.natural_image(rng, 1536, 1024, 3.0, edges=True)
    plain = synth.encode_jpeg(img, 88, "4:2:0", 0)
    outs = [ctx().process([synth.encode_jpeg(img, 88, "4:2:0", r)])[0] for r in (0, 1, 4, 96, 5000)]
    assert all(o[0] == 0 for o in outs)
    for o in outs[1:]:
        assert np.array_equal(o[1], outs[0][1])
    assert_same(outs[0][1], oracle.jpeg_decode(plain))
