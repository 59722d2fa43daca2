"""Per-bucket collation on the device: a BATCH_COLLATE batch stores the payloads of one bucket back to back, so every
bucket is one dense uint8 [n, h, w, c] array.  Pixels must be the ones the uncollated path (and the oracle) produce;
only their placement changes."""
import numpy as np
import pytest

import datago_b200 as dg
import oracle
from datago_b200 import synth
from gpu_common import assert_same, ctx, jpeg

pytestmark = pytest.mark.gpu

CFG224 = dict(crop_and_resize=True, default_image_size=224, downsampling_ratio=16, min_aspect_ratio=0.5, max_aspect_ratio=2.0)


def _run(c, inputs, forced=None, flags=0):
    b = c.batch(inputs, forced, flags)
    b.upload()
    b.run()
    host = np.empty(max(1, b.packed_bytes()), np.uint8)
    b.download_packed(host)
    b.sync()
    return b, host


def test_buckets_are_dense_arrays_with_oracle_pixels():
    rng = np.random.default_rng(71)
    inputs, forced = [], []
    for k in range(24):
        w, h = int(rng.integers(90, 700)), int(rng.integers(90, 700))
        if k % 3 == 0:
            inputs.append(jpeg(rng, w, h, q=88, rst=(4 if k % 2 else 0)))
        elif k % 3 == 1:
            inputs.append(rng.integers(0, 256, (h, w, 3), dtype=np.uint8))
        else:
            inputs.append(rng.integers(0, 256, (h, w), dtype=np.uint8))   # a mask: one channel, its own bucket
        forced.append(None)
    inputs.append(b"not a jpeg")   # failed items belong to no bucket
    forced.append(None)
    inputs.append(inputs[1])
    forced.append("1.900")          # forced key
    c = ctx(CFG224)
    b, host = _run(c, inputs, forced, dg.BATCH_COLLATE)
    buckets = b.buckets()
    assert buckets
    seen = []
    for bk in buckets:
        n, h, w, ch = bk["shape"]
        assert n == len(bk["items"]) and bk["items"] == sorted(bk["items"])
        assert bk["packed_offset"] % 256 == 0
        dense = host[bk["packed_offset"]:bk["packed_offset"] + bk["nbytes"]].reshape(n, h, w, ch)
        on_device = c.copy_to_host(bk["array"].ptr, bk["nbytes"]).reshape(n, h, w, ch)
        assert np.array_equal(dense, on_device)
        for pos, i in enumerate(bk["items"]):
            r = b.result(i)
            assert r.status == 0 and (r.width, r.height, r.channels) == (w, h, ch)
            assert r.plan.key.decode() == bk["key"]
            assert r.packed_offset == bk["packed_offset"] + pos * h * w * ch
            src = inputs[i]
            if isinstance(src, bytes):
                src = oracle.jpeg_decode(src)
            want, _ = oracle.crop_and_resize(CFG224, src, forced[i])
            got = dense[pos] if ch == 3 else dense[pos, :, :, 0]
            assert_same(got, want, f"item {i} in bucket {bk['key']}")
            seen.append(i)
    assert sorted(seen) == [i for i in range(len(inputs)) if i != 24]
    assert b.result(24).status != 0
    keys = [(bk["key"], bk["shape"][3]) for bk in buckets]
    assert len(set(keys)) == len(keys)
    b.close()


def test_collated_equals_uncollated_without_transform_on_odd_shapes():
    # decode-only: buckets are groups of equal decoded shape; odd sizes make the tight packing unaligned
    rng = np.random.default_rng(72)
    shapes = [(37, 53), (37, 53), (129, 65), (37, 53), (129, 65), (200, 100)]
    inputs = [jpeg(rng, w, h, sub=("4:4:4" if k % 2 else "4:2:0"), q=85) for k, (w, h) in enumerate(shapes)]
    inputs.append(jpeg(rng, 37, 53, gray=True))
    c = ctx(None)
    b0, h0 = _run(c, inputs, None, dg.BATCH_DECODE_ONLY)
    b1, h1 = _run(c, inputs, None, dg.BATCH_DECODE_ONLY | dg.BATCH_COLLATE)
    assert b0.buckets() == []
    bks = b1.buckets()
    assert sorted(bk["shape"] for bk in bks) == sorted([(3, 53, 37, 3), (2, 65, 129, 3), (1, 100, 200, 3), (1, 53, 37, 1)])
    for i in range(len(inputs)):
        r0, r1 = b0.result(i), b1.result(i)
        assert r0.status == 0 and r1.status == 0 and r0.nbytes == r1.nbytes
        assert np.array_equal(h0[r0.packed_offset:r0.packed_offset + r0.nbytes], h1[r1.packed_offset:r1.packed_offset + r1.nbytes]), i
    b0.close()
    b1.close()


def test_bucket_array_wraps_as_torch_tensor_without_copy():
    torch = pytest.importorskip("torch")
    rng = np.random.default_rng(73)
    raws = [rng.integers(0, 256, (300, 300, 3), dtype=np.uint8) for _ in range(5)]
    c = ctx(CFG224)
    b, host = _run(c, raws, None, dg.BATCH_COLLATE)
    (bk,) = b.buckets()
    t = torch.as_tensor(bk["array"], device="cuda:0")
    assert tuple(t.shape) == (5, 224, 224, 3) and t.dtype == torch.uint8 and t.data_ptr() == bk["array"].ptr
    assert np.array_equal(t.cpu().numpy().reshape(-1), host[bk["packed_offset"]:bk["packed_offset"] + bk["nbytes"]])
    b.close()


def test_items_with_unusable_tables_take_no_bucket_slot():
    # a Huffman table whose code lengths over-subscribe the code space is found on the host: the item fails before the
    # buckets are laid out; an item with damaged entropy data keeps its slot and reports a status
    rng = np.random.default_rng(72)
    good = [jpeg(rng, 300, 300, q=85) for _ in range(3)]
    bad_table = bytearray(good[0])
    dht = bad_table.index(b"\xff\xc4")
    assert bad_table[dht + 5] == 0 and bad_table[dht + 7] == 5   # the standard luminance DC table
    bad_table[dht + 5], bad_table[dht + 7] = 3, 2                # three codes of length 1, the symbol count unchanged
    cut = good[1][: len(good[1]) * 2 // 3]
    c = ctx(CFG224)
    b, host = _run(c, [good[0], bytes(bad_table), good[1], cut, good[2]], None, dg.BATCH_COLLATE)
    assert b.result(1).status == 6
    assert b.result(3).status == 3
    slots = [i for bk in b.buckets() for i in bk["items"]]
    assert sorted(slots) == [0, 2, 3, 4]
    for bk in b.buckets():
        n, h, w, ch = bk["shape"]
        dense = host[bk["packed_offset"]:bk["packed_offset"] + bk["nbytes"]].reshape(n, h, w, ch)
        for pos, i in enumerate(bk["items"]):
            if b.result(i).status == 0:
                assert_same(dense[pos], oracle.jpeg_to_payload([good[0], None, good[1], None, good[2]][i], CFG224)[0])
    b.close()
