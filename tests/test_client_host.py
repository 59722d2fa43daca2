"""Host-side pieces of the DatagoClient harness that need no GPU: config checks, file enumeration with rank slices,
local tar (webdataset) reading, sample grouping and key-hash sharding.  Mirrors the assertions of datago's own
multi-rank tests (src/generator_files.rs:362-424, src/generator_wds.rs:651-706): ranks are disjoint and cover."""
import io
import json
import os
import tarfile

import numpy as np
import pytest

import oracle
from datago_b200 import client


def _tar(path, entries):
    with tarfile.open(path, "w") as tf:
        for name, payload in entries:
            ti = tarfile.TarInfo(name)
            ti.size = len(payload)
            tf.addfile(ti, io.BytesIO(payload))


def test_check_config_mirrors_reference_rules():
    ok = dict(source_type="file", source_config=dict(root_path="/tmp", rank=0, world_size=1), limit=10, samples_buffer_size=4)
    assert client.DatagoClient._check_config(json.dumps(ok)) is not None
    for bad in (dict(ok, limit=0), dict(ok, samples_buffer_size=0),
                dict(ok, source_config=dict(root_path="/tmp", rank=2, world_size=2)),
                dict(ok, source_config=dict(root_path="/tmp", rank=0, world_size=0))):
        assert client.DatagoClient._check_config(json.dumps(bad)) is None
    assert client.DatagoClient._check_config("not json") is None
    assert client.DatagoClient._check_config(json.dumps(dict(limit=1))) is None


def test_enumerate_files_filters_limits_and_slices(tmp_path):
    for i in range(23):
        (tmp_path / f"img_{i:02d}.jpg").write_bytes(b"x")
    (tmp_path / "notes.txt").write_bytes(b"x")
    (tmp_path / "sub").mkdir()
    (tmp_path / "sub" / "deep.PNG").write_bytes(b"x")
    files = client.enumerate_files(str(tmp_path), 100)
    assert len(files) == 24 and not any(f.endswith(".txt") for f in files)
    assert len(client.enumerate_files(str(tmp_path), 5)) == 6        # ceil(1.1 * 5)
    r0 = client.enumerate_files(str(tmp_path), 100, 0, 2)
    r1 = client.enumerate_files(str(tmp_path), 100, 1, 2)
    assert len(r0) == 12 and len(r1) == 12 and not set(r0) & set(r1) and set(r0) | set(r1) == set(files)


def test_expand_shards(tmp_path):
    for i in range(3):
        (tmp_path / f"shard-{i:03d}.tar").write_bytes(b"")
    want = [str(tmp_path / f"shard-{i:03d}.tar") for i in range(3)]
    assert client.expand_shards(str(tmp_path / "shard-{000..002}.tar")) == want
    assert client.expand_shards(str(tmp_path / "shard-*.tar")) == want


def test_tar_samples_group_by_key_and_put_the_reference_image_first(tmp_path):
    path = str(tmp_path / "s.tar")
    _tar(path, [("a.json", b"{}"), ("a.mask.png", b"m"), ("a.jpg", b"J"), ("b.jpg", b"K"), ("b.txt", b"t"), ("c.cls", b"3")])
    got = [[n for n, _ in files] for _, files in client.tar_samples(path)]
    # key = basename without the LAST extension: "a.mask" is its own key (src/generator_wds.rs:133-138)
    assert got == [["a.json"], ["a.mask.png"], ["a.jpg"], ["b.jpg", "b.txt"], ["c.cls"]]
    _tar(path, [("x.json", b"{}"), ("x.png", b"m"), ("x.jpg", b"J"), ("y.txt", b"t"), ("y.jpg", b"K")])
    got = [[n for n, _ in files] for _, files in client.tar_samples(path)]
    assert got == [["x.jpg", "x.json", "x.png"], ["y.jpg", "y.txt"]]


def test_tar_key_hash_sharding_is_disjoint_and_covers(tmp_path):
    path = str(tmp_path / "s.tar")
    keys = ["%06d_%04d" % (0, i) for i in range(200)]
    _tar(path, [(k + ext, b"p") for k in keys for ext in (".jpg", ".json")])
    seen = []
    for rank in range(4):
        mine = [os.path.splitext(files[0][0])[0] for _, files in client.tar_samples(path, "jpg", rank, 4)]
        assert all(oracle.key_hash(k) % 4 == rank for k in mine)
        seen += mine
    assert sorted(seen) == keys


def test_image_payload_behaves_like_the_reference_python_payload():
    # src/structs.rs:191-224: __call__ -> PIL image, get_payload -> the plain record, other attributes -> the PIL image
    from datago_b200.client import ImagePayload
    a = np.arange(5 * 7 * 3, dtype=np.uint8).reshape(5, 7, 3)
    p = ImagePayload(a.tobytes(), 50, 70, 5, 7, 3, 8, False)
    assert p().size == (7, 5) and p().mode == "RGB"
    assert p.size == (7, 5) and p.mode == "RGB"          # delegated to the PIL image
    assert p.resize((3, 2)).size == (3, 2)
    q = p.get_payload()
    assert q is not p and q.data == p.data and (q.height, q.width, q.channels, q.original_width) == (5, 7, 3, 70)
    assert np.array_equal(p.to_numpy_array(), a)
    g = ImagePayload(a[:, :, 0].tobytes(), 5, 7, 5, 7, 1, 8, False)
    assert g().mode == "L" and g.to_numpy_array().shape == (5, 7)
    rgba = ImagePayload(np.zeros((2, 2, 4), np.uint8).tobytes(), 2, 2, 2, 2, 4, 8, False)
    assert rgba().mode == "RGBA"
    with pytest.raises(AttributeError):
        p.__cuda_array_interface__
    with pytest.raises(AttributeError):
        p.no_such_attribute_anywhere


def test_sample_auto_convert_and_logging():
    # src/structs.rs:279-351, src/client.rs:253-263
    from datago_b200 import client
    a = np.full((4, 6, 3), 9, np.uint8)
    s = client.Sample("k1", "src", client.ImagePayload(a.tobytes(), 4, 6, 4, 6, 3, 8, False), {"json": "{\"a\": 1}", "n": 3})
    s.additional_images["k1.mask"] = client.ImagePayload(a[:, :, 0].tobytes(), 4, 6, 4, 6, 1, 8, False)
    d = client.sample_to_python_types(s)
    assert d["id"] == "k1" and d["source"] == "src" and d["duplicate_state"] == 0
    assert d["attributes"] == {"json": "{\"a\": 1}", "n": "3"}
    assert d["image"].size == (6, 4) and d["additional_images"]["k1.mask"].mode == "L"
    assert d["masks"] == {} and d["latents"] == {} and d["tags"] == [] and d["coca_embedding"] == []
    first = client.initialize_logging("warn")
    assert client.initialize_logging() is False or first is False   # a second call reports that logging was set up already


def test_host_decode_of_png_masks_and_other_formats():
    # what the CUDA decoder does not take goes through Pillow to raw 8-bit pixels (src/worker_http.rs:186-201: masks are PNG)
    import io
    from PIL import Image
    rng = np.random.default_rng(3)
    mask = (rng.integers(0, 2, (40, 60)) * 255).astype(np.uint8)
    rgba = rng.integers(0, 256, (20, 30, 4), dtype=np.uint8)

    def enc(arr, fmt, **kw):
        b = io.BytesIO()
        Image.fromarray(arr).save(b, fmt, **kw)
        return b.getvalue()

    assert np.array_equal(client.decode_on_host(enc(mask, "PNG")), mask)
    assert np.array_equal(client.decode_on_host(enc(rgba, "PNG")), rgba)
    pal = Image.fromarray(rgba[:, :, :3]).quantize(16)
    b = io.BytesIO(); pal.save(b, "PNG")
    assert client.decode_on_host(b.getvalue()).shape == (20, 30, 3)
    prog = enc(rgba[:, :, :3], "JPEG", progressive=True)
    assert not client.is_baseline_jpeg(prog) and client.decode_on_host(prog).shape == (20, 30, 3)
    assert client.is_baseline_jpeg(enc(rgba[:, :, :3], "JPEG"))
    assert client.decode_on_host(b"not an image at all") is None
    # re-encoding of finished payloads (src/image_processing.rs:375-416)
    j = client.encode_payload(rgba[:, :, :3], "jpeg", 92)
    assert j[:2] == b"\xff\xd8" and Image.open(io.BytesIO(j)).size == (30, 20)
    p = client.encode_payload(mask, "png")
    assert p[:4] == b"\x89PNG" and np.array_equal(np.asarray(Image.open(io.BytesIO(p))), mask)
    enc_payload = client.ImagePayload(p, 40, 60, 40, 60, -1, 8, True)
    assert enc_payload().size == (60, 40)
