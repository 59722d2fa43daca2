"""The DatagoClient harness end to end on a GPU: samples from local files and local webdataset shards, payloads equal
to the oracle's, the reference's sample-level rules (bucket shared inside a sample, bad files skipped, ranks disjoint)."""
import io
import json
import os
import tarfile

import numpy as np
import pytest

import oracle
from datago_b200 import synth
from datago_b200.client import DatagoClient
from gpu_common import jpeg

pytestmark = pytest.mark.gpu

CFG = dict(crop_and_resize=True, default_image_size=256, downsampling_ratio=16, min_aspect_ratio=0.5, max_aspect_ratio=2.0)


def _drain(c):
    out = []
    while True:
        s = c.get_sample()
        if s is None:
            return out
        out.append(s)


def test_file_source_matches_oracle_and_skips_a_corrupt_file(tmp_path):
    rng = np.random.default_rng(51)
    datas = {}
    for i, (w, h) in enumerate([(320, 200), (200, 320), (256, 256), (500, 130), (123, 457)]):
        d = jpeg(rng, w, h, "4:2:0", 88, 4 if i % 2 else 0)
        (tmp_path / f"im{i}.jpg").write_bytes(d)
        datas[str(tmp_path / f"im{i}.jpg")] = d
    (tmp_path / "broken.jpg").write_bytes(b"\xff\xd8 this is not a jpeg")
    cfg = dict(source_type="file", source_config=dict(root_path=str(tmp_path)), image_config=CFG, limit=100, samples_buffer_size=8)
    samples = _drain(DatagoClient(json.dumps(cfg)))
    assert len(samples) == 5
    for s in samples:
        path = json.loads(s.id)
        want, p = oracle.jpeg_to_payload(datas[path], CFG)
        assert s.source == "filesystem"
        im = s.image
        assert (im.width, im.height, im.channels, im.bit_depth, im.is_encoded) == (p.target_w, p.target_h, 3, 8, False)
        assert (im.original_width, im.original_height) == (p.src_w, p.src_h)
        assert np.array_equal(im.to_numpy_array(), want)
        assert im.to_pil_image().size == (p.target_w, p.target_h)


def test_file_source_without_transform_returns_decoded_images(tmp_path):
    rng = np.random.default_rng(52)
    d = jpeg(rng, 111, 77)
    (tmp_path / "a.jpeg").write_bytes(d)
    cfg = dict(source_type="file", source_config=dict(root_path=str(tmp_path)), limit=4, samples_buffer_size=2)
    (s,) = _drain(DatagoClient(json.dumps(cfg)))
    assert np.array_equal(s.image.to_numpy_array(), oracle.jpeg_decode(d))


def test_two_ranks_are_disjoint_and_limit_is_respected(tmp_path):
    rng = np.random.default_rng(53)
    for i in range(12):
        (tmp_path / f"f{i:02d}.jpg").write_bytes(jpeg(rng, 64 + 8 * i, 80))
    ids = []
    for rank in range(2):
        cfg = dict(source_type="file", source_config=dict(root_path=str(tmp_path), rank=rank, world_size=2), limit=100, samples_buffer_size=4)
        ids.append({s.id for s in _drain(DatagoClient(json.dumps(cfg)))})
    assert len(ids[0]) == 6 and len(ids[1]) == 6 and not ids[0] & ids[1]
    cfg = dict(source_type="file", source_config=dict(root_path=str(tmp_path)), limit=5, samples_buffer_size=4)
    assert len(_drain(DatagoClient(json.dumps(cfg)))) == 5
    bad = dict(source_type="file", source_config=dict(root_path=str(tmp_path), rank=3, world_size=2), limit=5, samples_buffer_size=4)
    assert DatagoClient(json.dumps(bad)).get_sample() is None   # python/test_datago_edge_cases.py:224-245 of datago


def _write_shard(path, n, rng, first=0):
    keys, blobs = [], {}
    with tarfile.open(path, "w") as tf:
        for i in range(first, first + n):
            key = "%06d_%04d" % (0, i)
            w, h = int(rng.integers(10, 40)) * 8, int(rng.integers(10, 40)) * 8
            img = jpeg(rng, w, h, "4:4:4", 90)
            mask_arr = synth.ellipse_mask(rng, w, h)
            b = io.BytesIO()
            from PIL import Image
            Image.fromarray(mask_arr).save(b, "JPEG", quality=95)
            entries = [(key + ".json", json.dumps({"caption": f"sample {i}"}).encode()), (key + ".jpg", img), (key + ".jpeg", b.getvalue())]
            for name, payload in entries:
                ti = tarfile.TarInfo(name)
                ti.size = len(payload)
                tf.addfile(ti, io.BytesIO(payload))
            keys.append(key)
            blobs[key] = (img, b.getvalue())
    return keys, blobs


def test_webdataset_samples_share_one_bucket_and_carry_text(tmp_path):
    rng = np.random.default_rng(54)
    keys, blobs = _write_shard(str(tmp_path / "shard-000.tar"), 9, rng)
    cfg = dict(source_type="webdataset", source_config=dict(url=str(tmp_path / "shard-{000..000}.tar")), image_config=CFG,
               limit=100, samples_buffer_size=4, batch_size=4)
    samples = _drain(DatagoClient(json.dumps(cfg)))
    assert [s.id for s in samples] == keys
    for s in samples:
        img, mask = blobs[s.id]
        want, p = oracle.jpeg_to_payload(img, CFG)
        assert np.array_equal(s.image.to_numpy_array(), want)
        assert json.loads(s.attributes)["json"] == json.dumps({"caption": f"sample {int(s.id[-4:])}"})
        (name, extra), = s.additional_images.items()
        assert name.endswith(".jpeg") and extra.channels == 1
        assert (extra.width, extra.height) == (s.image.width, s.image.height)     # src/worker_wds.rs:68-76
        key = oracle.aspect_ratio_to_str(p.target_w, p.target_h)
        assert np.array_equal(extra.to_numpy_array(), oracle.jpeg_to_payload(mask, CFG, key)[0])


def test_webdataset_ranks_by_key_hash(tmp_path):
    rng = np.random.default_rng(55)
    keys, _ = _write_shard(str(tmp_path / "s.tar"), 16, rng)
    got = []
    for rank in range(2):
        cfg = dict(source_type="webdataset", source_config=dict(url=str(tmp_path / "s.tar"), rank=rank, world_size=2),
                   limit=100, samples_buffer_size=4)
        mine = [s.id for s in _drain(DatagoClient(json.dumps(cfg)))]
        assert all(oracle.key_hash(k) % 2 == rank for k in mine)
        got += mine
    assert sorted(got) == keys


def test_device_payloads_are_zero_copy_tensors(tmp_path):
    import torch
    rng = np.random.default_rng(56)
    d = jpeg(rng, 300, 200)
    (tmp_path / "a.jpg").write_bytes(d)
    cfg = dict(source_type="file", source_config=dict(root_path=str(tmp_path)), image_config=CFG, limit=4, samples_buffer_size=2,
               device_payloads=True)
    (s,) = _drain(DatagoClient(json.dumps(cfg)))
    t = torch.as_tensor(s.image, device="cuda")
    assert t.dtype == torch.uint8 and tuple(t.shape) == (s.image.height, s.image.width, 3)
    assert t.data_ptr() == s.image._device_ptr
    want, _ = oracle.jpeg_to_payload(d, CFG)
    assert np.array_equal(t.cpu().numpy(), want)
    assert np.array_equal(torch.from_dlpack(s.image).cpu().numpy(), want)


def test_image_to_rgb8_config_key_turns_gray_files_into_rgb(tmp_path):
    # src/worker_files.rs:385-413: a gray file with img_to_rgb8 comes back with three equal channels
    rng = np.random.default_rng(57)
    g = jpeg(rng, 150, 100, gray=True)
    (tmp_path / "g.jpg").write_bytes(g)
    for flag, channels in ((True, 3), (False, 1)):
        cfg = dict(source_type="file", source_config=dict(root_path=str(tmp_path)),
                   image_config=dict(CFG, image_to_rgb8=flag), limit=4, samples_buffer_size=2)
        (s,) = _drain(DatagoClient(json.dumps(cfg)))
        want, p = oracle.crop_and_resize(CFG, oracle.jpeg_decode(g))
        assert (s.image.channels, s.image.width, s.image.height) == (channels, p.target_w, p.target_h)
        got = s.image.to_numpy_array()
        assert np.array_equal(got, oracle.to_rgb8(want) if flag else want.reshape(got.shape))


def test_png_masks_ride_in_the_image_bucket_and_payloads_can_be_re_encoded(tmp_path):
    # a webdataset sample with a JPEG image and a PNG mask (the reference's masks are PNG, src/worker_http.rs:186-201):
    # the mask is decoded on the host, then bucketed, cropped and resized on the GPU with the image's key
    import io
    import tarfile
    from PIL import Image
    from datago_b200 import synth
    rng = np.random.default_rng(56)
    path = str(tmp_path / "m.tar")
    want = {}
    with tarfile.open(path, "w") as tf:
        for k in range(4):
            w, h = int(rng.integers(200, 500)), int(rng.integers(200, 500))
            img = synth.encode_jpeg(synth.natural_image(rng, w, h, 4.0, True), 90, "4:2:0", 0)
            mask = synth.ellipse_mask(rng, w, h)
            b = io.BytesIO(); Image.fromarray(mask).save(b, "PNG")
            key = f"s{k:03d}"
            for name, payload in ((key + ".jpg", img), (key + ".png", b.getvalue())):
                ti = tarfile.TarInfo(name); ti.size = len(payload); tf.addfile(ti, io.BytesIO(payload))
            want[key] = (img, mask)
    cfg = dict(source_type="webdataset", source_config=dict(url=path), image_config=CFG, limit=10, samples_buffer_size=4)
    samples = _drain(DatagoClient(json.dumps(cfg)))
    assert sorted(s.id for s in samples) == sorted(want)
    for s in samples:
        img, mask = want[s.id]
        payload, p = oracle.jpeg_to_payload(img, CFG)
        assert np.array_equal(s.image.to_numpy_array(), payload)
        (name, extra), = s.additional_images.items()
        assert name.endswith(".png") and extra.channels == 1 and (extra.width, extra.height) == (s.image.width, s.image.height)
        key = oracle.aspect_ratio_to_str(p.target_w, p.target_h)
        assert np.array_equal(extra.to_numpy_array(), oracle.crop_and_resize(CFG, mask, key)[0])
    # pre_encode_images: payloads come back as encoded files (src/image_processing.rs:375-416)
    cfg["image_config"] = dict(CFG, pre_encode_images=True, encode_format="png")
    for s in _drain(DatagoClient(json.dumps(cfg))):
        assert s.image.is_encoded and s.image.channels == -1 and bytes(s.image.data[:4]) == b"\x89PNG"
        payload, _ = oracle.jpeg_to_payload(want[s.id][0], CFG)
        assert np.array_equal(np.asarray(s.image.to_pil_image()), payload)      # PNG is lossless
