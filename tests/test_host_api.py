"""The C-ABI library on a machine without a GPU: it loads, exports what the header declares, and its host-side
planning (buckets, geometry, JPEG headers, sharding) agrees with the oracle.  No compute call is made here."""
import glob
import os
import re
import subprocess

import numpy as np
import pytest
from hypothesis import given, settings, strategies as st

import datago_b200 as dg
import oracle

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
CFG224 = dict(crop_and_resize=True, default_image_size=224, downsampling_ratio=16, min_aspect_ratio=0.5, max_aspect_ratio=2.0)
CFG1024 = dict(CFG224, default_image_size=1024, downsampling_ratio=32)


def _declared_symbols():
    names = []
    for path in glob.glob(os.path.join(ROOT, "include", "*.h")):
        for line in open(path):
            m = re.match(r"^DG_API\s+[\w\s\*]+?\b(dg_\w+)\(", line)
            if m:
                names.append(m.group(1))
    return names


def test_library_exports_every_declared_symbol():
    L = dg.lib()
    declared = _declared_symbols()
    assert len(declared) >= 25
    for name in declared:
        assert hasattr(L, name), name
    out = subprocess.run(["nm", "-D", "--defined-only", dg.library_path()], capture_output=True, text=True).stdout
    exported = set(re.findall(r"\bT (dg_\w+)", out))
    assert set(declared) <= exported
    assert set(dg.EXPORTS) == set(declared)


def test_no_cpu_path_without_a_device():
    import torch
    if torch.cuda.is_available():
        pytest.skip("a device is present")
    with pytest.raises(dg.DatagoB200Error) as e:
        dg.Context(0, CFG224)
    assert "no CPU path" in str(e.value)
    ctx = dg.Context(dg.DG_DEVICE_NONE, CFG224)
    with pytest.raises(dg.DatagoB200Error):
        ctx.batch([b"\xff\xd8\xff\xd9"])
    with pytest.raises(dg.DatagoB200Error) as e:
        dg.Feeder(0, CFG224)                      # the submit / wait front end has no CPU path either
    assert "no CPU path" in str(e.value)
    with pytest.raises(dg.DatagoB200Error):
        dg.Feeder(dg.DG_DEVICE_NONE, CFG224, lanes=1)


def test_reference_known_answers_through_the_c_abi():
    ctx = dg.Context(dg.DG_DEVICE_NONE, CFG224)
    # datago src/image_processing.rs:458-477
    assert ctx.closest_aspect_ratio(100, 100) == "1.000"
    assert ctx.closest_aspect_ratio(200, 100) == "1.900"
    assert ctx.closest_aspect_ratio(100, 200) == "0.526"
    p = ctx.plan_geometry(300, 200, 3, "1.000")
    assert (p.target_w, p.target_h, p.new_w, p.new_h, p.crop_left) == (224, 224, 336, 224, 56.0)
    p = ctx.plan_geometry(300, 200, 3, "1.900")
    assert (p.target_w, p.target_h) == (304, 160)
    p = ctx.plan_geometry(400, 200)
    assert (p.target_w, p.target_h) == (304, 160)
    assert ctx.plan_geometry(224, 224).identity == 1


@pytest.mark.parametrize("cfg", [CFG224, CFG1024, dict(CFG224, default_image_size=512), dict(CFG224, default_image_size=2048, downsampling_ratio=64),
                                 dict(CFG224, default_image_size=768, downsampling_ratio=8, min_aspect_ratio=0.25, max_aspect_ratio=4.0)])
def test_tables_match_oracle(cfg):
    ctx = dg.Context(dg.DG_DEVICE_NONE, cfg)
    assert ctx.bucket_table() == oracle.bucket_table(cfg)
    assert dg.size_list(cfg) == oracle.size_list(cfg)


@settings(max_examples=400, deadline=None)
@given(w=st.integers(1, 6000), h=st.integers(1, 6000), which=st.integers(0, 2))
def test_geometry_matches_oracle_bit_exact(w, h, which):
    cfg = [CFG224, CFG1024, dict(CFG224, default_image_size=2048, downsampling_ratio=64)][which]
    ctx = _ctx_cache(which, cfg)
    assert ctx.plan_geometry(w, h).as_tuple() == oracle.plan_geometry(cfg, w, h).as_tuple()


_CTX = {}


def _ctx_cache(which, cfg):
    if which not in _CTX:
        _CTX[which] = dg.Context(dg.DG_DEVICE_NONE, cfg)
    return _CTX[which]


def test_forced_keys_match_oracle():
    ctx = dg.Context(dg.DG_DEVICE_NONE, CFG1024)
    rng = np.random.default_rng(0)
    keys = [k for k, _, _, _ in ctx.bucket_table()]
    for _ in range(200):
        w, h = int(rng.integers(8, 4097)), int(rng.integers(8, 4097))
        k = keys[int(rng.integers(0, len(keys)))]
        assert ctx.plan_geometry(w, h, 3, k).as_tuple() == oracle.plan_geometry(CFG1024, w, h, k).as_tuple()
    with pytest.raises(dg.DatagoB200Error) as e:
        ctx.plan_geometry(100, 100, 3, "9.999")
    assert e.value.code == 8


def test_invalid_configs_are_rejected():
    # datago asserts on these (src/image_processing.rs:78-93)
    for bad in (dict(CFG224, default_image_size=0), dict(CFG224, downsampling_ratio=0), dict(CFG224, min_aspect_ratio=0.0),
                dict(CFG224, min_aspect_ratio=2.0, max_aspect_ratio=1.0)):
        with pytest.raises(dg.DatagoB200Error):
            dg.Context(dg.DG_DEVICE_NONE, bad)
    # no transform: bucket queries say so
    ctx = dg.Context(dg.DG_DEVICE_NONE, None)
    with pytest.raises(dg.DatagoB200Error) as e:
        ctx.closest_aspect_ratio(10, 10)
    assert e.value.code == 9


def test_aspect_ratio_to_str():
    for wh in [(304, 160), (224, 224), (1, 3), (1440, 704), (5, 7)]:
        assert dg.aspect_ratio_to_str(*wh) == oracle.aspect_ratio_to_str(*wh)


def test_jpeg_probe_matches_oracle(golden_dir):
    for path in sorted(glob.glob(os.path.join(golden_dir, "jpeg_*.jpg"))):
        data = open(path, "rb").read()
        a, b = dg.jpeg_probe(data), oracle.jpeg_info(data)
        assert (a.width, a.height, a.channels, a.hsamp, a.vsamp, a.mcux, a.mcuy, a.restart_interval) == \
               (b.width, b.height, b.channels, b.hsamp, b.vsamp, b.mcux, b.mcuy, b.restart_interval)
        assert a.scan_offset + a.scan_len == len(data)


def test_jpeg_probe_rejects_garbage():
    for bad, code in ((b"", 4), (b"not a jpeg at all", 4), (b"\xff\xd8\xff\xd9", 3), (b"\xff\xd8\xff\xe0\x00\x10JFIF", 3)):
        with pytest.raises(dg.DatagoB200Error) as e:
            dg.jpeg_probe(bad)
        assert e.value.code == code, bad
    # progressive JPEG: unsupported on this path
    import io
    from PIL import Image
    b = io.BytesIO()
    Image.fromarray(np.zeros((32, 32, 3), np.uint8)).save(b, "JPEG", progressive=True)
    with pytest.raises(dg.DatagoB200Error) as e:
        dg.jpeg_probe(b.getvalue())
    assert e.value.code == 5


def test_sharding_matches_oracle_and_reference_asserts():
    assert dg.rank_slice(10, 0, 2) == (0, 5) and dg.rank_slice(11, 1, 2) == (6, 11)
    assert [dg.rank_slice(13, r, 3) for r in range(3)] == [(0, 5), (5, 9), (9, 13)]
    with pytest.raises(dg.DatagoB200Error):
        dg.rank_slice(10, 2, 2)
    with pytest.raises(dg.DatagoB200Error):
        dg.rank_slice(10, 0, 0)
    for n in (0, 1, 7, 1024, 64000):
        for world in (1, 2, 3, 8):
            got = [dg.rank_slice(n, r, world) for r in range(world)]
            assert got == [oracle.rank_slice(n, r, world) for r in range(world)]
            assert got[0][0] == 0 and got[-1][1] == n and all(got[i][1] == got[i + 1][0] for i in range(world - 1))
    for k in ["", "a", "000001_0002", "x" * 7, "y" * 8, "z" * 9, "sample/ünï"]:
        assert dg.key_hash(k) == oracle.key_hash(k)
        assert dg.key_rank(k, 8) == oracle.key_hash(k) % 8


@settings(max_examples=300, deadline=None)
@given(data=st.binary(min_size=0, max_size=400), splice=st.integers(0, 700))
def test_header_parser_survives_garbage(data, splice):
    # random bytes, and random bytes spliced into a real header: a status or a plan, never a crash
    real = open(os.path.join(ROOT, "tests", "golden", "jpeg_420_q75_rst2.jpg"), "rb").read()
    for blob in (data, real[:splice] + data + real[splice + len(data):], real[:splice]):
        try:
            info = dg.jpeg_probe(blob)
            assert info.width > 0 and info.height > 0 and info.scan_offset + info.scan_len == len(blob)
        except dg.DatagoB200Error as e:
            assert e.code in (3, 4, 5, 6)


def test_bind_to_gpu_cpus_changes_nothing_without_a_device():
    # no CUDA device (or no NVML): the helper reports None and leaves the affinity mask alone
    import os
    before = os.sched_getaffinity(0)
    got = dg.bind_to_gpu_cpus(0)
    if got is None:
        assert os.sched_getaffinity(0) == before
    else:  # on a GPU box: a non-empty subset of the mask the process had
        assert set(got) <= before and set(got) == os.sched_getaffinity(0)
        os.sched_setaffinity(0, before)
