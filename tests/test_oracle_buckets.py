"""The oracle's bucket / geometry / sharding logic against the reference's own known answers."""
import json
import os

import pytest

import oracle

CFG224 = dict(default_image_size=224, downsampling_ratio=16, min_aspect_ratio=0.5, max_aspect_ratio=2.0)


def test_reference_closest_aspect_ratio_asserts():
    # datago src/image_processing.rs:458-460
    assert oracle.plan_geometry(CFG224, 100, 100).key.decode() == "1.000"
    assert oracle.plan_geometry(CFG224, 200, 100).key.decode() == "1.900"
    assert oracle.plan_geometry(CFG224, 100, 200).key.decode() == "0.526"


def test_reference_crop_and_resize_dims():
    # datago src/image_processing.rs:463-477: 300x200 forced "1.000" -> 224x224, forced "1.900" -> 304x160,
    # 400x200 automatic -> 304x160
    p = oracle.plan_geometry(CFG224, 300, 200, "1.000")
    assert (p.target_w, p.target_h) == (224, 224)
    p = oracle.plan_geometry(CFG224, 300, 200, "1.900")
    assert (p.target_w, p.target_h) == (304, 160)
    p = oracle.plan_geometry(CFG224, 400, 200)
    assert (p.target_w, p.target_h) == (304, 160)


def test_geometry_known_answer_300x200():
    p = oracle.plan_geometry(CFG224, 300, 200, "1.000")
    assert (p.new_w, p.new_h) == (336, 224)
    assert (p.crop_left, p.crop_top) == (56.0, 0.0)


def test_table_224():
    t = oracle.bucket_table(CFG224)
    assert [(k, w, h) for k, _, w, h in t] == [
        ("0.526", 160, 304), ("0.556", 160, 288), ("0.647", 176, 272), ("0.750", 192, 256), ("0.867", 208, 240),
        ("1.000", 224, 224), ("1.154", 240, 208), ("1.333", 256, 192), ("1.545", 272, 176), ("1.800", 288, 160),
        ("1.900", 304, 160)]
    assert len(oracle.size_list(CFG224)) == 20


@pytest.mark.parametrize("size,ratio", [(1024, 32), (512, 16), (2048, 64)])
def test_table_benchmark_configs(size, ratio):
    cfg = dict(CFG224, default_image_size=size, downsampling_ratio=ratio)
    t = oracle.bucket_table(cfg)
    assert len(oracle.size_list(cfg)) == 46 and len(t) == 27
    assert t[0][0] == "0.489" and t[-1][0] == "2.045"
    scale = size // 1024 if size >= 1024 else None
    if size == 1024:
        assert (t[0][2], t[0][3]) == (704, 1440) and (t[-1][2], t[-1][3]) == (1440, 704)
    # list invariants the reference checks (src/image_processing.rs:480-494, 652-679, 727-759)
    ars = [a for _, a, _, _ in t]
    assert ars == sorted(ars)
    for _, _, w, h in t:
        assert w % ratio == 0 and h % ratio == 0


def test_golden_tables_and_plans(golden_dir):
    kat = json.load(open(os.path.join(golden_dir, "buckets.json")))
    for name, rows in kat["tables"].items():
        size, ratio = (int(x) for x in name.split("/"))
        cfg = dict(CFG224, default_image_size=size, downsampling_ratio=ratio)
        assert [[k, w, h] for k, _, w, h in oracle.bucket_table(cfg)] == rows
    for row in kat["plans"]:
        cfg = dict(CFG224, default_image_size=row["size"], downsampling_ratio=row["ratio"])
        assert list(oracle.plan_geometry(cfg, row["w"], row["h"], row["forced"]).as_tuple()) == row["plan"]


def test_no_resize_when_already_target():
    # src/image_processing.rs:761-785
    p = oracle.plan_geometry(CFG224, 224, 224)
    assert p.identity == 1


def test_extreme_aspect_ratios_clamp():
    # src/image_processing.rs:701-725: very wide / very tall images land in the outermost buckets
    assert oracle.plan_geometry(CFG224, 10000, 100).key.decode() == "1.900"
    assert oracle.plan_geometry(CFG224, 100, 10000).key.decode() == "0.526"


def test_unknown_key():
    with pytest.raises(KeyError):
        oracle.plan_geometry(CFG224, 100, 100, "3.141")


def test_aspect_ratio_to_str():
    assert oracle.aspect_ratio_to_str(304, 160) == "1.900"
    assert oracle.aspect_ratio_to_str(224, 224) == "1.000"
    assert oracle.aspect_ratio_to_str(1, 3) == "0.333"


def test_rank_slices_reference_asserts():
    # datago src/generator_files.rs:190-231
    assert oracle.rank_slice(10, 0, 2) == (0, 5) and oracle.rank_slice(10, 1, 2) == (5, 10)
    assert oracle.rank_slice(11, 0, 2) == (0, 6) and oracle.rank_slice(11, 1, 2) == (6, 11)
    assert [oracle.rank_slice(13, r, 3) for r in range(3)] == [(0, 5), (5, 9), (9, 13)]
    assert oracle.rank_slice(10, 0, 1) == (0, 10)
    assert oracle.rank_slice(0, 0, 1) == (0, 0)
    with pytest.raises(ValueError):
        oracle.rank_slice(10, 0, 0)


def test_siphash_construction_against_published_vectors():
    # SipHash-2-4 reference vectors (key 00..0f, message 00..n-1): pins rounds, finalisation and byte order of the
    # construction whose 1-3 variant with a zero key is the shard hash.
    k0 = int.from_bytes(bytes(range(8)), "little")
    k1 = int.from_bytes(bytes(range(8, 16)), "little")
    assert oracle.siphash(k0, k1, 2, 4, b"") == 0x726FDB47DD0E0E31
    assert oracle.siphash(k0, k1, 2, 4, bytes(range(1))) == 0x74F839C593DC67FD
    assert oracle.siphash(k0, k1, 2, 4, bytes(range(8))) == 0x93F5F5799A932462
    assert oracle.siphash(k0, k1, 2, 4, bytes(range(15))) == 0xA129CA6149BE45E5


def test_key_hash_shards_are_disjoint_and_cover():
    keys = ["%06d_%04d" % (i // 1000, i % 1000) for i in range(4000)]
    for world in (2, 4, 8):
        ranks = [oracle.key_hash(k) % world for k in keys]
        counts = [ranks.count(r) for r in range(world)]
        assert sum(counts) == len(keys)
        assert min(counts) > 0.8 * len(keys) / world
