"""Submit / wait front end: many threads hand in single samples, the library batches them.  Every result must equal the
oracle's (and therefore the batch path's), whatever batch a sample happened to land in."""
import threading
import time
from concurrent.futures import ThreadPoolExecutor

import numpy as np
import pytest

import datago_b200 as dg
import oracle
from gpu_common import assert_same, jpeg

pytestmark = pytest.mark.gpu

CFG224 = dict(crop_and_resize=True, default_image_size=224, downsampling_ratio=16, min_aspect_ratio=0.5, max_aspect_ratio=2.0)


def _samples(seed, n):
    rng = np.random.default_rng(seed)
    out = []
    for k in range(n):
        w, h = int(rng.integers(60, 500)), int(rng.integers(60, 500))
        if k % 4 == 3:
            out.append(rng.integers(0, 256, (h, w, 3), dtype=np.uint8))
        else:
            out.append(jpeg(rng, w, h, sub=("4:4:4" if k % 5 == 0 else "4:2:0"), q=int(rng.integers(70, 96)), rst=(3 if k % 2 else 0)))
    return out


def _want(cfg, x, forced=None):
    dec = oracle.jpeg_decode(x) if isinstance(x, bytes) else x
    if cfg is None:
        return dec
    return oracle.crop_and_resize(cfg, dec, forced)[0]


def test_worker_threads_each_get_their_own_result():
    samples = _samples(81, 96)
    with dg.Feeder(0, CFG224, max_batch=16, max_wait_us=1500) as f:
        def work(i):
            return f.process_one(samples[i])
        with ThreadPoolExecutor(12) as pool:
            results = list(pool.map(work, range(len(samples))))
        for i, (st, out, r) in enumerate(results):
            assert st == 0, i
            want = _want(CFG224, samples[i])
            assert (r.height, r.width) == want.shape[:2]
            assert_same(out, want, f"sample {i}")
        st = f.stats()
        assert st["submitted"] == st["completed"] == len(samples) and st["failed"] == 0
        assert st["open_tickets"] == 0 and st["queued"] == 0
        assert st["batched_items"] == len(samples) and 1 < st["batches"] <= len(samples)
        assert 1 < st["largest_batch"] <= 16          # samples of different threads really shared launches


def test_host_buffer_at_submit_device_payload_and_forced_key():
    samples = _samples(82, 6)
    with dg.Feeder(0, CFG224, max_batch=8, max_wait_us=500) as f:
        ctx_plan = dg.lib().dg_feeder_ctx(f._h)
        assert ctx_plan
        # (a) caller-allocated buffer sized from a plan query, filled by wait()
        info = dg.jpeg_probe(samples[0])
        p = dg.Plan()
        assert dg.lib().dg_plan_geometry(ctx_plan, info.width, info.height, 3, None, dg.C.byref(p)) == 0
        buf = np.zeros((p.target_h, p.target_w, 3), np.uint8)
        t = f.submit(samples[0], host_out=buf)
        r = f.wait(t)
        assert r.status == 0 and not r.device_data and r.plan.key == p.key
        assert_same(buf, _want(CFG224, samples[0]), "host_out path")
        f.release(t)
        # (b) device-resident payload, valid until release
        t = f.submit(samples[1], forced_key="1.900")
        r = f.wait(t)
        assert r.status == 0 and r.device_data and (r.width, r.height) == (304, 160)
        ctx = dg.Context(0, CFG224)
        got = ctx.copy_to_host(r.device_data, r.nbytes).reshape(r.height, r.width, 3)
        assert_same(got, _want(CFG224, samples[1], "1.900"), "device payload")
        assert_same(f.fetch(t, r), got, "fetch")
        view = f.peek(t, r)                       # the library's own page-locked copy, no second host copy
        assert_same(np.array(view), got, "peek")
        f.release(t)
        ctx.close()
        # (c) too small a buffer is an error of the call, the ticket survives and can be fetched
        small = np.zeros(16, np.uint8)
        t = f.submit(samples[2], host_out=small)
        with pytest.raises(dg.DatagoB200Error):
            f.wait(t)
        r = f.wait(t)
        assert r.status == 0
        assert_same(f.fetch(t, r), _want(CFG224, samples[2]), "after a short buffer")
        f.release(t)
        with pytest.raises(dg.DatagoB200Error):
            f.release(t)


def test_failures_are_per_sample_and_decode_only_mode():
    good = _samples(83, 5)
    bad = [b"", b"\xff\xd8\xff", good[0][: len(good[0]) // 2], b"GIF89a" + bytes(100)]
    with dg.Feeder(0, None, max_batch=32, max_wait_us=3000, flags=dg.BATCH_DECODE_ONLY) as f:
        tickets = [f.submit(x) for x in good + bad]
        for i, (x, t) in enumerate(zip(good + bad, tickets)):
            r = f.wait(t)
            if i < len(good):
                assert r.status == 0, i
                assert_same(f.fetch(t, r), _want(None, x), f"decode-only {i}")
            else:
                assert r.status != 0, i
            f.release(t)
        st = f.stats()
        assert st["failed"] == len(bad) and st["completed"] == len(good) + len(bad)


def test_timeout_release_while_queued_and_shutdown_with_open_tickets():
    samples = _samples(84, 4)
    f = dg.Feeder(0, CFG224, lanes=1, max_batch=64, max_wait_us=400_000)
    t0 = f.submit(samples[0])
    assert f.wait(t0, timeout_s=0.01) is None        # the batch is still filling: not done, ticket stays valid
    t1 = f.submit(samples[1])
    f.release(t1)                                      # withdrawn before it ran
    r = f.wait(t0, timeout_s=30)
    assert r is not None and r.status == 0
    assert f.stats()["batched_items"] == 1
    assert_same(f.fetch(t0, r), _want(CFG224, samples[0]), "after timeout")
    t2 = f.submit(samples[2])                          # left open on purpose
    f.close()                                          # must not hang or leak with t0 unreleased and t2 queued
    assert t2 > t0


def test_backpressure_blocks_submit_until_a_lane_drains_the_queue():
    samples = _samples(85, 12)
    with dg.Feeder(0, CFG224, lanes=1, max_batch=4, max_wait_us=200, queue_limit=4) as f:
        tickets = []
        done = threading.Event()

        def producer():
            for x in samples:
                tickets.append(f.submit(x))
            done.set()
        th = threading.Thread(target=producer)
        th.start()
        assert done.wait(60)
        th.join()
        for i, t in enumerate(tickets):
            r = f.wait(t)
            assert r.status == 0
            assert_same(f.fetch(t, r), _want(CFG224, samples[i]), f"sample {i}")
            f.release(t)
        assert f.stats()["largest_batch"] <= 4
