"""Benchmark of the image hot path on B200: decoded(+bucketed) images/s on seeded synthetic inputs.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload c2|c0|c1|c3|c4] [--images M] [--impl reference]

A step is one pass of the path over the whole workload (default: the 8192-JPEG decode-throughput set, C2).  `value` is
measured with the inputs already in HBM (CUDA events around K back-to-back passes); `e2e` goes through the public batch
API from host bytes to host pixel buffers.  The default run then measures the local-file set (C0, decode + bucket
crop-resize) and the resize-only set (C1) in the same process, shorter, and reports them under `configs`.
Multi-GPU runs are weak-scaled: every rank owns one workload-sized shard of an N-times larger job (contiguous rank
slices, the rule datago's file source uses); `--workload c3` instead splits one fixed set of tar shards over the ranks
by key hash, datago's webdataset rule (strong scaling).  There is no collective on the data path; only the timing is
reduced across ranks.  `--impl reference` times the CPU implementation of the same path (the oracle port; the
reference's Rust crates cannot be built here) on all host cores.
"""
import argparse
import io
import json
import math
import os
import pickle
import statistics
import subprocess
import sys
import tarfile
import threading
import time
from concurrent.futures import ThreadPoolExecutor

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

import numpy as np  # noqa: E402

METRIC = "decoded+bucketed images/s"
LABELS = {
    "c0": "C0 local-file set: {n} 4:2:0 q90 JPEGs 256..2048, decode + 1024/32 bucket crop-resize",
    "c1": "C1 resize-only: {n} raw RGB buffers 512..4096, 512/16 buckets",
    "c2": "C2 JPEG decode throughput: {n} baseline 4:2:0 JPEGs 512..1536, q75-95, half with restart interval 4, decode to RGB8",
    "c3": "C3 webdataset-shaped: {n} samples (.jpg up to 2048 + .json) in local tar shards of 1000, key-hash dispatch, decode + 1024/32 bucket crop-resize",
    "c4": "C4 multi-payload: {n} samples of a 4:4:4 JPEG up to 4096 plus a same-size L8 mask, both into the image's 2048/64 bucket",
}


def load_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        return float(json.load(open(path))["hbm_gbs"]), "measured"
    return 6650.0, "fallback"


def load_traffic():
    """DRAM bytes per pixel of the post-entropy kernels as ncu counted them on a small case (profiles/traffic.json)."""
    path = os.path.join(ROOT, "profiles", "traffic.json")
    return json.load(open(path)) if os.path.exists(path) else {}


# ---- workloads ------------------------------------------------------------------------------------------------------
class Workload:
    """items: bytes (JPEG files) or numpy arrays (raw pixels); forced[i]: bucket key forced on item i or None;
    samples: how many samples the items make up (C4: two items per sample)."""

    def __init__(self, name, items, forced, samples, cfg):
        self.name, self.items, self.forced, self.samples, self.cfg = name, items, forced, samples, cfg


def _cached(tag, make, rank, barrier):
    """Generated once per box by rank 0 and shared through /dev/shm."""
    cache = f"/dev/shm/datago_b200_{tag}.pkl"
    if rank == 0 and not os.path.exists(cache):
        t = time.time()
        obj = make()
        with open(cache + ".tmp", "wb") as f:
            pickle.dump(obj, f, protocol=4)
        os.replace(cache + ".tmp", cache)
        print(f"[bench] generated {tag} in {time.time() - t:.1f}s", file=sys.stderr)
    barrier()
    with open(cache, "rb") as f:
        return pickle.load(f)


def shard_paths(count):
    """C3: seeded tar shards of 1000 samples under /dev/shm (written once per box)."""
    from datago_b200 import synth
    n_shards = (count + 999) // 1000
    d = f"/dev/shm/datago_b200_c3_{count}"
    paths = [os.path.join(d, f"shard-{s:05d}.tar") for s in range(n_shards)]
    if not all(os.path.exists(p) for p in paths):
        os.makedirs(d, exist_ok=True)
        t = time.time()
        import multiprocessing as mp
        jobs = [(paths[s] + ".tmp", s * 1000, min(1000, count - s * 1000)) for s in range(n_shards)]
        with mp.get_context("fork").Pool(max(1, (os.cpu_count() or 8) - 1)) as pool:
            pool.starmap(synth.write_shard, jobs)
        for p in paths:
            os.replace(p + ".tmp", p)
        print(f"[bench] wrote {n_shards} C3 shards in {time.time() - t:.1f}s", file=sys.stderr)
    return paths


def load_workload(name, count, rank, world, barrier, ctx_for_keys=None):
    from datago_b200 import synth
    import datago_b200 as dg
    cfg = synth.IMAGE_CONFIGS[name]
    procs = max(1, (os.cpu_count() or 8) - 1)
    if name == "c3":
        # datago's webdataset rule: every rank walks every shard and keeps the samples whose key hashes to it
        # (src/generator_wds.rs:140-148)
        if rank == 0:
            shard_paths(count)
        barrier()
        items = []
        for p in shard_paths(count):
            with tarfile.open(p) as tf:
                for m in tf:
                    stem, ext = os.path.splitext(m.name)
                    if ext == ".jpg" and dg.key_rank(stem, world) == rank:
                        items.append(tf.extractfile(m).read())
        return Workload(name, items, None, len(items), cfg)
    if name == "c4":
        pairs = _cached(f"c4_{count}", lambda: synth.make("c4", range(count), processes=procs), rank, barrier)
        start, end = dg.rank_slice(world * count, rank, world)
        items, forced = [], []
        for i in range(start, end):
            jpg, mask = pairs[i % count]
            info = dg.jpeg_probe(jpg)
            key = ctx_for_keys.plan_geometry(info.width, info.height, 3).key.decode()
            items += [jpg, mask]
            forced += [None, key]  # the mask goes into the image's bucket (src/worker_wds.rs:68-76)
        return Workload(name, items, forced, end - start, cfg)
    items = _cached(f"{name}_{count}", lambda: synth.make(name, range(count), processes=procs), rank, barrier)
    start, end = dg.rank_slice(world * count, rank, world)  # this rank's shard of the N x workload job
    return Workload(name, [items[i % count] for i in range(start, end)], None, end - start, cfg)


def workload_stats(wl):
    """Pixels and algorithmic bytes of one pass: coefficients 2 B per MCU-padded sample, RGB 3 B per pixel."""
    import datago_b200 as dg
    st = dict(pixels=0, compressed=0, coef_bytes=0, plane_bytes=0, rgb_bytes=0, rst_compressed=0, rst_coef_bytes=0)
    for it in wl.items:
        if isinstance(it, (bytes, bytearray)):
            i = dg.jpeg_probe(it)
            blocks = i.mcux * i.mcuy * (1 if i.channels == 1 else i.hsamp * i.vsamp + 2)
            st["pixels"] += i.width * i.height
            st["compressed"] += i.scan_len
            st["coef_bytes"] += blocks * 128      # 2 * s * P_mcu
            st["plane_bytes"] += blocks * 64
            st["rgb_bytes"] += i.width * i.height * i.channels
            if i.restart_interval:
                st["rst_compressed"] += i.scan_len
                st["rst_coef_bytes"] += blocks * 128
        else:
            st["pixels"] += it.shape[0] * it.shape[1]
            st["rgb_bytes"] += it.nbytes
    return st


class ClockSampler:
    QUERY = "clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap"

    def __init__(self, index):
        self.index, self.rows, self.proc = index, [], None

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits",
                                          "-i", str(self.index), "-lms", "100"], stdout=subprocess.PIPE, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append((time.time(), [c.strip() for c in line.split(",")]))

    def window(self, t0, t1):
        """Samples inside [t0, t1] are the ones reported; when the window is too short to hold three, all samples are
        (the sampler runs from the first warm-up pass on, so they are all under load)."""
        self.t0, self.t1 = t0, t1

    def stop(self):
        if not self.proc:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        self.thread.join(timeout=2)
        rows = list(self.rows)
        inside = [r for (t, r) in rows if getattr(self, "t0", 0) <= t <= getattr(self, "t1", float("inf"))]
        rows = inside if len(inside) >= 3 else [r for (_, r) in rows]
        num = lambda s: s.replace(".", "").isdigit()  # noqa: E731
        sm = [float(r[0]) for r in rows if r and num(r[0])]
        mx = [float(r[1]) for r in rows if len(r) > 1 and num(r[1])]
        pw = [float(r[2]) for r in rows if len(r) > 2 and num(r[2])]
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        reasons = [n for i, n in enumerate(names) if any(len(r) > 3 + i and r[3 + i] == "Active" for r in rows)]
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "power_w_max": max(pw) if pw else None, "samples": len(sm), "reasons": reasons}


# ---- CPU arm ----------------------------------------------------------------------------------------------------------
def cpu_baseline(wl, budget_s=12.0):
    """The oracle port on all host cores over a bounded sample of the workload (in samples per second)."""
    import oracle
    threads = os.cpu_count() or 1
    if wl.name == "c4":  # JPEGs decode + resize, masks resize into the same bucket (same size, same aspect ratio)
        parts = [([x for x in wl.items if isinstance(x, bytes)], 1), ([x for x in wl.items if not isinstance(x, bytes)], 2)]
    else:
        parts = [(wl.items, {"c0": 1, "c1": 2, "c2": 0, "c3": 1}[wl.name])]
    n_all = len(parts[0][0])
    probe_n = min(n_all, max(2 * threads, 8))
    t = time.time()
    for items, kind in parts:
        oracle.run_batch(items[:probe_n], kind, wl.cfg, threads)()
    per = max(1e-4, (time.time() - t) / probe_n)
    n = int(min(n_all, max(probe_n, budget_s / per)))
    calls = [oracle.run_batch(items[:n], kind, wl.cfg, threads) for items, kind in parts]
    t = time.time()
    ok = min(c() for c in calls)
    dt = time.time() - t
    return {"value": ok / dt, "unit": "images/s", "cores": threads, "kind": "port",
            "sample": f"first {n} of {n_all} samples of the workload, {dt:.1f}s wall; scalar C++ restatement, no SIMD decoder"}


def pil_yardstick(items, budget_s=5.0):
    """libjpeg-turbo through Pillow on a thread pool: an independent SIMD-optimised CPU decoder, for scale."""
    from PIL import Image
    threads = os.cpu_count() or 1
    items = [x for x in items if isinstance(x, bytes)]
    if not items:
        return None

    def one(b):
        return np.asarray(Image.open(io.BytesIO(b)).convert("RGB")).shape[0]
    n = min(len(items), 8 * threads)
    with ThreadPoolExecutor(threads) as ex:
        t = time.time()
        list(ex.map(one, items[:n]))
        dt = time.time() - t
        n2 = int(min(len(items), max(n, budget_s / max(dt / n, 1e-5))))
        t = time.time()
        list(ex.map(one, items[:n2]))
        dt = time.time() - t
    return {"value": n2 / dt, "unit": "images/s", "cores": threads, "sample": f"{n2} items, decode only, Python thread pool"}


# ---- GPU arm ----------------------------------------------------------------------------------------------------------
def parity_check(ctx, batch, wl, limit):
    """Outside the timed region: payloads of the resident batch against the oracle (first, last, largest, evenly spread)."""
    import oracle
    n = len(wl.items)
    size = lambda x: len(x) if isinstance(x, bytes) else x.size  # noqa: E731
    pick = sorted({0, n - 1, max(range(n), key=lambda i: size(wl.items[i])), *range(0, n, max(1, n // max(1, limit - 3)))})[:limit]

    def want(i):
        x, key = wl.items[i], (wl.forced[i] if wl.forced else None)
        if isinstance(x, bytes):
            return oracle.jpeg_to_payload(x, wl.cfg, key)[0]
        return oracle.crop_and_resize(wl.cfg, x, key)[0] if wl.cfg else x

    with ThreadPoolExecutor(os.cpu_count() or 4) as ex:
        wants = list(ex.map(want, pick))
    bad = 0
    for i, w in zip(pick, wants):
        r = batch.result(i)
        got = ctx.copy_to_host(r.device_data, int(r.nbytes)) if r.status == 0 else None
        if got is None or got.size != w.size or not np.array_equal(got, w.reshape(-1)):
            bad += 1
    return {"images": len(pick), "mismatches": bad, "checked_against": "oracle, bit-exact"}


def resize_bytes(ctx, wl):
    """crop_and_resize: C * P_used + C * tw * th per image, P_used = the source pixels that map into the crop."""
    import datago_b200 as dg
    total = out = 0
    for k, it in enumerate(wl.items):
        if isinstance(it, (bytes, bytearray)):
            i = dg.jpeg_probe(it)
            w_, h_, c_ = i.width, i.height, i.channels
        else:
            h_, w_ = it.shape[:2]
            c_ = 1 if it.ndim == 2 else it.shape[2]
        p = ctx.plan_geometry(w_, h_, c_, wl.forced[k] if wl.forced else None)
        scale = max(p.target_w / w_, p.target_h / h_)
        used = min(w_, math.ceil(p.target_w / scale)) * min(h_, math.ceil(p.target_h / scale))
        total += c_ * used + c_ * p.target_w * p.target_h
        out += c_ * p.target_w * p.target_h
    return total, out


def measure(wl, local_rank, world, barrier, all_max, steps, warmup, e2e_steps, chunk, feeder_threads, parity_limit,
            kernels_only, peak, traffic):
    """One workload on this rank's GPU: resident passes, per-stage pass, end-to-end passes.  Returns the report dict."""
    import torch
    import datago_b200 as dg
    cfg, items, forced = wl.cfg, wl.items, wl.forced
    stats = workload_stats(wl)
    stream = torch.cuda.Stream()
    ctx = dg.Context(local_rank, cfg, stream=stream.cuda_stream)
    out = {}

    # -- inputs resident in HBM: K passes of dg_batch_run on an uploaded batch, CUDA events on a parent stream that the
    #    library's stream waits on and is waited for
    b = ctx.batch(items, forced, 0)
    b.upload()
    b.sync()
    sampler = ClockSampler(local_rank)
    sampler.start()
    time.sleep(1.0)  # nvidia-smi needs a moment before its first sample
    for _ in range(warmup):
        b.run()
    b.sync()
    failed = [i for i in range(len(b)) if b.result(i).status != 0]
    assert not failed, f"{len(failed)} items failed, first {failed[:5]}"
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    parent, done = torch.cuda.Stream(), torch.cuda.Event()
    torch.cuda.synchronize()
    barrier()
    t_begin = time.time()
    e0.record(parent)
    stream.wait_event(e0)
    for _ in range(steps):
        b.run()
    done.record(stream)
    parent.wait_event(done)
    e1.record(parent)
    torch.cuda.synchronize()
    barrier()
    sampler.window(t_begin, time.time())
    elapsed_ms = all_max(e0.elapsed_time(e1))
    out["clocks"] = sampler.stop()
    b.sync()
    out["gpu_launches"] = b.counters()["kernel_launches"] * steps
    if parity_limit:
        out["parity_check"] = parity_check(ctx, b, wl, parity_limit)
    b.close()
    n_samples = all_max(wl.samples, op="sum")
    out["value"] = n_samples * steps / (elapsed_ms / 1000.0)
    out["ms_per_step"] = elapsed_ms / steps
    out["mpix_per_s"] = out["value"] * stats["pixels"] / max(1, wl.samples) / 1e6
    if stats["compressed"]:
        out["compressed_bits_per_pixel"] = round(8.0 * stats["compressed"] / stats["pixels"], 3)

    # -- per-kernel durations: one more pass with CUDA events around every stage.  A timing batch keeps all waves on one
    #    stream, so each event pair brackets a kernel that ran alone (the timed passes above overlap the waves).
    tb = ctx.batch(items, forced, dg.BATCH_TIMING)
    tb.upload()
    tb.run()
    tb.run()
    tb.sync()
    stage_ms = tb.stage_ms()  # of the last pass
    tb.close()
    bytes_of = {"unstuff": 2 * stats["compressed"],
                "huff_restart": stats["rst_compressed"] + stats["rst_coef_bytes"],
                "huff_spec": stats["compressed"] - stats["rst_compressed"] + stats["coef_bytes"] - stats["rst_coef_bytes"]}
    stages = {}
    for name, ms in stage_ms.items():
        if ms < 0.02:
            continue
        stages[name] = {"ms": round(ms, 3)}
        if bytes_of.get(name):
            stages[name]["gbs"] = round(bytes_of[name] / ms / 1e6, 1)
    out["stages"] = stages
    out["stage_pass"] = {"ms_serial_sum": round(sum(stage_ms.values()), 3),
                         "note": "stages timed in a one-stream pass; value is timed with the waves overlapped on two streams"}
    # The graded figure: the stages after entropy decoding on their algorithmic bytes -- coefficients in (2 bytes per
    # MCU-padded sample) plus pixels out (decoded RGB, or the bucket-sized payload when a resize follows, in which case
    # the resize kernels belong to the stage); a resize-only workload is graded on source pixels used + payload.
    post_ms = stage_ms.get("idct", 0.0) + stage_ms.get("color", 0.0)
    resize_ms = stage_ms.get("resize_h", 0.0) + stage_ms.get("resize_v", 0.0) + stage_ms.get("resize_shift", 0.0)
    roofline = None
    if cfg and cfg.get("crop_and_resize") and resize_ms > 0:
        rbytes, payload = resize_bytes(ctx, wl)
        out["resize"] = {"ms": round(resize_ms, 3), "bytes": rbytes, "gbs": round(rbytes / resize_ms / 1e6, 1),
                         "frac": round(rbytes / resize_ms / 1e6 / peak, 4)}
        if post_ms > 0:
            pbytes, pms, kern = stats["coef_bytes"] + payload, post_ms + resize_ms, "idct+color+resize"
        else:
            pbytes, pms, kern = rbytes, resize_ms, "resize_h+resize_v+resize_shift"
    else:
        pbytes, pms, kern = stats["coef_bytes"] + stats["rgb_bytes"], post_ms, "idct+color"
    if pms > 0:
        out["post_entropy"] = {"ms": round(pms, 3), "bytes": pbytes, "gbs": round(pbytes / pms / 1e6, 1),
                               "frac": round(pbytes / pms / 1e6 / peak, 4)}
        per_px = (traffic.get(wl.name) or {}).get("dram_bytes_per_pixel")
        roofline = {"kernel": kern, "bound": "hbm", "achieved": out["post_entropy"]["gbs"], "peak": peak, "unit": "GB/s",
                    "frac": out["post_entropy"]["frac"], "traffic": int(per_px * stats["pixels"]) if per_px else None,
                    "algorithmic_bytes": pbytes,
                    "longest_stage": max(stages, key=lambda k: stages[k]["ms"]) if stages else None}
    out["roofline"] = roofline
    huff_ms = stage_ms.get("huff_restart", 0.0) + stage_ms.get("huff_spec", 0.0)
    if huff_ms:
        sm_mhz = out["clocks"].get("sm_mhz") or 1965.0
        out["huffman"] = {"ms": round(huff_ms, 3),
                          "bits_per_cycle_per_sm": round(stats["compressed"] * 8 / (huff_ms / 1000.0 * sm_mhz * 1e6 * 148), 4)}
    if kernels_only:
        ctx.close()
        return out

    # -- end to end through the batch API: host bytes in, host pixels out.  Sub-batches alternate between two contexts
    #    (two streams), the way a host batcher drives the library, so that the device-to-host copy of one sub-batch
    #    overlaps the planning, upload and kernels of the next.
    # at least four sub-batches per pass, so that the two contexts have something to overlap on the smaller workloads
    chunk = max(1, min(chunk, (len(items) + 3) // 4))
    if wl.name == "c4":
        chunk += chunk % 2  # keep the two payloads of a sample in one sub-batch
    max_out = 0
    for c0 in range(0, len(items), chunk):
        with ctx.batch(items[c0:c0 + chunk], forced[c0:c0 + chunk] if forced else None, 0) as bb:
            max_out = max(max_out, bb.packed_bytes())
    lanes = [(ctx, torch.empty(max_out + 4096, dtype=torch.uint8).pin_memory().numpy()),
             (dg.Context(local_rank, cfg), torch.empty(max_out + 4096, dtype=torch.uint8).pin_memory().numpy())]
    h2d = d2h = 0

    def finish(bb):
        nonlocal h2d, d2h
        bb.sync()
        assert all(bb.result(i).status == 0 for i in range(0, len(bb), 97))
        c = bb.counters()
        h2d += c["h2d_bytes"]
        d2h += c["d2h_bytes"]
        bb.close()

    def e2e_pass(to_host=True):
        nonlocal h2d, d2h
        h2d = d2h = 0
        pending = [None, None]
        for k, c0 in enumerate(range(0, len(items), chunk)):
            lane_ctx, pin_np = lanes[k % 2]
            if pending[k % 2] is not None:
                finish(pending[k % 2])  # the pinned buffer of this lane is free again
            bb = lane_ctx.batch(items[c0:c0 + chunk], forced[c0:c0 + chunk] if forced else None, 0 if to_host else dg.BATCH_COLLATE)
            bb.upload()
            bb.run()
            if to_host:
                bb.download_packed(pin_np)  # one copy; payload i is pin_np[result(i).packed_offset:][:nbytes]
            pending[k % 2] = bb
        for bb in pending:
            if bb is not None:
                finish(bb)

    def timed(fn):
        torch.cuda.synchronize()
        barrier()
        t0 = time.perf_counter()
        for _ in range(e2e_steps):
            fn()
        torch.cuda.synchronize()
        dt = time.perf_counter() - t0
        barrier()
        return n_samples * e2e_steps / all_max(dt)

    e2e_pass()  # warm-up: grows the library's pinned and device block caches
    v = timed(e2e_pass)
    out["e2e"] = {"value": v, "unit": "images/s", "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
                  "steps": e2e_steps, "batch": chunk, "streams": 2}
    # Same, with the payloads left in HBM as per-bucket [n, h, w, c] arrays (what a training process on the same GPU
    # consumes): host bytes in, only the per-image status words come back.
    v = timed(lambda: e2e_pass(to_host=False))
    out["e2e_device_payloads"] = {"value": v, "unit": "images/s", "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
                                  "note": "payloads stay on the device, collated per bucket; not the headline e2e"}
    lanes[1][0].close()

    # Same host-to-host job through the per-sample front end: worker threads submit single samples and wait for them,
    # as datago's tokio workers would; the library cuts the batches (two lanes of up to 512 samples).
    if feeder_threads > 0 and not forced:
        flags = dg.BATCH_DECODE_ONLY if not (cfg and cfg.get("crop_and_resize")) else 0
        with dg.Feeder(local_rank, cfg, lanes=2, max_batch=min(chunk, 512), max_wait_us=2000, queue_limit=4 * chunk, flags=flags) as feeder:
            depth = 128  # samples each worker keeps in flight, so that the batches fill

            def worker(k):
                pending = []

                def fin(t):
                    r = feeder.wait(t)
                    assert r.status == 0
                    px = feeder.peek(t, r)  # the payload where the library's download left it: page-locked host memory
                    assert px.size == r.nbytes and int(px.flat[0]) + int(px.flat[-1]) >= 0
                    feeder.release(t)

                for i in range(k, len(items), feeder_threads):
                    if len(pending) == depth:
                        fin(pending.pop(0))
                    pending.append(feeder.submit(items[i]))
                for t in pending:
                    fin(t)

            def feeder_pass():
                ths = [threading.Thread(target=worker, args=(k,)) for k in range(feeder_threads)]
                for th in ths:
                    th.start()
                for th in ths:
                    th.join()

            feeder_pass()  # warm-up
            v = timed(feeder_pass)
            st = feeder.stats()
        out["e2e_feeder"] = {"value": v, "unit": "images/s", "threads": feeder_threads, "in_flight": feeder_threads * depth,
                             "mean_batch": round(st["batched_items"] / max(1, st["batches"]), 1),
                             "note": "per-sample dg_submit / dg_wait / dg_peek from Python worker threads; not the headline e2e"}
    ctx.close()
    return out


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="c2", choices=["c0", "c1", "c2", "c3", "c4"])
    ap.add_argument("--images", type=int, default=0, help="samples in the workload (default: the configuration's own count; c3: 8000)")
    ap.add_argument("--e2e-chunk", type=int, default=1024)
    ap.add_argument("--feeder-threads", type=int, default=16, help="worker threads of the submit / wait measurement (0: skip)")
    ap.add_argument("--kernels-only", action="store_true", help="resident passes and the per-stage pass only (profiling runs)")
    ap.add_argument("--no-side-configs", action="store_true", help="skip the shorter C0 and C1 measurements of the default run")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    args = ap.parse_args()

    from datago_b200 import synth
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    # C3 at its full size is 64 shards; the default here is 8 of them so that generating the shards stays within minutes
    count = args.images or (8000 if args.workload == "c3" else synth.COUNTS[args.workload])
    strong = args.workload == "c3"
    config = {"workload": LABELS[args.workload].format(n=count), "images_per_gpu": count if not strong else f"{count} / N by key hash",
              "sharding": "key-hash dispatch of one fixed shard set (dg_key_rank), no collective" if strong else
                          "contiguous rank slices of an N x workload job, no collective",
              "l2": "inputs and intermediates of one pass exceed the 126 MB L2 many times over; no explicit flush"}

    # ---------------- reference arm: the CPU path on the host cores ------------------------------------------------
    if args.impl == "reference":
        if rank != 0:
            return
        import datago_b200 as dg
        keys = dg.Context(dg.DG_DEVICE_NONE, synth.IMAGE_CONFIGS[args.workload]) if args.workload == "c4" else None
        wl = load_workload(args.workload, count, 0, 1, lambda: None, keys)
        vals, base = [], None
        for step in range(args.warmup + args.steps):
            base = cpu_baseline(wl, budget_s=8.0 if step >= args.warmup else 2.0)
            if step >= args.warmup:
                vals.append(base["value"])
        v = statistics.mean(vals)
        base["value"] = v
        print(json.dumps({"impl": "reference", "metric": METRIC, "value": v, "unit": "images/s", "n_gpus": args.gpus,
                          "steps": args.steps, "warmup": args.warmup, "ms_per_step": 1000.0 * count / v,
                          "higher_is_better": True, "scaling": "strong" if strong else "weak", "vs_baseline": None, "dtype": "u8",
                          "data": "synthetic", "config": config, "cpu_baseline": base,
                          "e2e": {"value": v, "unit": "images/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}))
        return

    # ---------------- our arm ------------------------------------------------------------------------------------------------
    import torch
    import torch.distributed as dist
    import datago_b200 as dg

    torch.cuda.set_device(local_rank)
    # several ranks on one box: host threads and the page-locked staging memory of each rank next to its GPU (a box may
    # have more than one socket).  A single rank keeps all cores: the CPU baseline of the same run uses them.
    bound = dg.bind_to_gpu_cpus(local_rank) if world > 1 and os.environ.get("DATAGO_B200_BENCH_BIND", "1") != "0" else None
    print(f"[bench] rank {rank}: host cores {'unchanged' if bound is None else f'{bound[0]}..{bound[-1]} ({len(bound)})'}", file=sys.stderr)
    # stdout carries the one JSON line: keep NCCL's own banner (NCCL_DEBUG=VERSION) and debug text off it
    if os.environ.get("NCCL_DEBUG", "").upper() == "VERSION":
        os.environ["NCCL_DEBUG"] = "WARN"
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))

    def barrier():
        if world > 1:
            dist.barrier()

    def all_max(x, op="max"):
        if world == 1:
            return x
        t = torch.tensor([float(x)], dtype=torch.float64, device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MAX if op == "max" else dist.ReduceOp.SUM)
        return float(t.item())

    peak, peak_src = load_peaks()
    traffic = load_traffic()
    keys = dg.Context(dg.DG_DEVICE_NONE, synth.IMAGE_CONFIGS[args.workload]) if args.workload == "c4" else None
    wl = load_workload(args.workload, count, rank, world, barrier, keys)
    e2e_steps = max(1, min(args.steps, 5))
    big = args.workload in ("c1", "c4")  # multi-megapixel items: the oracle needs seconds for a few of them
    rep = measure(wl, local_rank, world, barrier, all_max, args.steps, args.warmup, e2e_steps, args.e2e_chunk,
                  args.feeder_threads, 16 if big else 64, args.kernels_only, peak, traffic)
    line = {"metric": METRIC, "value": rep.pop("value"), "unit": "images/s", "n_gpus": world, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": rep.pop("ms_per_step"), "higher_is_better": True,
            "scaling": "strong" if strong else "weak", "vs_baseline": None, "dtype": "u8", "data": "synthetic", "config": config}
    if rep.get("roofline"):
        rep["roofline"]["peak_source"] = peak_src
    line.update(rep)
    if world == 1 and not args.no_cpu_baseline and not args.kernels_only:
        line["cpu_baseline"] = cpu_baseline(wl)
        y = pil_yardstick(wl.items)
        if y:
            line["cpu_baseline"]["pillow_libjpeg_turbo_decode"] = y

    # ---------------- the other single-GPU configurations, shorter, in the same process --------------------------------
    if args.workload == "c2" and not args.images and world == 1 and not args.kernels_only and not args.no_side_configs:
        configs = {}
        for name in ("c0", "c1"):
            side = load_workload(name, synth.COUNTS[name], 0, 1, lambda: None)
            r = measure(side, local_rank, 1, lambda: None, lambda x, op="max": x, max(3, args.steps // 4), 3, 2, args.e2e_chunk,
                        0, 8 if name == "c1" else 24, False, peak, traffic)
            r["workload"] = LABELS[name].format(n=synth.COUNTS[name])
            if not args.no_cpu_baseline:
                r["cpu_baseline"] = cpu_baseline(side, budget_s=6.0)
            configs[name] = r
            del side
        line["configs"] = configs
    if rank == 0:
        print(json.dumps(line))
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
