"""Benchmark of the image hot path on B200: decoded(+bucketed) images/s on seeded synthetic JPEGs.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload c2|c0|c1] [--images M] [--impl reference]

A step is one pass of the path over the whole workload (default: the 8192-JPEG decode-throughput set).  `value` is
measured with the compressed inputs already in HBM (CUDA events on the library's stream around K back-to-back passes);
`e2e` goes through the public batch API from host JPEG bytes to host pixel buffers.  Multi-GPU runs are weak-scaled:
every rank owns one workload-sized shard of an N-times larger job (contiguous rank slices, the rule datago's file
source uses) and there is no collective on the data path; only the timing is reduced across ranks.
`--impl reference` times the CPU implementation of the same path (the oracle port; the reference's Rust crates are not
buildable here) on all host cores.
"""
import argparse
import json
import os
import pickle
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

import numpy as np  # noqa: E402

METRIC = "decoded+bucketed images/s"


def load_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        return float(json.load(open(path))["hbm_gbs"]), "measured"
    return 6650.0, "fallback"


def dataset(workload, count, rank, world, barrier):
    """The seeded workload, generated once per box (rank 0) and shared through /dev/shm."""
    from datago_b200 import synth
    cache = f"/dev/shm/datago_b200_{workload}_{count}.pkl"
    if rank == 0 and not os.path.exists(cache):
        procs = max(1, (os.cpu_count() or 8) - 1)
        t = time.time()
        items = synth.make(workload, range(count), processes=procs)
        with open(cache + ".tmp", "wb") as f:
            pickle.dump(items, f, protocol=4)
        os.replace(cache + ".tmp", cache)
        print(f"[bench] generated {count} {workload} items on {procs} processes in {time.time() - t:.1f}s", file=sys.stderr)
    barrier()
    with open(cache, "rb") as f:
        return pickle.load(f)


class ClockSampler:
    QUERY = "clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap"

    def __init__(self, index):
        self.index = index
        self.rows = []
        self.proc = None

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
        self.rows = inside if len(inside) >= 3 else [r for (_, r) in rows]
        sm = [float(r[0]) for r in self.rows if r and r[0].replace(".", "").isdigit()]
        mx = [float(r[1]) for r in self.rows if len(r) > 1 and r[1].replace(".", "").isdigit()]
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        reasons = [n for i, n in enumerate(names) if any(len(r) > 3 + i and r[3 + i] == "Active" for r in self.rows)]
        pw = [float(r[2]) for r in self.rows if len(r) > 2 and r[2].replace(".", "").isdigit()]
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "power_w_max": max(pw) if pw else None, "samples": len(sm), "reasons": reasons}


def workload_stats(items, workload):
    """Pixels and algorithmic bytes of one pass: coefficients 2 B per MCU-padded sample, planes 1 B per sample, RGB 3 B per pixel."""
    import datago_b200 as dg
    st = dict(images=len(items), pixels=0, compressed=0, coef_bytes=0, plane_bytes=0, rgb_bytes=0, ecs_bits=0)
    for it in items:
        if isinstance(it, (bytes, bytearray)):
            i = dg.jpeg_probe(it)
            bpm = 1 if i.channels == 1 else i.hsamp * i.vsamp + 2
            blocks = i.mcux * i.mcuy * bpm
            st["pixels"] += i.width * i.height
            st["compressed"] += i.scan_len
            st["coef_bytes"] += blocks * 128      # 2 * s * P_mcu
            st["plane_bytes"] += blocks * 64
            st["rgb_bytes"] += i.width * i.height * i.channels
        else:
            st["pixels"] += it.shape[0] * it.shape[1]
            st["rgb_bytes"] += it.nbytes
    return st


def cpu_baseline(items, kind, cfg, budget_s=12.0):
    """The oracle port on all host cores over a bounded sample of the workload."""
    import oracle
    threads = os.cpu_count() or 1
    probe_n = min(len(items), max(2 * threads, 8))
    call = oracle.run_batch(items[:probe_n], kind, cfg, threads)
    t = time.time()
    call()
    per_image = max(1e-4, (time.time() - t) / probe_n)  # seconds per image with all threads busy
    n = int(min(len(items), max(probe_n, budget_s / per_image)))
    call = oracle.run_batch(items[:n], kind, cfg, threads)
    t = time.time()
    ok = call()
    dt = time.time() - t
    return {"value": ok / dt, "unit": "images/s", "cores": threads, "kind": "port",
            "sample": f"first {n} of {len(items)} items of the workload, {dt:.1f}s wall"}


def pil_yardstick(items, budget_s=6.0):
    """libjpeg-turbo through Pillow on a thread pool: an independent SIMD-optimised CPU decoder, for scale."""
    import io
    from concurrent.futures import ThreadPoolExecutor
    from PIL import Image
    threads = os.cpu_count() or 1

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
    return {"value": n2 / dt, "unit": "images/s", "cores": threads, "sample": f"{n2} items"}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="c2", choices=["c0", "c1", "c2"])
    ap.add_argument("--images", type=int, default=0)
    ap.add_argument("--e2e-chunk", type=int, default=1024)
    ap.add_argument("--feeder-threads", type=int, default=16, help="worker threads of the submit / wait measurement (0: skip)")
    ap.add_argument("--contexts", type=int, default=1, help="library contexts the resident workload is split over")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    args = ap.parse_args()

    from datago_b200 import synth
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    count = args.images or synth.COUNTS[args.workload]
    cfg = synth.IMAGE_CONFIGS[args.workload]
    kind = {"c0": 1, "c1": 2, "c2": 0}[args.workload]
    config = {"workload": {"c0": f"C0 local-file set: {count} 4:2:0 q90 JPEGs 256..2048, decode + 1024/32 bucket crop-resize",
                           "c1": f"C1 resize-only: {count} raw RGB buffers 512..4096, 512/16 buckets",
                           "c2": f"C2 JPEG decode throughput: {count} baseline 4:2:0 JPEGs 512..1536, q75-95, half with restart interval 4, decode to RGB8"}[args.workload],
              "images_per_gpu": count, "contexts": args.contexts, "sharding": "contiguous rank slices of an N x workload job, no collective",
              "l2": "inputs and intermediates of one pass exceed the 126 MB L2 many times over; no explicit flush"}

    # ---------------- reference arm: the CPU path on the host cores ------------------------------------------------
    if args.impl == "reference":
        if rank != 0:
            return
        items = dataset(args.workload, count, 0, 1, lambda: None)
        vals = []
        base = None
        for step in range(args.warmup + args.steps):
            base = cpu_baseline(items, kind, cfg, budget_s=8.0 if step >= args.warmup else 2.0)
            if step >= args.warmup:
                vals.append(base["value"])
        v = statistics.mean(vals)
        base["value"] = v
        print(json.dumps({"impl": "reference", "metric": METRIC, "value": v, "unit": "images/s", "n_gpus": args.gpus,
                          "steps": args.steps, "warmup": args.warmup, "ms_per_step": 1000.0 * count / v,
                          "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "u8",
                          "data": "synthetic", "config": config, "cpu_baseline": base,
                          "e2e": {"value": v, "unit": "images/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}))
        return

    # ---------------- our arm ------------------------------------------------------------------------------------------------
    import torch
    import torch.distributed as dist
    import datago_b200 as dg

    torch.cuda.set_device(local_rank)
    # stdout carries the one JSON line: keep NCCL's own banner (NCCL_DEBUG=VERSION) and debug text off it
    if os.environ.get("NCCL_DEBUG", "").upper() == "VERSION":
        os.environ["NCCL_DEBUG"] = "WARN"
    os.environ.setdefault("NCCL_DEBUG_FILE", "/dev/stderr")
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))

    def barrier():
        if world > 1:
            dist.barrier()

    items = dataset(args.workload, count, rank, world, barrier)
    quorum = world * count
    start, end = dg.rank_slice(quorum, rank, world)  # this rank's shard of the N x workload job
    items = [items[i % count] for i in range(start, end)]
    stats = workload_stats(items, args.workload)

    stream = torch.cuda.Stream()
    ctx = dg.Context(local_rank, cfg, stream=stream.cuda_stream)
    peak, peak_src = load_peaks()

    # -- inputs resident in HBM ---------------------------------------------------------------------------------------
    # The workload is split over `--contexts` library contexts (contiguous parts, one resident batch and one stream
    # each), the way the library is driven in production (a feeder lane per context): a step is one pass over every
    # part, queued back to back, so the parts' passes overlap each other within a step and from one step to the next.
    # CUDA events on a parent stream bracket all K steps: every context stream waits for the start event, the end
    # event waits for every context stream.
    n_ctx = max(1, min(args.contexts, len(items)))
    part = (len(items) + n_ctx - 1) // n_ctx
    streams = [stream] + [torch.cuda.Stream() for _ in range(n_ctx - 1)]
    ctxs = [ctx] + [dg.Context(local_rank, cfg, stream=st.cuda_stream) for st in streams[1:]]
    batches = []
    for k in range(n_ctx):
        b = ctxs[k].batch(items[k * part:(k + 1) * part], None, 0)
        b.upload()
        b.sync()
        batches.append(b)
    sampler = ClockSampler(local_rank)
    sampler.start()
    time.sleep(1.0)  # nvidia-smi needs a moment before its first sample
    for _ in range(args.warmup):
        for b in batches:
            b.run()
    for b in batches:
        b.sync()
        assert all(b.result(i).status == 0 for i in range(len(b))), "an image failed to decode"
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    parent = torch.cuda.Stream()
    done = [torch.cuda.Event() for _ in streams]
    torch.cuda.synchronize()
    barrier()
    t_begin = time.time()
    e0.record(parent)
    for st in streams:
        st.wait_event(e0)
    for _ in range(args.steps):
        for b in batches:
            b.run()
    for st, ev in zip(streams, done):
        ev.record(st)
        parent.wait_event(ev)
    e1.record(parent)
    torch.cuda.synchronize()
    barrier()
    sampler.window(t_begin, time.time())
    elapsed_ms = e0.elapsed_time(e1)
    clocks = sampler.stop()
    launches = 0
    for b in batches:
        b.sync()
        launches += b.counters()["kernel_launches"] * args.steps
        b.close()
    for c in ctxs[1:]:
        c.close()
    # Per-kernel durations: one more pass of the same workload with CUDA events around every stage.  A timing batch
    # keeps all waves on one stream, so each event pair brackets a kernel that ran alone (the timed passes above
    # overlap the waves on two streams).
    tb = ctx.batch(items, None, dg.BATCH_TIMING)
    tb.upload()
    tb.run()
    tb.run()
    tb.sync()
    stage_ms = tb.stage_ms()  # of the last pass
    serial_ms = sum(stage_ms.values())
    tb.close()
    t = torch.tensor([elapsed_ms], dtype=torch.float64, device="cuda")
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    elapsed_ms = float(t.item())
    value = world * len(items) * args.steps / (elapsed_ms / 1000.0)

    # -- end to end through the batch API: host bytes in, host pixels out ------------------------------------------
    # Sub-batches alternate between two contexts (two streams), the way a host batcher would drive the library, so
    # that the device-to-host copy of one sub-batch overlaps the planning, upload and kernels of the next.
    chunk = max(1, min(args.e2e_chunk, len(items)))
    e2e_steps = max(1, min(args.steps, 5))
    max_out = 0
    for c0 in range(0, len(items), chunk):
        with ctx.batch(items[c0:c0 + chunk], None, 0) as b:
            max_out = max(max_out, b.packed_bytes())
    lanes = [(ctx, torch.empty(max_out + 4096, dtype=torch.uint8).pin_memory().numpy()),
             (dg.Context(local_rank, cfg), torch.empty(max_out + 4096, dtype=torch.uint8).pin_memory().numpy())]
    h2d = d2h = 0

    def finish(pending):
        nonlocal h2d, d2h
        b, outs = pending
        b.sync()
        assert all(b.result(i).status == 0 for i in range(0, len(b), 97))
        c = b.counters()
        h2d += c["h2d_bytes"]
        d2h += c["d2h_bytes"]
        b.close()

    def e2e_pass(to_host=True):
        nonlocal h2d, d2h
        h2d = d2h = 0
        pending = [None, None]
        for k, c0 in enumerate(range(0, len(items), chunk)):
            lane_ctx, pin_np = lanes[k % 2]
            if pending[k % 2] is not None:
                finish(pending[k % 2])  # the pinned buffer of this lane is free again
            b = lane_ctx.batch(items[c0:c0 + chunk], None, 0 if to_host else dg.BATCH_COLLATE)
            b.upload()
            b.run()
            if to_host:
                b.download_packed(pin_np)  # one copy; payload i is pin_np[result(i).packed_offset:][:nbytes]
            outs = pin_np
            pending[k % 2] = (b, outs)
        for pnd in pending:
            if pnd is not None:
                finish(pnd)

    e2e_pass()  # warm-up: grows the library's pinned and device block caches
    torch.cuda.synchronize()
    barrier()
    t0 = time.perf_counter()
    for _ in range(e2e_steps):
        e2e_pass()
    torch.cuda.synchronize()
    e2e_s = time.perf_counter() - t0
    barrier()
    t = torch.tensor([e2e_s], dtype=torch.float64, device="cuda")
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    e2e_value = world * len(items) * e2e_steps / float(t.item())
    e2e_h2d, e2e_d2h = h2d, d2h

    # Same, with the payloads left in HBM as per-bucket [n, h, w, c] arrays (what a training process on the same GPU
    # consumes): host bytes in, only the per-image status words come back.
    barrier()
    t0 = time.perf_counter()
    for _ in range(e2e_steps):
        e2e_pass(to_host=False)
    torch.cuda.synchronize()
    dev_s = time.perf_counter() - t0
    barrier()
    t = torch.tensor([dev_s], dtype=torch.float64, device="cuda")
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    e2e_device = {"value": world * len(items) * e2e_steps / float(t.item()), "unit": "images/s",
                  "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
                  "note": "payloads stay on the device, collated per bucket; not the headline e2e"}

    # Same host-to-host job through the per-sample front end: worker threads submit single samples and wait for
    # them, as datago's tokio workers would; the library cuts the batches (two lanes of up to 512 samples).
    import threading
    n_workers = args.feeder_threads
    feeder_value = None
    if n_workers > 0:
        flags = dg.BATCH_DECODE_ONLY if not (cfg and cfg.get("crop_and_resize")) else 0
        with dg.Feeder(local_rank, cfg, lanes=2, max_batch=min(chunk, 512), max_wait_us=2000, queue_limit=4 * chunk, flags=flags) as feeder:
            # samples each worker keeps in flight: the batches fill to what arrives within max_wait_us, so the workers
            # have to keep a few hundred samples outstanding between them
            depth = 128

            def worker(k):
                # each worker keeps `depth` samples in flight and reads every payload where the library's download
                # left it (dg_peek: page-locked host memory), touching its first and last byte
                mine = list(range(k, len(items), n_workers))
                pending = []

                def finish(t):
                    r = feeder.wait(t)
                    assert r.status == 0
                    px = feeder.peek(t, r)
                    assert px.size == r.nbytes and int(px.flat[0]) + int(px.flat[-1]) >= 0
                    feeder.release(t)

                for i in mine:
                    if len(pending) == depth:
                        finish(pending.pop(0))
                    pending.append(feeder.submit(items[i]))
                for t in pending:
                    finish(t)

            def feeder_pass():
                ths = [threading.Thread(target=worker, args=(k,)) for k in range(n_workers)]
                for th in ths:
                    th.start()
                for th in ths:
                    th.join()

            feeder_pass()  # warm-up
            barrier()
            t0 = time.perf_counter()
            for _ in range(e2e_steps):
                feeder_pass()
            fs = time.perf_counter() - t0
            barrier()
            st = feeder.stats()
        t = torch.tensor([fs], dtype=torch.float64, device="cuda")
        if world > 1:
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        feeder_value = {"value": world * len(items) * e2e_steps / float(t.item()), "unit": "images/s", "threads": n_workers, "in_flight": n_workers * depth,
                        "mean_batch": round(st["batched_items"] / max(1, st["batches"]), 1),
                        "note": "per-sample dg_submit / dg_wait / dg_peek from Python worker threads, payloads in the library's page-locked host buffers; not the headline e2e"}

    if rank != 0:
        if world > 1:
            dist.destroy_process_group()
        return

    # -- roofline of the dominant kernel, from the stage events of the last timed pass -----------------------------
    bytes_of = {
        "unstuff": 2 * stats["compressed"],
        "coef_clear": stats["coef_bytes"],
        "huff_restart": None, "huff_spec": None,  # filled below (split by image class)
        "idct": stats["coef_bytes"] + stats["plane_bytes"],
        "color": stats["plane_bytes"] + stats["rgb_bytes"],
    }
    rst_items = [it for it in items if isinstance(it, (bytes, bytearray)) and dg.jpeg_probe(it).restart_interval]
    rst_stats = workload_stats(rst_items, args.workload) if rst_items else dict(compressed=0, coef_bytes=0)
    bytes_of["huff_restart"] = rst_stats["compressed"] + rst_stats["coef_bytes"]
    bytes_of["huff_spec"] = (stats["compressed"] - rst_stats["compressed"]) + (stats["coef_bytes"] - rst_stats["coef_bytes"])
    stages = {}
    for name, ms in stage_ms.items():
        if ms < 0.05:  # e.g. the coefficient clear, which only runs on a scratch block's first use
            continue
        b = bytes_of.get(name)
        stages[name] = {"ms": round(ms, 3)}
        if b:
            stages[name]["gbs"] = round(b / ms / 1e6, 1)
            stages[name]["frac"] = round(b / ms / 1e6 / peak, 4)
    # The roofline object grades the longest HBM-graded stage (IDCT, colour, resize).  Entropy decoding is serial bit
    # parsing: it is reported in bits per cycle (`huffman`) and, when it is the longest stage, named in `longest_stage`.
    longest = max(stages, key=lambda k: stages[k]["ms"]) if stages else None
    graded = [k for k in stages if not k.startswith("huff") and k != "unstuff"]
    top = max(graded, key=lambda k: stages[k]["ms"]) if graded else longest
    roofline = None
    if top:
        achieved = stages[top].get("gbs")
        # DRAM bytes per launch: dram__bytes_read + dram__bytes_write of one ncu capture on a 256 / 1024-image case of
        # this workload (profiles/), expressed per algorithmic byte and scaled to this pass by the units it processes
        # (traffic grows in proportion to the image count).  The entropy kernels move fewer bytes than the dense
        # coefficient array they fill: only the sectors that hold non-zero coefficients are written.
        ncu_bytes_per_algorithmic_byte = {"idct": 1.205, "color": 0.958, "huff_restart": 0.66, "huff_spec": 0.63}
        ratio = ncu_bytes_per_algorithmic_byte.get(top)
        roofline = {"kernel": top, "bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s",
                    "frac": round(achieved / peak, 4) if achieved else None,
                    "traffic": int(ratio * bytes_of[top]) if ratio and bytes_of.get(top) else None, "peak_source": peak_src,
                    "longest_stage": longest}
    post_ms = stage_ms.get("idct", 0.0) + stage_ms.get("color", 0.0)
    roofline_top = top
    post_bytes = stats["coef_bytes"] + stats["rgb_bytes"]
    post = {"ms": round(post_ms, 3), "bytes": post_bytes, "gbs": round(post_bytes / post_ms / 1e6, 1) if post_ms else None,
            "frac": round(post_bytes / post_ms / 1e6 / peak, 4) if post_ms else None}
    # crop_and_resize: C * P_used + C * tw * th per image, P_used = the source pixels that map into the crop
    resize = None
    resize_ms = stage_ms.get("resize_h", 0.0) + stage_ms.get("resize_v", 0.0) + stage_ms.get("resize_shift", 0.0)
    if cfg and cfg.get("crop_and_resize") and resize_ms > 0:
        import math
        rbytes = 0
        for it in items:
            if isinstance(it, (bytes, bytearray)):
                i = dg.jpeg_probe(it)
                w_, h_, c_ = i.width, i.height, i.channels
            else:
                h_, w_ = it.shape[:2]
                c_ = 1 if it.ndim == 2 else it.shape[2]
            p = ctx.plan_geometry(w_, h_, c_)
            scale = max(p.target_w / w_, p.target_h / h_)
            used = min(w_, math.ceil(p.target_w / scale)) * min(h_, math.ceil(p.target_h / scale))
            rbytes += c_ * used + c_ * p.target_w * p.target_h
        resize = {"ms": round(resize_ms, 3), "bytes": rbytes, "gbs": round(rbytes / resize_ms / 1e6, 1),
                  "frac": round(rbytes / resize_ms / 1e6 / peak, 4)}
    huff_ms = stage_ms.get("huff_restart", 0.0) + stage_ms.get("huff_spec", 0.0)
    sm_mhz = clocks.get("sm_mhz") or 1965.0
    huff = {"ms": round(huff_ms, 3),
            "bits_per_cycle_per_sm": round(stats["compressed"] * 8 / (huff_ms / 1000.0 * sm_mhz * 1e6 * 148), 4) if huff_ms else None}

    if roofline and roofline_top and roofline_top.startswith("resize") and resize:
        # the resize passes share one algorithmic figure (source pixels used + payload), reported over their sum
        roofline.update({"kernel": "resize_h+resize_v+resize_shift", "achieved": resize["gbs"], "frac": resize["frac"]})
    line = {"metric": METRIC, "value": value, "unit": "images/s", "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": elapsed_ms / args.steps, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": "u8", "data": "synthetic", "config": config,
            "mpix_per_s": value * stats["pixels"] / len(items) / 1e6,
            "e2e": {"value": e2e_value, "unit": "images/s", "h2d_bytes_per_step": e2e_h2d, "d2h_bytes_per_step": e2e_d2h,
                    "steps": e2e_steps, "batch": chunk, "streams": 2},
            "e2e_device_payloads": e2e_device, "e2e_feeder": feeder_value,
            "gpu_launches": launches, "clocks": clocks, "roofline": roofline, "stages": stages, "post_entropy": post, "resize": resize,
            "huffman": huff, "stage_pass": {"ms_serial_sum": round(serial_ms, 3), "note": "stages timed in a one-stream pass over the whole workload; value is timed with the workload split over `contexts` contexts, each overlapping its waves on two streams"}}
    if world == 1 and not args.no_cpu_baseline:
        line["cpu_baseline"] = cpu_baseline(items, kind, cfg)
        if args.workload != "c1":
            line["cpu_baseline"]["pillow_libjpeg_turbo_decode"] = pil_yardstick(items)
    print(json.dumps(line))
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
