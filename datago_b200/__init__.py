"""datago_b200: the B200 image path of datago (decode -> bucket -> resize -> crop) behind a C ABI.

This module is the thin Python side of include/datago_b200.h (ctypes, no torch needed).  Pixel work is
done by the CUDA library only; importing works without a GPU (bucket / geometry / sharding queries are
host code), but creating a device context or running a batch without one raises DatagoB200Error.
"""
import ctypes as C
import os

import numpy as np

from .build import build as _build

_HERE = os.path.dirname(os.path.abspath(__file__))

DG_DEVICE_NONE = -1
BATCH_DECODE_ONLY = 1
BATCH_TIMING = 2
BATCH_KEEP_COEFFICIENTS = 4
BATCH_COLLATE = 8
ITEM_TO_RGB8 = 1
STAGES = ("unstuff", "coef_clear", "huff_restart", "huff_spec", "idct", "color", "resize_h", "resize_v", "resize_shift",
          "to_rgb8")
STATUS_NAMES = {0: "ok", 1: "invalid", 2: "cuda", 3: "truncated", 4: "bad_marker", 5: "unsupported", 6: "bad_table",
                7: "bad_code", 8: "unknown_key", 9: "no_transform", 10: "sync_limit", 11: "too_large", 12: "timeout"}
E_TIMEOUT = 12


class DatagoB200Error(RuntimeError):
    def __init__(self, code, msg):
        super().__init__(f"[{STATUS_NAMES.get(code, code)}] {msg}")
        self.code = code


class ImageConfig(C.Structure):
    _fields_ = [("crop_and_resize", C.c_int32), ("default_image_size", C.c_uint32), ("downsampling_ratio", C.c_uint32),
                ("min_aspect_ratio", C.c_double), ("max_aspect_ratio", C.c_double)]

    @classmethod
    def from_dict(cls, d):
        """From the `image_config` object of datago's client JSON (missing numbers default to 0, as serde does)."""
        return cls(int(bool(d.get("crop_and_resize", False))), int(d.get("default_image_size", 0)),
                   int(d.get("downsampling_ratio", 0)), float(d.get("min_aspect_ratio", 0.0)),
                   float(d.get("max_aspect_ratio", 0.0)))


class Plan(C.Structure):
    _fields_ = [("src_w", C.c_uint32), ("src_h", C.c_uint32), ("channels", C.c_uint32), ("target_w", C.c_uint32),
                ("target_h", C.c_uint32), ("new_w", C.c_uint32), ("new_h", C.c_uint32), ("crop_left", C.c_double),
                ("crop_top", C.c_double), ("crop_w", C.c_double), ("crop_h", C.c_double), ("identity", C.c_int32),
                ("key", C.c_char * 16)]

    def as_tuple(self):
        return (self.key.decode(), self.target_w, self.target_h, self.new_w, self.new_h, self.crop_left,
                self.crop_top, self.crop_w, self.crop_h, self.identity)


class JpegInfo(C.Structure):
    _fields_ = [("width", C.c_uint32), ("height", C.c_uint32), ("channels", C.c_uint32), ("hsamp", C.c_uint32),
                ("vsamp", C.c_uint32), ("mcux", C.c_uint32), ("mcuy", C.c_uint32), ("restart_interval", C.c_uint32),
                ("scan_offset", C.c_uint64), ("scan_len", C.c_uint64)]


class Item(C.Structure):
    _fields_ = [("data", C.c_void_p), ("len", C.c_uint64), ("raw_w", C.c_uint32), ("raw_h", C.c_uint32),
                ("raw_c", C.c_uint32), ("flags", C.c_uint32), ("forced_key", C.c_char_p)]


class _ItemBytes(C.Structure):
    """Same layout as Item with `data` typed as char*: assigning a bytes object to it is the cheapest way ctypes
    offers to take the address of its buffer (and it keeps the object alive)."""
    _fields_ = [("data", C.c_char_p), ("len", C.c_uint64), ("raw_w", C.c_uint32), ("raw_h", C.c_uint32),
                ("raw_c", C.c_uint32), ("flags", C.c_uint32), ("forced_key", C.c_char_p)]


class Result(C.Structure):
    _fields_ = [("status", C.c_int32), ("original_width", C.c_uint32), ("original_height", C.c_uint32),
                ("width", C.c_uint32), ("height", C.c_uint32), ("channels", C.c_uint32), ("bit_depth", C.c_uint32),
                ("nbytes", C.c_uint64), ("device_data", C.c_void_p), ("plan", Plan), ("packed_offset", C.c_uint64)]


class Bucket(C.Structure):
    _fields_ = [("key", C.c_char * 16), ("n", C.c_uint32), ("width", C.c_uint32), ("height", C.c_uint32),
                ("channels", C.c_uint32), ("nbytes", C.c_uint64), ("device_data", C.c_void_p),
                ("packed_offset", C.c_uint64), ("items", C.POINTER(C.c_int32))]


class CtxCounters(C.Structure):
    _fields_ = [("items", C.c_uint64 * 13), ("batches", C.c_uint64), ("bytes_in", C.c_uint64), ("bytes_out", C.c_uint64)]


LOG_FN = C.CFUNCTYPE(None, C.c_int, C.c_char_p, C.c_void_p)


class FeederConfig(C.Structure):
    _fields_ = [("lanes", C.c_uint32), ("max_batch", C.c_uint32), ("max_wait_us", C.c_uint32),
                ("queue_limit", C.c_uint32), ("batch_flags", C.c_uint32), ("reserved", C.c_uint32)]


class FeederStats(C.Structure):
    _fields_ = [("submitted", C.c_uint64), ("completed", C.c_uint64), ("failed", C.c_uint64), ("batches", C.c_uint64),
                ("batched_items", C.c_uint64), ("largest_batch", C.c_uint32), ("queued", C.c_uint32),
                ("open_tickets", C.c_uint32), ("reserved", C.c_uint32)]


class DeviceArray:
    """A dense uint8 array in device memory owned by a batch; speaks __cuda_array_interface__ (version 3), so
    torch.as_tensor / cupy.asarray wrap it without a copy.  Keep the batch alive while it is in use."""

    def __init__(self, ptr, shape, owner):
        self.ptr, self.shape, self._owner = int(ptr), tuple(int(v) for v in shape), owner

    @property
    def __cuda_array_interface__(self):
        return {"shape": self.shape, "typestr": "|u1", "data": (self.ptr, False), "version": 3, "strides": None}


_lib = None


def library_path():
    return os.path.join(_HERE, "libdatago_b200.so")


def lib():
    """The loaded CUDA library; built on first use when the .so is missing or older than its sources."""
    global _lib
    if _lib is not None:
        return _lib
    path = library_path()
    if not os.path.exists(path) or os.environ.get("DATAGO_B200_REBUILD"):
        path = _build()
    L = C.CDLL(path)
    vp, u32p, u64p = C.c_void_p, C.POINTER(C.c_uint32), C.POINTER(C.c_uint64)
    sig = {
        "dg_last_error": (C.c_char_p, []),
        "dg_version": (C.c_char_p, []),
        "dg_ctx_create": (C.c_int, [C.c_int, C.POINTER(ImageConfig), C.POINTER(vp)]),
        "dg_ctx_create_on_stream": (C.c_int, [C.c_int, C.POINTER(ImageConfig), vp, C.POINTER(vp)]),
        "dg_ctx_destroy": (None, [vp]),
        "dg_ctx_stream": (vp, [vp]),
        "dg_ctx_get_counters": (C.c_int, [vp, C.POINTER(CtxCounters)]),
        "dg_set_log_callback": (None, [LOG_FN, vp]),
        "dg_size_list": (C.c_int, [C.POINTER(ImageConfig), C.c_int, vp, vp]),
        "dg_bucket_table": (C.c_int, [vp, C.c_int, vp, vp, vp, vp]),
        "dg_closest_aspect_ratio": (C.c_int, [vp, C.c_int32, C.c_int32, C.c_char_p]),
        "dg_aspect_ratio_to_str": (None, [C.c_uint32, C.c_uint32, C.c_char_p]),
        "dg_plan_geometry": (C.c_int, [vp, C.c_uint32, C.c_uint32, C.c_uint32, C.c_char_p, C.POINTER(Plan)]),
        "dg_jpeg_probe": (C.c_int, [C.c_char_p, C.c_uint64, C.POINTER(JpegInfo)]),
        "dg_rank_slice": (C.c_int, [C.c_uint64, C.c_uint64, C.c_uint64, u64p, u64p]),
        "dg_key_hash": (C.c_uint64, [C.c_char_p, C.c_uint64]),
        "dg_key_rank": (C.c_uint64, [C.c_char_p, C.c_uint64, C.c_uint64]),
        "dg_batch_create": (C.c_int, [vp, C.POINTER(Item), C.c_int, C.c_uint32, C.POINTER(vp)]),
        "dg_batch_upload": (C.c_int, [vp]),
        "dg_batch_run": (C.c_int, [vp]),
        "dg_batch_download": (C.c_int, [vp, C.POINTER(vp)]),
        "dg_batch_download_packed": (C.c_int, [vp, vp, C.c_uint64]),
        "dg_batch_packed_bytes": (C.c_uint64, [vp]),
        "dg_batch_sync": (C.c_int, [vp]),
        "dg_batch_result": (C.c_int, [vp, C.c_int, C.POINTER(Result)]),
        "dg_batch_bucket_count": (C.c_int, [vp]),
        "dg_batch_bucket": (C.c_int, [vp, C.c_int, C.POINTER(Bucket)]),
        "dg_batch_stage_ms": (C.c_int, [vp, C.POINTER(C.c_float)]),
        "dg_batch_counters": (C.c_int, [vp, u64p, u64p, u32p]),
        "dg_batch_huffman_stats": (C.c_int, [vp, u64p]),
        "dg_batch_debug": (C.c_int, [vp, C.c_int, C.POINTER(vp), u64p, C.POINTER(vp)]),
        "dg_batch_destroy": (None, [vp]),
        "dg_process": (C.c_int, [vp, C.POINTER(Item), C.c_int, C.c_uint32, C.POINTER(vp), C.POINTER(Result)]),
        "dg_copy_to_host": (C.c_int, [vp, vp, vp, C.c_uint64]),
        "dg_feeder_create": (C.c_int, [C.c_int, C.POINTER(ImageConfig), C.POINTER(FeederConfig), C.POINTER(vp)]),
        "dg_feeder_ctx": (vp, [vp]),
        "dg_submit": (C.c_int, [vp, C.POINTER(Item), vp, C.c_uint64, u64p]),
        "dg_wait": (C.c_int, [vp, C.c_uint64, C.c_uint64, C.POINTER(Result)]),
        "dg_fetch": (C.c_int, [vp, C.c_uint64, vp, C.c_uint64]),
        "dg_peek": (C.c_int, [vp, C.c_uint64, C.POINTER(vp)]),
        "dg_release": (C.c_int, [vp, C.c_uint64]),
        "dg_feeder_get_stats": (C.c_int, [vp, C.POINTER(FeederStats)]),
        "dg_feeder_destroy": (None, [vp]),
        "dg_resize_device_static": (C.c_int, [vp, vp, C.c_uint32, C.c_uint32, C.c_uint32, C.c_char_p, vp, C.POINTER(Plan)]),
    }
    for name, (res, args) in sig.items():
        fn = getattr(L, name)
        fn.restype = res
        fn.argtypes = args
    _lib = L
    return L


EXPORTS = ("dg_set_log_callback dg_ctx_get_counters dg_last_error dg_version dg_ctx_create dg_ctx_create_on_stream dg_ctx_destroy dg_ctx_stream dg_size_list "
           "dg_bucket_table dg_closest_aspect_ratio dg_aspect_ratio_to_str dg_plan_geometry dg_jpeg_probe dg_rank_slice "
           "dg_key_hash dg_key_rank dg_batch_create dg_batch_upload dg_batch_run dg_batch_download dg_batch_sync "
           "dg_batch_download_packed dg_batch_packed_bytes dg_batch_bucket_count dg_batch_bucket "
           "dg_batch_result dg_batch_stage_ms dg_batch_counters dg_batch_huffman_stats dg_batch_debug dg_batch_destroy dg_process "
           "dg_copy_to_host dg_resize_device_static dg_feeder_create dg_feeder_ctx dg_submit dg_wait dg_fetch dg_peek dg_release "
           "dg_feeder_get_stats dg_feeder_destroy").split()


def _shape(result):
    """numpy shape of a payload: H x W for one channel, H x W x C otherwise."""
    return (result.height, result.width) if result.channels == 1 else (result.height, result.width, result.channels)


def _check(rc):
    if rc:
        raise DatagoB200Error(rc, lib().dg_last_error().decode())


_log_keep = None


def bind_to_gpu_cpus(device):
    """Restricts the calling process (and the threads it starts afterwards: the library's host pool, Python workers) to
    the host cores NVML reports as local to CUDA device `device`, so that the page-locked staging memory the library
    allocates is placed on that socket and the device-to-host copies of one rank do not cross the inter-socket link.  To
    be called before the first Context of the process.  Changes nothing on the GPU.  Returns the cores, or None when NVML,
    the PCI id or a non-empty intersection with the current affinity mask is not available (nothing is changed then)."""
    import os
    try:
        import pynvml
        import torch
        pr = torch.cuda.get_device_properties(device)
        bus_id = f"{pr.pci_domain_id:08x}:{pr.pci_bus_id:02x}:{pr.pci_device_id:02x}.0"
        pynvml.nvmlInit()
        try:
            h = pynvml.nvmlDeviceGetHandleByPciBusId(bus_id.encode())
            words = (max(os.sched_getaffinity(0)) + 64) // 64
            mask = pynvml.nvmlDeviceGetCpuAffinity(h, max(words, 16))
        finally:
            pynvml.nvmlShutdown()
        cpus = {64 * i + b for i, word in enumerate(mask) for b in range(64) if (int(word) >> b) & 1}
        cpus &= os.sched_getaffinity(0)
        if not cpus:
            return None
        os.sched_setaffinity(0, cpus)
        return sorted(cpus)
    except Exception:  # noqa: BLE001 - a missing NVML, an old torch, a container without the call: all mean "do not bind"
        return None


def set_log_callback(fn):
    """fn(level, message) receives one line per dropped item (level 1 = error) and the library's own warnings;
    None removes it.  The counterpart of the `log` records datago writes for failed samples."""
    global _log_keep
    if fn is None:
        lib().dg_set_log_callback(C.cast(None, LOG_FN), None)
        _log_keep = None
        return
    cb = LOG_FN(lambda level, msg, user: fn(int(level), msg.decode(errors="replace")))
    lib().dg_set_log_callback(cb, None)
    _log_keep = cb


# ---- host-only helpers ----------------------------------------------------------------------------------------------
def size_list(image_config):
    cfg = ImageConfig.from_dict(image_config)
    w = np.zeros(4096, np.uint32)
    h = np.zeros(4096, np.uint32)
    n = lib().dg_size_list(C.byref(cfg), 4096, w.ctypes.data, h.ctypes.data)
    return [(int(w[i]), int(h[i])) for i in range(n)]


def aspect_ratio_to_str(w, h):
    b = C.create_string_buffer(16)
    lib().dg_aspect_ratio_to_str(w, h, b)
    return b.value.decode()


def jpeg_probe(data: bytes):
    info = JpegInfo()
    _check(lib().dg_jpeg_probe(data, len(data), C.byref(info)))
    return info


def rank_slice(quorum, rank, world_size):
    s, e = C.c_uint64(), C.c_uint64()
    _check(lib().dg_rank_slice(quorum, rank, world_size, C.byref(s), C.byref(e)))
    return int(s.value), int(e.value)


def key_hash(key: str):
    b = key.encode()
    return int(lib().dg_key_hash(b, len(b)))


def key_rank(key: str, world_size: int):
    b = key.encode()
    return int(lib().dg_key_rank(b, len(b), world_size))


# ---- context and batches --------------------------------------------------------------------------------------------
class Context:
    """One device + stream + (optional) aspect-ratio transform; the counterpart of the `Option<ARAwareTransform>`
    a DatagoClient holds (src/client.rs:92-95 of datago)."""

    def __init__(self, device=0, image_config=None, stream=None):
        self._h = C.c_void_p()
        cfg = ImageConfig.from_dict(image_config) if image_config else None
        ref = C.byref(cfg) if cfg is not None else None
        if stream is None:
            _check(lib().dg_ctx_create(device, ref, C.byref(self._h)))
        else:
            _check(lib().dg_ctx_create_on_stream(device, ref, C.c_void_p(stream), C.byref(self._h)))
        self.device = device
        self.image_config = image_config

    def close(self):
        if self._h:
            lib().dg_ctx_destroy(self._h)
            self._h = C.c_void_p()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    @property
    def stream(self):
        return lib().dg_ctx_stream(self._h)

    def bucket_table(self):
        """[(key, aspect ratio, w, h)] sorted by aspect ratio."""
        w = np.zeros(4096, np.uint32)
        h = np.zeros(4096, np.uint32)
        ar = np.zeros(4096, np.float64)
        keys = C.create_string_buffer(16 * 4096)
        n = lib().dg_bucket_table(self._h, 4096, w.ctypes.data, h.ctypes.data, ar.ctypes.data, C.addressof(keys))
        return [(keys.raw[16 * i:16 * i + 16].split(b"\0")[0].decode(), float(ar[i]), int(w[i]), int(h[i]))
                for i in range(n)]

    def closest_aspect_ratio(self, w, h):
        b = C.create_string_buffer(16)
        _check(lib().dg_closest_aspect_ratio(self._h, w, h, b))
        return b.value.decode()

    def plan_geometry(self, w, h, channels=3, forced_key=None):
        p = Plan()
        _check(lib().dg_plan_geometry(self._h, w, h, channels, forced_key.encode() if forced_key else None, C.byref(p)))
        return p

    def batch(self, inputs, forced_keys=None, flags=0, to_rgb8=None):
        return Batch(self, inputs, forced_keys, flags, to_rgb8)

    def process(self, inputs, forced_keys=None, flags=0, to_rgb8=None):
        """create + upload + run + download + sync in one go: list of (status, numpy array or None, Result)."""
        with self.batch(inputs, forced_keys, flags, to_rgb8) as b:
            b.upload()
            b.run()
            outs = b.download()
            b.sync()
            res = [b.result(i) for i in range(len(b))]
        return [(r.status, o if r.status == 0 else None, r) for r, o in zip(res, outs)]

    def resize_device_static(self, src_ptr, w, h, channels, dst_ptr, forced_key=None):
        """crop_and_resize of one device-resident image using only the library's built-in scratch array: for hosts
        that must not allocate device memory while running.  src_ptr / dst_ptr are device addresses owned by the
        caller (dst sized from plan_geometry).  Returns the plan.  Raises too_large beyond the 32 MiB scratch."""
        p = Plan()
        _check(lib().dg_resize_device_static(self._h, C.c_void_p(src_ptr), w, h, channels,
                                             forced_key.encode() if forced_key else None, C.c_void_p(dst_ptr), C.byref(p)))
        return p

    def counters(self):
        """Items finished by this context per status name, batches, bytes in and out."""
        c = CtxCounters()
        _check(lib().dg_ctx_get_counters(self._h, C.byref(c)))
        items = {STATUS_NAMES[i]: int(c.items[i]) for i in range(13) if c.items[i]}
        return dict(items=items, batches=int(c.batches), bytes_in=int(c.bytes_in), bytes_out=int(c.bytes_out))

    def copy_to_host(self, device_ptr, nbytes):
        out = np.empty(nbytes, np.uint8)
        _check(lib().dg_copy_to_host(self._h, out.ctypes.data, C.c_void_p(device_ptr), nbytes))
        return out


class Batch:
    """A batch of samples.  inputs: bytes (JPEG files) or numpy uint8 arrays HxW / HxWxC (raw pixels).
    to_rgb8: True, or one bool per input: datago's `image_to_rgb8` (gray -> RGB, RGBA composited over gray)."""

    def __init__(self, ctx, inputs, forced_keys=None, flags=0, to_rgb8=None):
        self.ctx = ctx
        self._flags = flags
        self._n = len(inputs)
        self._items = (Item * max(1, self._n))()
        as_bytes = (_ItemBytes * max(1, self._n)).from_buffer(self._items)
        self._keep = [as_bytes]
        for i, x in enumerate(inputs):
            item_flags = ITEM_TO_RGB8 if (to_rgb8 is True or (to_rgb8 and to_rgb8[i])) else 0
            if type(x) is bytes:
                it = as_bytes[i]
                it.data = x
                it.len = len(x)
                it.flags = item_flags
                if forced_keys and forced_keys[i]:
                    it.forced_key = forced_keys[i].encode()
                continue
            it = self._items[i]
            it.flags = item_flags
            if isinstance(x, (bytes, bytearray, memoryview)):
                buf = (C.c_char * len(x)).from_buffer_copy(bytes(x))
                self._keep.append(buf)
                it.data = C.cast(buf, C.c_void_p)
                it.len = len(x)
            else:
                a = np.ascontiguousarray(x, np.uint8)
                self._keep.append(a)
                it.data = a.ctypes.data
                it.len = a.nbytes
                it.raw_h, it.raw_w = a.shape[:2]
                it.raw_c = 1 if a.ndim == 2 else a.shape[2]
            if forced_keys and forced_keys[i]:
                it.forced_key = forced_keys[i].encode()
        self._h = C.c_void_p()
        _check(lib().dg_batch_create(ctx._h, self._items, self._n, flags, C.byref(self._h)))
        self._outs = None

    def __len__(self):
        return self._n

    def __enter__(self):
        return self

    def __exit__(self, *a):
        self.close()

    def close(self):
        if self._h:
            lib().dg_batch_destroy(self._h)
            self._h = C.c_void_p()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def upload(self):
        _check(lib().dg_batch_upload(self._h))

    def run(self):
        _check(lib().dg_batch_run(self._h))

    def sync(self):
        _check(lib().dg_batch_sync(self._h))

    def result(self, i):
        r = Result()
        _check(lib().dg_batch_result(self._h, i, C.byref(r)))
        return r

    def host_buffers(self):
        """numpy arrays shaped like each ok payload (None for failed items)."""
        outs = []
        for i in range(self._n):
            r = self.result(i)
            if r.status:
                outs.append(None)
            else:
                outs.append(np.empty(_shape(r), np.uint8))
        return outs

    def download(self, outs=None):
        """Queue device->host copies into `outs` (from host_buffers()); valid after sync()."""
        if outs is None:
            outs = self.host_buffers()
        ptrs = (C.c_void_p * max(1, self._n))(*[o.ctypes.data if o is not None else None for o in outs])
        self._outs = outs
        _check(lib().dg_batch_download(self._h, ptrs))
        return outs

    def packed_bytes(self):
        return int(lib().dg_batch_packed_bytes(self._h))

    def download_packed(self, host_buffer):
        """Queue ONE device->host copy of every payload into `host_buffer` (a writable uint8 numpy array, ideally
        pinned); payload i then sits at result(i).packed_offset.  Valid after sync()."""
        self._outs = host_buffer
        _check(lib().dg_batch_download_packed(self._h, host_buffer.ctypes.data, host_buffer.nbytes))

    def buckets(self):
        """Buckets of a BATCH_COLLATE batch: list of dicts with key, shape (n, h, w, c), items (batch indices in
        storage order), packed_offset and `array`, a DeviceArray over the dense [n, h, w, c] block."""
        out = []
        for k in range(lib().dg_batch_bucket_count(self._h)):
            bk = Bucket()
            _check(lib().dg_batch_bucket(self._h, k, C.byref(bk)))
            shape = (bk.n, bk.height, bk.width, bk.channels)
            out.append(dict(key=bk.key.decode(), shape=shape, items=[int(bk.items[j]) for j in range(bk.n)],
                            packed_offset=int(bk.packed_offset), nbytes=int(bk.nbytes),
                            array=DeviceArray(bk.device_data, shape, self)))
        return out

    def stage_ms(self):
        ms = (C.c_float * len(STAGES))()
        _check(lib().dg_batch_stage_ms(self._h, ms))
        return dict(zip(STAGES, [float(v) for v in ms]))

    def counters(self):
        h2d, d2h, k = C.c_uint64(), C.c_uint64(), C.c_uint32()
        _check(lib().dg_batch_counters(self._h, C.byref(h2d), C.byref(d2h), C.byref(k)))
        return dict(h2d_bytes=int(h2d.value), d2h_bytes=int(d2h.value), kernel_launches=int(k.value))

    def huffman_stats(self):
        out = (C.c_uint64 * 3)()
        _check(lib().dg_batch_huffman_stats(self._h, out))
        return dict(chunks=int(out[0]), rounds=int(out[1]), subsequence_decodes=int(out[2]))

    def debug_coefficients(self, i):
        """int16 [blocks, 64] coefficients of JPEG item i in scan order (single-wave batches created with
        BATCH_KEEP_COEFFICIENTS, after sync)."""
        coef, nb = C.c_void_p(), C.c_uint64()
        _check(lib().dg_batch_debug(self._h, i, C.byref(coef), C.byref(nb), None))
        raw = self.ctx.copy_to_host(coef.value, int(nb.value) * 128)
        return raw.view(np.int16).reshape(int(nb.value), 64)

    def debug_decoded(self, i):
        """The full-size decoded image of JPEG item i (single-wave batches, after sync).  When a resize reads it, its
        rows are padded to 16 bytes in device memory; the padding is dropped here."""
        r = self.result(i)
        dec = C.c_void_p()
        _check(lib().dg_batch_debug(self._h, i, None, None, C.byref(dec)))
        h, w, c = r.original_height, r.original_width, r.channels
        resized = self.ctx.image_config is not None and not (self._flags & BATCH_DECODE_ONLY) and not r.plan.identity
        pitch = (w * c + 15) // 16 * 16 if resized else w * c
        raw = self.ctx.copy_to_host(dec.value, pitch * h).reshape(h, pitch)[:, :w * c]
        return np.ascontiguousarray(raw).reshape((h, w, 3) if c == 3 else (h, w))


class Feeder:
    """Submit / wait front end (dg_feeder): threads submit single samples, the library batches them for the GPU.
    ctypes releases the GIL inside every call, so Python threads overlap the way datago's tokio workers do."""

    def __init__(self, device=0, image_config=None, lanes=0, max_batch=0, max_wait_us=0, queue_limit=0, flags=0):
        self._h = C.c_void_p()
        cfg = ImageConfig.from_dict(image_config) if image_config else None
        fc = FeederConfig(lanes, max_batch, max_wait_us, queue_limit, flags, 0)
        _check(lib().dg_feeder_create(device, C.byref(cfg) if cfg is not None else None, C.byref(fc), C.byref(self._h)))

    def close(self):
        if self._h:
            lib().dg_feeder_destroy(self._h)
            self._h = C.c_void_p()

    def __enter__(self):
        return self

    def __exit__(self, *a):
        self.close()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def submit(self, x, forced_key=None, host_out=None, to_rgb8=False):
        """x: bytes (a JPEG file) or a numpy uint8 array HxW / HxWx3.  host_out: optional writable uint8 array the
        payload is copied into by wait().  Returns the ticket."""
        it = Item()
        if isinstance(x, (bytes, bytearray, memoryview)):
            keep = bytes(x)
            it.data = C.cast(C.c_char_p(keep), C.c_void_p)
            it.len = len(keep)
        else:
            keep = np.ascontiguousarray(x, np.uint8)
            it.data = keep.ctypes.data
            it.len = keep.nbytes
            it.raw_h, it.raw_w = keep.shape[:2]
            it.raw_c = 1 if keep.ndim == 2 else keep.shape[2]
        if forced_key:
            it.forced_key = forced_key.encode()
        if to_rgb8:
            it.flags = ITEM_TO_RGB8
        t = C.c_uint64()
        _check(lib().dg_submit(self._h, C.byref(it), host_out.ctypes.data if host_out is not None else None,
                               host_out.nbytes if host_out is not None else 0, C.byref(t)))
        return int(t.value)

    def wait(self, ticket, timeout_s=None):
        """Result of the ticket, or None when timeout_s ran out first."""
        r = Result()
        ns = 0xFFFFFFFFFFFFFFFF if timeout_s is None else int(timeout_s * 1e9)
        rc = lib().dg_wait(self._h, ticket, ns, C.byref(r))
        if rc == E_TIMEOUT:
            return None
        _check(rc)
        return r

    def fetch(self, ticket, result):
        """The payload of a finished ticket as a numpy array (H x W x 3, or H x W for one channel)."""
        out = np.empty(_shape(result), np.uint8)
        _check(lib().dg_fetch(self._h, ticket, out.ctypes.data, out.nbytes))
        return out

    def peek(self, ticket, result):
        """The payload of a finished ticket as a numpy view of the feeder's own page-locked host buffer (no copy);
        valid until release()."""
        ptr = C.c_void_p()
        _check(lib().dg_peek(self._h, ticket, C.byref(ptr)))
        shape = _shape(result)
        return np.ctypeslib.as_array(C.cast(ptr, C.POINTER(C.c_uint8)), shape=(int(result.nbytes),)).reshape(shape)

    def release(self, ticket):
        _check(lib().dg_release(self._h, ticket))

    def process_one(self, x, forced_key=None, to_rgb8=False):
        """submit + wait + fetch + release: (status, array or None, Result) -- the blocking call a worker thread makes."""
        t = self.submit(x, forced_key, to_rgb8=to_rgb8)
        try:
            r = self.wait(t)
            return r.status, (self.fetch(t, r) if r.status == 0 else None), r
        finally:
            self.release(t)

    def stats(self):
        st = FeederStats()
        _check(lib().dg_feeder_get_stats(self._h, C.byref(st)))
        return {k: int(getattr(st, k)) for k, _ in FeederStats._fields_ if k != "reserved"}
