"""ctypes front end of the CPU oracle (oracle/oracle.cpp).  TEST INFRASTRUCTURE ONLY.

Only the test-suite, the smoke check and the benchmark's CPU-baseline leg may import this
package; the shipped library never does.
"""
import ctypes as C
import os

import numpy as np

from .build import build as _build

MODE_FIR = 0     # fast_image_resize-style 16-bit coefficients (the reference's resizer)
MODE_PILLOW = 1  # Pillow's 22-bit coefficients (used to pin the arithmetic against PIL)

STATUS = {0: "ok", 1: "truncated", 2: "bad_marker", 3: "unsupported", 4: "bad_table", 5: "bad_code"}


class Plan(C.Structure):
    _fields_ = [("src_w", C.c_uint32), ("src_h", C.c_uint32), ("target_w", C.c_uint32), ("target_h", C.c_uint32),
                ("new_w", C.c_uint32), ("new_h", C.c_uint32), ("crop_left", C.c_double), ("crop_top", C.c_double),
                ("crop_w", C.c_double), ("crop_h", C.c_double), ("identity", C.c_int32), ("key", C.c_char * 16)]

    def as_tuple(self):
        return (self.key.decode(), self.target_w, self.target_h, self.new_w, self.new_h, self.crop_left,
                self.crop_top, self.crop_w, self.crop_h, self.identity)


class JpegInfo(C.Structure):
    _fields_ = [("width", C.c_int32), ("height", C.c_int32), ("channels", C.c_int32), ("hsamp", C.c_int32),
                ("vsamp", C.c_int32), ("mcux", C.c_int32), ("mcuy", C.c_int32), ("restart_interval", C.c_int32),
                ("blocks", C.c_int32 * 3)]


class Item(C.Structure):
    _fields_ = [("data", C.c_void_p), ("len", C.c_uint64), ("raw_w", C.c_uint32), ("raw_h", C.c_uint32),
                ("raw_c", C.c_uint32), ("pad", C.c_uint32)]


_lib = None


def lib():
    global _lib
    if _lib is None:
        _lib = C.CDLL(_build())
        _lib.orc_key_hash.restype = C.c_uint64
        _lib.orc_key_hash.argtypes = [C.c_char_p, C.c_size_t]
        _lib.orc_siphash.restype = C.c_uint64
        _lib.orc_siphash.argtypes = [C.c_uint64, C.c_uint64, C.c_int, C.c_int, C.c_char_p, C.c_size_t]
        _lib.orc_plan_geometry.argtypes = [C.c_uint32, C.c_uint32, C.c_double, C.c_double, C.c_uint32, C.c_uint32,
                                           C.c_char_p, C.POINTER(Plan)]
        _lib.orc_resample.argtypes = [C.c_void_p, C.c_int, C.c_int, C.c_int, C.c_double, C.c_double, C.c_double,
                                      C.c_double, C.c_void_p, C.c_int, C.c_int, C.c_int]
        _lib.orc_crop_and_resize.argtypes = [C.c_uint32, C.c_uint32, C.c_double, C.c_double, C.c_void_p, C.c_uint32,
                                             C.c_uint32, C.c_int, C.c_char_p, C.c_void_p, C.POINTER(Plan), C.c_int]
        _lib.orc_jpeg_info.argtypes = [C.c_char_p, C.c_size_t, C.POINTER(JpegInfo)]
        _lib.orc_jpeg_decode.argtypes = [C.c_char_p, C.c_size_t, C.c_void_p]
        _lib.orc_jpeg_decode_variant.argtypes = [C.c_char_p, C.c_size_t, C.c_void_p, C.c_int, C.c_int, C.c_int]
        _lib.orc_jpeg_decode_stages.argtypes = [C.c_char_p, C.c_size_t] + [C.c_void_p] * 7
        _lib.orc_jpeg_to_payload.argtypes = [C.c_char_p, C.c_size_t, C.c_uint32, C.c_uint32, C.c_double, C.c_double,
                                             C.c_char_p, C.c_void_p, C.POINTER(Plan), C.c_int]
        _lib.orc_bucket_table.argtypes = [C.c_uint32, C.c_uint32, C.c_double, C.c_double, C.c_int, C.c_void_p,
                                          C.c_void_p, C.c_void_p, C.c_void_p]
        _lib.orc_size_list.argtypes = [C.c_uint32, C.c_uint32, C.c_double, C.c_double, C.c_int, C.c_void_p, C.c_void_p]
        _lib.orc_rank_slice.argtypes = [C.c_uint64, C.c_uint64, C.c_uint64, C.POINTER(C.c_uint64), C.POINTER(C.c_uint64)]
        _lib.orc_coeffs.argtypes = [C.c_int, C.c_double, C.c_double, C.c_int, C.c_int, C.c_void_p, C.c_void_p,
                                    C.c_void_p, C.c_int, C.POINTER(C.c_int32)]
        _lib.orc_run_batch.argtypes = [C.POINTER(Item), C.c_int, C.c_int, C.c_uint32, C.c_uint32, C.c_double,
                                       C.c_double, C.c_int, C.POINTER(C.c_uint64), C.POINTER(C.c_uint64)]
        _lib.orc_aspect_ratio_to_str.argtypes = [C.c_uint32, C.c_uint32, C.c_char_p]
        _lib.orc_to_rgb8.argtypes = [C.c_void_p, C.c_uint64, C.c_int, C.c_void_p]
    return _lib


class OracleError(RuntimeError):
    def __init__(self, code):
        super().__init__(f"oracle status {code} ({STATUS.get(code, '?')})")
        self.code = code


def _cfg(cfg):
    return (int(cfg["default_image_size"]), int(cfg["downsampling_ratio"]), float(cfg["min_aspect_ratio"]),
            float(cfg["max_aspect_ratio"]))


def size_list(cfg):
    w = np.zeros(4096, np.uint32)
    h = np.zeros(4096, np.uint32)
    n = lib().orc_size_list(*_cfg(cfg), 4096, w.ctypes.data, h.ctypes.data)
    return [(int(w[i]), int(h[i])) for i in range(n)]


def bucket_table(cfg):
    """[(key, ar, w, h)] sorted by aspect ratio."""
    w = np.zeros(4096, np.uint32)
    h = np.zeros(4096, np.uint32)
    ar = np.zeros(4096, np.float64)
    keys = C.create_string_buffer(16 * 4096)
    n = lib().orc_bucket_table(*_cfg(cfg), 4096, w.ctypes.data, h.ctypes.data, ar.ctypes.data, keys)
    return [(keys.raw[16 * i:16 * i + 16].split(b"\0")[0].decode(), float(ar[i]), int(w[i]), int(h[i]))
            for i in range(n)]


def aspect_ratio_to_str(w, h):
    b = C.create_string_buffer(16)
    lib().orc_aspect_ratio_to_str(w, h, b)
    return b.value.decode()


def plan_geometry(cfg, w, h, forced_key=None):
    p = Plan()
    rc = lib().orc_plan_geometry(*_cfg(cfg), w, h, forced_key.encode() if forced_key else None, C.byref(p))
    if rc:
        raise KeyError(f"bucket key {forced_key!r} not in table (rc {rc})")
    return p


def resample(src, box, out_wh, mode=MODE_FIR):
    """One Lanczos3 convolution resize of box=(left, top, width, height) of src (H,W[,C] u8) into out_wh=(w,h)."""
    src = np.ascontiguousarray(src, np.uint8)
    h, w = src.shape[:2]
    c = 1 if src.ndim == 2 else src.shape[2]
    dw, dh = out_wh
    dst = np.empty((dh, dw) if src.ndim == 2 else (dh, dw, c), np.uint8)
    rc = lib().orc_resample(src.ctypes.data, w, h, c, *[float(b) for b in box], dst.ctypes.data, dw, dh, mode)
    assert rc == 0
    return dst


def coeffs(in_size, in0, in1, out_size, mode=MODE_FIR):
    start = np.zeros(out_size, np.int32)
    size = np.zeros(out_size, np.int32)
    cap = (int(np.ceil(3.0 * max(1.0, (in1 - in0) / out_size))) * 2 + 1) * out_size
    k = np.zeros(cap, np.int32)
    prec = C.c_int32()
    window = lib().orc_coeffs(in_size, in0, in1, out_size, mode, start.ctypes.data, size.ctypes.data, k.ctypes.data,
                              cap, C.byref(prec))
    return start, size, k.reshape(out_size, window), prec.value


def crop_and_resize(cfg, src, forced_key=None, mode=MODE_FIR):
    src = np.ascontiguousarray(src, np.uint8)
    h, w = src.shape[:2]
    c = 1 if src.ndim == 2 else src.shape[2]
    p = plan_geometry(cfg, w, h, forced_key)
    dst = np.empty((p.target_h, p.target_w) if src.ndim == 2 else (p.target_h, p.target_w, c), np.uint8)
    rc = lib().orc_crop_and_resize(*_cfg(cfg), src.ctypes.data, w, h, c, forced_key.encode() if forced_key else None,
                                   dst.ctypes.data, C.byref(p), mode)
    assert rc == 0
    return dst, p


def to_rgb8(src):
    """convert_to_rgb8 of an HxW or HxWxC uint8 image (C = 1..4): HxWx3."""
    src = np.ascontiguousarray(src, np.uint8)
    h, w = src.shape[:2]
    c = 1 if src.ndim == 2 else src.shape[2]
    dst = np.empty((h, w, 3), np.uint8)
    assert lib().orc_to_rgb8(src.ctypes.data, h * w, c, dst.ctypes.data) == 0
    return dst


def jpeg_info(data: bytes):
    info = JpegInfo()
    rc = lib().orc_jpeg_info(data, len(data), C.byref(info))
    if rc:
        raise OracleError(rc)
    return info


def jpeg_decode(data: bytes):
    info = jpeg_info(data)
    shape = (info.height, info.width, 3) if info.channels == 3 else (info.height, info.width)
    out = np.empty(shape, np.uint8)
    rc = lib().orc_jpeg_decode(data, len(data), out.ctypes.data)
    if rc:
        raise OracleError(rc)
    return out


def jpeg_decode_variant(data: bytes, idct=0, upsample=0, color=0):
    """Decode with another published IDCT (1: 12-bit stb-style), upsampling (1: two rounded passes, 2: bias 8 in both
    phases) or colour arithmetic (1: 14-bit constants); (0, 0, 0) is jpeg_decode."""
    info = jpeg_info(data)
    shape = (info.height, info.width, 3) if info.channels == 3 else (info.height, info.width)
    out = np.empty(shape, np.uint8)
    rc = lib().orc_jpeg_decode_variant(data, len(data), out.ctypes.data, idct, upsample, color)
    if rc:
        raise OracleError(rc)
    return out


def jpeg_decode_stages(data: bytes):
    """(coefficients per component [blocks,64] int16, MCU-padded planes per component, pixels)."""
    info = jpeg_info(data)
    ncomp = 3 if info.channels == 3 else 1
    coefs = [np.zeros((info.blocks[c], 64), np.int16) for c in range(ncomp)]
    planes = []
    for c in range(ncomp):
        hs, vs = (info.hsamp, info.vsamp) if c == 0 else (1, 1)
        planes.append(np.zeros((info.mcuy * vs * 8, info.mcux * hs * 8), np.uint8))
    shape = (info.height, info.width, 3) if info.channels == 3 else (info.height, info.width)
    out = np.empty(shape, np.uint8)
    cp = [a.ctypes.data for a in coefs] + [None] * (3 - ncomp)
    pp = [a.ctypes.data for a in planes] + [None] * (3 - ncomp)
    rc = lib().orc_jpeg_decode_stages(data, len(data), *cp, *pp, out.ctypes.data)
    if rc:
        raise OracleError(rc)
    return coefs, planes, out


def jpeg_to_payload(data: bytes, cfg=None, forced_key=None, mode=MODE_FIR):
    """image_to_payload for a JPEG: (pixels, plan or None)."""
    if cfg is None:
        return jpeg_decode(data), None
    info = jpeg_info(data)
    p = plan_geometry(cfg, info.width, info.height, forced_key)
    shape = (p.target_h, p.target_w, 3) if info.channels == 3 else (p.target_h, p.target_w)
    out = np.empty(shape, np.uint8)
    rc = lib().orc_jpeg_to_payload(data, len(data), *_cfg(cfg), forced_key.encode() if forced_key else None,
                                   out.ctypes.data, C.byref(p), mode)
    if rc:
        raise OracleError(rc)
    return out, p


def key_hash(key: str) -> int:
    b = key.encode()
    return int(lib().orc_key_hash(b, len(b)))


def siphash(k0, k1, c, d, data: bytes) -> int:
    return int(lib().orc_siphash(k0, k1, c, d, data, len(data)))


def rank_slice(n, rank, world):
    s, e = C.c_uint64(), C.c_uint64()
    rc = lib().orc_rank_slice(n, rank, world, C.byref(s), C.byref(e))
    if rc:
        raise ValueError("rank must be < world_size and world_size > 0")
    return int(s.value), int(e.value)


def run_batch(items, kind, cfg=None, threads=1):
    """Timed CPU baseline: items = list of bytes (JPEG) or numpy HWC arrays (raw).  Returns ok count."""
    arr = (Item * len(items))()
    keep = []
    for i, it in enumerate(items):
        if isinstance(it, (bytes, bytearray)):
            buf = C.create_string_buffer(bytes(it), len(it))
            keep.append(buf)
            arr[i].data = C.addressof(buf)
            arr[i].len = len(it)
        else:
            a = np.ascontiguousarray(it, np.uint8)
            keep.append(a)
            arr[i].data = a.ctypes.data
            arr[i].len = a.nbytes
            arr[i].raw_h, arr[i].raw_w = a.shape[:2]
            arr[i].raw_c = 1 if a.ndim == 2 else a.shape[2]
    size, ratio, mn, mx = _cfg(cfg) if cfg else (0, 1, 1.0, 1.0)
    ok, sink = C.c_uint64(), C.c_uint64()

    def call():
        lib().orc_run_batch(arr, len(items), kind, size, ratio, mn, mx, threads, C.byref(ok), C.byref(sink))
        return int(ok.value)
    call.keep = keep
    return call
