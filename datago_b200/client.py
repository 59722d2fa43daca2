"""`DatagoClient`-shaped host harness over the C ABI.

It mirrors the surface of datago's pyo3 module for the two sources that need no network
(src/client.rs:80-243 of datago): `DatagoClient(json_config)`, `start()`, `get_sample()`, `stop()`, with `Sample` and
`ImagePayload` objects carrying the reference's field names (src/structs.rs:52-71, 240-272).  IO (directory walk,
tar reading, sample grouping, rank sharding) is host work done the way the reference's generators do it; every pixel
goes through the CUDA library in batches.

Differences that are stated, not hidden:
  * `source_type` "webdataset" reads LOCAL tar shards (`url` is a path, a glob or a {a..b} brace pattern); the reference
    streams them over HTTP (src/generator_wds.rs:56-204);
  * baseline JPEG payloads are decoded by the CUDA library; every other image type a sample may carry (PNG masks above
    all, src/worker_http.rs:186-201, but also progressive JPEG, BMP, GIF, WebP) is decoded on the host by Pillow to raw
    8-bit pixels, the way the reference hands them to the `image` crate, and then takes the library's raw-pixel path
    (bucket, crop and resize on the GPU).  `pre_encode_images` re-encodes finished payloads on the host as well
    (src/image_processing.rs:375-416);
  * two opt-in keys the reference ignores: `"device"` (CUDA ordinal, default LOCAL_RANK or 0) and `"batch_size"`;
    `"device_payloads": true` keeps the pixels on the GPU (`ImagePayload.__cuda_array_interface__` / `__dlpack__`).
"""
import glob
import json
import logging
import os
import queue
import re
import tarfile
import threading

import numpy as np

from . import BATCH_DECODE_ONLY, Context, DatagoB200Error, aspect_ratio_to_str, jpeg_probe, key_rank, rank_slice

log = logging.getLogger("datago_b200")

IMG_TYPES = ("jpg", "jpeg", "png")          # src/worker_wds.rs:11
TEXT_TYPES = ("cls", "json", "txt")         # src/worker_wds.rs:10
FILE_EXTENSIONS = ("jpg", "jpeg", "png", "bmp", "gif", "webp")  # src/generator_files.rs:50
TIMEOUT_S = 300                             # src/client.rs:12


class ImagePayload:
    """The fields of datago's ImagePayload; `data` is host bytes, or empty when the payload stayed on the device."""

    def __init__(self, data=b"", original_height=0, original_width=0, height=0, width=0, channels=0, bit_depth=0,
                 is_encoded=False, device_ptr=0, keepalive=None):
        self.data = data
        self.original_height, self.original_width = original_height, original_width
        self.height, self.width, self.channels, self.bit_depth = height, width, channels, bit_depth
        self.is_encoded = is_encoded
        self._device_ptr = device_ptr
        self._keepalive = keepalive  # the batch that owns the device memory

    def _shape(self):
        return (self.height, self.width, self.channels) if self.channels > 1 else (self.height, self.width)

    def to_numpy_array(self):
        """src/structs.rs:154-188"""
        if self.is_encoded:
            import io
            from PIL import Image
            return np.asarray(Image.open(io.BytesIO(self.data)).convert("RGB"))
        if self._device_ptr and not len(self.data):
            return self._keepalive.ctx.copy_to_host(self._device_ptr, self.height * self.width * self.channels).reshape(self._shape())
        return np.frombuffer(self.data, np.uint8).reshape(self._shape())

    def to_pil_image(self):
        """src/structs.rs:103-151: mode L for one channel, RGBA for four, RGB otherwise."""
        from PIL import Image
        if self.is_encoded:
            import io
            return Image.open(io.BytesIO(self.data))
        a = self.to_numpy_array()
        if self.channels == 1:
            return Image.fromarray(a.reshape(self.height, self.width)).convert("L")
        if self.channels == 4:
            return Image.fromarray(a).convert("RGBA")
        return Image.fromarray(a)

    # PythonImagePayload (src/structs.rs:191-224): calling the payload gives the PIL image, get_payload() a copy of the
    # plain record, and any other attribute is looked up on the PIL image, so a payload can be used where a PIL image
    # is expected (payload.size, payload.resize(...), payload.mode ...).
    def __call__(self):
        return self.to_pil_image()

    def get_payload(self):
        return ImagePayload(bytes(self.data), self.original_height, self.original_width, self.height, self.width,
                            self.channels, self.bit_depth, self.is_encoded, self._device_ptr, self._keepalive)

    def __getattr__(self, attr):
        # only reached for names the payload itself does not have
        if attr.startswith("_"):
            raise AttributeError(attr)
        return getattr(self.to_pil_image(), attr)

    @property
    def __cuda_array_interface__(self):
        if not self._device_ptr:
            raise AttributeError("payload is not device resident")
        return {"shape": self._shape(), "typestr": "|u1", "data": (self._device_ptr, False), "version": 3}

    def __dlpack__(self, stream=None):
        import torch
        return torch.as_tensor(self, device="cuda").__dlpack__(stream=stream)

    def __dlpack_device__(self):
        import torch
        return torch.as_tensor(self, device="cuda").__dlpack_device__()


def _empty_payload():
    return ImagePayload()


class Sample:
    """src/structs.rs:240-272"""

    def __init__(self, id, source, image, attributes=None):
        self.id, self.source, self.image = id, source, image
        self._attributes = attributes or {}
        self.duplicate_state = 0
        self.masks, self.additional_images, self.latents = {}, {}, {}
        self.coca_embedding, self.tags = [], []

    @property
    def attributes(self):
        return json.dumps(self._attributes)


def sample_to_python_types(sample):
    """src/structs.rs:279-351: the sample as a dict of plain Python types with PIL images; attribute values that are
    not strings arrive JSON-encoded."""
    return {
        "id": sample.id, "source": sample.source, "duplicate_state": sample.duplicate_state,
        "attributes": {k: (v if isinstance(v, str) else json.dumps(v)) for k, v in sample._attributes.items()},
        "tags": list(sample.tags), "coca_embedding": list(sample.coca_embedding),
        "latents": {k: {"data": bytes(v.data), "len": v.len} for k, v in sample.latents.items()},
        "image": sample.image.to_pil_image(),
        "masks": {k: m.to_pil_image() for k, m in sample.masks.items()},
        "additional_images": {k: m.to_pil_image() for k, m in sample.additional_images.items()},
    }


_logging_initialised = False


def initialize_logging(log_level=None):
    """src/client.rs:253-263: set up the logger once; False when it had been set up before.  The level comes from
    `log_level`, else from RUST_LOG (the variable the reference's env_logger reads), else "error"."""
    global _logging_initialised
    if _logging_initialised:
        return False
    level = (os.environ.get("RUST_LOG") or log_level or "error").split(",")[0].strip().upper()
    level = {"WARN": "WARNING", "TRACE": "DEBUG", "OFF": "CRITICAL"}.get(level, level)
    logging.basicConfig(level=getattr(logging, level, logging.ERROR), format="[%(asctime)s %(levelname)s %(name)s] %(message)s")
    log.setLevel(getattr(logging, level, logging.ERROR))
    _logging_initialised = True
    return True


# ---- host-side codecs around the GPU path ---------------------------------------------------------------------------
def is_baseline_jpeg(data):
    """True when the CUDA decoder takes the file (baseline, Huffman, 8 bit): a header-only look."""
    try:
        jpeg_probe(data)
        return True
    except DatagoB200Error:
        return False


def decode_on_host(data):
    """Any image Pillow reads -> raw uint8 pixels shaped (H, W) or (H, W, C), C in 2..4, as `image::load_from_memory`
    yields Luma8 / LumaA8 / Rgb8 / Rgba8 (src/worker_wds.rs:45).  Palette images become RGB or RGBA, 1-bit and 16-bit
    gray become 8-bit gray.  Returns None when the bytes are no image."""
    import io
    from PIL import Image
    try:
        im = Image.open(io.BytesIO(data))
        im.load()
    except Exception:  # noqa: BLE001
        return None
    if im.mode == "P":
        im = im.convert("RGBA" if "transparency" in im.info else "RGB")
    elif im.mode in ("1", "I;16", "I;16B", "I", "F"):
        im = im.convert("L")
    elif im.mode not in ("L", "LA", "RGB", "RGBA"):
        im = im.convert("RGB")
    return np.ascontiguousarray(np.asarray(im, dtype=np.uint8))


def encode_payload(pixels, encode_format="jpeg", jpeg_quality=92):
    """src/image_processing.rs:375-416: the payload re-encoded as JPEG (given quality) or PNG (fast compression)."""
    import io
    from PIL import Image
    im = Image.fromarray(pixels)
    out = io.BytesIO()
    if str(encode_format).lower() == "png":
        im.save(out, "PNG", compress_level=1)
    else:
        if im.mode in ("RGBA", "LA"):
            im = im.convert("RGB" if im.mode == "RGBA" else "L")  # JPEG has no alpha channel
        im.save(out, "JPEG", quality=int(jpeg_quality))
    return out.getvalue()


# ---- generators ---------------------------------------------------------------------------------------------------------
def enumerate_files(root_path, limit, rank=0, world_size=1, random_sampling=False):
    """src/generator_files.rs:44-125: walk, extension filter, take 2*limit, contiguous rank slice, optional shuffle,
    submit at most ceil(1.1 * limit)."""
    files = []
    for dirpath, _, names in os.walk(root_path, followlinks=False):
        for n in names:
            if n.lower().endswith(FILE_EXTENSIONS):
                files.append(os.path.join(dirpath, n))
                if len(files) >= limit * 2:
                    break
        if len(files) >= limit * 2:
            break
    if world_size > 1:
        start, end = rank_slice(len(files), rank, world_size)
        files = files[start:end]
    if random_sampling:
        np.random.default_rng().shuffle(files)
    return files[: int(np.ceil(1.1 * limit))]


def expand_shards(url):
    """{a..b} brace ranges and globs, as the reference expands shard lists (src/generator_wds.rs:244-300)."""
    m = re.search(r"\{(\d+)\.\.(\d+)\}", url)
    if m:
        width = len(m.group(1))
        return [p for i in range(int(m.group(1)), int(m.group(2)) + 1)
                for p in expand_shards(url[:m.start()] + str(i).zfill(width) + url[m.end():])]
    hits = sorted(glob.glob(url))
    return hits if hits else [url]


def tar_samples(path, reference_image_type="jpg", rank=0, world_size=1):
    """Consecutive tar entries with the same key (basename without the last extension) form a sample; with
    world_size > 1 an entry is kept only if hash(key) % world_size == rank; the reference image goes first.
    src/generator_wds.rs:116-203."""
    current_key, current = None, []

    def finish():
        current.sort(key=lambda it: 0 if it[0].endswith(reference_image_type) else 1)  # stable, like sort_by
        return list(current)

    with tarfile.open(path, "r") as tf:
        for entry in tf:
            if not entry.isfile():
                continue
            key = os.path.splitext(os.path.basename(entry.name))[0]
            if world_size > 1 and key_rank(key, world_size) != rank:
                continue
            if current_key is None:
                current_key = key
            if key != current_key and current:
                yield path, finish()
                current.clear()
                current_key = key
            current.append((entry.name, tf.extractfile(entry).read()))
    if current:
        yield path, finish()


# ---- client ----------------------------------------------------------------------------------------------------------------
class DatagoClient:
    def __init__(self, str_config):
        self.is_valid = False
        self.is_started = False
        self._thread = None
        self._stop = threading.Event()
        self._reader_stop = threading.Event()
        self._buffers = [None, None]
        cfg = self._check_config(str_config)
        if cfg is None:
            return
        self.config = cfg
        self.source_type = cfg.get("source_type", "db")
        if self.source_type not in ("file", "webdataset"):
            log.error("source_type %r needs the network; this harness serves 'file' and 'webdataset' (local shards)", self.source_type)
            return
        self.limit = int(cfg["limit"])
        self._queue = queue.Queue(maxsize=int(cfg["samples_buffer_size"]))
        self.image_config = cfg.get("image_config")
        self.batch_size = int(cfg.get("batch_size", 256))
        self.device_payloads = bool(cfg.get("device_payloads", False))
        ic = self.image_config or {}
        self.pre_encode = bool(ic.get("pre_encode_images", False))        # src/image_processing.rs:60-70
        self.encode_format = str(ic.get("encode_format", "jpeg"))
        self.jpeg_quality = int(ic.get("jpeg_quality", 92))
        device = int(cfg.get("device", os.environ.get("LOCAL_RANK", 0)))
        tfm = self.image_config if self.image_config and self.image_config.get("crop_and_resize") else None
        self.ctx = Context(device, tfm)  # raises when no CUDA device: there is no CPU path
        self.is_valid = True

    @staticmethod
    def _check_config(str_config):
        """src/client.rs:38-78"""
        try:
            cfg = json.loads(str_config)
            for key in ("source_config", "limit", "samples_buffer_size"):
                if key not in cfg:
                    raise KeyError(key)
        except Exception as e:  # noqa: BLE001
            log.error("Failed to parse config: %s", e)
            return None
        if int(cfg["samples_buffer_size"]) == 0:
            log.error("Samples buffer size must be greater than 0")
            return None
        if int(cfg["limit"]) == 0:
            log.error("Limit must be greater than 0")
            return None
        world = int(cfg["source_config"].get("world_size", 1) or 0) if "world_size" in cfg["source_config"] else 1
        rank = int(cfg["source_config"].get("rank", 0))
        if world == 0:
            log.error("World size must be greater than 0")
            return None
        if rank >= world:
            log.error("Rank must be less than world size")
            return None
        return cfg

    # -- lifecycle (src/client.rs:139-243) ----------------------------------------------------------------------------
    def start(self):
        if not self.is_valid or self.is_started:
            return
        self._stop.clear()
        self._reader_stop.clear()
        self._thread = threading.Thread(target=self._run, daemon=True)
        self._thread.start()
        self.is_started = True

    def get_sample(self):
        if not self.is_valid:
            return None
        if not self.is_started:
            self.start()
        try:
            s = self._queue.get(timeout=TIMEOUT_S)
        except queue.Empty:
            log.warning("Timeout waiting for sample, stopping the client")
            self.stop()
            return None
        if s is None:
            self.stop()
        return s

    def get_sample_auto_convert(self):
        """src/client.rs:207-215: the next sample as a dict of Python types with PIL images, or None."""
        s = self.get_sample()
        return None if s is None else sample_to_python_types(s)

    def stop(self):
        self._stop.set()
        if self._thread and self._thread is not threading.current_thread():
            while self._thread.is_alive():  # unblock a producer stuck on a full queue
                try:
                    self._queue.get_nowait()
                except queue.Empty:
                    pass
                self._thread.join(timeout=0.05)
        self.is_started = False

    def __iter__(self):
        while True:
            s = self.get_sample()
            if s is None:
                return
            yield s

    # -- engine ----------------------------------------------------------------------------------------------------------------
    def _units(self):
        """Yields (sample id, source, [(filename, bytes)...]) with the reference image first."""
        sc = self.config["source_config"]
        rank, world = int(sc.get("rank", 0)), int(sc.get("world_size", 1) or 1)
        if self.source_type == "file":
            for path in enumerate_files(sc["root_path"], self.limit, rank, world, bool(sc.get("random_sampling", False))):
                try:
                    with open(path, "rb") as f:
                        yield json.dumps(path), "filesystem", [(path, f.read())]
                except OSError as e:
                    log.error("Failed to load image from path %s: %s", path, e)
        else:
            ref = sc.get("reference_image_type", "jpg")
            shards = expand_shards(sc["url"])
            if sc.get("random_sampling"):
                np.random.default_rng().shuffle(shards)
            for shard in shards:
                for source, files in tar_samples(shard, ref, rank, world):
                    key = os.path.splitext(os.path.basename(files[0][0]))[0]
                    yield key, source, files

    def _run(self):
        """The engine: a reader thread walks files / shards ahead of this thread (datago's generator task), and this
        thread keeps one batch on the GPU while it plans the next (datago's worker pool): a batch is launched -- host
        planning, upload, kernels and the packed download queued on the context's stream -- before the previous one is
        waited for and turned into samples.  Samples leave in source order."""
        produced = 0
        units_q = queue.Queue(maxsize=max(4 * self.batch_size, 16))
        reader = threading.Thread(target=self._read_ahead, args=(units_q,), daemon=True)
        reader.start()
        in_flight, flight_units = None, 0
        try:
            pending, lane, eof = [], 0, False
            while not self._stop.is_set():
                room = self.limit - produced - flight_units - len(pending)
                if not eof and room > 0 and len(pending) < self.batch_size:
                    try:
                        unit = units_q.get(timeout=0.1)
                    except queue.Empty:  # the reader is still at work (or the client is being stopped)
                        continue
                    if unit is None:
                        eof = True
                    else:
                        pending.append(unit)
                    continue
                if pending:  # a full batch, the last units below the limit, or the end of the source
                    launched = self._launch(pending, lane)
                    lane ^= 1
                    if in_flight is not None:
                        produced += self._finish(in_flight)
                    in_flight, flight_units, pending = launched, len(pending), []
                    continue
                if in_flight is not None:  # samples that failed leave room below the limit: the loop reads on
                    produced += self._finish(in_flight)
                    in_flight, flight_units = None, 0
                    continue
                break
        except Exception:  # noqa: BLE001
            log.exception("datago_b200 worker failed")
        finally:
            self._reader_stop.set()
            if in_flight is not None:
                try:
                    in_flight[0].sync()
                    in_flight[0].close()
                except Exception:  # noqa: BLE001
                    pass
            while reader.is_alive():  # unblock a reader stuck on a full queue
                try:
                    units_q.get_nowait()
                except queue.Empty:
                    pass
                reader.join(timeout=0.05)
            self._put(None)

    def _read_ahead(self, units_q):
        try:
            for unit in self._units():
                while not (self._stop.is_set() or self._reader_stop.is_set()):
                    try:
                        units_q.put(unit, timeout=0.1)
                        break
                    except queue.Full:
                        continue
                else:
                    return
        except Exception:  # noqa: BLE001
            log.exception("datago_b200 reader failed")
        finally:
            while not (self._stop.is_set() or self._reader_stop.is_set()):
                try:
                    units_q.put(None, timeout=0.1)
                    break
                except queue.Full:
                    continue

    def _host_buffer(self, lane, nbytes):
        """The lane's landing buffer for packed downloads: page-locked when torch can provide it (a copy into pageable
        memory is staged by the driver at a fraction of the link rate), grown on demand."""
        buf = self._buffers[lane]
        if buf is None or buf.nbytes < nbytes:
            want = max(nbytes, 1 << 20) * 5 // 4
            try:
                import torch
                buf = torch.empty(want, dtype=torch.uint8).pin_memory().numpy()
            except Exception:  # noqa: BLE001 - no torch, or no page-locked memory to be had
                buf = np.empty(want, np.uint8)
            self._buffers[lane] = buf
        return buf

    def _put(self, s):
        while not self._stop.is_set():
            try:
                self._queue.put(s, timeout=0.1)
                return True
            except queue.Full:
                continue
        return False

    def _launch(self, units, lane):
        """Queues one GPU batch for all image payloads of `units`; returns what _finish needs.  Later payloads of a
        sample are forced into the bucket of its first image (src/worker_wds.rs:68-76); the key comes from the
        header-only plan, so the whole sample rides in one batch."""
        inputs, keys, slots = [], [], []  # slots: (unit index, filename, is first image)
        has_tfm = self.ctx.image_config is not None
        for ui, (_, _, files) in enumerate(units):
            sample_key = None
            for name, data in files:
                ext = os.path.splitext(name)[1].lstrip(".").lower()
                if self.source_type == "webdataset" and ext not in IMG_TYPES:
                    continue
                forced = sample_key
                if not is_baseline_jpeg(data):
                    pixels = decode_on_host(data)  # PNG masks and whatever else the CUDA decoder does not take
                    if pixels is not None:
                        data = pixels
                if has_tfm and sample_key is None:
                    try:
                        if isinstance(data, np.ndarray):
                            h_, w_, c_ = data.shape[0], data.shape[1], (1 if data.ndim == 2 else data.shape[2])
                        else:
                            info = jpeg_probe(data)
                            w_, h_, c_ = info.width, info.height, info.channels
                        p = self.ctx.plan_geometry(w_, h_, c_)
                        sample_key = aspect_ratio_to_str(p.target_w, p.target_h)
                    except DatagoB200Error:
                        pass  # the item fails in the batch as well and the sample is handled there
                inputs.append(data)
                keys.append(forced)
                slots.append((ui, name))
        # `image_to_rgb8` of image_config applies to every image payload the file and webdataset workers produce
        # (src/worker_files.rs:19-30, src/worker_wds.rs:45-53 pass the client's ImageEncoding unchanged)
        to_rgb8 = True if (self.image_config or {}).get("image_to_rgb8") else None
        batch = self.ctx.batch(inputs, keys, 0 if has_tfm else BATCH_DECODE_ONLY, to_rgb8=to_rgb8)
        batch.upload()
        batch.run()
        buf = None
        if not self.device_payloads and len(batch):
            buf = self._host_buffer(lane, batch.packed_bytes())
            batch.download_packed(buf)  # one copy; payload i lands at result(i).packed_offset
        return batch, units, slots, buf

    def _finish(self, launched):
        """Waits for a launched batch and puts its samples on the queue; returns how many it made."""
        batch, units, slots, buf = launched
        batch.sync()
        made = 0
        payloads = {}
        for i, (ui, name) in enumerate(slots):
            r = batch.result(i)
            if r.status != 0:
                log.error("decode failed for %s (status %d)", name, r.status)
                continue
            if self.pre_encode and not self.device_payloads:
                px = buf[r.packed_offset:r.packed_offset + r.nbytes].reshape(r.height, r.width, r.channels)
                pl = ImagePayload(data=encode_payload(px, self.encode_format, self.jpeg_quality),
                                  original_height=r.original_height, original_width=r.original_width, height=r.height,
                                  width=r.width, channels=-1, bit_depth=8, is_encoded=True)
            else:
                pl = ImagePayload(data=b"" if self.device_payloads else buf[r.packed_offset:r.packed_offset + r.nbytes].tobytes(), original_height=r.original_height,
                                  original_width=r.original_width, height=r.height, width=r.width, channels=r.channels,
                                  bit_depth=8, is_encoded=False, device_ptr=r.device_data if self.device_payloads else 0,
                                  keepalive=batch if self.device_payloads else None)
            payloads.setdefault(ui, []).append((name, pl))
        if not self.device_payloads:
            batch.close()
        for ui, (sid, source, files) in enumerate(units):
            sample = self._assemble(sid, source, files, payloads.get(ui, []))
            if sample is None:
                continue
            if not self._put(sample):
                break
            made += 1
        return made

    def _assemble(self, sid, source, files, imgs):
        if self.source_type == "file":
            if not imgs:
                return None  # src/worker_files.rs:63-70: the sample is dropped
            return Sample(sid, source, imgs[0][1])
        sc = self.config["source_config"]
        ref = sc.get("reference_image_type", "jpg")
        sample, attributes = None, {}
        for name, pl in imgs:  # src/worker_wds.rs:78-131
            ext = os.path.splitext(name)[1].lstrip(".")
            if ext == ref:
                if sample is None:
                    sample = Sample(sid, source, pl)
                else:
                    sample.image = pl
            else:
                if sample is None:
                    sample = Sample(sid, source, _empty_payload())
                sample.additional_images[name] = pl
        for name, data in files:  # src/worker_wds.rs:139-144
            ext = os.path.splitext(name)[1].lstrip(".")
            if ext in TEXT_TYPES:
                attributes[ext] = data.decode("utf-8", errors="replace")
        if sample is None:
            return None
        sample._attributes = attributes
        return sample
