/*
 * datago_b200 -- C ABI of the B200 image path that replaces datago's per-sample
 * "decode -> bucket -> resize -> crop" routine.
 *
 * datago (Rust) has no FFI seam for this path: the work happens in ordinary Rust calls into the
 * `image` and `fast_image_resize` crates.  This header cuts the seam at those calls; each entry point
 * names the datago source line(s) it stands in for (paths relative to the datago tree).
 *
 * Conventions
 *   - plain C, POD structs, no exceptions; every function that can fail returns a dg_status (0 = ok)
 *     and leaves a message readable with dg_last_error() on the calling thread;
 *   - a dg_ctx is bound to one CUDA device and one stream; calls on one ctx are serialised by an
 *     internal lock, so the tokio worker threads of src/worker_files.rs:83-121 may share it;
 *   - the CUDA path is the only path: there is no CPU fallback.  dg_ctx_create fails when no
 *     device is usable.
 */
#ifndef DATAGO_B200_H
#define DATAGO_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#if defined(__GNUC__)
#define DG_API __attribute__((visibility("default")))
#else
#define DG_API
#endif

typedef enum dg_status {
    DG_OK = 0,
    DG_E_INVALID = 1,      /* bad argument */
    DG_E_CUDA = 2,         /* a CUDA runtime call failed; see dg_last_error */
    DG_E_TRUNCATED = 3,    /* JPEG ends early (headers or entropy-coded data) */
    DG_E_BAD_MARKER = 4,   /* not a JPEG / marker structure broken */
    DG_E_UNSUPPORTED = 5,  /* progressive, arithmetic, 12-bit, CMYK, unsupported sampling */
    DG_E_BAD_TABLE = 6,    /* Huffman / quantisation table missing or malformed */
    DG_E_BAD_CODE = 7,     /* entropy decoding met a code that is not in the table */
    DG_E_UNKNOWN_KEY = 8,  /* forced aspect-ratio key is not a bucket (datago panics: image_processing.rs:335) */
    DG_E_NO_TRANSFORM = 9, /* a bucket query on a ctx created without crop_and_resize */
    DG_E_SYNC_LIMIT = 10,  /* entropy decoder did not converge within its iteration cap */
    DG_E_TOO_LARGE = 11,   /* input exceeds a stated size limit: an image whose header declares more than 512 MiB of
                              decoded pixels (the `image` crate's default allocation limit; DATAGO_B200_MAX_IMAGE_MB
                              at context creation changes it), or an entropy-coded segment of 4 GiB */
    DG_E_TIMEOUT = 12      /* dg_wait: the sample has not finished within the given time (the ticket stays valid) */
} dg_status;

/* image_config of the client JSON: ImageTransformConfig, src/image_processing.rs:43-70 (the fields on this path). */
typedef struct dg_image_config {
    int32_t crop_and_resize;
    uint32_t default_image_size;
    uint32_t downsampling_ratio;
    double min_aspect_ratio;
    double max_aspect_ratio;
} dg_image_config;

/* Geometry of crop_and_resize for one image: src/image_processing.rs:259-310. */
typedef struct dg_plan {
    uint32_t src_w, src_h, channels; /* decoded size; 3 = RGB8, 1 = L8 */
    uint32_t target_w, target_h;     /* bucket size = output size */
    uint32_t new_w, new_h;           /* size after the first (whole-image) resize */
    double crop_left, crop_top;      /* CropBox::fit_src_into_dst_size(new_w, new_h, target_w, target_h, None) */
    double crop_w, crop_h;
    int32_t identity;                /* 1: source already has the bucket size and is returned unchanged (:266-267) */
    char key[16];                    /* bucket key, format!("{:.3}", w / h) */
} dg_plan;

typedef struct dg_jpeg_info {
    uint32_t width, height, channels; /* channels of the decoded image: 3 or 1 */
    uint32_t hsamp, vsamp;            /* luma sampling factors (2,2 = 4:2:0; 1,1 = 4:4:4) */
    uint32_t mcux, mcuy, restart_interval;
    uint64_t scan_offset, scan_len;   /* entropy-coded segment within the file */
} dg_jpeg_info;

/* One unit of work of a batch. */
typedef struct dg_item {
    const uint8_t* data;   /* JPEG file bytes, or raw interleaved 8-bit pixels when raw_w > 0 (host memory) */
    uint64_t len;
    uint32_t raw_w, raw_h, raw_c; /* raw input: size and channels (1 = L8, 2 = LA8, 3 = RGB8, 4 = RGBA8); 0 for JPEG input */
    uint32_t flags;        /* DG_ITEM_* */
    const char* forced_key; /* NULL or "": bucket chosen from the image's own aspect ratio; else the key to force
                               (the "same bucket for every payload of a sample" rule, src/worker_wds.rs:68-76) */
} dg_item;

/* dg_item.flags.
 * DG_ITEM_TO_RGB8: ImageEncoding.img_to_rgb8 (`image_to_rgb8` of the client JSON, src/image_processing.rs:27,63): after
 * crop_and_resize a payload that is not RGB8 is converted by convert_to_rgb8 (:163-186, applied at :366-372):
 * one-channel images repeat their value in three channels, RGBA is composited over an opaque (128,128,128)
 * background (source-over in f32, truncated to 8 bits), and the payload reports channels = 3.  datago sets it for
 * the main image and never for masks / additional images (src/worker_http.rs:188-192).
 * Images with an alpha channel (LA8, RGBA8) are resized as fast_image_resize does it for U8x2 / U8x4 pixels
 * (src/image_processing.rs:269-274): colour multiplied by alpha before each convolution resize and divided by it
 * afterwards; without the flag the payload keeps its 2 or 4 channels. */
enum { DG_ITEM_TO_RGB8 = 1u };

/* Per-item outcome: the fields of ImagePayload (src/structs.rs:52-71) plus where the pixels are. */
typedef struct dg_result {
    int32_t status;               /* dg_status of this item */
    uint32_t original_width, original_height;
    uint32_t width, height, channels, bit_depth;
    uint64_t nbytes;              /* width * height * channels */
    const uint8_t* device_data;   /* HWC, row-major, tightly packed, in device memory owned by the batch */
    dg_plan plan;                 /* valid when the ctx has a transform */
    uint64_t packed_offset;       /* where dg_batch_download_packed puts this payload, from its host base */
} dg_result;

/* One bucket of a DG_BATCH_COLLATE batch: n same-shape payloads stored back to back, i.e. one dense uint8
 * [n][height][width][channels] array -- what a training loop stacks from the `ImagePayload`s of one aspect-ratio
 * bucket after src/structs.rs:154-188 (to_numpy_array) has copied each of them. */
typedef struct dg_bucket {
    char key[16];                /* bucket key; "" for batches without a transform (grouped by decoded shape) */
    uint32_t n, width, height, channels;
    uint64_t nbytes;             /* n * height * width * channels */
    const uint8_t* device_data;  /* device memory owned by the batch */
    uint64_t packed_offset;      /* where dg_batch_download_packed puts the array, from its host base */
    const int32_t* items;        /* n batch indices: items[k] is the item stored at position k (batch order kept) */
} dg_bucket;

typedef struct dg_ctx dg_ctx;
typedef struct dg_batch dg_batch;

enum {
    DG_BATCH_DECODE_ONLY = 1u,  /* ignore the ctx transform: payload = decoded image (image_to_payload with img_tfm None) */
    DG_BATCH_TIMING = 2u,       /* record CUDA events around each stage of dg_batch_run */
    DG_BATCH_KEEP_COEFFICIENTS = 4u, /* leave the decoded coefficients in place for dg_batch_debug (they are normally
                                        zeroed again as they are consumed) */
    DG_BATCH_COLLATE = 8u       /* lay the payloads out bucket by bucket, see dg_batch_bucket */
};

/* Stages reported by dg_batch_stage_ms. */
enum { DG_STAGE_UNSTUFF = 0, DG_STAGE_COEF_CLEAR, DG_STAGE_HUFF_RESTART, DG_STAGE_HUFF_SPEC, DG_STAGE_IDCT, DG_STAGE_COLOR,
       DG_STAGE_RESIZE_H, DG_STAGE_RESIZE_V, DG_STAGE_RESIZE_SHIFT, DG_STAGE_TO_RGB8, DG_STAGE_COUNT };

DG_API const char* dg_last_error(void);
DG_API const char* dg_version(void);

/* ---- logging and counters --------------------------------------------------------------------------------------------
 * datago reports every sample it drops through the `log` crate (src/worker_files.rs:63-70, src/worker_wds.rs:134-137) and
 * lets the embedding process choose the sink (initialize_logging, src/client.rs:253-263).  Here the embedding process
 * installs a callback; the library calls it from the thread that runs dg_batch_sync / the feeder lanes, once per failed
 * item (DG_LOG_ERROR: "item 17: truncated (status 3)") and for rare conditions of the library itself (DG_LOG_WARN).
 * NULL removes the callback (the default: silent).  The callback must not call back into the library. */
enum { DG_LOG_ERROR = 1, DG_LOG_WARN = 2, DG_LOG_INFO = 3, DG_LOG_DEBUG = 4 };
typedef void (*dg_log_fn)(int level, const char* message, void* user);
DG_API void dg_set_log_callback(dg_log_fn fn, void* user);

/* Items a context has finished, by dg_status (index = status code, [0] = succeeded), counted in dg_batch_sync:
 * the per-reason drop counters a data-loading service exports. */
#define DG_STATUS_COUNT 13
typedef struct dg_ctx_counters {
    uint64_t items[DG_STATUS_COUNT];
    uint64_t batches, bytes_in, bytes_out;  /* batches synchronised; compressed / raw bytes uploaded; payload bytes produced */
} dg_ctx_counters;

/* ---- context ------------------------------------------------------------------------------------------------ */
/* DatagoClient::new builds the transform once (src/client.rs:92-95 -> image_processing.rs:77-120).
 * cfg NULL or crop_and_resize == 0: no transform (payloads are the decoded images).
 * Invalid configs (size 0, ratio 0, min_ar <= 0, max_ar < min_ar) return DG_E_INVALID where datago asserts (:78-93). */
#define DG_DEVICE_NONE (-1) /* planning-only ctx: bucket / geometry queries work, every pixel entry point fails */
DG_API int dg_ctx_create(int device, const dg_image_config* cfg, dg_ctx** out);
/* Same, running on a caller-owned CUDA stream (a cudaStream_t passed as void*). */
DG_API int dg_ctx_create_on_stream(int device, const dg_image_config* cfg, void* cuda_stream, dg_ctx** out);
DG_API void dg_ctx_destroy(dg_ctx* ctx);
/* The cudaStream_t all work of this ctx is queued on. */
DG_API void* dg_ctx_stream(dg_ctx* ctx);
DG_API int dg_ctx_get_counters(dg_ctx* ctx, dg_ctx_counters* out);

/* ---- bucket logic (host only; no device work) ------------------------------------------------------------------- */
/* build_image_size_list, src/image_processing.rs:188-219: the raw list, duplicates kept. Returns the count. */
DG_API int dg_size_list(const dg_image_config* cfg, int max_n, uint32_t* w, uint32_t* h);
/* The key -> size map sorted by aspect ratio (get_ar_aware_transform, :96-119). keys: 16 bytes per entry. Returns the count. */
DG_API int dg_bucket_table(const dg_ctx* ctx, int max_n, uint32_t* w, uint32_t* h, double* ar, char* keys);
/* ARAwareTransform::get_closest_aspect_ratio, :222-252. */
DG_API int dg_closest_aspect_ratio(const dg_ctx* ctx, int32_t w, int32_t h, char key_out[16]);
/* aspect_ratio_to_str, :130-133. */
DG_API void dg_aspect_ratio_to_str(uint32_t w, uint32_t h, char key_out[16]);
/* Geometry half of crop_and_resize, :259-310. */
DG_API int dg_plan_geometry(const dg_ctx* ctx, uint32_t w, uint32_t h, uint32_t channels, const char* forced_key, dg_plan* out);
/* Header-only look at a JPEG (what image::ImageReader learns before decode(), src/worker_files.rs:14-16). */
DG_API int dg_jpeg_probe(const uint8_t* data, uint64_t len, dg_jpeg_info* out);

/* ---- sharding (host only) ----------------------------------------------------------------------------------------- */
/* get_data_slice_multirank, src/generator_files.rs:24-42. DG_E_INVALID when rank >= world_size (datago asserts). */
DG_API int dg_rank_slice(uint64_t quorum, uint64_t rank, uint64_t world_size, uint64_t* start, uint64_t* end);
/* hash_fn, src/generator_wds.rs:50-54: Rust's DefaultHasher over the key string. */
DG_API uint64_t dg_key_hash(const char* key, uint64_t len);
/* The rank a webdataset key belongs to, src/generator_wds.rs:140-148. */
DG_API uint64_t dg_key_rank(const char* key, uint64_t len, uint64_t world_size);

/* ---- batches: image::load_from_memory + image_to_payload for many samples at once ---------------------------- */
/* Replaces, per item, the decode call (src/worker_files.rs:8-17, src/worker_wds.rs:45, src/worker_http.rs:64)
 * followed by image_to_payload (src/image_processing.rs:341-431).
 * create: parses headers, plans geometry, builds device descriptors and filter tables, copies the compressed
 *         (or raw) bytes into pinned staging.  Items whose header is bad keep a non-zero status and are skipped,
 *         as datago drops a sample whose decode fails (src/worker_files.rs:63-70).
 * upload: host -> device copies (async on the ctx stream).
 * run:    all kernels (async).  May be called repeatedly on an uploaded batch.
 * download: device -> host copy of every ok item into host_out[i] (entries may be NULL to skip).
 * sync:   waits for the stream and collects per-item device status words.
 */
DG_API int dg_batch_create(dg_ctx* ctx, const dg_item* items, int n, uint32_t flags, dg_batch** out);
DG_API int dg_batch_upload(dg_batch* b);
DG_API int dg_batch_run(dg_batch* b);
DG_API int dg_batch_download(dg_batch* b, uint8_t* const* host_out);
/* One device -> host copy for the whole batch: payload i lands at host_base + result.packed_offset (256-byte aligned
 * slots).  dg_batch_packed_bytes gives the size the buffer needs.  Prefer this for large batches: thousands of separate
 * asynchronous copies fill the driver's submission queue and stall the calling thread. */
DG_API int dg_batch_download_packed(dg_batch* b, uint8_t* host_base, uint64_t capacity);
DG_API uint64_t dg_batch_packed_bytes(const dg_batch* b);
DG_API int dg_batch_sync(dg_batch* b);
DG_API int dg_batch_result(const dg_batch* b, int i, dg_result* out);
/* Buckets of a DG_BATCH_COLLATE batch, in order of first appearance.  Items that dg_batch_create rejected (bad header
 * or tables, unknown key, too large) belong to no bucket.  An item whose entropy-coded data turns out to be damaged is
 * only found on the device: it keeps its slot, the slot's pixels are undefined and its dg_result.status is non-zero
 * after dg_batch_sync -- consumers of a bucket array must look at the status of items[k].  Images and
 * masks of one key differ in channels and form separate buckets.  Per-item results stay valid (they point into the
 * bucket arrays).  0 buckets for a batch created without the flag. */
DG_API int dg_batch_bucket_count(const dg_batch* b);
DG_API int dg_batch_bucket(const dg_batch* b, int k, dg_bucket* out);
/* Milliseconds per stage of the last dg_batch_run of a DG_BATCH_TIMING batch (after dg_batch_sync). */
DG_API int dg_batch_stage_ms(const dg_batch* b, float ms[DG_STAGE_COUNT]);
/* Bytes copied host->device by upload, and kernels launched by one run. */
DG_API int dg_batch_counters(const dg_batch* b, uint64_t* h2d_bytes, uint64_t* d2h_bytes, uint32_t* kernel_launches);
/* Counters of the speculative entropy decoder over the last run: chunks of subsequences processed, synchronisation
 * rounds, subsequence decodes (guess + re-decodes + write pass).  Synchronises the stream. */
DG_API int dg_batch_huffman_stats(dg_batch* b, uint64_t out[3]);
/* Intermediate device buffers, for stage-by-stage parity tests: coefficient words (int16, scan order) and, for
 * decode+resize batches, the full-size decoded image of item i (its rows padded to a multiple of 16 bytes unless the
 * item's plan is an identity). */
DG_API int dg_batch_debug(const dg_batch* b, int i, const int16_t** coef, uint64_t* nblocks, const uint8_t** decoded);
DG_API void dg_batch_destroy(dg_batch* b);

/* One call doing create + upload + run + download + sync + destroy; results[i] (optional) receive the outcomes
 * (device_data is NULL there: the batch is gone). */
DG_API int dg_process(dg_ctx* ctx, const dg_item* items, int n, uint32_t flags, uint8_t* const* host_out, dg_result* results);

/* ---- submit / wait: single samples from many threads, batched for the GPU ----------------------------------------
 * datago calls the decode + image_to_payload pair once per sample from num_cpus tokio worker threads, all at once
 * (src/worker_files.rs:83-121,150-152; src/worker_wds.rs:183-227; src/worker_http.rs:276-332).  A feeder keeps that
 * calling pattern: any number of threads call dg_submit / dg_wait concurrently; lane threads inside the feeder gather
 * the queued samples into batches (up to max_batch, or whatever is there once the oldest sample has waited
 * max_wait_us) and run them through the batch entry points above, so results are the batch path's results.
 *   dg_submit   copies the sample's bytes (the caller's buffer is free again on return, like the `&item.buffer` borrow
 *               of src/worker_wds.rs:45) and returns a ticket; blocks while queue_limit samples are already waiting
 *               (the bounded-concurrency role of DATAGO_MAX_TASKS).  host_out may be NULL.
 *   dg_wait     blocks up to timeout_ns (UINT64_MAX: no limit) for the ticket; fills *out.  With a host_out given at
 *               submit it also copies the payload there, on the calling thread; out->device_data is then NULL.
 *               Without one, out->device_data points at the payload in device memory until dg_release, and
 *               dg_fetch copies it to host memory once the caller has sized a buffer from out->nbytes.
 *   dg_release  ends the ticket (any state); every ticket must be released.  A ticket belongs to one thread at a time.
 * A sample that fails (bad JPEG, unknown forced key) completes with that status in out->status, as datago logs and drops
 * such a sample (src/worker_files.rs:63-70); the dg_wait call itself still returns DG_OK. */
typedef struct dg_feeder dg_feeder;
typedef uint64_t dg_ticket;

typedef struct dg_feeder_config {  /* zero fields take the default */
    uint32_t lanes;        /* batches in flight, each with its own context and thread (default 2, at most 8) */
    uint32_t max_batch;    /* samples per batch (default 512) */
    uint32_t max_wait_us;  /* longest time a queued sample waits for its batch to fill (default 2000) */
    uint32_t queue_limit;  /* dg_submit blocks while this many samples are queued (default 4 * max_batch) */
    uint32_t batch_flags;  /* 0 or DG_BATCH_DECODE_ONLY */
    uint32_t reserved;
} dg_feeder_config;

typedef struct dg_feeder_stats {
    uint64_t submitted, completed, failed; /* failed: completed with a non-zero status */
    uint64_t batches, batched_items;
    uint32_t largest_batch, queued, open_tickets, reserved;
} dg_feeder_stats;

DG_API int dg_feeder_create(int device, const dg_image_config* image_config, const dg_feeder_config* config, dg_feeder** out);
/* A context with the feeder's transform, for dg_plan_geometry / dg_closest_aspect_ratio / dg_bucket_table queries. */
DG_API const dg_ctx* dg_feeder_ctx(const dg_feeder* f);
DG_API int dg_submit(dg_feeder* f, const dg_item* item, uint8_t* host_out, uint64_t host_capacity, dg_ticket* ticket);
DG_API int dg_wait(dg_feeder* f, dg_ticket ticket, uint64_t timeout_ns, dg_result* out);
DG_API int dg_fetch(dg_feeder* f, dg_ticket ticket, uint8_t* host_out, uint64_t capacity);
/* The payload where the feeder's own device -> host copy left it (page-locked host memory of the library), valid until
 * dg_release: lets a caller consume the pixels without a second host copy. */
DG_API int dg_peek(dg_feeder* f, dg_ticket ticket, const uint8_t** host_data);
DG_API int dg_release(dg_feeder* f, dg_ticket ticket);
DG_API int dg_feeder_get_stats(dg_feeder* f, dg_feeder_stats* out);
/* Stops the lanes, fails what is still queued, frees everything (device payloads of unreleased tickets included).
 * No other call on the feeder may be in progress or follow. */
DG_API void dg_feeder_destroy(dg_feeder* f);

/* crop_and_resize of ONE image that is already in device memory, without any device allocation.
 * No counterpart in datago: it exists for hosts that must not let a library allocate device memory while they run
 * (a training process whose framework allocator owns all of HBM, a loop that cannot afford the device-wide
 * synchronisation an allocation can imply, a service with a no-allocation-after-start-up rule).
 * device_src: w * h * channels interleaved 8-bit pixels, any alignment; the library loads no byte outside those
 * w * h * channels, so the image may end where its allocation ends.  device_dst: room for the bucket's target_w *
 * target_h * channels bytes (learn the size first with dg_plan_geometry).  The work runs on the ctx stream (see
 * dg_ctx_stream), a non-blocking stream that is not ordered with any stream of the caller: device_src must be
 * complete, and device_dst free to be written, before the call; the result is complete when the call returns.  Descriptors, filter tables and the images between
 * passes live in one 32 MiB array inside the library image, held by every GPU that loads the library until exit.
 * Limit: intermediates + tables must fit those 32 MiB; the intermediates are bounded by
 * new_w * channels * (max(src_h, new_h) + 2 * new_h) bytes (new_w, new_h from dg_plan_geometry), e.g. a 4096 x 4096
 * RGB source into a 1024-class bucket needs about 19 MiB.  Larger inputs get DG_E_TOO_LARGE and nothing is launched.
 * The first call on a device looks up the array's device address; make that call before any stream capture.
 * All calls share the array and it keeps whatever the last call left (nothing in it needs clearing: every byte is
 * written before it is read), so two calls that overlap on the same GPU -- two contexts, two streams -- race; calls
 * on one ctx are serialised and the function returns after its work has completed. */
DG_API int dg_resize_device_static(dg_ctx* ctx, const uint8_t* device_src, uint32_t w, uint32_t h, uint32_t channels,
                            const char* forced_key, uint8_t* device_dst, dg_plan* plan_out);

/* Device -> host copy helper for callers without a CUDA binding (tests). */
DG_API int dg_copy_to_host(dg_ctx* ctx, void* dst, const void* device_src, uint64_t nbytes);

#ifdef __cplusplus
}
#endif
#endif
