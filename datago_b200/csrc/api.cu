// C ABI of the B200 image path (declared in include/datago_b200.h) and the batch scheduler behind it.
//
// A batch is planned on the host (headers, bucket geometry, filter tables, device descriptors), its inputs are
// staged in pinned memory and uploaded with a handful of large copies, and its images run through the kernels
// in "waves": groups of images whose intermediates (unstuffed streams, coefficients, planes, full-size decoded
// images, resize intermediates) share one scratch block that the next wave reuses.
#include <cuda.h>  // CUtensorMap and the enumerations of cuTensorMapEncodeTiled; the entry point itself comes through the runtime
#include <cuda_runtime.h>

#include <algorithm>
#include <atomic>
#include <array>
#include <cmath>
#include <cstdarg>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <map>
#include <memory>
#include <mutex>
#include <string>
#include <thread>
#include <unordered_map>
#include <vector>

#include "host.h"
#include "host_pool.h"
#include "kernels.h"

using namespace dg;

// ---------------------------------------------------------------------------------------------------------------
// errors
// ---------------------------------------------------------------------------------------------------------------
static thread_local char g_err[512] = "";

static int fail(int code, const char* fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_err, sizeof g_err, fmt, ap);
    va_end(ap);
    return code;
}

int dg::dg_set_error(int code, const char* msg) { return fail(code, "%s", msg); }

#define CU(call)                                                                                         \
    do {                                                                                                 \
        cudaError_t e_ = (call);                                                                         \
        if (e_ != cudaSuccess) return fail(DG_E_CUDA, "%s: %s (%s:%d)", #call, cudaGetErrorString(e_), __FILE__, __LINE__); \
    } while (0)

// ---- logging ----------------------------------------------------------------------------------------------------------
static std::mutex g_log_mu;
static dg_log_fn g_log_fn = nullptr;
static void* g_log_user = nullptr;

extern "C" void dg_set_log_callback(dg_log_fn fn, void* user) {
    std::lock_guard<std::mutex> lock(g_log_mu);
    g_log_fn = fn;
    g_log_user = user;
}

static void log_line(int level, const char* fmt, ...) {
    dg_log_fn fn;
    void* user;
    {
        std::lock_guard<std::mutex> lock(g_log_mu);
        fn = g_log_fn;
        user = g_log_user;
    }
    if (!fn) return;
    char buf[256];
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(buf, sizeof buf, fmt, ap);
    va_end(ap);
    fn(level, buf, user);
}

static const char* status_name(int st) {
    static const char* const names[DG_STATUS_COUNT] = {"ok", "invalid", "cuda", "truncated", "bad_marker", "unsupported", "bad_table",
                                                       "bad_code", "unknown_key", "no_transform", "sync_limit", "too_large", "timeout"};
    return st >= 0 && st < DG_STATUS_COUNT ? names[st] : "?";
}

extern "C" const char* dg_last_error(void) { return g_err; }
extern "C" const char* dg_version(void) { return "datago_b200 0.1 (sm_100a)"; }

// ---------------------------------------------------------------------------------------------------------------
// context: device, stream, transform, caches of device and pinned blocks
// ---------------------------------------------------------------------------------------------------------------
namespace {

struct Block {
    void* ptr = nullptr;
    size_t size = 0;
    bool busy = false;
    size_t zero_prefix = 0;  // scratch blocks: leading bytes known to be zero (the coefficient region, see dg_batch_run)
};

// Grow-only cache: a batch borrows blocks and hands them back; nothing is freed before the ctx goes away, so steady
// state makes no allocation calls.
struct BlockCache {
    bool pinned;
    std::vector<Block> blocks;
    explicit BlockCache(bool p) : pinned(p) {}
    int acquire(size_t size, int* index, bool keep_zero_prefix = false) {
        if (size == 0) size = 256;
        int best = -1;
        for (size_t i = 0; i < blocks.size(); ++i)
            if (!blocks[i].busy && blocks[i].size >= size && (best < 0 || blocks[i].size < blocks[best].size)) best = (int)i;
        if (best < 0) {
            // replace the largest idle block that is too small, so the cache does not pile up stale sizes
            int victim = -1;
            for (size_t i = 0; i < blocks.size(); ++i)
                if (!blocks[i].busy && (victim < 0 || blocks[i].size > blocks[victim].size)) victim = (int)i;
            Block nb;
            nb.size = size + size / 8 + 4096;
            if (victim >= 0) {
                if (pinned) cudaFreeHost(blocks[victim].ptr); else cudaFree(blocks[victim].ptr);
                blocks[victim] = Block();
            }
            cudaError_t e = pinned ? cudaHostAlloc(&nb.ptr, nb.size, cudaHostAllocDefault) : cudaMalloc(&nb.ptr, nb.size);
            if (e != cudaSuccess) {
                cudaGetLastError();  // a failed allocation must not surface again as the next healthy batch's error
                return fail(DG_E_CUDA, "%s of %zu bytes: %s", pinned ? "cudaHostAlloc" : "cudaMalloc", nb.size, cudaGetErrorString(e));
            }
            if (victim >= 0) { blocks[victim] = nb; best = victim; }
            else { blocks.push_back(nb); best = (int)blocks.size() - 1; }
        }
        blocks[best].busy = true;
        if (!keep_zero_prefix) blocks[best].zero_prefix = 0;
        *index = best;
        return DG_OK;
    }
    void release(int index) { if (index >= 0) blocks[index].busy = false; }
    void clear() {
        for (auto& b : blocks) if (b.ptr) { if (pinned) cudaFreeHost(b.ptr); else cudaFree(b.ptr); }
        blocks.clear();
    }
};

inline size_t align_up(size_t v, size_t a) { return (v + a - 1) / a * a; }

}  // namespace

struct dg_ctx {
    int device = 0;
    cudaStream_t stream = nullptr;   // everything the caller can observe is ordered on this stream
    cudaStream_t stream2 = nullptr;  // odd waves of a batch run here, concurrently with the even ones
    cudaStream_t aux[2] = {nullptr, nullptr};  // per lane: the restart-interval decoder runs beside the speculative one
    cudaEvent_t ev_fork = nullptr, ev_join = nullptr;
    cudaEvent_t ev_aux_go[2] = {nullptr, nullptr}, ev_aux_done[2] = {nullptr, nullptr};
    bool own_stream = false;
    bool has_tfm = false;
    dg_image_config cfg{};
    Transform tfm;
    std::mutex mu;
    BlockCache dev{false}, pin{true};
    // Lanczos tables built so far, by (input size, box, output size): data sets repeat image sizes, and every epoch
    // repeats all of them, while a table costs two sin() per weight.  Dropped wholesale when it outgrows its cap.
    std::map<std::array<uint64_t, 4>, std::shared_ptr<const FilterTable>> table_cache;
    size_t table_cache_bytes = 0, table_cache_cap = (size_t)512 << 20;
    size_t wave_bytes = (size_t)13 << 30;  // coefficient bytes per wave (upper bound; waves are balanced below it)
    // Plane bytes per IDCT + colour launch pair.  Launching the two kernels in groups of images whose planes fit the L2
    // used to pay; with the present colour kernel the tails of many small launches cost more than the plane reads from
    // DRAM, so the default is one pair per wave (DATAGO_B200_L2_GROUP_MB restores the grouping).
    size_t l2_group_bytes = (size_t)1 << 40;
    // Three-component 4:2:0 images take the fused path (luma never leaves the SM); DATAGO_B200_FUSED=0 sends them through
    // the general IDCT and colour kernels instead (for measurements and for testing that path on the common sampling).
    bool fused_path = true;
    // Horizontal resize passes run on the tensor cores where their geometry fits; DATAGO_B200_HMMA=0 keeps them on the
    // dp2a kernel (measurements, and the test-suite's coverage of that kernel).
    bool hmma = true;
    unsigned int conv_timeouts_seen = 0;
    dg_ctx_counters counters{};  // guarded by mu
    // Largest decoded image accepted (width * height * channels bytes); the `image` crate's default allocation limit is 512 MiB.
    uint64_t max_image_bytes = (uint64_t)512 << 20;
};

// cuTensorMapEncodeTiled, looked up through the runtime (the library does not link against the driver library).
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                  const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
static EncodeTiledFn encode_tiled_fn() {
    static const EncodeTiledFn fn = [] {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult q = cudaDriverEntryPointSymbolNotFound;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) != cudaSuccess || q != cudaDriverEntryPointSuccess) p = nullptr;
        return (EncodeTiledFn)p;
    }();
    return fn;
}

static int ctx_create(int device, const dg_image_config* cfg, void* stream, bool have_stream, dg_ctx** out) {
    if (!out) return fail(DG_E_INVALID, "out is NULL");
    *out = nullptr;
    if (device != DG_DEVICE_NONE) {
        int count = 0;
        cudaError_t e = cudaGetDeviceCount(&count);
        if (e != cudaSuccess || count == 0)
            return fail(DG_E_CUDA, "no usable CUDA device (%s); this library has no CPU path", e != cudaSuccess ? cudaGetErrorString(e) : "count is 0");
        if (device < 0 || device >= count) return fail(DG_E_INVALID, "device %d out of range (%d present)", device, count);
    }
    dg_ctx* c = new dg_ctx();
    c->device = device;
    if (cfg && cfg->crop_and_resize) {
        if (!config_valid(*cfg)) { delete c; return fail(DG_E_INVALID, "image_config: size, ratio and aspect-ratio bounds must be positive and ordered"); }
        c->cfg = *cfg;
        c->tfm = make_transform(*cfg);
        c->has_tfm = !c->tfm.buckets.empty();
        if (!c->has_tfm) { delete c; return fail(DG_E_INVALID, "image_config yields an empty bucket table"); }
    }
    if (device == DG_DEVICE_NONE) { *out = c; return DG_OK; }  // planning only: bucket and geometry queries
    if (cudaSetDevice(device) != cudaSuccess) { delete c; return fail(DG_E_CUDA, "cudaSetDevice(%d) failed", device); }
    if (have_stream) c->stream = (cudaStream_t)stream;
    else {
        if (cudaStreamCreateWithFlags(&c->stream, cudaStreamNonBlocking) != cudaSuccess) { delete c; return fail(DG_E_CUDA, "cudaStreamCreate failed"); }
        c->own_stream = true;
    }
    if (cudaStreamCreateWithFlags(&c->stream2, cudaStreamNonBlocking) != cudaSuccess ||
        cudaEventCreateWithFlags(&c->ev_fork, cudaEventDisableTiming) != cudaSuccess ||
        cudaEventCreateWithFlags(&c->ev_join, cudaEventDisableTiming) != cudaSuccess ||
        cudaStreamCreateWithFlags(&c->aux[0], cudaStreamNonBlocking) != cudaSuccess ||
        cudaStreamCreateWithFlags(&c->aux[1], cudaStreamNonBlocking) != cudaSuccess ||
        cudaEventCreateWithFlags(&c->ev_aux_go[0], cudaEventDisableTiming) != cudaSuccess ||
        cudaEventCreateWithFlags(&c->ev_aux_go[1], cudaEventDisableTiming) != cudaSuccess ||
        cudaEventCreateWithFlags(&c->ev_aux_done[0], cudaEventDisableTiming) != cudaSuccess ||
        cudaEventCreateWithFlags(&c->ev_aux_done[1], cudaEventDisableTiming) != cudaSuccess) {
        delete c;
        return fail(DG_E_CUDA, "creating the second stream failed");
    }
    if (const char* mb = getenv("DATAGO_B200_L2_GROUP_MB")) { long v = atol(mb); if (v >= 1) c->l2_group_bytes = (size_t)v << 20; }
    if (const char* mb = getenv("DATAGO_B200_TABLE_CACHE_MB")) { long v = atol(mb); if (v >= 0) c->table_cache_cap = (size_t)v << 20; }
    if (const char* v = getenv("DATAGO_B200_FUSED")) c->fused_path = atoi(v) != 0;
    if (const char* v = getenv("DATAGO_B200_HMMA")) c->hmma = atoi(v) != 0;
    if (!encode_tiled_fn()) c->hmma = false;  // a driver without tensor maps: every horizontal pass takes the dp2a kernel
    if (const char* mb = getenv("DATAGO_B200_MAX_IMAGE_MB")) { long v = atol(mb); if (v >= 1) c->max_image_bytes = (uint64_t)v << 20; }
    if (const char* mb = getenv("DATAGO_B200_WAVE_MB")) { long v = atol(mb); if (v >= 16) c->wave_bytes = (size_t)v << 20; }
    *out = c;
    return DG_OK;
}

extern "C" int dg_ctx_create(int device, const dg_image_config* cfg, dg_ctx** out) { return ctx_create(device, cfg, nullptr, false, out); }
extern "C" int dg_ctx_create_on_stream(int device, const dg_image_config* cfg, void* s, dg_ctx** out) { return ctx_create(device, cfg, s, true, out); }

extern "C" void dg_ctx_destroy(dg_ctx* c) {
    if (!c) return;
    if (c->device == DG_DEVICE_NONE) { delete c; return; }
    cudaSetDevice(c->device);
    cudaStreamSynchronize(c->stream);
    cudaStreamSynchronize(c->stream2);
    c->dev.clear();
    c->pin.clear();
    cudaEventDestroy(c->ev_fork);
    cudaEventDestroy(c->ev_join);
    for (int i = 0; i < 2; ++i) {
        cudaStreamSynchronize(c->aux[i]);
        cudaEventDestroy(c->ev_aux_go[i]);
        cudaEventDestroy(c->ev_aux_done[i]);
        cudaStreamDestroy(c->aux[i]);
    }
    cudaStreamDestroy(c->stream2);
    if (c->own_stream) cudaStreamDestroy(c->stream);
    delete c;
}

extern "C" void* dg_ctx_stream(dg_ctx* c) { return c ? (void*)c->stream : nullptr; }

extern "C" int dg_ctx_get_counters(dg_ctx* c, dg_ctx_counters* out) {
    if (!c || !out) return fail(DG_E_INVALID, "NULL argument");
    std::lock_guard<std::mutex> lock(c->mu);
    *out = c->counters;
    return DG_OK;
}

// ---------------------------------------------------------------------------------------------------------------
// host-only entry points
// ---------------------------------------------------------------------------------------------------------------
extern "C" int dg_size_list(const dg_image_config* cfg, int max_n, uint32_t* w, uint32_t* h) {
    if (!cfg || !config_valid(*cfg)) return 0;
    auto l = image_size_list(*cfg);
    for (int i = 0; i < (int)l.size() && i < max_n; ++i) { w[i] = l[i].first; h[i] = l[i].second; }
    return (int)l.size();
}

extern "C" int dg_bucket_table(const dg_ctx* c, int max_n, uint32_t* w, uint32_t* h, double* ar, char* keys) {
    if (!c || !c->has_tfm) return 0;
    const auto& b = c->tfm.buckets;
    for (int i = 0; i < (int)b.size() && i < max_n; ++i) {
        if (w) w[i] = b[i].w;
        if (h) h[i] = b[i].h;
        if (ar) ar[i] = b[i].ar;
        if (keys) memcpy(keys + 16 * i, b[i].key, 16);
    }
    return (int)b.size();
}

extern "C" int dg_closest_aspect_ratio(const dg_ctx* c, int32_t w, int32_t h, char key_out[16]) {
    if (!c || !key_out) return fail(DG_E_INVALID, "NULL argument");
    if (!c->has_tfm) return fail(DG_E_NO_TRANSFORM, "ctx has no crop_and_resize transform");
    memcpy(key_out, c->tfm.buckets[c->tfm.closest(w, h)].key, 16);
    return DG_OK;
}

extern "C" void dg_aspect_ratio_to_str(uint32_t w, uint32_t h, char key_out[16]) { format_key(w, h, key_out); }

extern "C" int dg_plan_geometry(const dg_ctx* c, uint32_t w, uint32_t h, uint32_t channels, const char* forced_key, dg_plan* out) {
    if (!c || !out || w == 0 || h == 0) return fail(DG_E_INVALID, "NULL argument or empty image");
    if (!c->has_tfm) return fail(DG_E_NO_TRANSFORM, "ctx has no crop_and_resize transform");
    int rc = plan_geometry(c->tfm, w, h, channels, forced_key, out);
    if (rc) return fail(rc, "aspect ratio key '%s' is not in the bucket table", forced_key ? forced_key : "");
    return DG_OK;
}

extern "C" int dg_jpeg_probe(const uint8_t* data, uint64_t len, dg_jpeg_info* out) {
    if (!data || !out) return fail(DG_E_INVALID, "NULL argument");
    JpegHeader h;
    int rc = parse_jpeg_header(data, len, h);
    if (rc) return fail(rc, "JPEG header rejected (status %d)", rc);
    out->width = h.width; out->height = h.height; out->channels = h.ncomp == 1 ? 1 : 3;
    out->hsamp = h.hs; out->vsamp = h.vs; out->mcux = h.mcux; out->mcuy = h.mcuy; out->restart_interval = h.restart;
    out->scan_offset = h.scan_off; out->scan_len = h.scan_len;
    return DG_OK;
}

extern "C" int dg_rank_slice(uint64_t quorum, uint64_t rank, uint64_t world, uint64_t* start, uint64_t* end) {
    if (world == 0 || rank >= world || !start || !end) return fail(DG_E_INVALID, "rank must be less than world size");
    const uint64_t chunk = quorum / world, rem = quorum % world;
    *start = rank < rem ? rank * (chunk + 1) : rem * (chunk + 1) + (rank - rem) * chunk;
    *end = rank + 1 <= rem ? (rank + 1) * (chunk + 1) : rem * (chunk + 1) + (rank + 1 - rem) * chunk;
    return DG_OK;
}

extern "C" uint64_t dg_key_hash(const char* key, uint64_t len) { return siphash13_str(key, len); }
extern "C" uint64_t dg_key_rank(const char* key, uint64_t len, uint64_t world) { return world ? siphash13_str(key, len) % world : 0; }

// ---------------------------------------------------------------------------------------------------------------
// batch planning
// ---------------------------------------------------------------------------------------------------------------
namespace {

// Appends arrays to one host image of the batch's device metadata; offsets become device pointers after upload.
struct Meta {
    std::vector<uint8_t> bytes;
    size_t put(const void* src, size_t n, size_t align = 16) {
        size_t off = align_up(bytes.size(), align);
        bytes.resize(off + n);
        if (n) memcpy(bytes.data() + off, src, n);
        return off;
    }
    template <typename T> size_t put(const std::vector<T>& v, size_t align = 16) { return put(v.data(), v.size() * sizeof(T), align); }
};

struct OwnerMapOff {  // OwnerMap with meta offsets instead of pointers
    size_t first = 0, coarse = 0;
    uint32_t n = 0, shift = 6, total = 0;
};

OwnerMapOff put_owner_map(Meta& m, const std::vector<uint32_t>& first /* n + 1 */) {
    OwnerMapOff o;
    o.n = (uint32_t)first.size() - 1;
    o.total = first.back();
    o.shift = 6;
    std::vector<uint32_t> coarse((o.total >> o.shift) + 1, 0);
    uint32_t owner = 0;
    for (size_t k = 0; k < coarse.size(); ++k) {
        const uint32_t idx = (uint32_t)k << o.shift;
        while (owner + 1 < o.n && first[owner + 1] <= idx) ++owner;
        coarse[k] = owner;
    }
    o.first = m.put(first);
    o.coarse = m.put(coarse);
    return o;
}

struct ItemPlan {
    int status = DG_OK;
    bool is_jpeg = false, transform = false;
    uint32_t w = 0, h = 0, c = 0;  // decoded / raw size
    dg_plan plan{};
    uint32_t out_w = 0, out_h = 0;
    size_t out_off = 0, out_bytes = 0;  // in the output arena
    bool to_rgb = false;                // convert_to_rgb8 follows the pipeline: it writes c channels at pipe_off,
    uint32_t c_out = 0;                 // the conversion writes the c_out = 3 channel payload at out_off
    size_t pipe_off = 0;                // where decode / resize / copy put their result (== out_off unless to_rgb)
    size_t raw_in_off = 0;              // raw pixel inputs: offset in the input arena
    uint32_t src_pitch = 0;             // bytes per row of the image a resize reads (raw input or decoded JPEG): rows are
                                        // padded to 16 bytes when a resize follows, tight otherwise
    JpegHeader* hdr = nullptr;
    int wave = -1, wave_local = -1;     // JPEG index inside its wave
    size_t coef_off_blocks = 0, decoded_off = 0;
    uint32_t nblocks = 0;
};

struct WavePlan {
    int first_item = 0, last_item = 0;  // [first, last)
    std::vector<JpegDesc> descs;
    std::vector<uint32_t> spec_list, restart_list, restart_first, block_first, color_first;
    std::vector<std::array<uint32_t, 4>> groups;  // (first block, block count, first colour tile, tile count) per L2 group
    // descs [fused_first, descs.size()) take the fused 4:2:0 path: prefix sums of their chroma blocks and tiles, and
    // their own launch groups (first chroma block, count, first tile, count)
    uint32_t fused_first = 0;
    uint32_t n_huge = 0;  // leading entries of spec_list (sorted longest first) with more than kSpecHugeBytes of entropy-coded data
    std::vector<uint32_t> fchroma_first, ftile_first;
    std::vector<std::array<uint32_t, 4>> fgroups;
    std::vector<ConvPass> passes[4];    // H1, V1, H2, V2
    std::vector<uint32_t> pass_first[4];
    uint32_t mma_tiles[4] = {0, 0, 0, 0};  // tiles of the passes that take the tensor-core kernel; those passes come first
    std::vector<CopyJob> copies;
    std::vector<uint32_t> copy_first;
    std::vector<ToRgbJob> torgb;
    std::vector<uint32_t> torgb_first;
    // alpha images: multiply before / divide after each of the two resizes (0: before H1, 1: after V1, 2: before H2, 3: after V2)
    std::vector<AlphaJob> alpha[4];
    std::vector<uint32_t> alpha_first[4];
    // scratch layout (bytes from the wave scratch base)
    size_t us_bytes = 0, coef_blocks = 0, plane_bytes = 0, decoded_bytes = 0, mid_bytes = 0, nseg = 0;
    size_t off_us = 0, off_uslen = 0, off_segstart = 0, off_segfound = 0, off_coef = 0, off_planes = 0, off_decoded = 0, off_mid = 0, total = 0;
    // meta offsets
    size_t m_descs = 0, m_spec = 0, m_restart_list = 0, m_passes[4] = {0, 0, 0, 0}, m_copies = 0, m_torgbs = 0, m_alphas[4] = {0, 0, 0, 0};
    OwnerMapOff m_restart, m_blocks, m_color, m_fchroma, m_ftile, m_pass[4], m_copy, m_torgb, m_alpha[4];
};

struct StageEvent { int stage; cudaEvent_t a, b; };

// One same-shape group of a DG_BATCH_COLLATE batch: its payloads sit back to back, i.e. they are one [n, h, w, c] array.
struct BucketPlan {
    char key[16] = {0};
    uint32_t w = 0, h = 0, c = 0;
    size_t off = 0;  // in the output arena
    std::vector<int32_t> items;
};

}  // namespace

struct dg_batch {
    dg_ctx* ctx = nullptr;
    uint32_t flags = 0;
    int n = 0;
    std::vector<ItemPlan> items;
    std::vector<JpegHeader> headers;
    std::vector<WavePlan> waves;
    std::vector<BucketPlan> buckets;
    Meta meta;
    // persistent device block: [meta | status | blob | raw inputs | outputs]
    int blk_persist = -1, blk_scratch = -1, blk_scratch2 = -1, blk_pin = -1, blk_pin_status = -1;
    uint8_t* d_persist = nullptr;
    uint8_t* d_scratch = nullptr;   // scratch of the even waves
    uint8_t* d_scratch2 = nullptr;  // scratch of the odd waves (same block when the batch has one wave)
    uint8_t* h_pin = nullptr;       // pinned image of [meta | status zeros | blob]
    uint32_t* h_status = nullptr;   // pinned, n words
    size_t off_meta = 0, off_status = 0, off_blob = 0, off_rawin = 0, off_out = 0, persist_bytes = 0;
    size_t blob_bytes = 0, rawin_bytes = 0, out_bytes = 0, pin_bytes = 0;
    size_t arena_bytes = 0;  // out_bytes plus the pre-conversion images of DG_ITEM_TO_RGB8 items (never downloaded)
    uint32_t n_huff = 0;
    size_t m_huff = 0, m_qt = 0, m_tables = 0, meta_total = 0;  // meta_total: meta.bytes plus the filter tables behind it
    std::vector<const uint8_t*> raw_src;  // caller memory of raw items (used inside dg_batch_create only)
    uint64_t h2d = 0, d2h = 0;
    uint32_t launches = 0;
    bool uploaded = false, ran = false;
    bool counted = false;    // its items have been added to the context's counters
    bool used_hmma = false;  // a pass of this batch ran on the tensor-core resize kernel, whose waits are bounded
    std::vector<StageEvent> events;
    float stage_ms[DG_STAGE_COUNT] = {0};
};

namespace {

struct Planner {
    dg_ctx* ctx;
    dg_batch* b;
    bool final_round = true;   // device addresses are final: tensor maps are encoded (the sizing round skips them)
    std::atomic<bool> tmap_failed{false};  // a tensor map could not be encoded (items are planned on several threads)
    std::unordered_map<std::string, uint32_t> huff_ids, qt_ids;
    std::vector<HuffTable> huff_pool;
    std::vector<uint32_t> qt_pool;  // 32 words per table, the layout JpegWave::qt32 documents
    std::map<std::array<uint64_t, 4>, std::pair<size_t, const FilterTable*>> table_ids;  // key -> (word offset, table)
    std::vector<std::shared_ptr<const FilterTable>> tables;  // keeps the batch's tables alive whatever the ctx cache does
    // Tables of the batch in pool order: (word offset, table).  The pool itself is never materialised on the host heap:
    // dg_batch_create packs every table straight into the page-locked staging buffer (tens of MB per batch, and a fresh
    // heap block of that size costs more in page faults than the copy).
    size_t table_words_total = 0;
    std::vector<std::pair<size_t, const FilterTable*>> table_list;
    void pack_tables(uint32_t* dst) const { for (const auto& e : table_list) e.second->pack(dst + e.first); }


    // Most batches repeat a handful of tables (every libjpeg-encoded file carries the same four Huffman tables), so the
    // tables seen last are compared byte-wise before anything is hashed.
    std::vector<std::pair<const JpegHeader::RawHuff*, uint32_t>> recent_huff;
    std::vector<std::pair<const uint16_t*, uint32_t>> recent_qt;
    template <typename P> static void remember(std::vector<std::pair<P, uint32_t>>& v, P p, uint32_t id) {
        if (v.size() >= 8) v.pop_back();
        v.insert(v.begin(), std::make_pair(p, id));
    }

    int huff_id(const JpegHeader::RawHuff& raw, uint32_t* id) {
        for (const auto& r : recent_huff)
            if (r.first->count == raw.count && memcmp(r.first->bits, raw.bits, 17) == 0 && memcmp(r.first->vals, raw.vals, (size_t)std::max(raw.count, 0)) == 0) { *id = r.second; return DG_OK; }
        const int rc = huff_id_slow(raw, id);
        if (!rc) remember(recent_huff, &raw, *id);
        return rc;
    }
    int huff_id_slow(const JpegHeader::RawHuff& raw, uint32_t* id) {
        std::string key((const char*)raw.bits, 17);
        key.append((const char*)raw.vals, 256);
        auto it = huff_ids.find(key);
        if (it != huff_ids.end()) { *id = it->second; return DG_OK; }
        HuffTable t;
        if (!build_huff_table(raw, t)) return DG_E_BAD_TABLE;
        *id = (uint32_t)huff_pool.size();
        huff_pool.push_back(t);
        huff_ids.emplace(std::move(key), *id);
        return DG_OK;
    }
    uint32_t qt_id(const uint16_t* q) {
        for (const auto& r : recent_qt)
            if (memcmp(r.first, q, 128) == 0) return r.second;
        const uint32_t id = qt_id_slow(q);
        remember(recent_qt, q, id);
        return id;
    }
    uint32_t qt_id_slow(const uint16_t* q) {
        std::string key((const char*)q, 128);
        auto it = qt_ids.find(key);
        if (it != qt_ids.end()) return it->second;
        uint32_t id = (uint32_t)(qt_pool.size() / 32);
        for (int i = 0; i < 32; ++i) qt_pool.push_back((uint32_t)q[2 * i] | ((uint32_t)q[2 * i + 1] << 24));
        qt_ids.emplace(std::move(key), id);
        return id;
    }
    static std::array<uint64_t, 4> table_key(int in_size, double in0, double in1, int out_size) {
        std::array<uint64_t, 4> key;
        key[0] = (uint64_t)in_size << 32 | (uint32_t)out_size;
        memcpy(&key[1], &in0, 8);
        memcpy(&key[2], &in1, 8);
        key[3] = 0;
        return key;
    }
    std::shared_ptr<const FilterTable> cached(const std::array<uint64_t, 4>& key) const {
        auto it = ctx->table_cache.find(key);
        return it == ctx->table_cache.end() ? nullptr : it->second;
    }
    void remember_in_ctx(const std::array<uint64_t, 4>& key, const std::shared_ptr<const FilterTable>& t) {
        const size_t bytes = t->words() * 4 + 4 * (t->start.size() + t->size.size()) + 2 * t->k.size();
        if (ctx->table_cache_bytes + bytes > ctx->table_cache_cap) { ctx->table_cache.clear(); ctx->table_cache_bytes = 0; }
        if (ctx->table_cache.emplace(key, t).second) ctx->table_cache_bytes += bytes;
    }
    void adopt(const std::array<uint64_t, 4>& key, std::shared_ptr<const FilterTable> t) {
        tables.push_back(t);
        const size_t off = align_up(table_words_total, 4);
        table_words_total = off + t->words();
        table_list.emplace_back(off, t.get());
        table_ids.emplace(key, std::make_pair(off, t.get()));
    }
    // returns the table and its word offset in the pool
    const FilterTable* table(int in_size, double in0, double in1, int out_size, size_t* word_off) {
        const auto key = table_key(in_size, in0, in1, out_size);
        auto it = table_ids.find(key);
        if (it == table_ids.end()) {
            std::shared_ptr<const FilterTable> t = cached(key);
            if (!t) {
                t = std::make_shared<const FilterTable>(make_filter_table(in_size, in0, in1, out_size));
                remember_in_ctx(key, t);
            }
            adopt(key, t);
            it = table_ids.find(key);
        }
        *word_off = it->second.first;
        return it->second.second;
    }
    // Builds the filter tables a set of plans will ask for on all host cores (the weights cost a sin() each).
    void prebuild_tables(const std::vector<const dg_plan*>& plans) {
        struct Req { std::array<uint64_t, 4> key; int in_size; double in0, in1; int out_size; std::shared_ptr<const FilterTable> t; };
        std::vector<Req> reqs;
        std::map<std::array<uint64_t, 4>, int> seen;
        auto want = [&](int in_size, double in0, double in1, int out_size) {
            const auto key = table_key(in_size, in0, in1, out_size);
            if (table_ids.count(key) || seen.count(key)) return;
            seen[key] = 1;
            if (auto t = cached(key)) { adopt(key, t); return; }
            reqs.push_back(Req{key, in_size, in0, in1, out_size, nullptr});
        };
        for (const dg_plan* pp : plans) {
            const dg_plan& p = *pp;
            if (p.identity) continue;
            if (p.new_w != p.src_w) want((int)p.src_w, 0.0, (double)p.src_w, (int)p.new_w);
            if (p.new_h != p.src_h) want((int)p.src_h, 0.0, (double)p.src_h, (int)p.new_h);
            if ((double)p.target_w != p.crop_w || p.crop_left != std::round(p.crop_left))
                want((int)p.new_w, p.crop_left, p.crop_left + p.crop_w, (int)p.target_w);
            if ((double)p.target_h != p.crop_h || p.crop_top != std::round(p.crop_top))
                want((int)p.new_h, p.crop_top, p.crop_top + p.crop_h, (int)p.target_h);
        }
        if (reqs.empty()) return;
        HostPool::get().run(reqs.size(), [&](size_t i) {
            reqs[i].t = std::make_shared<const FilterTable>(make_filter_table(reqs[i].in_size, reqs[i].in0, reqs[i].in1, reqs[i].out_size));
        }, 2);
        for (Req& r : reqs) { remember_in_ctx(r.key, r.t); adopt(r.key, r.t); }
    }
};

// One image's chain of convolution passes (see kernels_resize.cu).  Buffers are described by byte offsets first and
// turned into pointers when the device blocks are known.
struct PassDraft {
    int stage;  // 0 H1, 1 V1, 2 H2, 3 V2
    size_t tab_off;
    const FilterTable* tab;
    uint32_t t0, count;       // outputs along the filtered axis
    uint32_t other;           // extent along the other axis
    // resolved when chaining
};

}  // namespace

// Whether the tensor-core horizontal pass can take outputs [t0, t0 + out_w) of table T: the source bytes under every
// 8-byte output tile and under every 64-byte strip must fit what a CTA stages (see conv_h_mma in kernels_resize.cu).
static bool hmma_fits(const FilterTable& T, uint32_t t0, uint32_t out_w, uint32_t C, int32_t origin, uint32_t* box_pieces) {
    const uint32_t row_bytes = out_w * C;
    auto lo = [&](uint32_t j) { return ((T.start[t0 + j / C] - origin) * (int32_t)C) & ~15; };
    auto hi = [&](uint32_t j) { const uint32_t x = std::min(out_w - 1, j / C); return (T.start[t0 + x] + T.size[t0 + x] - origin) * (int32_t)C; };
    for (uint32_t j = 0; j < row_bytes; j += 8)
        if (hi(j + 7) - lo(j) > (int32_t)kHMmaMaxBand) return false;
    int32_t widest = 0;
    for (uint32_t j = 0; j < row_bytes; j += kHMmaStrip) {
        if (lo(j) < 0) return false;  // the copy's first coordinate
        widest = std::max(widest, hi(j + kHMmaStrip - 1) - lo(j));
    }
    if (widest > (int32_t)kHMmaMaxSpan) return false;
    *box_pieces = ((uint32_t)(widest + 15) / 16) | 1u;  // odd: the staged rows then start in different shared-memory banks
    return true;
}

// The source of a tensor-core horizontal pass as rows of 32-bit words: `rows` rows of `pitch` bytes from `src` (16-byte
// aligned, pitch a multiple of 16); one copy brings box_pieces * 16 bytes of 32 consecutive rows.  Words and rows outside
// the array read as zero (the kernel multiplies them by zero weights or never stores their results).
static bool encode_source_map(ConvPass& cp) {
    static_assert(sizeof(CUtensorMap) == sizeof(cp.tmap), "tensor map size");
    const EncodeTiledFn fn = encode_tiled_fn();
    if (!fn) return false;
    const cuuint64_t gdim[2] = {cp.src_pitch / 4, cp.out_h};
    const cuuint64_t gstride[1] = {cp.src_pitch};
    const cuuint32_t box[2] = {cp.box_pieces * 4, 32};
    const cuuint32_t estride[2] = {1, 1};
    CUtensorMap m;
    const CUresult r = fn(&m, CU_TENSOR_MAP_DATA_TYPE_UINT32, 2, const_cast<uint8_t*>(cp.src), gdim, gstride, box, estride,
                          CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                          CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return false;
    memcpy(cp.tmap, &m, sizeof m);
    return true;
}

// Whether the tensor-core vertical pass can take output rows [t0, t0 + out_h) of table T: the source rows under the eight
// output rows of a warp and under the 64 of a CTA must fit what a CTA stages (see k_conv_v_mma in kernels_resize.cu).
// box: rows of a tensor-map box | boxes per chunk << 16; src_rows: source rows the pass reads, from row 0 of its source.
static bool vmma_fits(const FilterTable& T, uint32_t t0, uint32_t out_h, int32_t origin, uint32_t* box, uint32_t* src_rows) {
    int32_t tallest = 0, last = 0;
    for (uint32_t y0 = 0; y0 < out_h; y0 += kVMmaRows) {
        const uint32_t y1 = std::min(out_h, y0 + kVMmaRows) - 1;
        const int32_t lo = T.start[t0 + y0] - origin;
        if (lo < 0) return false;
        int32_t hi = lo;
        for (uint32_t y = y0; y <= y1; ++y) {
            if (T.start[t0 + y] < T.start[t0 + y0]) return false;  // the windows move down with the output rows
            hi = std::max(hi, T.start[t0 + y] + T.size[t0 + y] - origin);
        }
        tallest = std::max(tallest, hi - lo);
        last = std::max(last, hi);
        for (uint32_t yw = y0; yw <= y1; yw += 8) {
            const uint32_t yl = std::min(y1, yw + 7);
            int32_t bhi = 0;
            for (uint32_t y = yw; y <= yl; ++y) {
                if (T.start[t0 + y] < T.start[t0 + yw]) return false;
                bhi = std::max(bhi, T.start[t0 + y] + T.size[t0 + y]);
            }
            // the kernel takes the band's end from the warp's last row
            if (bhi != T.start[t0 + yl] + T.size[t0 + yl] || bhi - T.start[t0 + yw] > (int32_t)kVMmaMaxBand) return false;
        }
    }
    if (tallest <= 0 || tallest > (int32_t)kVMmaMaxSpan) return false;
    const uint32_t boxes = ((uint32_t)tallest + 255) / 256;
    const uint32_t rows = (uint32_t)align_up(((size_t)tallest + boxes - 1) / boxes, 8);
    *box = rows | boxes << 16;
    *src_rows = (uint32_t)last;
    return true;
}

// The source of a tensor-core vertical pass as rows of bytes: one copy brings 64 bytes of `box rows` consecutive rows, laid
// out with the 64-byte swizzle.  Bytes and rows outside the array read as zero.
static bool encode_source_map_v(ConvPass& cp, uint32_t src_rows) {
    const EncodeTiledFn fn = encode_tiled_fn();
    if (!fn) return false;
    const cuuint64_t gdim[2] = {cp.src_pitch, src_rows};
    const cuuint64_t gstride[1] = {cp.src_pitch};
    const cuuint32_t box[2] = {64, cp.box_pieces & 0xFFFFu};
    const cuuint32_t estride[2] = {1, 1};
    CUtensorMap m;
    const CUresult r = fn(&m, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<uint8_t*>(cp.src), gdim, gstride, box, estride,
                          CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_64B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                          CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return false;
    memcpy(cp.tmap, &m, sizeof m);
    return true;
}

// Plans the resize of one image: appends passes / copy jobs to the wave.  src: device pointer of the source image
// (tight pitch), dst: device pointer of the payload (tight pitch), mid: scratch for intermediates.
// caller_owned_src: the source is memory of the caller with nothing guaranteed around it (the batch path's sources sit
// in padded arenas of the library): the pass that reads it is then planned so that no load leaves the image's bytes.
static void plan_resize(Planner& pl, WavePlan& wv, const dg_plan& p, uint32_t C, const uint8_t* src, uint32_t src_pitch, uint8_t* dst,
                        uint8_t* mid_base, size_t* mid_used, bool caller_owned_src = false) {
    const uint32_t w = p.src_w, h = p.src_h, tw = p.target_w, th = p.target_h;
    auto add_copy = [&](const uint8_t* s, uint32_t pitch, uint32_t row_bytes, uint32_t rows) {
        CopyJob j;
        j.src = s; j.dst = dst; j.src_pitch = pitch; j.row_bytes = row_bytes; j.rows = rows; j.tile_first = 0;
        wv.copies.push_back(j);
    };
    if (p.identity) { add_copy(src, src_pitch, w * C, h); return; }
    const bool h1 = p.new_w != w, v1 = p.new_h != h;
    const bool h2 = (double)tw != p.crop_w || p.crop_left != std::round(p.crop_left);
    const bool v2 = (double)th != p.crop_h || p.crop_top != std::round(p.crop_top);
    size_t o_h1 = 0, o_v1 = 0, o_h2 = 0, o_v2 = 0;
    const FilterTable* T_h1 = h1 ? pl.table((int)w, 0.0, (double)w, (int)p.new_w, &o_h1) : nullptr;
    const FilterTable* T_v1 = v1 ? pl.table((int)h, 0.0, (double)h, (int)p.new_h, &o_v1) : nullptr;
    const FilterTable* T_h2 = h2 ? pl.table((int)p.new_w, p.crop_left, p.crop_left + p.crop_w, (int)tw, &o_h2) : nullptr;
    const FilterTable* T_v2 = v2 ? pl.table((int)p.new_h, p.crop_top, p.crop_top + p.crop_h, (int)th, &o_v2) : nullptr;
    // region of the resized (new_w x new_h) image that the crop step reads
    int ca, cb, ra, rb;
    if (h2) { ca = T_h2->first_in(); cb = T_h2->last_in(0, (int)tw); } else { ca = (int)p.crop_left; cb = ca + (int)tw; }
    if (v2) { ra = T_v2->first_in(); rb = T_v2->last_in(0, (int)th); } else { ra = (int)p.crop_top; rb = ra + (int)th; }
    // rows of the horizontally resized image that the vertical pass reads
    int ma, mb;
    if (v1) { ma = T_v1->start[ra]; mb = T_v1->last_in(ra, rb); } else { ma = ra; mb = rb; }

    struct Buf { const uint8_t* ptr; uint32_t pitch; int col0, row0; };  // origin in the current coordinate system
    Buf cur{src, src_pitch, 0, 0};
    const int n_pass = (int)h1 + (int)v1 + (int)h2 + (int)v2;
    int done = 0;
    // Images with an alpha channel: fast_image_resize multiplies the colour channels by alpha before each convolution
    // resize and divides afterwards (a resize that only copies touches no value).  The multiplied copy of a source that
    // must stay intact (the batch's input) goes to the scratch area; otherwise both steps work in place.
    const bool alpha = C == 2 || C == 4;
    auto add_alpha = [&](int slot, const uint8_t* s, uint32_t spitch, uint8_t* d, uint32_t dpitch, uint32_t width, uint32_t rows, bool divide) {
        AlphaJob j;
        memset(&j, 0, sizeof j);
        j.src = s; j.dst = d; j.src_pitch = spitch; j.dst_pitch = dpitch; j.width = width; j.rows = rows; j.channels = C; j.divide = divide ? 1 : 0;
        wv.alpha[slot].push_back(j);
    };
    auto premultiplied_copy = [&](int slot) {  // of the whole source image
        const uint32_t pitch = (uint32_t)align_up((size_t)w * C, 16);
        uint8_t* pm = mid_base + *mid_used;
        *mid_used += align_up((size_t)pitch * h, 256);
        add_alpha(slot, src, src_pitch, pm, pitch, w, h, false);
        cur = Buf{pm, pitch, 0, 0};
    };
    if (alpha && (h1 || v1)) premultiplied_copy(0);
    auto next_dst = [&](uint32_t out_w, uint32_t out_h, uint32_t* pitch) -> uint8_t* {
        if (done + 1 == n_pass) { *pitch = tw * C; return dst; }
        *pitch = (uint32_t)align_up((size_t)out_w * C, 16);
        uint8_t* ptr = mid_base + *mid_used;
        *mid_used += align_up((size_t)*pitch * out_h, 256);
        return ptr;
    };
    auto emit = [&](int stage, bool horizontal, const FilterTable* T, size_t tab_off, uint32_t t0, uint32_t out_w, uint32_t out_h,
                    const uint8_t* s, int32_t origin, uint32_t spitch, uint8_t* d, uint32_t dpitch) {
        ConvPass cp;
        memset(&cp, 0, sizeof cp);
        cp.src = s; cp.dst = d; cp.src_pitch = spitch; cp.dst_pitch = dpitch; cp.out_w = out_w; cp.out_h = out_h;
        cp.channels = C; cp.src_origin = origin; cp.t0 = t0; cp.tab_n = (uint32_t)T->n; cp.window = (uint32_t)T->window;
        cp.precision = (uint32_t)T->precision; cp.tab_off = tab_off;
        const bool guarded = caller_owned_src && s >= src && s < src + (size_t)src_pitch * h;
        if (horizontal) {
            cp.fast = 1;
            if (guarded) { cp.guard_lo = src; cp.guard_hi = src + (size_t)w * h * C; }
            else if (pl.ctx->hmma && (((uintptr_t)s | spitch) & 15) == 0 && hmma_fits(*T, t0, out_w, C, origin, &cp.box_pieces)) {
                cp.fast = 2;
                if (pl.final_round && !encode_source_map(cp)) pl.tmap_failed = true;
            }
        } else {
            const uintptr_t bits = (uintptr_t)s | (uintptr_t)d | spitch | dpitch;
            cp.fast = (bits & 15) == 0 && (uint32_t)T->window <= kVFastMaxWindow && (size_t)align_up((size_t)out_w * C, 16) <= spitch &&
                      (size_t)align_up((size_t)out_w * C, 16) <= dpitch;
            // the vector path reads whole 16-byte chunks: in caller memory they must end inside the row they start in
            if (guarded && (size_t)(s - src) % spitch + align_up((size_t)out_w * C, 16) > spitch) cp.fast = 0;
            uint32_t src_rows = 0;
            if (cp.fast && !guarded && pl.ctx->hmma && vmma_fits(*T, t0, out_h, origin, &cp.box_pieces, &src_rows)) {
                cp.fast = 2;
                if (pl.final_round && !encode_source_map_v(cp, src_rows)) pl.tmap_failed = true;
            }
        }
        cp.tiles_x = conv_tiles_x(cp, !horizontal);
        wv.passes[stage].push_back(cp);
        ++done;
    };
    if (h1) {  // source rows [ma, mb) -> columns [ca, cb)
        uint32_t pitch;
        const uint32_t ow = (uint32_t)(cb - ca), oh = (uint32_t)(mb - ma);
        uint8_t* d = next_dst(ow, oh, &pitch);
        emit(0, true, T_h1, o_h1, (uint32_t)ca, ow, oh, cur.ptr + (size_t)(ma - cur.row0) * cur.pitch, cur.col0, cur.pitch, d, pitch);
        cur = Buf{d, pitch, ca, ma};
    }
    if (v1) {  // rows [ma, mb) -> rows [ra, rb), columns [ca, cb)
        uint32_t pitch;
        const uint32_t ow = (uint32_t)(cb - ca), oh = (uint32_t)(rb - ra);
        uint8_t* d = next_dst(ow, oh, &pitch);
        emit(1, false, T_v1, o_v1, (uint32_t)ra, ow, oh, cur.ptr + (size_t)(ca - cur.col0) * C, cur.row0, cur.pitch, d, pitch);
        cur = Buf{d, pitch, ca, ra};
    }
    if (alpha && (h1 || v1)) {  // the first resize is complete: divide its result (region [ca, cb) x [ra, rb)) in place
        uint8_t* region = const_cast<uint8_t*>(cur.ptr) + (size_t)(ra - cur.row0) * cur.pitch + (size_t)(ca - cur.col0) * C;
        add_alpha(1, region, cur.pitch, region, cur.pitch, (uint32_t)(cb - ca), (uint32_t)(rb - ra), true);
    }
    if (alpha && (h2 || v2)) {  // the second resize multiplies again
        if (cur.ptr == src) premultiplied_copy(2);
        else {
            uint8_t* region = const_cast<uint8_t*>(cur.ptr) + (size_t)(ra - cur.row0) * cur.pitch + (size_t)(ca - cur.col0) * C;
            add_alpha(2, region, cur.pitch, region, cur.pitch, (uint32_t)(cb - ca), (uint32_t)(rb - ra), false);
        }
    }
    if (h2) {  // columns [ca, cb) -> output columns [0, tw), rows [ra, rb)
        uint32_t pitch;
        const uint32_t oh = (uint32_t)(rb - ra);
        uint8_t* d = next_dst(tw, oh, &pitch);
        emit(2, true, T_h2, o_h2, 0, tw, oh, cur.ptr + (size_t)(ra - cur.row0) * cur.pitch, cur.col0, cur.pitch, d, pitch);
        cur = Buf{d, pitch, 0, ra};
        ca = 0;
    }
    if (v2) {  // rows [ra, rb) -> output rows [0, th)
        uint32_t pitch;
        uint8_t* d = next_dst(tw, th, &pitch);
        emit(3, false, T_v2, o_v2, 0, tw, th, cur.ptr + (size_t)(ca - cur.col0) * C, cur.row0, cur.pitch, d, pitch);
        cur = Buf{d, pitch, 0, 0};
    }
    if (alpha && (h2 || v2)) add_alpha(3, dst, tw * C, dst, tw * C, tw, th, true);
    if (n_pass == 0)  // same scale, integral crop: a strided copy
        add_copy(src + (size_t)ra * src_pitch + (size_t)ca * C, src_pitch, tw * C, th);
}

// worst-case scratch of the intermediates of one image's resize
static size_t resize_mid_bound(const dg_plan& p, uint32_t C) {
    if (p.identity) return 0;
    if (C == 2 || C == 4) {  // plus the pre-multiplied copy of the source
        const size_t pm = align_up(align_up((size_t)p.src_w * C, 16) * p.src_h, 256);
        const size_t a = align_up((size_t)p.new_w * C, 16) * (size_t)(std::max(p.src_h, p.new_h) + 8);
        const size_t b = align_up((size_t)p.new_w * C, 16) * (size_t)(p.new_h + 8);
        return pm + align_up(a, 256) + 2 * align_up(b, 256);
    }
    const size_t a = align_up((size_t)p.new_w * C, 16) * (size_t)(std::max(p.src_h, p.new_h) + 8);
    const size_t b = align_up((size_t)p.new_w * C, 16) * (size_t)(p.new_h + 8);
    return align_up(a, 256) + 2 * align_up(b, 256);
}

// Runs fn(0..n-1) on the process-wide host pool; small counts stay on the calling thread.
template <typename F> static void parallel_items(int n, F&& fn) {
    HostPool::get().run((size_t)std::max(n, 0), [&fn](size_t i) { fn((int)i); }, 64);
}

static int abandon(dg_batch* b, int rc) {
    dg_ctx* ctx = b->ctx;
    ctx->dev.release(b->blk_persist);
    ctx->dev.release(b->blk_scratch);
    ctx->dev.release(b->blk_scratch2);
    ctx->pin.release(b->blk_pin);
    ctx->pin.release(b->blk_pin_status);
    delete b;
    return rc;
}

extern "C" int dg_batch_create(dg_ctx* ctx, const dg_item* items, int n, uint32_t flags, dg_batch** out) {
    if (!ctx || !out || n < 0 || (n > 0 && !items)) return fail(DG_E_INVALID, "NULL argument");
    *out = nullptr;
    if (ctx->device == DG_DEVICE_NONE) return fail(DG_E_INVALID, "planning-only context: pixel work needs a CUDA device (there is no CPU path)");
    std::lock_guard<std::mutex> lock(ctx->mu);
    CU(cudaSetDevice(ctx->device));
    dg_batch* b = new dg_batch();
    b->ctx = ctx; b->flags = flags; b->n = n;
    b->items.resize(n);
    b->headers.resize(n);
    b->raw_src.assign(n, nullptr);
    const bool transform = ctx->has_tfm && !(flags & DG_BATCH_DECODE_ONLY);
    Planner pl{ctx, b};

    // ---- pass 1: headers, geometry, arena layout -----------------------------------------------------------------------
    // Header parsing and geometry are independent per item and run on several host threads for large batches; the arena
    // offsets are then assigned in item order.
    auto inspect = [&](int i) {
        ItemPlan& it = b->items[i];
        const dg_item& src = items[i];
        it.transform = transform;
        if (!src.data) { it.status = DG_E_INVALID; return; }
        const bool want_rgb = (src.flags & DG_ITEM_TO_RGB8) != 0;
        if (src.raw_w) {
            if (src.raw_h == 0 || src.raw_c < 1 || src.raw_c > 4 ||
                src.len < (uint64_t)src.raw_w * src.raw_h * src.raw_c) { it.status = DG_E_INVALID; return; }
            it.w = src.raw_w; it.h = src.raw_h; it.c = src.raw_c;
        } else {
            JpegHeader& h = b->headers[i];
            it.status = parse_jpeg_header(src.data, src.len, h);
            if (it.status) return;
            if (h.scan_len > 0xFFFFFF00ull) { it.status = DG_E_TOO_LARGE; return; }
            // Everything the host can tell about the tables is settled here, before the output arena is laid out, so
            // that an item that fails on them takes no slot of a collated bucket.  (The dequantiser multiplies by one
            // byte: 16-bit quantisation tables are not on this path.)
            for (uint32_t c = 0; c < h.ncomp && c < 3; ++c) {
                for (int k = 0; k < 64; ++k)
                    if (h.qt[h.comp_tq[c]][k] > 255) { it.status = DG_E_UNSUPPORTED; return; }
                if (!huff_lengths_valid(h.dc[h.comp_td[c]]) || !huff_lengths_valid(h.ac[h.comp_ta[c]])) { it.status = DG_E_BAD_TABLE; return; }
            }
            it.is_jpeg = true; it.hdr = &h;
            it.w = h.width; it.h = h.height; it.c = h.ncomp == 1 ? 1 : 3;
        }
        // A header can declare far more pixels than its bytes could ever hold (a forged SOF of 65535 x 65535 plans tens
        // of GB).  datago decodes through the `image` crate, whose default limits refuse such a file and drop that one
        // sample (src/worker_files.rs:14-16, 63-70); here the item alone gets DG_E_TOO_LARGE.
        if ((uint64_t)it.w * it.h * it.c > ctx->max_image_bytes) { it.status = DG_E_TOO_LARGE; return; }
        if (transform) {
            it.status = plan_geometry(ctx->tfm, it.w, it.h, it.c, src.forced_key, &it.plan);
            if (it.status) return;
            it.out_w = it.plan.target_w; it.out_h = it.plan.target_h;
        } else {
            it.out_w = it.w; it.out_h = it.h;
            it.plan.src_w = it.w; it.plan.src_h = it.h; it.plan.channels = it.c;
        }
        it.to_rgb = want_rgb && it.c != 3;
        it.c_out = it.to_rgb ? 3 : it.c;
        it.out_bytes = (size_t)it.out_w * it.out_h * it.c_out;
        it.src_pitch = it.w * it.c;
        if (transform && !it.plan.identity && (it.c == 1 || it.c == 3)) it.src_pitch = (uint32_t)align_up((size_t)it.w * it.c, 16);
    };
    parallel_items(n, inspect);
    size_t blob = 0, rawin = 0, outb = 0;
    for (int i = 0; i < n; ++i) {
        ItemPlan& it = b->items[i];
        if (it.status) continue;
        it.out_off = outb;
        outb += align_up(it.out_bytes, 256);
        if (it.is_jpeg) blob += align_up(b->headers[i].scan_len, 16) + 16;
        else { it.raw_in_off = rawin; rawin += align_up((size_t)it.src_pitch * it.h, 256); b->raw_src[i] = items[i].data; }
    }
    if (flags & DG_BATCH_COLLATE) {
        // Re-lay the output arena bucket by bucket (buckets in order of first appearance, items in batch order):
        // payloads of one bucket are packed without gaps, so the bucket is a dense [n, h, w, c] array on the device.
        for (int i = 0; i < n; ++i) {
            ItemPlan& it = b->items[i];
            if (it.status) continue;
            BucketPlan* bk = nullptr;
            for (BucketPlan& cand : b->buckets)
                if (cand.w == it.out_w && cand.h == it.out_h && cand.c == it.c_out && memcmp(cand.key, it.plan.key, 16) == 0) { bk = &cand; break; }
            if (!bk) {
                b->buckets.emplace_back();
                bk = &b->buckets.back();
                memcpy(bk->key, it.plan.key, 16);
                bk->w = it.out_w; bk->h = it.out_h; bk->c = it.c_out;
            }
            bk->items.push_back(i);
        }
        outb = 0;
        for (BucketPlan& bk : b->buckets) {
            bk.off = outb;
            const size_t each = (size_t)bk.w * bk.h * bk.c;
            for (size_t k = 0; k < bk.items.size(); ++k) b->items[bk.items[k]].out_off = bk.off + k * each;
            outb = align_up(bk.off + bk.items.size() * each, 256);
        }
    }
    b->blob_bytes = blob; b->rawin_bytes = rawin; b->out_bytes = outb;
    // pre-conversion images live behind the payloads, addressed from the same base
    size_t arena = align_up(outb, 256);
    for (ItemPlan& it : b->items) {
        if (it.status) continue;
        it.pipe_off = it.out_off;
        if (it.to_rgb) { it.pipe_off = arena; arena += align_up((size_t)it.out_w * it.out_h * it.c, 256); }
    }
    b->arena_bytes = arena;

    // ---- pass 2: waves ----------------------------------------------------------------------------------------------------
    // Few, large, equally sized waves: large because the entropy kernels fill the GPU only with hundreds of images per
    // launch, at least two (when there is enough work) so that the two streams of dg_batch_run overlap them.
    {
        std::vector<size_t> need_coef(n, 0), need_big(n, 0);
        size_t total_coef = 0, total_big = 0;
        for (int i = 0; i < n; ++i) {
            ItemPlan& it = b->items[i];
            if (it.status) continue;
            if (it.is_jpeg) {
                const JpegHeader& h = *it.hdr;
                it.nblocks = h.mcux * h.mcuy * (h.ncomp == 1 ? 1 : h.hs * h.vs + 2);
                need_coef[i] = (size_t)it.nblocks * 128;
                if (transform) need_big[i] += align_up((size_t)it.src_pitch * it.h, 256);
            }
            if (transform) need_big[i] += resize_mid_bound(it.plan, it.c);
            total_coef += need_coef[i];
            total_big += need_big[i];
        }
        size_t n_waves = std::max<size_t>(1, std::max((total_coef + ctx->wave_bytes - 1) / ctx->wave_bytes,
                                                      (total_big + 2 * ctx->wave_bytes - 1) / (2 * ctx->wave_bytes)));
        if (n_waves == 1 && total_coef + total_big > ((size_t)1 << 30)) n_waves = 2;
        const size_t coef_cap = total_coef / n_waves + 1, big_cap = total_big / n_waves + 1;
        WavePlan* wv = nullptr;
        size_t coef_bytes = 0, big_bytes = 0;
        for (int i = 0; i < n; ++i) {
            ItemPlan& it = b->items[i];
            if (it.status) continue;
            if (!wv || (coef_bytes >= coef_cap && coef_cap > 1) || (big_bytes >= big_cap && big_cap > 1 && total_coef == 0)) {
                b->waves.emplace_back();
                wv = &b->waves.back();
                wv->first_item = i;
                coef_bytes = big_bytes = 0;
            }
            coef_bytes += need_coef[i]; big_bytes += need_big[i];
            it.wave = (int)b->waves.size() - 1;
            wv->last_item = i + 1;
        }
    }

    // ---- pass 3: per-wave scratch layout and JPEG descriptors ------------------------------------------------------
    size_t scratch_max = 0, blob_off = 0;
    for (WavePlan& wv : b->waves) {
        size_t us = 0, planes = 0, decoded = 0, mids = 0, blocks = 0, segs = 0;
        // Descriptors are built in item order, then arranged so that the images of the general path come first and those
        // of the fused 4:2:0 path after them: each class then owns one contiguous range of the coefficient array.
        std::vector<JpegDesc> built;
        std::vector<int> built_item;
        for (int i = wv.first_item; i < wv.last_item; ++i) {
            ItemPlan& it = b->items[i];
            if (it.status || it.wave < 0) continue;
            if (transform) mids += resize_mid_bound(it.plan, it.c);
            if (!it.is_jpeg) continue;
            const JpegHeader& h = *it.hdr;
            JpegDesc d;
            memset(&d, 0, sizeof d);
            for (uint32_t c = 0; c < 3 && !it.status; ++c) {
                const uint32_t cc = c < h.ncomp ? c : 0;
                for (int k = 0; k < 64; ++k)  // the dequantiser multiplies by one byte: 16-bit tables are not on this path
                    if (h.qt[h.comp_tq[cc]][k] > 255) it.status = DG_E_UNSUPPORTED;
                if (it.status) break;
                d.qt[c] = pl.qt_id(h.qt[h.comp_tq[cc]]);
                int rc = pl.huff_id(h.dc[h.comp_td[cc]], &d.dc_tab[c]);
                if (!rc) rc = pl.huff_id(h.ac[h.comp_ta[cc]], &d.ac_tab[c]);
                if (rc) it.status = rc;
            }
            if (it.status) continue;  // nothing has been laid out for this image yet
            d.raw_off = blob_off; d.raw_len = (uint32_t)h.scan_len;
            blob_off += align_up(h.scan_len, 16) + 16;
            d.us_off = us; us += align_up(h.scan_len + 32, 16);
            d.nblocks = it.nblocks;
            d.width = h.width; d.height = h.height; d.mcux = h.mcux; d.mcuy = h.mcuy;
            d.ncomp = h.ncomp; d.hs = h.hs; d.vs = h.vs; d.bpm = h.ncomp == 1 ? 1 : h.hs * h.vs + 2;
            for (uint32_t c = 0; c < 3; ++c) {
                const uint32_t hs = c == 0 ? h.hs : 1, vs = c == 0 ? h.vs : 1;
                d.plane_pitch[c] = h.mcux * hs * 8;
                d.plane_rows[c] = h.mcuy * vs * 8;
            }
            d.restart = h.restart;
            const uint32_t mcus = h.mcux * h.mcuy;
            d.nseg = h.restart ? (mcus + h.restart - 1) / h.restart : 1;
            d.seg_off = (uint32_t)segs; segs += d.nseg;
            d.item = (uint32_t)i;
            if (transform) { d.out_off = decoded; it.decoded_off = decoded; decoded += align_up((size_t)it.src_pitch * it.h, 256); d.out_pitch = it.src_pitch; }
            else { d.out_off = it.pipe_off; d.out_pitch = it.w * it.c; }
            built.push_back(d);
            built_item.push_back(i);
        }
        std::vector<size_t> order;
        for (int pass = 0; pass < 2; ++pass)
            for (size_t k = 0; k < built.size(); ++k)
                if ((int)(ctx->fused_path && fused_decode(built[k].ncomp, built[k].hs, built[k].vs, built[k].width)) == pass) order.push_back(k);
        uint32_t color_total = 0, restart_total = 0, fchroma_total = 0, ftile_total = 0;
        size_t group_bytes = 0, fgroup_bytes = 0;
        wv.block_first.push_back(0);
        wv.color_first.push_back(0);
        wv.groups.push_back({0, 0, 0, 0});
        wv.fchroma_first.push_back(0);
        wv.ftile_first.push_back(0);
        wv.fgroups.push_back({0, 0, 0, 0});
        wv.restart_first.push_back(0);
        wv.fused_first = (uint32_t)built.size();
        for (size_t k : order) {
            JpegDesc d = built[k];
            ItemPlan& it = b->items[built_item[k]];
            const bool fused = ctx->fused_path && fused_decode(d.ncomp, d.hs, d.vs, d.width);
            d.block_off = blocks;
            it.coef_off_blocks = blocks;
            blocks += it.nblocks;
            // the fused path keeps no luma plane
            for (uint32_t c = fused ? 1 : 0; c < d.ncomp; ++c) { d.plane_off[c] = planes; planes += align_up((size_t)d.plane_pitch[c] * d.plane_rows[c], 256); }
            it.wave_local = (int)wv.descs.size();
            if (d.restart) { wv.restart_list.push_back((uint32_t)wv.descs.size()); restart_total += d.nseg; wv.restart_first.push_back(restart_total); }
            else wv.spec_list.push_back((uint32_t)wv.descs.size());
            if (fused && wv.fused_first == (uint32_t)built.size()) wv.fused_first = (uint32_t)wv.descs.size();
            wv.descs.push_back(d);
            // images whose planes fit the L2 budget together share one IDCT launch and one colour launch
            if (!fused) {
                wv.block_first.push_back((uint32_t)blocks);
                const uint32_t ntiles = color_tiles(d.width, d.mcuy);
                color_total += ntiles;
                wv.color_first.push_back(color_total);
                const size_t pbytes = (size_t)it.nblocks * 64;
                if (wv.groups.back()[1] && group_bytes + pbytes > ctx->l2_group_bytes) {
                    wv.groups.push_back({(uint32_t)(blocks - it.nblocks), 0, color_total - ntiles, 0});
                    group_bytes = 0;
                }
                group_bytes += pbytes;
                wv.groups.back()[1] += it.nblocks;
                wv.groups.back()[3] += ntiles;
            } else {
                const uint32_t nchroma = 2 * d.mcux * d.mcuy, ntiles = fused_tiles(d.width, d.mcuy);
                fchroma_total += nchroma;
                ftile_total += ntiles;
                wv.fchroma_first.push_back(fchroma_total);
                wv.ftile_first.push_back(ftile_total);
                const size_t pbytes = (size_t)nchroma * 64;
                if (wv.fgroups.back()[1] && fgroup_bytes + pbytes > ctx->l2_group_bytes) {
                    wv.fgroups.push_back({fchroma_total - nchroma, 0, ftile_total - ntiles, 0});
                    fgroup_bytes = 0;
                }
                fgroup_bytes += pbytes;
                wv.fgroups.back()[1] += nchroma;
                wv.fgroups.back()[3] += ntiles;
            }
        }
        // longest streams first: one CTA decodes one image, and the launch ends with its slowest CTA
        std::stable_sort(wv.spec_list.begin(), wv.spec_list.end(),
                         [&](uint32_t a, uint32_t c) { return wv.descs[a].raw_len > wv.descs[c].raw_len; });
        wv.n_huge = 0;
        // (at most kSpecHugeMax of them: one such CTA fills an SM, so they trade throughput for a shorter critical path)
        while (wv.n_huge < wv.spec_list.size() && wv.n_huge < kSpecHugeMax && wv.descs[wv.spec_list[wv.n_huge]].raw_len > kSpecHugeBytes) ++wv.n_huge;
        wv.us_bytes = us; wv.coef_blocks = blocks; wv.plane_bytes = planes; wv.decoded_bytes = decoded; wv.mid_bytes = mids; wv.nseg = segs;
        size_t o = 0;
        wv.off_coef = o; o += align_up(blocks * 128, 256);  // first: the zero prefix of a scratch block is tracked from offset 0
        wv.off_us = o; o += align_up(us, 256);
        wv.off_uslen = o; o += align_up(wv.descs.size() * 4, 256);
        wv.off_segfound = o; o += align_up(wv.descs.size() * 4, 256);
        wv.off_segstart = o; o += align_up(segs * 4, 256);
        wv.off_planes = o; o += align_up(planes, 256);
        wv.off_decoded = o; o += align_up(decoded, 256);
        wv.off_mid = o; o += align_up(mids, 256);
        wv.total = o;
        scratch_max = std::max(scratch_max, o);
    }

    // ---- device and pinned blocks (addresses are needed by the resize descriptors) ------------------------------------
    // persistent layout: [status | blob | raw inputs | outputs | meta]; meta size is known only after planning the
    // resize passes, so it gets a bound: descriptors + tables are small next to the pixel buffers.
    int rc = ctx->dev.acquire(std::max<size_t>(scratch_max, 256), &b->blk_scratch, true);
    if (rc) return abandon(b, rc);
    b->d_scratch = (uint8_t*)ctx->dev.blocks[b->blk_scratch].ptr;
    b->d_scratch2 = b->d_scratch;
    if (b->waves.size() > 1) {
        rc = ctx->dev.acquire(std::max<size_t>(scratch_max, 256), &b->blk_scratch2, true);
        if (rc) return abandon(b, rc);
        b->d_scratch2 = (uint8_t*)ctx->dev.blocks[b->blk_scratch2].ptr;
    }

    b->off_status = 0;  // n status words, then 4 counters of the speculative Huffman kernel
    b->off_blob = align_up((size_t)n * 4 + 32, 256);
    b->off_rawin = b->off_blob + align_up(blob, 256);
    b->off_out = b->off_rawin + align_up(rawin, 256);
    const size_t fixed_bytes = b->off_out + align_up(b->arena_bytes, 256);

    // Resize descriptors hold device addresses inside the persistent block, whose size depends on the metadata that
    // contains them.  So the passes are planned twice: once against a stand-in base to size the metadata (filter
    // tables are cached, the second round is cheap), once with the real base address.
    if (transform) {
        std::vector<const dg_plan*> plans;
        for (const ItemPlan& it : b->items)
            if (!it.status && it.wave >= 0) plans.push_back(&it.plan);
        pl.prebuild_tables(plans);
    }
    for (int round = 0; round < 2; ++round) {
        uint8_t* baseP = round == 0 ? b->d_scratch : b->d_persist;
        pl.final_round = round == 1;
        for (size_t wi = 0; wi < b->waves.size(); ++wi) {
            WavePlan& wv = b->waves[wi];
            uint8_t* const kBaseS = (wi & 1) ? b->d_scratch2 : b->d_scratch;
            for (int s = 0; s < 4; ++s) { wv.passes[s].clear(); wv.pass_first[s].clear(); }
            wv.copies.clear(); wv.copy_first.clear();
            wv.torgb.clear(); wv.torgb_first.clear();
            for (int a = 0; a < 4; ++a) { wv.alpha[a].clear(); wv.alpha_first[a].clear(); }
            // Every item is planned on its own (the filter tables are all there by now, so the planner is only read):
            // its intermediates get the slice of the wave's scratch that its worst-case bound reserves, and its passes
            // and jobs are appended to the wave's lists in item order afterwards.
            const int n_wave_items = wv.last_item - wv.first_item;
            std::vector<size_t> mid_at((size_t)n_wave_items + 1, 0);
            for (int k = 0; k < n_wave_items; ++k) {
                const ItemPlan& it = b->items[wv.first_item + k];
                mid_at[k + 1] = mid_at[k] + ((transform && !it.status && it.wave >= 0) ? resize_mid_bound(it.plan, it.c) : 0);
            }
            size_t mid_used = mid_at[n_wave_items];
            std::vector<WavePlan> parts((size_t)n_wave_items);
            std::atomic<bool> overflow{false};
            parallel_items(n_wave_items, [&](int k) {
                ItemPlan& it = b->items[wv.first_item + k];
                if (it.status || it.wave < 0) return;
                // encoding a tensor map is a driver call and wants a current context, which the pool's threads do not
                // have by themselves
                static thread_local int bound_device = -1;
                if (bound_device != ctx->device) { if (cudaSetDevice(ctx->device) != cudaSuccess) { pl.tmap_failed = true; return; } bound_device = ctx->device; }
                WavePlan& part = parts[k];
                const uint8_t* src = it.is_jpeg ? kBaseS + wv.off_decoded + it.decoded_off : baseP + b->off_rawin + it.raw_in_off;
                uint8_t* dst = baseP + b->off_out + it.pipe_off;
                const uint8_t* converted_from = dst;
                if (transform) {
                    size_t used = 0;
                    plan_resize(pl, part, it.plan, it.c, src, it.src_pitch, dst, kBaseS + wv.off_mid + mid_at[k], &used);
                    if (used > mid_at[k + 1] - mid_at[k]) overflow = true;
                } else if (!it.is_jpeg) {  // raw pixels, no transform: the payload is the input (JPEGs decode straight into dst)
                    if (it.to_rgb) converted_from = src;  // the conversion reads the input itself
                    else {
                        CopyJob j;
                        j.src = src; j.dst = dst; j.src_pitch = it.w * it.c; j.row_bytes = it.w * it.c; j.rows = it.h; j.tile_first = 0;
                        part.copies.push_back(j);
                    }
                }
                if (it.to_rgb) {
                    ToRgbJob j;
                    j.src = converted_from; j.dst = baseP + b->off_out + it.out_off; j.npx = it.out_w * it.out_h; j.channels = it.c;
                    j.tile_first = 0; j.pad = 0;
                    part.torgb.push_back(j);
                }
            });
            if (overflow) mid_used = wv.mid_bytes + 1;
            for (const WavePlan& part : parts) {
                for (int s = 0; s < 4; ++s) wv.passes[s].insert(wv.passes[s].end(), part.passes[s].begin(), part.passes[s].end());
                for (int a = 0; a < 4; ++a) wv.alpha[a].insert(wv.alpha[a].end(), part.alpha[a].begin(), part.alpha[a].end());
                wv.copies.insert(wv.copies.end(), part.copies.begin(), part.copies.end());
                wv.torgb.insert(wv.torgb.end(), part.torgb.begin(), part.torgb.end());
            }
            if (mid_used > wv.mid_bytes) return abandon(b, fail(DG_E_INVALID, "internal: resize scratch bound exceeded"));
            for (int s = 0; s < 4; ++s) {
                uint32_t t = 0;
                wv.pass_first[s].push_back(0);
                std::stable_partition(wv.passes[s].begin(), wv.passes[s].end(), [](const ConvPass& cp) { return cp.fast == 2; });
                wv.mma_tiles[s] = 0;
                for (ConvPass& cp : wv.passes[s]) {
                    cp.tile_first = t;
                    t += conv_tiles(cp, (s & 1) != 0);
                    wv.pass_first[s].push_back(t);
                    if (cp.fast == 2) wv.mma_tiles[s] = t;
                }
            }
            uint32_t t = 0;
            wv.copy_first.push_back(0);
            for (CopyJob& j : wv.copies) {
                j.tile_first = t;
                t += (uint32_t)(((uint64_t)j.row_bytes * j.rows + kCopyTileBytes - 1) / kCopyTileBytes);
                wv.copy_first.push_back(t);
            }
            for (int a = 0; a < 4; ++a) {
                t = 0;
                wv.alpha_first[a].push_back(0);
                for (AlphaJob& j : wv.alpha[a]) {
                    j.tile_first = t;
                    t += (j.width * j.rows + kAlphaTilePx - 1) / kAlphaTilePx;
                    wv.alpha_first[a].push_back(t);
                }
            }
            t = 0;
            wv.torgb_first.push_back(0);
            for (ToRgbJob& j : wv.torgb) {
                j.tile_first = t;
                t += (j.npx + kToRgbTilePx - 1) / kToRgbTilePx;
                wv.torgb_first.push_back(t);
            }
        }
        // meta image
        Meta& m = b->meta;
        m.bytes.clear();
        b->m_huff = m.put(pl.huff_pool, 16);
        b->n_huff = (uint32_t)pl.huff_pool.size();
        b->m_qt = m.put(pl.qt_pool, 16);
        for (WavePlan& wv : b->waves) {
            wv.m_descs = m.put(wv.descs, 16);
            wv.m_spec = m.put(wv.spec_list);
            wv.m_restart_list = m.put(wv.restart_list);
            wv.m_restart = put_owner_map(m, wv.restart_first);
            wv.m_blocks = put_owner_map(m, wv.block_first);
            wv.m_color = put_owner_map(m, wv.color_first);
            wv.m_fchroma = put_owner_map(m, wv.fchroma_first);
            wv.m_ftile = put_owner_map(m, wv.ftile_first);
            for (int s = 0; s < 4; ++s) {
                wv.m_passes[s] = m.put(wv.passes[s], 64);
                if (wv.pass_first[s].empty()) wv.pass_first[s].push_back(0);
                wv.m_pass[s] = put_owner_map(m, wv.pass_first[s]);
            }
            wv.m_copies = m.put(wv.copies, 16);
            if (wv.copy_first.empty()) wv.copy_first.push_back(0);
            wv.m_copy = put_owner_map(m, wv.copy_first);
            for (int a = 0; a < 4; ++a) {
                wv.m_alphas[a] = m.put(wv.alpha[a], 16);
                if (wv.alpha_first[a].empty()) wv.alpha_first[a].push_back(0);
                wv.m_alpha[a] = put_owner_map(m, wv.alpha_first[a]);
            }
            wv.m_torgbs = m.put(wv.torgb, 16);
            if (wv.torgb_first.empty()) wv.torgb_first.push_back(0);
            wv.m_torgb = put_owner_map(m, wv.torgb_first);
        }
        // the filter tables follow the rest of the metadata; they are written into the staging buffer directly
        b->m_tables = align_up(m.bytes.size(), 256);
        b->meta_total = b->m_tables + pl.table_words_total * 4;
        if (round == 0) {
            b->off_meta = fixed_bytes;
            b->persist_bytes = fixed_bytes + align_up(b->meta_total, 256);
            rc = ctx->dev.acquire(b->persist_bytes, &b->blk_persist);
            if (rc) return abandon(b, rc);
            b->d_persist = (uint8_t*)ctx->dev.blocks[b->blk_persist].ptr;
            bool pointers = transform;  // resize passes and copy jobs carry device pointers: lay them out again for real
            for (const WavePlan& wv : b->waves) pointers = pointers || !wv.copies.empty() || !wv.torgb.empty();  // (alpha jobs only exist with a transform)
            if (!pointers) break;
        }
    }
    if (pl.tmap_failed) return abandon(b, fail(DG_E_CUDA, "cuTensorMapEncodeTiled rejected the source of a horizontal resize pass"));

    // ---- pinned staging: [status zeros | blob | raw pixel inputs] + meta ------------------------------------------
    // Raw inputs are staged too: a copy from pageable caller memory is serialised by the driver at a fraction of the
    // link rate, while host threads fill page-locked memory in parallel and the upload becomes one large transfer.
    const size_t staged_head = b->off_rawin + align_up(rawin, 256);
    b->pin_bytes = staged_head + align_up(b->meta_total, 256);
    rc = ctx->pin.acquire(b->pin_bytes, &b->blk_pin);
    if (!rc) rc = ctx->pin.acquire(std::max<size_t>((size_t)n * 4, 256), &b->blk_pin_status);
    if (rc) return abandon(b, rc);
    b->h_pin = (uint8_t*)ctx->pin.blocks[b->blk_pin].ptr;
    b->h_status = (uint32_t*)ctx->pin.blocks[b->blk_pin_status].ptr;
    memset(b->h_pin, 0, b->off_blob);
    {
        std::vector<std::pair<int, size_t>> jobs;  // (item, offset in the blob): same order as the descriptors' raw_off
        size_t off = 0;
        for (WavePlan& wv : b->waves)
            for (int i = wv.first_item; i < wv.last_item; ++i) {
                const ItemPlan& it = b->items[i];
                if (it.status || !it.is_jpeg || it.wave_local < 0) continue;
                jobs.emplace_back(i, off);
                off += align_up(it.hdr->scan_len, 16) + 16;
            }
        parallel_items((int)jobs.size(), [&](int k) {
            const int i = jobs[k].first;
            const JpegHeader& h = *b->items[i].hdr;
            uint8_t* dst = b->h_pin + b->off_blob + jobs[k].second;
            memcpy(dst, items[i].data + h.scan_off, h.scan_len);
            memset(dst + h.scan_len, 0, align_up(h.scan_len, 16) + 16 - h.scan_len);
        });
    }
    if (rawin) {
        struct Piece { uint8_t* dst; const uint8_t* src; size_t len; uint32_t rows, pitch; };  // rows == 0: one flat run of len bytes
        std::vector<Piece> pieces;  // 4 MB pieces, so that a few large images still spread over the threads
        for (int i = 0; i < n; ++i) {
            const ItemPlan& it = b->items[i];
            if (it.status || it.is_jpeg || !b->raw_src[i]) continue;
            const size_t row = (size_t)it.w * it.c, bytes = row * it.h;
            uint8_t* dst = b->h_pin + b->off_rawin + it.raw_in_off;
            if (it.src_pitch == row) {
                for (size_t o = 0; o < bytes; o += (size_t)4 << 20)
                    pieces.push_back({dst + o, b->raw_src[i] + o, std::min(bytes - o, (size_t)4 << 20), 0, 0});
            } else {  // rows are re-pitched on the way: a piece is a run of whole rows
                const size_t rows_per = std::max<size_t>(1, ((size_t)4 << 20) / row);
                for (size_t y = 0; y < it.h; y += rows_per)
                    pieces.push_back({dst + y * it.src_pitch, b->raw_src[i] + y * row, row, (uint32_t)std::min<size_t>(rows_per, it.h - y), it.src_pitch});
            }
        }
        HostPool::get().run(pieces.size(), [&](size_t k) {
            const Piece& pc = pieces[k];
            if (!pc.rows) { memcpy(pc.dst, pc.src, pc.len); return; }
            for (uint32_t y = 0; y < pc.rows; ++y) memcpy(pc.dst + (size_t)y * pc.pitch, pc.src + (size_t)y * pc.len, pc.len);
        }, 1);
    }
    b->raw_src.clear();  // caller memory is not needed after this call
    memcpy(b->h_pin + staged_head, b->meta.bytes.data(), b->meta.bytes.size());
    {
        uint32_t* pool = reinterpret_cast<uint32_t*>(b->h_pin + staged_head + b->m_tables);
        const auto& list = pl.table_list;
        HostPool::get().run(list.size(), [&](size_t k) { list[k].second->pack(pool + list[k].first); }, 8);
    }
    *out = b;
    return DG_OK;
}

extern "C" int dg_batch_upload(dg_batch* b) {
    if (!b) return fail(DG_E_INVALID, "NULL batch");
    dg_ctx* ctx = b->ctx;
    std::lock_guard<std::mutex> lock(ctx->mu);
    CU(cudaSetDevice(ctx->device));
    b->h2d = 0;
    // status zeros + compressed blob + raw pixel inputs (contiguous in the staging buffer and on the device)
    const size_t head = b->off_rawin + align_up(b->rawin_bytes, 256);
    CU(cudaMemcpyAsync(b->d_persist, b->h_pin, head, cudaMemcpyHostToDevice, ctx->stream));
    b->h2d += head;
    // metadata
    CU(cudaMemcpyAsync(b->d_persist + b->off_meta, b->h_pin + head, b->meta_total, cudaMemcpyHostToDevice, ctx->stream));
    b->h2d += b->meta_total;
    b->uploaded = true;
    return DG_OK;
}

static OwnerMap resolve(const dg_batch* b, const OwnerMapOff& o) {
    OwnerMap m;
    const uint8_t* base = b->d_persist + b->off_meta;
    m.first = (const uint32_t*)(base + o.first);
    m.coarse = (const uint32_t*)(base + o.coarse);
    m.n = o.n; m.shift = o.shift; m.total = o.total;
    return m;
}

static int batch_run_locked(dg_batch* b);

extern "C" int dg_batch_run(dg_batch* b) {
    if (!b) return fail(DG_E_INVALID, "NULL batch");
    if (!b->uploaded) return fail(DG_E_INVALID, "dg_batch_run before dg_batch_upload");
    dg_ctx* ctx = b->ctx;
    std::lock_guard<std::mutex> lock(ctx->mu);
    const int rc = batch_run_locked(b);
    if (rc != DG_OK) {  // a pass that stopped half-way leaves no guarantee about the scratch contents
        if (b->blk_scratch >= 0) ctx->dev.blocks[b->blk_scratch].zero_prefix = 0;
        if (b->blk_scratch2 >= 0) ctx->dev.blocks[b->blk_scratch2].zero_prefix = 0;
    }
    return rc;
}

static int batch_run_locked(dg_batch* b) {
    dg_ctx* ctx = b->ctx;
    CU(cudaSetDevice(ctx->device));
    cudaStream_t s = ctx->stream;
    const uint8_t* meta = b->d_persist + b->off_meta;
    const bool timing = (b->flags & DG_BATCH_TIMING) != 0;
    // Waves alternate between two streams and two scratch blocks, so the serial, latency-bound entropy decoding of one
    // wave overlaps the bandwidth-hungry reconstruction of the other.  A timing batch stays on one stream: its stage
    // events then bracket kernels that ran alone.
    const bool two_lanes = !timing && b->waves.size() > 1;
    const bool transform = ctx->has_tfm && !(b->flags & DG_BATCH_DECODE_ONLY);
    size_t ev = 0;
    auto mark = [&](int stage, bool begin) -> cudaError_t {
        if (!timing) return cudaSuccess;
        if (begin) {
            if (ev == b->events.size()) {
                StageEvent se{stage, nullptr, nullptr};
                cudaError_t e = cudaEventCreate(&se.a);
                if (e == cudaSuccess) e = cudaEventCreate(&se.b);
                if (e != cudaSuccess) return e;
                b->events.push_back(se);
            }
            b->events[ev].stage = stage;
            return cudaEventRecord(b->events[ev].a, s);
        }
        return cudaEventRecord(b->events[ev++].b, s);
    };
    b->launches = 0;
    if (b->ran) CU(cudaMemsetAsync(b->d_persist + b->off_status, 0, align_up((size_t)b->n * 4, 8) + 32, s));  // status words of the previous run
    if (two_lanes) {
        CU(cudaEventRecord(ctx->ev_fork, ctx->stream));
        CU(cudaStreamWaitEvent(ctx->stream2, ctx->ev_fork, 0));
    }
    for (size_t wi = 0; wi < b->waves.size(); ++wi) {
        WavePlan& wv = b->waves[wi];
        uint8_t* sc = (wi & 1) ? b->d_scratch2 : b->d_scratch;
        // everything of the scratch block beyond this wave's coefficient region is about to be overwritten
        const size_t coef_bytes = wv.coef_blocks * 128;
        Block& scratch_blk = ctx->dev.blocks[(wi & 1) ? b->blk_scratch2 : b->blk_scratch];
        if (scratch_blk.zero_prefix > coef_bytes) scratch_blk.zero_prefix = coef_bytes;
        // the scratch block belongs to the lane, so in one-stream mode an odd wave must wait for nothing extra:
        // stream order already serialises the waves
        s = (two_lanes && (wi & 1)) ? ctx->stream2 : ctx->stream;
        if (!wv.descs.empty()) {
            JpegWave w;
            memset(&w, 0, sizeof w);
            w.descs = (const JpegDesc*)(meta + wv.m_descs);
            w.n = (uint32_t)wv.descs.size();
            w.raw = b->d_persist + b->off_blob;
            w.us = sc + wv.off_us;
            w.us_len = (uint32_t*)(sc + wv.off_uslen);
            w.seg_start = (uint32_t*)(sc + wv.off_segstart);
            w.seg_found = (uint32_t*)(sc + wv.off_segfound);
            w.coef = (int16_t*)(sc + wv.off_coef);
            w.planes = sc + wv.off_planes;
            w.out = transform ? sc + wv.off_decoded : b->d_persist + b->off_out;
            w.status = (uint32_t*)(b->d_persist + b->off_status);
            w.spec_stats = (unsigned long long*)(b->d_persist + b->off_status + align_up((size_t)b->n * 4, 8));
            w.huff = (const HuffTable*)(meta + b->m_huff);
            w.n_huff = b->n_huff;
            w.qt32 = (const uint32_t*)(meta + b->m_qt);
            w.spec_list = (const uint32_t*)(meta + wv.m_spec);
            w.n_spec = (uint32_t)wv.spec_list.size();
            w.restart_list = (const uint32_t*)(meta + wv.m_restart_list);
            w.restart_segs = resolve(b, wv.m_restart);
            w.blocks = resolve(b, wv.m_blocks);
            w.color_tiles = resolve(b, wv.m_color);
            w.fused_first = wv.fused_first;
            w.fused_chroma = resolve(b, wv.m_fchroma);
            w.fused_tiles = resolve(b, wv.m_ftile);
            CU(mark(DG_STAGE_UNSTUFF, true));
            launch_unstuff(w, s);
            ++b->launches;
            CU(mark(DG_STAGE_UNSTUFF, false));
            // The entropy decoders write only non-zero coefficients, so the coefficient region must be zero beforehand.
            // The IDCT zeroes the rows it found non-zero after reading them, which keeps the region zero from one wave
            // to the next on the same scratch block; only a part that was not a coefficient region before is cleared.
            const bool rezero = !(b->flags & DG_BATCH_KEEP_COEFFICIENTS);
            CU(mark(DG_STAGE_COEF_CLEAR, true));
            if (coef_bytes > scratch_blk.zero_prefix)
                CU(cudaMemsetAsync((uint8_t*)w.coef + scratch_blk.zero_prefix, 0, coef_bytes - scratch_blk.zero_prefix, s));
            scratch_blk.zero_prefix = rezero ? coef_bytes : 0;
            CU(mark(DG_STAGE_COEF_CLEAR, false));
            // The two entropy kernels work on disjoint images and are both latency bound: outside timing mode they run
            // side by side, the restart-interval one on the lane's auxiliary stream.
            // The auxiliary stream of the lane takes what can run beside the speculative decoder: the restart-interval
            // decoder, and the speculative decoder's widest CTAs for the few longest images of the wave.
            const uint32_t n_huge = wv.n_huge;
            const bool aux_restart = !timing && w.restart_segs.total && w.n_spec;
            const bool aux_huge = n_huge && w.n_spec > n_huge;  // also in a timing batch: the two launches are one stage
            const int lane = (int)(wi & 1);
            cudaStream_t aux = ctx->aux[lane];
            if (w.n_spec) {  // the longest images first: they decide when the stage ends
                CU(mark(DG_STAGE_HUFF_SPEC, true));
                if (aux_restart || aux_huge) {
                    CU(cudaEventRecord(ctx->ev_aux_go[lane], s));
                    CU(cudaStreamWaitEvent(aux, ctx->ev_aux_go[lane], 0));
                }
                launch_huff_spec(w, n_huge, s, aux_huge ? aux : s);
                b->launches += (n_huge ? 1 : 0) + (w.n_spec > n_huge ? 1 : 0);
                if (timing && aux_huge) {  // the stage ends when both launches have
                    CU(cudaEventRecord(ctx->ev_aux_done[lane], aux));
                    CU(cudaStreamWaitEvent(s, ctx->ev_aux_done[lane], 0));
                }
                CU(mark(DG_STAGE_HUFF_SPEC, false));
            }
            if (w.restart_segs.total) {
                CU(mark(DG_STAGE_HUFF_RESTART, true));
                launch_huff_restart(w, aux_restart ? aux : s);
                ++b->launches;
                CU(mark(DG_STAGE_HUFF_RESTART, false));
            }
            if (!timing && (aux_restart || aux_huge)) {
                CU(cudaEventRecord(ctx->ev_aux_done[lane], aux));
                CU(cudaStreamWaitEvent(s, ctx->ev_aux_done[lane], 0));
            }
            for (const auto& g : wv.groups) {
                if (!g[1]) continue;
                CU(mark(DG_STAGE_IDCT, true));
                launch_idct(w, g[0], g[1], rezero, s);
                ++b->launches;
                CU(mark(DG_STAGE_IDCT, false));
                CU(mark(DG_STAGE_COLOR, true));
                launch_color(w, g[2], g[3], s);
                ++b->launches;
                CU(mark(DG_STAGE_COLOR, false));
            }
            for (const auto& g : wv.fgroups) {  // 4:2:0: chroma planes first, then luma IDCT + upsampling + colour in one kernel
                if (!g[1]) continue;
                CU(mark(DG_STAGE_IDCT, true));
                launch_idct_chroma(w, g[0], g[1], rezero, s);
                ++b->launches;
                CU(mark(DG_STAGE_IDCT, false));
                CU(mark(DG_STAGE_COLOR, true));
                launch_luma_color(w, g[2], g[3], rezero, s);
                ++b->launches;
                CU(mark(DG_STAGE_COLOR, false));
            }
        }
        if (transform) {
            const uint32_t* tables = (const uint32_t*)(meta + b->m_tables);
            static const int kStageOf[4] = {DG_STAGE_RESIZE_H, DG_STAGE_RESIZE_V, DG_STAGE_RESIZE_SHIFT, DG_STAGE_RESIZE_SHIFT};
            auto alpha_step = [&](int a) -> int {
                if (wv.alpha[a].empty()) return DG_OK;
                CU(mark(DG_STAGE_RESIZE_SHIFT, true));
                launch_alpha((const AlphaJob*)(meta + wv.m_alphas[a]), resolve(b, wv.m_alpha[a]), s);
                ++b->launches;
                CU(mark(DG_STAGE_RESIZE_SHIFT, false));
                return DG_OK;
            };
            for (int st = 0; st < 4; ++st) {
                if (st == 0 || st == 2) { const int rc = alpha_step(st); if (rc) return rc; }                 // multiply before a resize
                if (!wv.passes[st].empty()) {
                    CU(mark(kStageOf[st], true));
                    const ConvPass* passes = (const ConvPass*)(meta + wv.m_passes[st]);
                    if (st & 1) launch_conv_v(passes, resolve(b, wv.m_pass[st]), tables, wv.mma_tiles[st], s);
                    else launch_conv_h(passes, resolve(b, wv.m_pass[st]), tables, wv.mma_tiles[st], s);
                    b->used_hmma = b->used_hmma || wv.mma_tiles[st] != 0;
                    ++b->launches;
                    CU(mark(kStageOf[st], false));
                }
                if (st == 1 || st == 3) { const int rc = alpha_step(st); if (rc) return rc; }                 // divide after it
            }
        }
        if (!wv.copies.empty()) {
            CU(mark(DG_STAGE_RESIZE_SHIFT, true));
            launch_copy((const CopyJob*)(meta + wv.m_copies), resolve(b, wv.m_copy), s);
            ++b->launches;
            CU(mark(DG_STAGE_RESIZE_SHIFT, false));
        }
        if (!wv.torgb.empty()) {
            CU(mark(DG_STAGE_TO_RGB8, true));
            launch_to_rgb8((const ToRgbJob*)(meta + wv.m_torgbs), resolve(b, wv.m_torgb), s);
            ++b->launches;
            CU(mark(DG_STAGE_TO_RGB8, false));
        }
    }
    if (two_lanes) {
        CU(cudaEventRecord(ctx->ev_join, ctx->stream2));
        CU(cudaStreamWaitEvent(ctx->stream, ctx->ev_join, 0));
    }
    CU(cudaGetLastError());
    b->ran = true;
    return DG_OK;
}

extern "C" int dg_batch_download(dg_batch* b, uint8_t* const* host_out) {
    if (!b || !host_out) return fail(DG_E_INVALID, "NULL argument");
    dg_ctx* ctx = b->ctx;
    std::lock_guard<std::mutex> lock(ctx->mu);
    CU(cudaSetDevice(ctx->device));
    b->d2h = 0;
    for (int i = 0; i < b->n; ++i) {
        const ItemPlan& it = b->items[i];
        if (it.status || !host_out[i]) continue;
        CU(cudaMemcpyAsync(host_out[i], b->d_persist + b->off_out + it.out_off, it.out_bytes, cudaMemcpyDeviceToHost, ctx->stream));
        b->d2h += it.out_bytes;
    }
    return DG_OK;
}

extern "C" uint64_t dg_batch_packed_bytes(const dg_batch* b) { return b ? b->out_bytes : 0; }

extern "C" int dg_batch_download_packed(dg_batch* b, uint8_t* host_base, uint64_t capacity) {
    if (!b || !host_base) return fail(DG_E_INVALID, "NULL argument");
    if (capacity < b->out_bytes) return fail(DG_E_INVALID, "packed download needs %zu bytes, the buffer holds %llu", b->out_bytes, (unsigned long long)capacity);
    dg_ctx* ctx = b->ctx;
    std::lock_guard<std::mutex> lock(ctx->mu);
    CU(cudaSetDevice(ctx->device));
    if (b->out_bytes) CU(cudaMemcpyAsync(host_base, b->d_persist + b->off_out, b->out_bytes, cudaMemcpyDeviceToHost, ctx->stream));
    b->d2h = b->out_bytes;
    return DG_OK;
}

static int device_status_to_code(uint32_t bits) {
    if (bits == 0) return DG_OK;
    if (bits & kStSyncLimit) return DG_E_SYNC_LIMIT;
    if (bits & kStBadMarker) return DG_E_BAD_MARKER;
    if (bits & (kStBadCode | kStCoefRange)) return DG_E_BAD_CODE;
    return DG_E_TRUNCATED;
}

extern "C" int dg_batch_sync(dg_batch* b) {
    if (!b) return fail(DG_E_INVALID, "NULL batch");
    dg_ctx* ctx = b->ctx;
    std::lock_guard<std::mutex> lock(ctx->mu);
    CU(cudaSetDevice(ctx->device));
    if (b->ran) {
        CU(cudaMemcpyAsync(b->h_status, b->d_persist + b->off_status, (size_t)b->n * 4, cudaMemcpyDeviceToHost, ctx->stream));
        b->d2h += (size_t)b->n * 4;
    }
    CU(cudaStreamSynchronize(ctx->stream));
    if (b->ran && b->used_hmma) {
        // the tensor-core resize pass bounds its waits for asynchronous copies; a wait that ran out left garbage behind
        const unsigned int t = read_conv_timeouts(ctx->stream);
        if (t != ctx->conv_timeouts_seen) {
            ctx->conv_timeouts_seen = t;
            return fail(DG_E_CUDA, "resize: a copy into shared memory did not complete in time (%u CTAs gave up); the batch's pixels are not valid", t);
        }
    }
    if (b->ran) {
        for (int i = 0; i < b->n; ++i)
            if (b->items[i].status == DG_OK && b->h_status[i]) b->items[i].status = device_status_to_code(b->h_status[i]);
        if (!b->counted) {  // once per batch, however often it is run and synchronised
            b->counted = true;
            ++ctx->counters.batches;
            ctx->counters.bytes_in += b->blob_bytes + b->rawin_bytes;
            for (int i = 0; i < b->n; ++i) {
                const int st = b->items[i].status;
                ++ctx->counters.items[st >= 0 && st < DG_STATUS_COUNT ? st : DG_E_INVALID];
                if (st == DG_OK) ctx->counters.bytes_out += b->items[i].out_bytes;
                else log_line(DG_LOG_ERROR, "item %d: %s (status %d)", i, status_name(st), st);  // the sample is dropped
            }
        }
        if (b->flags & DG_BATCH_TIMING) {
            for (float& v : b->stage_ms) v = 0.f;
            for (const StageEvent& se : b->events) {
                float ms = 0.f;
                if (cudaEventElapsedTime(&ms, se.a, se.b) == cudaSuccess) b->stage_ms[se.stage] += ms;
            }
        }
    }
    return DG_OK;
}

extern "C" int dg_batch_result(const dg_batch* b, int i, dg_result* out) {
    if (!b || !out || i < 0 || i >= b->n) return fail(DG_E_INVALID, "bad index");
    const ItemPlan& it = b->items[i];
    memset(out, 0, sizeof *out);
    out->status = it.status;
    out->original_width = it.w; out->original_height = it.h;
    if (it.status == DG_OK) {
        out->width = it.out_w; out->height = it.out_h; out->channels = it.c_out; out->bit_depth = 8;
        out->nbytes = it.out_bytes;
        out->device_data = b->d_persist + b->off_out + it.out_off;
        out->packed_offset = it.out_off;
    }
    out->plan = it.plan;
    return DG_OK;
}

extern "C" int dg_batch_bucket_count(const dg_batch* b) { return b ? (int)b->buckets.size() : 0; }

extern "C" int dg_batch_bucket(const dg_batch* b, int k, dg_bucket* out) {
    if (!b || !out || k < 0 || k >= (int)b->buckets.size()) return fail(DG_E_INVALID, "bad bucket index (is this a DG_BATCH_COLLATE batch?)");
    const BucketPlan& bk = b->buckets[k];
    memset(out, 0, sizeof *out);
    memcpy(out->key, bk.key, 16);
    out->n = (uint32_t)bk.items.size();
    out->width = bk.w; out->height = bk.h; out->channels = bk.c;
    out->nbytes = (uint64_t)bk.items.size() * bk.w * bk.h * bk.c;
    out->device_data = b->d_persist + b->off_out + bk.off;
    out->packed_offset = bk.off;
    out->items = bk.items.data();
    return DG_OK;
}

extern "C" int dg_batch_stage_ms(const dg_batch* b, float ms[DG_STAGE_COUNT]) {
    if (!b || !ms) return fail(DG_E_INVALID, "NULL argument");
    memcpy(ms, b->stage_ms, sizeof b->stage_ms);
    return DG_OK;
}

extern "C" int dg_batch_counters(const dg_batch* b, uint64_t* h2d, uint64_t* d2h, uint32_t* launches) {
    if (!b) return fail(DG_E_INVALID, "NULL batch");
    if (h2d) *h2d = b->h2d;
    if (d2h) *d2h = b->d2h;
    if (launches) *launches = b->launches;
    return DG_OK;
}

extern "C" int dg_batch_huffman_stats(dg_batch* b, uint64_t out[3]) {
    if (!b || !out) return fail(DG_E_INVALID, "NULL argument");
    dg_ctx* ctx = b->ctx;
    std::lock_guard<std::mutex> lock(ctx->mu);
    CU(cudaSetDevice(ctx->device));
    CU(cudaMemcpyAsync(out, b->d_persist + b->off_status + align_up((size_t)b->n * 4, 8), 24, cudaMemcpyDeviceToHost, ctx->stream));
    CU(cudaStreamSynchronize(ctx->stream));
    return DG_OK;
}

extern "C" int dg_batch_debug(const dg_batch* b, int i, const int16_t** coef, uint64_t* nblocks, const uint8_t** decoded) {
    if (!b || i < 0 || i >= b->n) return fail(DG_E_INVALID, "bad index");
    const ItemPlan& it = b->items[i];
    if (it.status || !it.is_jpeg || it.wave < 0) return fail(DG_E_INVALID, "item has no JPEG intermediates");
    if ((int)b->waves.size() != 1) return fail(DG_E_INVALID, "intermediates are only kept for single-wave batches");
    const WavePlan& wv = b->waves[it.wave];
    if (coef) *coef = (const int16_t*)(b->d_scratch + wv.off_coef) + it.coef_off_blocks * 64;
    if (nblocks) *nblocks = it.nblocks;
    const bool transform = b->ctx->has_tfm && !(b->flags & DG_BATCH_DECODE_ONLY);
    if (decoded) *decoded = transform ? b->d_scratch + wv.off_decoded + it.decoded_off : b->d_persist + b->off_out + it.pipe_off;
    return DG_OK;
}

extern "C" void dg_batch_destroy(dg_batch* b) {
    if (!b) return;
    dg_ctx* ctx = b->ctx;
    std::lock_guard<std::mutex> lock(ctx->mu);
    cudaSetDevice(ctx->device);
    cudaStreamSynchronize(ctx->stream);
    for (StageEvent& se : b->events) { cudaEventDestroy(se.a); cudaEventDestroy(se.b); }
    ctx->dev.release(b->blk_persist);
    ctx->dev.release(b->blk_scratch);
    ctx->dev.release(b->blk_scratch2);
    ctx->pin.release(b->blk_pin);
    ctx->pin.release(b->blk_pin_status);
    delete b;
}

extern "C" int dg_process(dg_ctx* ctx, const dg_item* items, int n, uint32_t flags, uint8_t* const* host_out, dg_result* results) {
    dg_batch* b = nullptr;
    int rc = dg_batch_create(ctx, items, n, flags, &b);
    if (rc) return rc;
    rc = dg_batch_upload(b);
    if (!rc) rc = dg_batch_run(b);
    if (!rc && host_out) rc = dg_batch_download(b, host_out);
    if (!rc) rc = dg_batch_sync(b);
    if (!rc && results)
        for (int i = 0; i < n; ++i) { dg_batch_result(b, i, &results[i]); results[i].device_data = nullptr; }
    dg_batch_destroy(b);
    return rc;
}

extern "C" int dg_copy_to_host(dg_ctx* ctx, void* dst, const void* src, uint64_t nbytes) {
    if (!ctx || !dst || !src || ctx->device == DG_DEVICE_NONE) return fail(DG_E_INVALID, "NULL argument or planning-only context");
    std::lock_guard<std::mutex> lock(ctx->mu);
    CU(cudaSetDevice(ctx->device));
    CU(cudaMemcpyAsync(dst, src, nbytes, cudaMemcpyDeviceToHost, ctx->stream));
    CU(cudaStreamSynchronize(ctx->stream));
    return DG_OK;
}

// ---------------------------------------------------------------------------------------------------------------
// Allocation-free crop_and_resize of one device-resident image.
//
// Some hosts cannot let a library allocate device memory once they are running: a training process whose framework
// allocator has already reserved all of HBM (a cudaMalloc would fail, or force that allocator to give its cache
// back), a latency-critical loop that cannot take the device-wide synchronisation an allocation may imply, or a
// service with a "no allocation after start-up" rule.  For them this entry point does the same work as a one-image
// batch -- same planner, same convolution kernels -- but takes everything it needs beyond the caller's input and
// output buffers (pass descriptors, filter tables, the intermediate images between passes) from one fixed array that
// is part of the library image.  Every GPU that loads the library holds those kStaticScratchBytes until the
// process exits.
// ---------------------------------------------------------------------------------------------------------------
namespace {

constexpr size_t kStaticScratchBytes = (size_t)32 << 20;
static __device__ __align__(256) unsigned char g_static_scratch[kStaticScratchBytes];

// In host code `g_static_scratch` is only a handle for the runtime, not an address a kernel can use; the device
// address is looked up once per device, with that device current.
constexpr int kMaxDevices = 64;
std::mutex g_static_mu;
unsigned char* g_static_ptr[kMaxDevices] = {nullptr};

int static_scratch_for(int device, unsigned char** out) {
    if (device < 0 || device >= kMaxDevices) return fail(DG_E_INVALID, "device ordinal %d not supported here", device);
    std::lock_guard<std::mutex> lock(g_static_mu);
    if (!g_static_ptr[device]) {
        void* p = nullptr;
        cudaError_t e = cudaGetSymbolAddress(&p, g_static_scratch);
        if (e != cudaSuccess || !p) return fail(DG_E_CUDA, "cudaGetSymbolAddress(static scratch): %s", cudaGetErrorString(e));
        g_static_ptr[device] = (unsigned char*)p;
    }
    *out = g_static_ptr[device];
    return DG_OK;
}

}  // namespace

extern "C" int dg_resize_device_static(dg_ctx* ctx, const uint8_t* device_src, uint32_t w, uint32_t h, uint32_t channels,
                                       const char* forced_key, uint8_t* device_dst, dg_plan* plan_out) {
    if (!ctx || !device_src || !device_dst || w == 0 || h == 0 || (channels != 1 && channels != 3))
        return fail(DG_E_INVALID, "NULL argument, empty image, or channels not 1 / 3");
    if (ctx->device == DG_DEVICE_NONE) return fail(DG_E_INVALID, "planning-only context: pixel work needs a CUDA device");
    if (!ctx->has_tfm) return fail(DG_E_NO_TRANSFORM, "ctx has no crop_and_resize transform");
    dg_plan plan;
    int rc = plan_geometry(ctx->tfm, w, h, channels, forced_key, &plan);
    if (rc) return fail(rc, "aspect ratio key '%s' is not in the bucket table", forced_key ? forced_key : "");
    if (plan_out) *plan_out = plan;

    std::lock_guard<std::mutex> lock(ctx->mu);
    CU(cudaSetDevice(ctx->device));
    unsigned char* scratch = nullptr;
    rc = static_scratch_for(ctx->device, &scratch);  // first call on a device: symbol look-up
    if (rc) return rc;

    // intermediates go to the top part of the array, metadata to the bottom part
    const size_t mid_bound = align_up(resize_mid_bound(plan, channels), 256);
    if (mid_bound + 65536 > kStaticScratchBytes)
        return fail(DG_E_TOO_LARGE, "image needs %zu bytes of intermediates; the static scratch holds %zu in total", mid_bound, kStaticScratchBytes);
    unsigned char* mid_base = scratch + (kStaticScratchBytes - mid_bound);
    const size_t meta_cap = kStaticScratchBytes - mid_bound;

    Planner pl{ctx, nullptr};
    WavePlan wv;
    size_t mid_used = 0;
    plan_resize(pl, wv, plan, channels, device_src, w * channels, device_dst, mid_base, &mid_used, true);
    if (mid_used > mid_bound) return fail(DG_E_TOO_LARGE, "internal: intermediates exceed their bound");
    Meta m;
    std::vector<uint32_t> packed(pl.table_words_total);
    pl.pack_tables(packed.data());
    const size_t m_tables = m.put(packed, 16);
    size_t m_passes[4];
    OwnerMapOff m_pass[4], m_copy;
    for (int s = 0; s < 4; ++s) {
        uint32_t t = 0;
        wv.pass_first[s].push_back(0);
        for (ConvPass& cp : wv.passes[s]) {  // at most one pass per stage here, so the tensor-core passes trivially come first
            cp.tile_first = t;
            t += conv_tiles(cp, (s & 1) != 0);
            wv.pass_first[s].push_back(t);
            if (cp.fast == 2) wv.mma_tiles[s] = t;
        }
        m_passes[s] = m.put(wv.passes[s], 64);
        m_pass[s] = put_owner_map(m, wv.pass_first[s]);
    }
    {
        uint32_t t = 0;
        wv.copy_first.push_back(0);
        for (CopyJob& j : wv.copies) {
            j.tile_first = t;
            t += (uint32_t)(((uint64_t)j.row_bytes * j.rows + kCopyTileBytes - 1) / kCopyTileBytes);
            wv.copy_first.push_back(t);
        }
    }
    const size_t m_copies = m.put(wv.copies, 16);
    m_copy = put_owner_map(m, wv.copy_first);
    if (m.bytes.size() > meta_cap)
        return fail(DG_E_TOO_LARGE, "filter tables (%zu bytes) and intermediates (%zu bytes) exceed the %zu-byte static scratch",
                    m.bytes.size(), mid_bound, kStaticScratchBytes);

    cudaStream_t s = ctx->stream;
    // nothing in the array has to start at zero: the metadata is overwritten here and every intermediate pixel is
    // written by a pass before the next pass reads it
    CU(cudaMemcpyAsync(scratch, m.bytes.data(), m.bytes.size(), cudaMemcpyHostToDevice, s));
    auto map_at = [&](const OwnerMapOff& o) {
        OwnerMap r;
        r.first = (const uint32_t*)(scratch + o.first);
        r.coarse = (const uint32_t*)(scratch + o.coarse);
        r.n = o.n; r.shift = o.shift; r.total = o.total;
        return r;
    };
    const uint32_t* tables = (const uint32_t*)(scratch + m_tables);
    for (int st = 0; st < 4; ++st) {
        if (wv.passes[st].empty()) continue;
        const ConvPass* passes = (const ConvPass*)(scratch + m_passes[st]);
        if (st & 1) launch_conv_v(passes, map_at(m_pass[st]), tables, wv.mma_tiles[st], s);
        else launch_conv_h(passes, map_at(m_pass[st]), tables, wv.mma_tiles[st], s);
    }
    if (!wv.copies.empty()) launch_copy((const CopyJob*)(scratch + m_copies), map_at(m_copy), s);
    CU(cudaGetLastError());
    CU(cudaStreamSynchronize(s));  // the host-side metadata image dies with this frame
    return DG_OK;
}
