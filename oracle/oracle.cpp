// CPU oracle for the datago per-sample image path.  TEST INFRASTRUCTURE ONLY.
//
// This file is the checker the CUDA path is compared with; it is never linked
// into, imported by or called from the shipped library.  Only the test-suite,
// the smoke check and the benchmark's CPU-baseline leg load it.
//
// What it restates (paths are relative to the datago source tree):
//   * bucket table / closest aspect ratio / crop geometry:
//       src/image_processing.rs:77-120 (get_ar_aware_transform),
//       :130-133 (aspect_ratio_to_str), :188-219 (build_image_size_list),
//       :222-252 (get_closest_aspect_ratio), :254-338 (crop_and_resize).
//     These are pinned by the reference's own known-answer tests
//     (src/image_processing.rs:441-478).
//   * the two `fast_image_resize::Resizer::resize` calls made at
//       src/image_processing.rs:288-323.  fast_image_resize 5.5.0 is a
//     third-party crate whose source is not part of the datago tree; the
//     restatement follows the Pillow resampling algorithm it documents itself
//     as derived from (f64 Lanczos3 weights, normalised, quantised to 16-bit
//     fixed point with the largest precision whose maximum coefficient stays
//     below 2^15, horizontal pass then vertical pass with an 8-bit
//     intermediate).  MODE_PILLOW switches only the quantisation to Pillow's
//     own 22-bit coefficients, which pins the rest of the arithmetic
//     bit-exactly against PIL.Image.resize(LANCZOS, box=...).
//   * the decode call sites src/worker_files.rs:8-17, src/worker_wds.rs:45,
//     src/worker_http.rs:64 (`image` 0.25.9 -> zune-jpeg 0.5.12, also absent):
//     ITU-T T.81 baseline sequential Huffman decoding, followed by the
//     libjpeg-family reconstruction (13-bit "islow" integer IDCT, triangle
//     chroma upsampling, 16-bit fixed-point YCbCr->RGB).  This reconstruction
//     is pinned bit-exactly against libjpeg-turbo (through Pillow) by the
//     test-suite.  PARITY UNPINNED against zune-jpeg itself: no golden pixel
//     exists anywhere in the reference's tests and its decoder cannot be run.
//   * sample sharding: src/generator_files.rs:24-42 (contiguous rank slices,
//     pinned by :190-240) and src/generator_wds.rs:50-54,140-148
//     (DefaultHasher(key) % world_size; DefaultHasher is SipHash-1-3 with a
//     zero key, `str` hashing appends 0xFF).
//
// Plain scalar C++ on purpose: one obvious loop per step, no SIMD, no tables
// shared with the CUDA code.
#include <algorithm>
#include <atomic>
#include <cmath>
#include <cstdint>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <map>
#include <string>
#include <thread>
#include <vector>

#define ORC_API extern "C" __attribute__((visibility("default")))

// ---------------------------------------------------------------------------
// 1. Buckets and geometry
// ---------------------------------------------------------------------------
namespace {

struct Bucket {
    double ar;        // the 3-decimal key parsed back to f64 (image_processing.rs:110-114)
    std::string key;  // format!("{:.3}", w / h)
    uint32_t w, h;
};

std::string ar_key(uint32_t w, uint32_t h) {
    char buf[64];
    snprintf(buf, sizeof buf, "%.3f", (double)w / (double)h);  // exact decimal rounding, as Rust's {:.3}
    return buf;
}

// image_processing.rs:188-219
std::vector<std::pair<uint32_t, uint32_t>> size_list(uint32_t size, uint32_t ratio, double mn, double mx) {
    std::vector<std::pair<uint32_t, uint32_t>> out;
    uint32_t patch = size / ratio;
    double psq = (double)(uint32_t)(patch * patch);
    uint32_t min_pw = (uint32_t)std::ceil(std::sqrt(psq * mn));
    uint32_t max_pw = (uint32_t)std::floor(std::sqrt(psq * mx));
    for (uint32_t pw = min_pw; pw <= max_pw; ++pw) {
        uint32_t ph = (uint32_t)std::floor(psq / (double)pw);
        out.push_back({pw * ratio, ph * ratio});
    }
    uint32_t min_ph = (uint32_t)std::ceil(std::sqrt(psq / mx));
    uint32_t max_ph = (uint32_t)std::floor(std::sqrt(psq / mn));
    for (uint32_t ph = min_ph; ph <= max_ph; ++ph) {
        uint32_t pw = (uint32_t)std::floor(psq / (double)ph);
        out.push_back({pw * ratio, ph * ratio});
    }
    return out;
}

// image_processing.rs:77-120.  Later list entries overwrite earlier ones on an equal key.
std::vector<Bucket> bucket_table(uint32_t size, uint32_t ratio, double mn, double mx) {
    std::map<std::string, std::pair<uint32_t, uint32_t>> m;
    for (auto& wh : size_list(size, ratio, mn, mx)) m[ar_key(wh.first, wh.second)] = wh;
    std::vector<Bucket> t;
    for (auto& kv : m) t.push_back({strtod(kv.first.c_str(), nullptr), kv.first, kv.second.first, kv.second.second});
    std::sort(t.begin(), t.end(), [](const Bucket& a, const Bucket& b) { return a.ar < b.ar; });
    return t;
}

// image_processing.rs:222-252.  Ties go to the right neighbour.
int closest_bucket(const std::vector<Bucket>& t, int w, int h) {
    double target = (double)w / (double)h;
    size_t lo = 0, hi = t.size();
    while (lo < hi) {
        size_t mid = (lo + hi) / 2;
        if (t[mid].ar < target) lo = mid + 1; else hi = mid;
    }
    size_t idx = lo;
    if (idx < t.size() && t[idx].ar == target) return (int)idx;
    if (idx == 0) return 0;
    if (idx == t.size()) return (int)t.size() - 1;
    double left = std::fabs(target - t[idx - 1].ar), right = std::fabs(t[idx].ar - target);
    return left < right ? (int)idx - 1 : (int)idx;
}

}  // namespace

struct orc_plan {
    uint32_t src_w, src_h;
    uint32_t target_w, target_h;  // bucket size
    uint32_t new_w, new_h;        // size after the first resize
    double crop_left, crop_top, crop_w, crop_h;  // box of the second resize
    int32_t identity;             // 1: source already has the bucket size, returned untouched
    char key[16];
};

// Fills up to max_n entries sorted by aspect ratio; returns the table size.
ORC_API int orc_bucket_table(uint32_t size, uint32_t ratio, double mn, double mx, int max_n,
                             uint32_t* w, uint32_t* h, double* ar, char* keys /* 16 bytes each */) {
    auto t = bucket_table(size, ratio, mn, mx);
    for (int i = 0; i < (int)t.size() && i < max_n; ++i) {
        w[i] = t[i].w; h[i] = t[i].h; ar[i] = t[i].ar;
        snprintf(keys + 16 * i, 16, "%s", t[i].key.c_str());
    }
    return (int)t.size();
}

ORC_API int orc_size_list(uint32_t size, uint32_t ratio, double mn, double mx, int max_n, uint32_t* w, uint32_t* h) {
    auto l = size_list(size, ratio, mn, mx);
    for (int i = 0; i < (int)l.size() && i < max_n; ++i) { w[i] = l[i].first; h[i] = l[i].second; }
    return (int)l.size();
}

ORC_API void orc_aspect_ratio_to_str(uint32_t w, uint32_t h, char* out16) {
    snprintf(out16, 16, "%s", ar_key(w, h).c_str());
}

// crop_and_resize geometry, image_processing.rs:259-310.  forced_key NULL or "" = automatic bucket.
// Returns 0, or -1 when the key is not in the table (the reference panics there, :335).
ORC_API int orc_plan_geometry(uint32_t size, uint32_t ratio, double mn, double mx, uint32_t w, uint32_t h,
                              const char* forced_key, orc_plan* p) {
    auto t = bucket_table(size, ratio, mn, mx);
    if (t.empty()) return -2;
    int idx = -1;
    if (forced_key && forced_key[0]) {
        for (int i = 0; i < (int)t.size(); ++i) if (t[i].key == forced_key) idx = i;
        if (idx < 0) return -1;
    } else {
        idx = closest_bucket(t, (int)w, (int)h);
    }
    memset(p, 0, sizeof *p);
    p->src_w = w; p->src_h = h;
    p->target_w = t[idx].w; p->target_h = t[idx].h;
    snprintf(p->key, sizeof p->key, "%s", t[idx].key.c_str());
    if (w == p->target_w && h == p->target_h) {
        p->identity = 1; p->new_w = w; p->new_h = h; p->crop_w = w; p->crop_h = h;
        return 0;
    }
    double sx = (double)p->target_w / (double)w, sy = (double)p->target_h / (double)h;
    double scale = sx > sy ? sx : sy;
    p->new_w = (uint32_t)std::round((double)w * scale);
    p->new_h = (uint32_t)std::round((double)h * scale);
    // CropBox::fit_src_into_dst_size(new_w, new_h, tw, th, None): centred box with the target's aspect.
    double width = p->new_w, height = p->new_h;
    double image_ratio = width / height, required = (double)p->target_w / (double)p->target_h;
    double cw, ch;
    if (std::fabs(image_ratio - required) < 2.220446049250313e-16) { cw = width; ch = height; }
    else if (image_ratio >= required) { cw = required * height; ch = height; }
    else { cw = width; ch = width / required; }
    p->crop_w = cw; p->crop_h = ch;
    p->crop_left = (width - cw) * 0.5;
    p->crop_top = (height - ch) * 0.5;
    return 0;
}

// ---------------------------------------------------------------------------
// 2. Lanczos3 convolution resize
// ---------------------------------------------------------------------------
namespace {

enum { MODE_FIR = 0, MODE_PILLOW = 1 };

double sinc(double x) { if (x == 0.0) return 1.0; double a = x * M_PI; return std::sin(a) / a; }
double lanczos3(double x) { return (x >= -3.0 && x < 3.0) ? sinc(x) * sinc(x / 3.0) : 0.0; }

struct Coeffs {
    std::vector<int32_t> start, size;  // per output sample: first input sample and tap count
    std::vector<int32_t> k;            // window * out taps, fixed point
    int window = 0, precision = 0;
};

// Weights for resampling in[in0, in1) of an axis of length in_size into out_size samples.
Coeffs make_coeffs(int in_size, double in0, double in1, int out_size, int mode) {
    Coeffs c;
    double scale = (in1 - in0) / (double)out_size;
    double fscale = scale < 1.0 ? 1.0 : scale;
    double radius = 3.0 * fscale;
    c.window = (int)std::ceil(radius) * 2 + 1;
    std::vector<double> kf((size_t)c.window * out_size, 0.0);
    c.start.resize(out_size); c.size.resize(out_size);
    double maxw = 0.0;
    bool first = true;
    for (int ox = 0; ox < out_size; ++ox) {
        double in_center = in0 + ((double)ox + 0.5) * scale;
        double* k = &kf[(size_t)ox * c.window];
        int n = 0, bstart, bend;
        double ww = 0.0;
        if (mode == MODE_PILLOW) {
            // Pillow: xmin/xmax are truncations of center -/+ support + 0.5, weight at (x - center + 0.5) / fscale.
            double ss = 1.0 / fscale;
            int xmin = (int)(in_center - radius + 0.5); if (xmin < 0) xmin = 0;
            int xmax = (int)(in_center + radius + 0.5); if (xmax > in_size) xmax = in_size;
            for (int x = 0; x < xmax - xmin; ++x) { double w = lanczos3(((double)(x + xmin) - in_center + 0.5) * ss); k[n++] = w; ww += w; }
            bstart = xmin; bend = xmax;
        } else {
            // fast_image_resize: floor/ceil window, leading and trailing zero weights dropped.
            double recip = 1.0 / fscale;
            double lo = std::floor(in_center - radius); if (lo < 0.0) lo = 0.0;
            double hi = std::ceil(in_center + radius); if (hi > (double)in_size) hi = (double)in_size;
            int xmin = (int)lo, xmax = (int)hi;
            double center = in_center - 0.5;
            bstart = xmin; bend = xmax;
            for (int x = xmin; x < xmax; ++x) {
                double w = lanczos3(((double)x - center) * recip);
                if (x == bstart && w == 0.0) bstart += 1; else { k[n++] = w; ww += w; }
            }
            for (int i = n - 1; i >= 0; --i) { if (bend <= bstart || k[i] != 0.0) break; bend -= 1; }
        }
        if (ww != 0.0) for (int i = 0; i < n; ++i) k[i] /= ww;
        c.start[ox] = bstart; c.size[ox] = bend - bstart;
        for (int i = 0; i < c.window; ++i) if (first || k[i] > maxw) { maxw = k[i]; first = false; }
    }
    c.k.resize(kf.size());
    if (mode == MODE_PILLOW) {
        c.precision = 22;
        for (size_t i = 0; i < kf.size(); ++i)
            c.k[i] = kf[i] < 0 ? (int32_t)(-0.5 + kf[i] * (double)(1 << 22)) : (int32_t)(0.5 + kf[i] * (double)(1 << 22));
    } else {
        int precision = 0;
        for (int cur = 0; cur < 22; ++cur) {
            precision = cur;
            int32_t next = (int32_t)std::round(maxw * (double)(1 << (precision + 1)));
            if (next >= (1 << 15)) break;
        }
        c.precision = precision;
        double s = (double)((int64_t)1 << precision);
        for (size_t i = 0; i < kf.size(); ++i) c.k[i] = (int32_t)(int16_t)std::round(kf[i] * s);
    }
    return c;
}

inline uint8_t clip8(int32_t v, int precision) { v >>= precision; return (uint8_t)(v < 0 ? 0 : v > 255 ? 255 : v); }

// src rows [row0, row0 + rows) of a (sw x sh x C) image -> dst (out_w x rows x C)
void horiz_pass(const uint8_t* src, int sw, int C, int row0, int rows, uint8_t* dst, int out_w, const Coeffs& co) {
    for (int y = 0; y < rows; ++y) {
        const uint8_t* s = src + (size_t)(row0 + y) * sw * C;
        uint8_t* d = dst + (size_t)y * out_w * C;
        for (int x = 0; x < out_w; ++x) {
            const int32_t* k = &co.k[(size_t)x * co.window];
            for (int ch = 0; ch < C; ++ch) {
                int32_t ss = 1 << (co.precision - 1);
                for (int i = 0; i < co.size[x]; ++i) ss += k[i] * (int32_t)s[(size_t)(co.start[x] + i) * C + ch];
                d[(size_t)x * C + ch] = clip8(ss, co.precision);
            }
        }
    }
}

// src (w x ? x C), columns [col0, col0 + w_out) -> dst (w_out x out_h x C); co.start is relative to src row 0
void vert_pass(const uint8_t* src, int sw, int C, int col0, int w_out, uint8_t* dst, int out_h, const Coeffs& co) {
    for (int y = 0; y < out_h; ++y) {
        const int32_t* k = &co.k[(size_t)y * co.window];
        uint8_t* d = dst + (size_t)y * w_out * C;
        for (int x = 0; x < w_out * C; ++x) {
            int32_t ss = 1 << (co.precision - 1);
            for (int i = 0; i < co.size[y]; ++i) ss += k[i] * (int32_t)src[((size_t)(co.start[y] + i) * sw + col0) * C + x];
            d[x] = clip8(ss, co.precision);
        }
    }
}

// Alpha handling of fast_image_resize for 8-bit pixels with an alpha channel (U8x2 = luma + alpha, U8x4 = RGBA), which
// its Resizer applies around every convolution resize (`use_alpha`, on by default): colour channels are multiplied by
// alpha before the convolution and divided by it afterwards; alpha itself is convolved like any channel.  Restated from
// the crate's published scalar code (mul_div_255, and a 16-bit reciprocal table for the division); not checkable here.
inline uint8_t mul_div_255(uint32_t a, uint32_t b) { const uint32_t t = a * b + 128; return (uint8_t)(((t >> 8) + t) >> 8); }
inline uint32_t recip_alpha(uint32_t a) { return a ? ((255u * (1u << 17)) / a + 1) >> 1 : 0; }
inline uint8_t div_and_clip(uint32_t v, uint32_t recip) { const uint32_t r = (v * recip + (1u << 15)) >> 16; return (uint8_t)(r > 255 ? 255 : r); }

void alpha_multiply(uint8_t* px, size_t n, int C) {
    for (size_t i = 0; i < n; ++i) {
        uint8_t* q = px + i * C;
        for (int c = 0; c + 1 < C; ++c) q[c] = mul_div_255(q[c], q[C - 1]);
    }
}
void alpha_divide(uint8_t* px, size_t n, int C) {
    for (size_t i = 0; i < n; ++i) {
        uint8_t* q = px + i * C;
        const uint32_t r = recip_alpha(q[C - 1]);
        for (int c = 0; c + 1 < C; ++c) q[c] = div_and_clip(q[c], r);
    }
}

// One `Resizer::resize` call with Convolution(Lanczos3) and a floating-point source box.
void resample(const uint8_t* src, int sw, int sh, int C, double left, double top, double bw, double bh,
              uint8_t* dst, int dw, int dh, int mode) {
    bool need_h = (double)dw != bw || left != std::round(left);
    bool need_v = (double)dh != bh || top != std::round(top);
    std::vector<uint8_t> premultiplied;
    const bool alpha = (C == 2 || C == 4) && (need_h || need_v);  // a plain copy touches no pixel value
    if (alpha) {
        premultiplied.assign(src, src + (size_t)sw * sh * C);
        alpha_multiply(premultiplied.data(), (size_t)sw * sh, C);
        src = premultiplied.data();
    }
    if (need_h && need_v) {
        Coeffs hc = make_coeffs(sw, left, left + bw, dw, mode), vc = make_coeffs(sh, top, top + bh, dh, mode);
        int y_first = vc.start[0], y_last = vc.start[dh - 1] + vc.size[dh - 1];
        int tmp_h = y_last - y_first;
        std::vector<uint8_t> tmp((size_t)dw * tmp_h * C);
        horiz_pass(src, sw, C, y_first, tmp_h, tmp.data(), dw, hc);
        for (auto& s : vc.start) s -= y_first;
        vert_pass(tmp.data(), dw, C, 0, dw, dst, dh, vc);
    } else if (need_h) {
        Coeffs hc = make_coeffs(sw, left, left + bw, dw, mode);
        horiz_pass(src, sw, C, (int)top, dh, dst, dw, hc);
    } else if (need_v) {
        Coeffs vc = make_coeffs(sh, top, top + bh, dh, mode);
        vert_pass(src, sw, C, (int)left, dw, dst, dh, vc);
    } else {
        for (int y = 0; y < dh; ++y)
            memcpy(dst + (size_t)y * dw * C, src + ((size_t)((int)top + y) * sw + (int)left) * C, (size_t)dw * C);
    }
    if (alpha) alpha_divide(dst, (size_t)dw * dh, C);
}

}  // namespace

ORC_API int orc_resample(const uint8_t* src, int sw, int sh, int C, double left, double top, double bw, double bh,
                         uint8_t* dst, int dw, int dh, int mode) {
    if (sw <= 0 || sh <= 0 || dw <= 0 || dh <= 0 || C < 1 || C > 4) return -1;
    resample(src, sw, sh, C, left, top, bw, bh, dst, dw, dh, mode);
    return 0;
}

// Fixed-point weights of one axis, for comparing coefficient tables (returns the window).
ORC_API int orc_coeffs(int in_size, double in0, double in1, int out_size, int mode, int32_t* start, int32_t* size,
                       int32_t* k, int k_cap, int32_t* precision) {
    Coeffs c = make_coeffs(in_size, in0, in1, out_size, mode);
    for (int i = 0; i < out_size; ++i) { start[i] = c.start[i]; size[i] = c.size[i]; }
    for (int i = 0; i < (int)c.k.size() && i < k_cap; ++i) k[i] = c.k[i];
    *precision = c.precision;
    return c.window;
}

// crop_and_resize (image_processing.rs:254-338) on an interleaved u8 image with C channels.
// dst must hold target_w * target_h * C bytes (see orc_plan_geometry).
ORC_API int orc_crop_and_resize(uint32_t size, uint32_t ratio, double mn, double mx, const uint8_t* src, uint32_t w,
                                uint32_t h, int C, const char* forced_key, uint8_t* dst, orc_plan* plan, int mode) {
    orc_plan p;
    int rc = orc_plan_geometry(size, ratio, mn, mx, w, h, forced_key, &p);
    if (rc) return rc;
    if (plan) *plan = p;
    if (p.identity) { memcpy(dst, src, (size_t)w * h * C); return 0; }
    std::vector<uint8_t> mid((size_t)p.new_w * p.new_h * C);
    resample(src, (int)w, (int)h, C, 0.0, 0.0, (double)w, (double)h, mid.data(), (int)p.new_w, (int)p.new_h, mode);
    resample(mid.data(), (int)p.new_w, (int)p.new_h, C, p.crop_left, p.crop_top, p.crop_w, p.crop_h, dst,
             (int)p.target_w, (int)p.target_h, mode);
    return 0;
}

// convert_to_rgb8 (image_processing.rs:163-186), applied by image_to_payload after crop_and_resize when
// `img_to_rgb8` is set and the image is not RGB8 already (:366-372).
//   1 channel (Luma8): the `image` crate's to_rgb8 repeats the value in all three channels (pinned by :891-904);
//   2 channels (LumaA8): the same on the luma byte, alpha dropped;
//   3 channels: unchanged (:907-920);
//   4 channels (Rgba8): every pixel is composited over an opaque (128,128,128) background with the crate's
//     `Pixel::blend`: source-over in f32 on values scaled to 0..1, the result scaled back by 255 and converted to
//     u8 by truncation; alpha 255 copies the pixel, alpha 0 keeps the background.  The reference's own test
//     (:847-888) pins alpha 0 / 255 exactly and (200,100,50,128) -> (164,114,89) within 2; the f32 operation order
//     below is a restatement of the published algorithm, PARITY UNPINNED beyond that test.
// Compiled with -ffp-contract=off: every operation rounds once, as the Rust code does.
ORC_API int orc_to_rgb8(const uint8_t* src, uint64_t npx, int C, uint8_t* dst) {
    if (C < 1 || C > 4) return 1;
    const float max_t = 255.0f;
    for (uint64_t i = 0; i < npx; ++i) {
        const uint8_t* s = src + i * (uint64_t)C;
        uint8_t* d = dst + i * 3;
        if (C <= 2) { d[0] = d[1] = d[2] = s[0]; continue; }
        if (C == 3) { d[0] = s[0]; d[1] = s[1]; d[2] = s[2]; continue; }
        if (s[3] == 255) { d[0] = s[0]; d[1] = s[1]; d[2] = s[2]; continue; }
        if (s[3] == 0) { d[0] = d[1] = d[2] = 128; continue; }
        const float bg_a = 255.0f / max_t, fg_a = (float)s[3] / max_t;
        const float alpha_final = bg_a + fg_a - bg_a * fg_a;
        for (int c = 0; c < 3; ++c) {
            const float bg = 128.0f / max_t, fg = (float)s[c] / max_t;
            const float bg_pre = bg * bg_a, fg_pre = fg * fg_a;
            const float out_pre = fg_pre + bg_pre * (1.0f - fg_a);
            const float out = out_pre / alpha_final;
            d[c] = (uint8_t)(max_t * out);
        }
    }
    return 0;
}

// ---------------------------------------------------------------------------
// 3. Baseline JPEG decode
// ---------------------------------------------------------------------------
namespace {

const uint8_t ZIGZAG[64] = {0,  1,  8,  16, 9,  2,  3,  10, 17, 24, 32, 25, 18, 11, 4,  5,  12, 19, 26, 33, 40, 48,
                            41, 34, 27, 20, 13, 6,  7,  14, 21, 28, 35, 42, 49, 56, 57, 50, 43, 36, 29, 22, 15, 23,
                            30, 37, 44, 51, 58, 59, 52, 45, 38, 31, 39, 46, 53, 60, 61, 54, 47, 55, 62, 63};

struct HuffTable {
    bool present = false;
    uint8_t bits[17] = {0};
    uint8_t vals[256] = {0};
    int32_t mincode[17], maxcode[18], valptr[17];
    void build() {  // T.81 Annex C / F.2.2.3
        int code = 0, k = 0;
        for (int l = 1; l <= 16; ++l) {
            valptr[l] = k; mincode[l] = code;
            code += bits[l]; k += bits[l];
            maxcode[l] = bits[l] ? code - 1 : -1;
            code <<= 1;
        }
        maxcode[17] = 0x7fffffff;
    }
};

struct Component { int id, h, v, tq, td, ta; int bw, bh; /* blocks per row/col incl. MCU padding */ int dw, dh; /* real samples */ };

struct Jpeg {
    int width = 0, height = 0, ncomp = 0, hmax = 1, vmax = 1, mcux = 0, mcuy = 0, restart = 0;
    Component comp[3];
    uint16_t qt[4][64];  // natural order
    bool qt_present[4] = {false, false, false, false};
    HuffTable dc[4], ac[4];
    const uint8_t* scan = nullptr;
    size_t scan_len = 0;
};

enum { ORC_OK = 0, ORC_E_TRUNCATED = 1, ORC_E_BAD_MARKER = 2, ORC_E_UNSUPPORTED = 3, ORC_E_BAD_TABLE = 4, ORC_E_BAD_CODE = 5 };

int parse_headers(const uint8_t* d, size_t n, Jpeg& j) {
    if (n < 4 || d[0] != 0xFF || d[1] != 0xD8) return ORC_E_BAD_MARKER;
    size_t p = 2;
    bool have_sof = false;
    while (true) {
        if (p + 4 > n) return ORC_E_TRUNCATED;
        if (d[p] != 0xFF) return ORC_E_BAD_MARKER;
        while (p < n && d[p] == 0xFF) ++p;  // fill bytes
        if (p >= n) return ORC_E_TRUNCATED;
        uint8_t m = d[p++];
        if (m == 0xD8 || (m >= 0xD0 && m <= 0xD7) || m == 0x01) continue;
        if (m == 0xD9) return ORC_E_TRUNCATED;
        if (p + 2 > n) return ORC_E_TRUNCATED;
        size_t len = ((size_t)d[p] << 8) | d[p + 1];
        if (len < 2 || p + len > n) return ORC_E_TRUNCATED;
        const uint8_t* s = d + p + 2;
        size_t sl = len - 2;
        if (m == 0xDB) {  // DQT
            size_t q = 0;
            while (q < sl) {
                int pq = s[q] >> 4, tq = s[q] & 15; ++q;
                if (tq > 3 || pq > 1) return ORC_E_BAD_TABLE;
                if (q + (pq ? 128 : 64) > sl) return ORC_E_TRUNCATED;
                for (int i = 0; i < 64; ++i) {
                    uint16_t v = pq ? (uint16_t)((s[q] << 8) | s[q + 1]) : s[q];
                    q += pq ? 2 : 1;
                    j.qt[tq][ZIGZAG[i]] = v;
                }
                j.qt_present[tq] = true;
            }
        } else if (m == 0xC4) {  // DHT
            size_t q = 0;
            while (q < sl) {
                if (q + 17 > sl) return ORC_E_TRUNCATED;
                int tc = s[q] >> 4, th = s[q] & 15; ++q;
                if (tc > 1 || th > 3) return ORC_E_BAD_TABLE;
                HuffTable& t = tc ? j.ac[th] : j.dc[th];
                int total = 0;
                t.bits[0] = 0;
                for (int i = 1; i <= 16; ++i) { t.bits[i] = s[q++]; total += t.bits[i]; }
                if (total > 256 || q + total > sl) return ORC_E_BAD_TABLE;
                memset(t.vals, 0, sizeof t.vals);
                for (int i = 0; i < total; ++i) t.vals[i] = s[q++];
                t.build(); t.present = true;
            }
        } else if (m == 0xC0 || m == 0xC1) {  // SOF0 / SOF1 (sequential Huffman)
            if (sl < 6) return ORC_E_TRUNCATED;
            if (s[0] != 8) return ORC_E_UNSUPPORTED;
            j.height = (s[1] << 8) | s[2]; j.width = (s[3] << 8) | s[4]; j.ncomp = s[5];
            if (j.width == 0 || j.height == 0) return ORC_E_UNSUPPORTED;
            if (j.ncomp != 1 && j.ncomp != 3) return ORC_E_UNSUPPORTED;
            if (sl < (size_t)(6 + 3 * j.ncomp)) return ORC_E_TRUNCATED;
            for (int i = 0; i < j.ncomp; ++i) {
                Component& c = j.comp[i];
                c.id = s[6 + 3 * i]; c.h = s[7 + 3 * i] >> 4; c.v = s[7 + 3 * i] & 15; c.tq = s[8 + 3 * i];
                if (c.h < 1 || c.h > 2 || c.v < 1 || c.v > 2 || c.tq > 3) return ORC_E_UNSUPPORTED;
            }
            if (j.ncomp == 1) { j.comp[0].h = j.comp[0].v = 1; }  // a single-component scan is never interleaved
            else if (j.comp[1].h != 1 || j.comp[1].v != 1 || j.comp[2].h != 1 || j.comp[2].v != 1) return ORC_E_UNSUPPORTED;
            j.hmax = j.comp[0].h; j.vmax = j.comp[0].v;
            j.mcux = (j.width + 8 * j.hmax - 1) / (8 * j.hmax);
            j.mcuy = (j.height + 8 * j.vmax - 1) / (8 * j.vmax);
            for (int i = 0; i < j.ncomp; ++i) {
                Component& c = j.comp[i];
                c.bw = j.mcux * c.h; c.bh = j.mcuy * c.v;
                c.dw = (j.width * c.h + j.hmax - 1) / j.hmax; c.dh = (j.height * c.v + j.vmax - 1) / j.vmax;
            }
            have_sof = true;
        } else if (m >= 0xC2 && m <= 0xCF && m != 0xC4 && m != 0xC8 && m != 0xCC) {
            return ORC_E_UNSUPPORTED;  // progressive, lossless, arithmetic
        } else if (m == 0xDD) {
            if (sl < 2) return ORC_E_TRUNCATED;
            j.restart = (s[0] << 8) | s[1];
        } else if (m == 0xDA) {  // SOS
            if (!have_sof) return ORC_E_BAD_MARKER;
            if (sl < 1 || s[0] != j.ncomp || sl < (size_t)(4 + 2 * j.ncomp)) return ORC_E_UNSUPPORTED;
            for (int i = 0; i < j.ncomp; ++i) {
                if (s[1 + 2 * i] != j.comp[i].id) return ORC_E_UNSUPPORTED;
                j.comp[i].td = s[2 + 2 * i] >> 4; j.comp[i].ta = s[2 + 2 * i] & 15;
                if (j.comp[i].td > 3 || j.comp[i].ta > 3 || !j.dc[j.comp[i].td].present || !j.ac[j.comp[i].ta].present) return ORC_E_BAD_TABLE;
                if (!j.qt_present[j.comp[i].tq]) return ORC_E_BAD_TABLE;
            }
            j.scan = d + p + len; j.scan_len = n - (p + len);
            return ORC_OK;
        }
        p += len;
    }
}

struct BitReader {
    const uint8_t* d; size_t n, p = 0;
    uint32_t acc = 0; int cnt = 0;
    bool hit_marker = false; uint8_t marker = 0;
    BitReader(const uint8_t* d_, size_t n_) : d(d_), n(n_) {}
    void fill() {
        while (cnt <= 24) {
            uint32_t b = 0;
            if (!hit_marker && p < n) {
                b = d[p];
                if (b == 0xFF) {
                    size_t q = p + 1;
                    while (q < n && d[q] == 0xFF) ++q;
                    uint8_t nx = q < n ? d[q] : 0xD9;
                    if (nx == 0) p = q + 1;
                    else { hit_marker = true; marker = nx; b = 0; }
                } else ++p;
            }
            acc |= b << (24 - cnt); cnt += 8;
        }
    }
    int bits(int k) { if (k == 0) return 0; fill(); int v = (int)(acc >> (32 - k)); acc <<= k; cnt -= k; return v; }
    int peek16() { fill(); return (int)(acc >> 16); }
    void skip(int k) { acc <<= k; cnt -= k; }
    // byte-align and consume an RSTn marker
    bool restart() {
        acc = 0; cnt = 0;
        if (!hit_marker) {  // stuffed stream did not stop at a marker yet: look for it
            while (p + 1 < n && !(d[p] == 0xFF && d[p + 1] >= 0xD0 && d[p + 1] <= 0xD7)) ++p;
            if (p + 1 >= n) return false;
            p += 2; return true;
        }
        if (marker < 0xD0 || marker > 0xD7) return false;
        while (p < n && d[p] == 0xFF) ++p;
        ++p; hit_marker = false; return true;
    }
};

int decode_symbol(BitReader& br, const HuffTable& t) {  // T.81 F.2.2.3 DECODE
    int look = br.peek16(), code = 0;
    for (int l = 1; l <= 16; ++l) {
        code = look >> (16 - l);
        if (t.maxcode[l] >= 0 && code <= t.maxcode[l] && code >= t.mincode[l]) {
            br.skip(l);
            return t.vals[t.valptr[l] + code - t.mincode[l]];
        }
    }
    return -1;
}

inline int extend(int v, int s) { return v < (1 << (s - 1)) ? v - (1 << s) + 1 : v; }

// Entropy-decode every block.  coef[c] holds bw*bh blocks of 64 int16 in natural order.
int decode_scan(const Jpeg& j, std::vector<int16_t> coef[3]) {
    BitReader br(j.scan, j.scan_len);
    int pred[3] = {0, 0, 0};
    int total = j.mcux * j.mcuy;
    for (int c = 0; c < j.ncomp; ++c) coef[c].assign((size_t)j.comp[c].bw * j.comp[c].bh * 64, 0);
    for (int m = 0; m < total; ++m) {
        if (j.restart && m && m % j.restart == 0) {
            if (!br.restart()) return ORC_E_TRUNCATED;
            pred[0] = pred[1] = pred[2] = 0;
        }
        int my = m / j.mcux, mx = m % j.mcux;
        for (int c = 0; c < j.ncomp; ++c) {
            const Component& cp = j.comp[c];
            for (int by = 0; by < cp.v; ++by)
                for (int bx = 0; bx < cp.h; ++bx) {
                    int16_t* blk = &coef[c][((size_t)(my * cp.v + by) * cp.bw + (mx * cp.h + bx)) * 64];
                    int s = decode_symbol(br, j.dc[cp.td]);
                    if (s < 0 || s > 11) return ORC_E_BAD_CODE;
                    int diff = s ? extend(br.bits(s), s) : 0;
                    pred[c] += diff;
                    blk[0] = (int16_t)pred[c];
                    for (int k = 1; k < 64;) {
                        int rs = decode_symbol(br, j.ac[cp.ta]);
                        if (rs < 0) return ORC_E_BAD_CODE;
                        int r = rs >> 4, sz = rs & 15;
                        if (sz == 0) { if (r == 15) { k += 16; continue; } break; }
                        k += r;
                        if (k > 63) return ORC_E_BAD_CODE;
                        blk[ZIGZAG[k]] = (int16_t)extend(br.bits(sz), sz);
                        ++k;
                    }
                }
        }
    }
    return ORC_OK;
}

// Reconstruction variants.  The default (0, 0, 0) is the libjpeg family, which the test-suite pins bit-exactly against
// libjpeg-turbo.  zune-jpeg, the decoder datago links, is not available here; the alternatives below are the other
// published choices for the three steps whose arithmetic differs between baseline decoders, so that the distance
// between the families can be measured (tests/test_oracle_variants.py prints and bounds it).
//   idct:     0 = 13-bit "islow" (libjpeg jidctint);  1 = 12-bit constants, rounding 512 >> 10 after the column pass and
//             65536 + (128 << 17) >> 17 after the row pass (the stb_image factorisation, which zune-jpeg's scalar IDCT
//             is understood to follow)
//   upsample: 0 = one rounding per sample, (3 * (3 near + far) + (3 near' + far') + 8 or 7) >> 4 (libjpeg "fancy" h2v2);
//             1 = two passes with an 8-bit intermediate, (3 near + far + 2) >> 2 vertically, then the same horizontally;
//             2 = one rounding with the bias 8 in both phases (stb_image)
//   colour:   0 = 16-bit constants 91881 / 22554 / 46802 / 116130, rounding 32768 per chroma term (libjpeg);
//             1 = 14-bit constants 22970 / 5638 / 11700 / 29032 on Y * 16384 with one rounding of 8192
struct Variant { int idct = 0, upsample = 0, color = 0; };
thread_local Variant g_variant;

// 12-bit IDCT of the stb_image family: dequantise, columns (round 512, shift 10), rows (round 65536 + (128 << 17), shift 17).
void idct_stb12(const int16_t* in, const uint16_t* q, uint8_t* out, int stride) {
    auto f2f = [](double x) { return (int32_t)(x * 4096.0 + 0.5); };
    int32_t val[64];
    auto kernel = [&](int32_t s0, int32_t s1, int32_t s2, int32_t s3, int32_t s4, int32_t s5, int32_t s6, int32_t s7,
                      int32_t& x0, int32_t& x1, int32_t& x2, int32_t& x3, int32_t& t0, int32_t& t1, int32_t& t2, int32_t& t3) {
        int32_t p2 = s2, p3 = s6;
        int32_t p1 = (p2 + p3) * f2f(0.5411961);
        t2 = p1 + p3 * f2f(-1.847759065);
        t3 = p1 + p2 * f2f(0.765366865);
        p2 = s0; p3 = s4;
        t0 = (p2 + p3) * 4096;
        t1 = (p2 - p3) * 4096;
        x0 = t0 + t3; x3 = t0 - t3; x1 = t1 + t2; x2 = t1 - t2;
        t0 = s7; t1 = s5; t2 = s3; t3 = s1;
        p3 = t0 + t2;
        int32_t p4 = t1 + t3;
        p1 = t0 + t3; p2 = t1 + t2;
        int32_t p5 = (p3 + p4) * f2f(1.175875602);
        t0 = t0 * f2f(0.298631336); t1 = t1 * f2f(2.053119869); t2 = t2 * f2f(3.072711026); t3 = t3 * f2f(1.501321110);
        p1 = p5 + p1 * f2f(-0.899976223); p2 = p5 + p2 * f2f(-2.562915447);
        p3 = p3 * f2f(-1.961570560); p4 = p4 * f2f(-0.390180644);
        t3 += p1 + p4; t2 += p2 + p3; t1 += p2 + p4; t0 += p1 + p3;
    };
    for (int i = 0; i < 8; ++i) {
        int32_t s[8];
        for (int r = 0; r < 8; ++r) s[r] = (int32_t)in[r * 8 + i] * (int32_t)q[r * 8 + i];
        int32_t x0, x1, x2, x3, t0, t1, t2, t3;
        kernel(s[0], s[1], s[2], s[3], s[4], s[5], s[6], s[7], x0, x1, x2, x3, t0, t1, t2, t3);
        x0 += 512; x1 += 512; x2 += 512; x3 += 512;
        val[i] = (x0 + t3) >> 10; val[56 + i] = (x0 - t3) >> 10;
        val[8 + i] = (x1 + t2) >> 10; val[48 + i] = (x1 - t2) >> 10;
        val[16 + i] = (x2 + t1) >> 10; val[40 + i] = (x2 - t1) >> 10;
        val[24 + i] = (x3 + t0) >> 10; val[32 + i] = (x3 - t0) >> 10;
    }
    for (int i = 0; i < 8; ++i) {
        const int32_t* v = val + i * 8;
        int32_t x0, x1, x2, x3, t0, t1, t2, t3;
        kernel(v[0], v[1], v[2], v[3], v[4], v[5], v[6], v[7], x0, x1, x2, x3, t0, t1, t2, t3);
        const int32_t rnd = 65536 + (128 << 17);
        x0 += rnd; x1 += rnd; x2 += rnd; x3 += rnd;
        auto c8 = [](int32_t x) { return (uint8_t)(x < 0 ? 0 : x > 255 ? 255 : x); };
        uint8_t* o = out + i * stride;
        o[0] = c8((x0 + t3) >> 17); o[7] = c8((x0 - t3) >> 17);
        o[1] = c8((x1 + t2) >> 17); o[6] = c8((x1 - t2) >> 17);
        o[2] = c8((x2 + t1) >> 17); o[5] = c8((x2 - t1) >> 17);
        o[3] = c8((x3 + t0) >> 17); o[4] = c8((x3 - t0) >> 17);
    }
}

// 13-bit "islow" integer IDCT with dequantisation, +128 and clamp.
void idct_islow(const int16_t* in, const uint16_t* q, uint8_t* out, int stride) {
    const int CB = 13, P1 = 2;
    const int32_t F_0_298 = 2446, F_0_390 = 3196, F_0_541 = 4433, F_0_765 = 6270, F_0_899 = 7373, F_1_175 = 9633,
                  F_1_501 = 12299, F_1_847 = 15137, F_1_961 = 16069, F_2_053 = 16819, F_2_562 = 20995, F_3_072 = 25172;
    int32_t ws[64];
    for (int pass = 0; pass < 2; ++pass) {
        for (int i = 0; i < 8; ++i) {
            int32_t x[8];
            if (pass == 0) for (int r = 0; r < 8; ++r) x[r] = (int32_t)in[r * 8 + i] * (int32_t)q[r * 8 + i];
            else for (int r = 0; r < 8; ++r) x[r] = ws[i * 8 + r];
            int32_t z2 = x[2], z3 = x[6];
            int32_t z1 = (z2 + z3) * F_0_541;
            int32_t tmp2 = z1 + z3 * (-F_1_847), tmp3 = z1 + z2 * F_0_765;
            int32_t tmp0 = (int32_t)((uint32_t)(x[0] + x[4]) << CB), tmp1 = (int32_t)((uint32_t)(x[0] - x[4]) << CB);
            int32_t tmp10 = tmp0 + tmp3, tmp13 = tmp0 - tmp3, tmp11 = tmp1 + tmp2, tmp12 = tmp1 - tmp2;
            tmp0 = x[7]; tmp1 = x[5]; tmp2 = x[3]; tmp3 = x[1];
            z1 = tmp0 + tmp3; z2 = tmp1 + tmp2; z3 = tmp0 + tmp2; int32_t z4 = tmp1 + tmp3;
            int32_t z5 = (z3 + z4) * F_1_175;
            tmp0 *= F_0_298; tmp1 *= F_2_053; tmp2 *= F_3_072; tmp3 *= F_1_501;
            z1 *= -F_0_899; z2 *= -F_2_562; z3 *= -F_1_961; z4 *= -F_0_390;
            z3 += z5; z4 += z5;
            tmp0 += z1 + z3; tmp1 += z2 + z4; tmp2 += z2 + z3; tmp3 += z1 + z4;
            int32_t o[8] = {tmp10 + tmp3, tmp11 + tmp2, tmp12 + tmp1, tmp13 + tmp0,
                            tmp13 - tmp0, tmp12 - tmp1, tmp11 - tmp2, tmp10 - tmp3};
            if (pass == 0) {
                int sh = CB - P1;
                for (int r = 0; r < 8; ++r) ws[r * 8 + i] = (o[r] + (1 << (sh - 1))) >> sh;
            } else {
                int sh = CB + P1 + 3;
                for (int r = 0; r < 8; ++r) {
                    int32_t v = ((o[r] + (1 << (sh - 1))) >> sh) + 128;
                    out[i * stride + r] = (uint8_t)(v < 0 ? 0 : v > 255 ? 255 : v);
                }
            }
        }
    }
}

inline uint8_t clamp8(int v) { return (uint8_t)(v < 0 ? 0 : v > 255 ? 255 : v); }

struct Decoded {
    Jpeg j;
    std::vector<int16_t> coef[3];
    std::vector<uint8_t> plane[3];  // MCU-padded, pitch = bw*8
};

int decode_to_planes(const uint8_t* d, size_t n, Decoded& o) {
    int rc = parse_headers(d, n, o.j);
    if (rc) return rc;
    rc = decode_scan(o.j, o.coef);
    if (rc) return rc;
    for (int c = 0; c < o.j.ncomp; ++c) {
        const Component& cp = o.j.comp[c];
        int pitch = cp.bw * 8;
        o.plane[c].assign((size_t)pitch * cp.bh * 8, 0);
        for (int by = 0; by < cp.bh; ++by)
            for (int bx = 0; bx < cp.bw; ++bx)
                (g_variant.idct == 1 ? idct_stb12 : idct_islow)(&o.coef[c][((size_t)by * cp.bw + bx) * 64], o.j.qt[cp.tq], &o.plane[c][(size_t)by * 8 * pitch + bx * 8], pitch);
    }
    return ORC_OK;
}

// Full-resolution chroma sample (x, y) from a subsampled plane, triangle filter with edge replication
// at the real (not MCU-padded) sample extent.
struct Upsampler {
    const uint8_t* p; int pitch, dw, dh, h, v;  // h, v: luma/chroma ratio per axis (1 or 2)
    int colsum(int cx, int y) const {  // vertical step: 3*near + far (v == 2) or 4*sample scaled like it
        if (v == 1) return p[(size_t)y * pitch + cx];
        int cy = y >> 1, far = (y & 1) ? cy + 1 : cy - 1;
        if (far < 0) far = 0;
        if (far > dh - 1) far = dh - 1;
        return 3 * p[(size_t)cy * pitch + cx] + p[(size_t)far * pitch + cx];
    }
    // two-pass variant: the vertical step rounds to 8 bits on its own
    int vround(int cx, int y) const { return v == 1 ? p[(size_t)y * pitch + cx] : (colsum(cx, y) + 2) >> 2; }
    int at(int x, int y) const {
        if (h == 1 && v == 1) return p[(size_t)y * pitch + x];
        if (h == 2 && dw <= 2) return p[(size_t)(y / v) * pitch + (x >> 1)];  // libjpeg replicates when the plane is <= 2 wide
        if (g_variant.upsample == 1) {
            if (h == 1) return vround(x, y);
            const int cx = x >> 1, t = vround(cx, y);
            const int nb = (x & 1) ? std::min(cx + 1, dw - 1) : std::max(cx - 1, 0);
            return (3 * t + vround(nb, y) + 2) >> 2;
        }
        if (g_variant.upsample == 2 && h == 2 && v == 2) {
            const int cx = x >> 1, t = colsum(cx, y);
            const int nb = (x & 1) ? std::min(cx + 1, dw - 1) : std::max(cx - 1, 0);
            return (3 * t + colsum(nb, y) + 8) >> 4;
        }
        if (h == 1) return (colsum(x, y) + ((y & 1) ? 2 : 1)) >> 2;  // h1v2: bias 1 on the upper row, 2 on the lower
        int cx = x >> 1;
        if (v == 1) {  // h2v1
            int t = p[(size_t)y * pitch + cx];
            if (x & 1) return cx == dw - 1 ? t : (3 * t + p[(size_t)y * pitch + cx + 1] + 2) >> 2;
            return cx == 0 ? t : (3 * t + p[(size_t)y * pitch + cx - 1] + 1) >> 2;
        }
        int t = colsum(cx, y);
        if (x & 1) {
            if (cx == dw - 1 && dw > 1) return (t * 4 + 7) >> 4;
            return (t * 3 + colsum(cx + 1, y) + 7) >> 4;  // dw == 1 reads the padded neighbour, as libjpeg does
        }
        if (cx == 0) return (t * 4 + 8) >> 4;
        return (t * 3 + colsum(cx - 1, y) + 8) >> 4;
    }
};

int decode_rgb(const uint8_t* d, size_t n, uint8_t* out, Decoded& o) {
    int rc = decode_to_planes(d, n, o);
    if (rc) return rc;
    const Jpeg& j = o.j;
    int W = j.width, H = j.height;
    if (j.ncomp == 1) {
        int pitch = j.comp[0].bw * 8;
        for (int y = 0; y < H; ++y) memcpy(out + (size_t)y * W, &o.plane[0][(size_t)y * pitch], W);
        return ORC_OK;
    }
    Upsampler ub{o.plane[1].data(), j.comp[1].bw * 8, j.comp[1].dw, j.comp[1].dh, j.hmax, j.vmax};
    Upsampler ur{o.plane[2].data(), j.comp[2].bw * 8, j.comp[2].dw, j.comp[2].dh, j.hmax, j.vmax};
    int ypitch = j.comp[0].bw * 8;
    for (int y = 0; y < H; ++y)
        for (int x = 0; x < W; ++x) {
            int Y = o.plane[0][(size_t)y * ypitch + x];
            int cb = ub.at(x, y) - 128, cr = ur.at(x, y) - 128;
            // 16-bit fixed point: 1.40200, 0.34414, 0.71414, 1.77200
            int r = Y + ((91881 * cr + 32768) >> 16);
            int g = Y + ((-22554 * cb - 46802 * cr + 32768) >> 16);
            int b = Y + ((116130 * cb + 32768) >> 16);
            if (g_variant.color == 1) {  // 14-bit constants, one rounding
                r = (Y * 16384 + 22970 * cr + 8192) >> 14;
                g = (Y * 16384 - 5638 * cb - 11700 * cr + 8192) >> 14;
                b = (Y * 16384 + 29032 * cb + 8192) >> 14;
            }
            uint8_t* px = out + ((size_t)y * W + x) * 3;
            px[0] = clamp8(r); px[1] = clamp8(g); px[2] = clamp8(b);
        }
    return ORC_OK;
}

}  // namespace

struct orc_jpeg_info_t {
    int32_t width, height, channels;  // channels of the decoded image: 3 (RGB) or 1 (L)
    int32_t hsamp, vsamp;             // luma sampling factors
    int32_t mcux, mcuy, restart_interval;
    int32_t blocks[3];                // MCU-padded block counts per component
};

ORC_API int orc_jpeg_info(const uint8_t* d, size_t n, orc_jpeg_info_t* info) {
    Jpeg j;
    int rc = parse_headers(d, n, j);
    if (rc) return rc;
    memset(info, 0, sizeof *info);
    info->width = j.width; info->height = j.height; info->channels = j.ncomp == 1 ? 1 : 3;
    info->hsamp = j.hmax; info->vsamp = j.vmax; info->mcux = j.mcux; info->mcuy = j.mcuy; info->restart_interval = j.restart;
    for (int c = 0; c < j.ncomp; ++c) info->blocks[c] = j.comp[c].bw * j.comp[c].bh;
    return 0;
}

// Decode to interleaved RGB (3 components) or L (1 component); out holds width*height*channels bytes.
ORC_API int orc_jpeg_decode(const uint8_t* d, size_t n, uint8_t* out) {
    Decoded o;
    return decode_rgb(d, n, out, o);
}

// Decode with another published choice for the IDCT, the chroma upsampling and the colour constants (see Variant); used
// only to measure how far the decoder families lie apart.
ORC_API int orc_jpeg_decode_variant(const uint8_t* d, size_t n, uint8_t* out, int idct, int upsample, int color) {
    g_variant = Variant{idct, upsample, color};
    Decoded o;
    const int rc = decode_rgb(d, n, out, o);
    g_variant = Variant{};
    return rc;
}

// Stage outputs for kernel-by-kernel parity: coefficients in scan order per component (blocks raster order within
// the component, natural order within a block) and the MCU-padded 8-bit planes after the IDCT.
ORC_API int orc_jpeg_decode_stages(const uint8_t* d, size_t n, int16_t* coef0, int16_t* coef1, int16_t* coef2,
                                   uint8_t* plane0, uint8_t* plane1, uint8_t* plane2, uint8_t* out) {
    Decoded o;
    std::vector<uint8_t> tmp;
    if (!out) {
        Jpeg j;
        int rc = parse_headers(d, n, j);
        if (rc) return rc;
        tmp.resize((size_t)j.width * j.height * 3);
        out = tmp.data();
    }
    int rc = decode_rgb(d, n, out, o);
    if (rc) return rc;
    int16_t* cs[3] = {coef0, coef1, coef2};
    uint8_t* ps[3] = {plane0, plane1, plane2};
    for (int c = 0; c < o.j.ncomp; ++c) {
        if (cs[c]) memcpy(cs[c], o.coef[c].data(), o.coef[c].size() * 2);
        if (ps[c]) memcpy(ps[c], o.plane[c].data(), o.plane[c].size());
    }
    return 0;
}

// image_to_payload (image_processing.rs:341-431) for a JPEG: decode, then crop_and_resize when size > 0.
// out must hold target_w*target_h*channels (or width*height*channels without a transform).
ORC_API int orc_jpeg_to_payload(const uint8_t* d, size_t n, uint32_t size, uint32_t ratio, double mn, double mx,
                                const char* forced_key, uint8_t* out, orc_plan* plan, int mode) {
    Jpeg j;
    int rc = parse_headers(d, n, j);
    if (rc) return rc;
    int C = j.ncomp == 1 ? 1 : 3;
    if (size == 0) { Decoded o; return decode_rgb(d, n, out, o); }
    std::vector<uint8_t> full((size_t)j.width * j.height * C);
    { Decoded o; rc = decode_rgb(d, n, full.data(), o); if (rc) return rc; }
    return orc_crop_and_resize(size, ratio, mn, mx, full.data(), (uint32_t)j.width, (uint32_t)j.height, C, forced_key, out, plan, mode);
}

// ---------------------------------------------------------------------------
// 4. Sharding
// ---------------------------------------------------------------------------
// generator_files.rs:24-42
ORC_API int orc_rank_slice(uint64_t quorum, uint64_t rank, uint64_t world, uint64_t* start, uint64_t* end) {
    if (world == 0 || rank >= world) return -1;
    uint64_t chunk = quorum / world, rem = quorum % world;
    *start = rank < rem ? rank * (chunk + 1) : rem * (chunk + 1) + (rank - rem) * chunk;
    *end = (rank + 1) <= rem ? (rank + 1) * (chunk + 1) : rem * (chunk + 1) + (rank + 1 - rem) * chunk;
    return 0;
}

namespace {
inline uint64_t rotl(uint64_t x, int b) { return (x << b) | (x >> (64 - b)); }
struct Sip13 {
    uint64_t v0 = 0x736f6d6570736575ULL, v1 = 0x646f72616e646f6dULL, v2 = 0x6c7967656e657261ULL, v3 = 0x7465646279746573ULL;
    void round() {
        v0 += v1; v1 = rotl(v1, 13); v1 ^= v0; v0 = rotl(v0, 32);
        v2 += v3; v3 = rotl(v3, 16); v3 ^= v2;
        v0 += v3; v3 = rotl(v3, 21); v3 ^= v0;
        v2 += v1; v1 = rotl(v1, 17); v1 ^= v2; v2 = rotl(v2, 32);
    }
};
}  // namespace

// SipHash-c-d of `n` bytes under key (k0, k1).  Exposed so that the test-suite can pin the construction with
// the published SipHash-2-4 vectors; the shard rule uses c=1, d=3, key (0,0).
ORC_API uint64_t orc_siphash(uint64_t k0, uint64_t k1, int c_rounds, int d_rounds, const uint8_t* m, size_t n) {
    Sip13 s;
    s.v0 ^= k0; s.v1 ^= k1; s.v2 ^= k0; s.v3 ^= k1;
    size_t i = 0;
    for (; i + 8 <= n; i += 8) {
        uint64_t w = 0;
        for (int b = 0; b < 8; ++b) w |= (uint64_t)m[i + b] << (8 * b);
        s.v3 ^= w;
        for (int r = 0; r < c_rounds; ++r) s.round();
        s.v0 ^= w;
    }
    uint64_t last = (uint64_t)(n & 0xff) << 56;
    for (int b = 0; i + b < n; ++b) last |= (uint64_t)m[i + b] << (8 * b);
    s.v3 ^= last;
    for (int r = 0; r < c_rounds; ++r) s.round();
    s.v0 ^= last;
    s.v2 ^= 0xff;
    for (int r = 0; r < d_rounds; ++r) s.round();
    return s.v0 ^ s.v1 ^ s.v2 ^ s.v3;
}

// Rust's DefaultHasher over a `str`: SipHash-1-3, key (0,0), the bytes followed by one 0xFF byte.
ORC_API uint64_t orc_key_hash(const uint8_t* key, size_t len) {
    std::vector<uint8_t> m(key, key + len);
    m.push_back(0xFF);
    return orc_siphash(0, 0, 1, 3, m.data(), m.size());
}

// ---------------------------------------------------------------------------
// 5. Multi-threaded driver: the timed CPU baseline (one worker per requested thread, as the reference's
//    tokio pool with DATAGO_MAX_TASKS = cores, src/worker_files.rs:83-88,150-152)
// ---------------------------------------------------------------------------
struct orc_item {
    const uint8_t* data;  // JPEG bytes, or raw interleaved pixels when raw_w > 0
    uint64_t len;
    uint32_t raw_w, raw_h, raw_c;
    uint32_t pad;
};

// kind 0: decode only; 1: decode + crop_and_resize; 2: raw crop_and_resize.  Outputs are produced into
// per-thread scratch and discarded (checksummed into *sink so the work cannot be optimised away).
ORC_API int orc_run_batch(const orc_item* items, int n, int kind, uint32_t size, uint32_t ratio, double mn, double mx,
                          int threads, uint64_t* ok_count, uint64_t* sink) {
    std::atomic<int> next{0};
    std::atomic<uint64_t> ok{0}, acc{0};
    auto work = [&]() {
        std::vector<uint8_t> out;
        for (;;) {
            int i = next.fetch_add(1);
            if (i >= n) break;
            const orc_item& it = items[i];
            int rc;
            if (kind == 2) {
                orc_plan p;
                if (orc_plan_geometry(size, ratio, mn, mx, it.raw_w, it.raw_h, nullptr, &p)) continue;
                out.resize((size_t)p.target_w * p.target_h * it.raw_c);
                rc = orc_crop_and_resize(size, ratio, mn, mx, it.data, it.raw_w, it.raw_h, (int)it.raw_c, nullptr, out.data(), nullptr, MODE_FIR);
            } else {
                orc_jpeg_info_t info;
                if (orc_jpeg_info(it.data, it.len, &info)) continue;
                size_t need = (size_t)info.width * info.height * info.channels;
                if (kind == 1) {
                    orc_plan p;
                    if (orc_plan_geometry(size, ratio, mn, mx, info.width, info.height, nullptr, &p)) continue;
                    need = (size_t)p.target_w * p.target_h * info.channels;
                }
                out.resize(need);
                rc = orc_jpeg_to_payload(it.data, it.len, kind == 1 ? size : 0, ratio, mn, mx, nullptr, out.data(), nullptr, MODE_FIR);
            }
            if (rc == 0) { ok.fetch_add(1); acc.fetch_add(out[out.size() / 2] + out[0]); }
        }
    };
    std::vector<std::thread> pool;
    for (int t = 0; t < threads; ++t) pool.emplace_back(work);
    for (auto& t : pool) t.join();
    *ok_count = ok.load();
    if (sink) *sink = acc.load();
    return 0;
}
