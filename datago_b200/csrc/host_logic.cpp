// Host-side planning for the image path: everything datago decides per sample before pixels move.
#include <algorithm>
#include <cmath>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <unordered_map>

#include "host.h"

namespace dg {

// ---------------------------------------------------------------------------------------------------------------
// Buckets.  datago: ImageTransformConfig::get_ar_aware_transform (src/image_processing.rs:77-120),
// build_image_size_list (:188-219), get_closest_aspect_ratio (:222-252), crop_and_resize (:259-310).
// All arithmetic is IEEE double, as in the Rust source, so the results are bit-identical.
// ---------------------------------------------------------------------------------------------------------------
bool config_valid(const dg_image_config& c) {
    return c.crop_and_resize && c.default_image_size > 0 && c.downsampling_ratio > 0 && c.min_aspect_ratio > 0.0 &&
           c.max_aspect_ratio >= c.min_aspect_ratio;
}

void format_key(uint32_t w, uint32_t h, char out[16]) {
    // Rust's {:.3} and C's %.3f both round the exact binary value to three decimals.
    snprintf(out, 16, "%.3f", (double)w / (double)h);
}

std::vector<std::pair<uint32_t, uint32_t>> image_size_list(const dg_image_config& c) {
    std::vector<std::pair<uint32_t, uint32_t>> sizes;
    const uint32_t ratio = c.downsampling_ratio;
    const uint32_t patch = c.default_image_size / ratio;
    const double area = (double)(uint32_t)(patch * patch);
    // patch widths first, then patch heights: the same (w, h) may be listed twice
    uint32_t lo = (uint32_t)std::ceil(std::sqrt(area * c.min_aspect_ratio));
    uint32_t hi = (uint32_t)std::floor(std::sqrt(area * c.max_aspect_ratio));
    for (uint32_t pw = lo; pw <= hi; ++pw) sizes.emplace_back(pw * ratio, (uint32_t)std::floor(area / (double)pw) * ratio);
    lo = (uint32_t)std::ceil(std::sqrt(area / c.max_aspect_ratio));
    hi = (uint32_t)std::floor(std::sqrt(area / c.min_aspect_ratio));
    for (uint32_t ph = lo; ph <= hi; ++ph) sizes.emplace_back((uint32_t)std::floor(area / (double)ph) * ratio, ph * ratio);
    return sizes;
}

Transform make_transform(const dg_image_config& c) {
    // HashMap<String, (u32, u32)> with insert(): a later size replaces an earlier one under the same key
    std::unordered_map<std::string, std::pair<uint32_t, uint32_t>> by_key;
    for (const auto& wh : image_size_list(c)) {
        char key[16];
        format_key(wh.first, wh.second, key);
        by_key[key] = wh;
    }
    Transform t;
    for (const auto& kv : by_key) {
        BucketEntry e;
        e.ar = strtod(kv.first.c_str(), nullptr);  // the key parsed back, not w / h
        snprintf(e.key, sizeof e.key, "%s", kv.first.c_str());
        e.w = kv.second.first;
        e.h = kv.second.second;
        t.buckets.push_back(e);
    }
    std::sort(t.buckets.begin(), t.buckets.end(), [](const BucketEntry& a, const BucketEntry& b) { return a.ar < b.ar; });
    return t;
}

int Transform::find(const char* key) const {
    for (size_t i = 0; i < buckets.size(); ++i)
        if (strcmp(buckets[i].key, key) == 0) return (int)i;
    return -1;
}

int Transform::closest(int32_t w, int32_t h) const {
    const double target = (double)w / (double)h;
    const int n = (int)buckets.size();
    int idx = (int)(std::lower_bound(buckets.begin(), buckets.end(), target,
                                     [](const BucketEntry& b, double v) { return b.ar < v; }) - buckets.begin());
    if (idx < n && buckets[idx].ar == target) return idx;
    if (idx == 0) return 0;
    if (idx == n) return n - 1;
    const double dl = std::fabs(target - buckets[idx - 1].ar), dr = std::fabs(buckets[idx].ar - target);
    return dl < dr ? idx - 1 : idx;  // a tie goes right
}

int plan_geometry(const Transform& t, uint32_t w, uint32_t h, uint32_t channels, const char* forced_key, dg_plan* out) {
    int idx;
    if (forced_key && forced_key[0]) {
        idx = t.find(forced_key);
        if (idx < 0) return DG_E_UNKNOWN_KEY;
    } else {
        idx = t.closest((int32_t)w, (int32_t)h);
    }
    const BucketEntry& b = t.buckets[idx];
    dg_plan p;
    memset(&p, 0, sizeof p);
    p.src_w = w; p.src_h = h; p.channels = channels;
    p.target_w = b.w; p.target_h = b.h;
    memcpy(p.key, b.key, sizeof p.key);
    if (w == b.w && h == b.h) {
        p.identity = 1;
        p.new_w = w; p.new_h = h; p.crop_w = w; p.crop_h = h;
        *out = p;
        return DG_OK;
    }
    const double sx = (double)b.w / (double)w, sy = (double)b.h / (double)h;
    const double scale = sx > sy ? sx : sy;
    p.new_w = (uint32_t)std::round((double)w * scale);  // f64::round: half away from zero
    p.new_h = (uint32_t)std::round((double)h * scale);
    // fast_image_resize CropBox::fit_src_into_dst_size with the default (0.5, 0.5) centring
    const double fw = (double)p.new_w, fh = (double)p.new_h;
    const double have = fw / fh, want = (double)b.w / (double)b.h;
    if (std::fabs(have - want) < 2.220446049250313e-16) { p.crop_w = fw; p.crop_h = fh; }
    else if (have >= want) { p.crop_w = want * fh; p.crop_h = fh; }
    else { p.crop_w = fw; p.crop_h = fw / want; }
    p.crop_left = (fw - p.crop_w) * 0.5;
    p.crop_top = (fh - p.crop_h) * 0.5;
    *out = p;
    return DG_OK;
}

// ---------------------------------------------------------------------------------------------------------------
// Lanczos3 filter tables: what fast_image_resize 5.x precomputes for ResizeAlg::Convolution(FilterType::Lanczos3)
// on 8-bit pixels (datago calls it at src/image_processing.rs:293-298 and :312-323).  Weights are evaluated and
// normalised in f64, then quantised to int16 with the largest precision that keeps the biggest weight below 2^15.
// ---------------------------------------------------------------------------------------------------------------
static inline double sinc_pi(double x) {
    if (x == 0.0) return 1.0;
    const double a = x * M_PI;
    return std::sin(a) / a;
}
static inline double lanczos3_weight(double x) { return (x >= -3.0 && x < 3.0) ? sinc_pi(x) * sinc_pi(x / 3.0) : 0.0; }

FilterTable make_filter_table(int in_size, double in0, double in1, int out_size) {
    FilterTable t;
    t.n = out_size;
    const double scale = (in1 - in0) / (double)out_size;
    const double fscale = std::max(scale, 1.0);
    const double radius = 3.0 * fscale;
    const double inv = 1.0 / fscale;
    t.window = (int)std::ceil(radius) * 2 + 1;
    t.start.resize(out_size);
    t.size.resize(out_size);
    std::vector<double> w((size_t)t.window * out_size, 0.0);  // [out][tap] while building
    double wmax = 0.0;
    for (int o = 0; o < out_size; ++o) {
        const double centre = in0 + ((double)o + 0.5) * scale;
        int lo = (int)std::max(std::floor(centre - radius), 0.0);
        int hi = (int)std::min(std::ceil(centre + radius), (double)in_size);
        double* row = &w[(size_t)o * t.window];
        int cnt = 0, first = lo, last = hi;
        double sum = 0.0;
        const double c = centre - 0.5;
        for (int x = lo; x < hi; ++x) {
            const double v = lanczos3_weight(((double)x - c) * inv);
            if (x == first && v == 0.0) { ++first; continue; }  // leading zero weights are not stored
            row[cnt++] = v;
            sum += v;
        }
        for (int i = cnt - 1; i >= 0 && last > first && row[i] == 0.0; --i) --last;  // nor trailing ones
        if (sum != 0.0) for (int i = 0; i < cnt; ++i) row[i] /= sum;
        t.start[o] = first;
        t.size[o] = last - first;
        for (int i = 0; i < t.window; ++i) wmax = (o == 0 && i == 0) ? row[i] : std::max(wmax, row[i]);
    }
    int precision = 0;
    for (int p = 0; p < 22; ++p) {
        precision = p;
        if ((int32_t)std::round(wmax * (double)(1 << (p + 1))) >= (1 << 15)) break;
    }
    t.precision = precision;
    const double q = (double)((int64_t)1 << precision);
    t.k.assign((size_t)t.window * out_size, 0);
    for (int o = 0; o < out_size; ++o)
        for (int i = 0; i < t.window; ++i)
            t.k[(size_t)i * out_size + o] = (int16_t)std::round(w[(size_t)o * t.window + i] * q);
    return t;
}

int FilterTable::last_in(int lo, int hi) const {
    int m = 0;
    for (int i = lo; i < hi; ++i) m = std::max(m, start[i] + size[i]);
    return m;
}

void FilterTable::pack(uint32_t* dst) const {
    memcpy(dst, start.data(), (size_t)n * 4);
    memcpy(dst + n, size.data(), (size_t)n * 4);
    uint16_t* kk = (uint16_t*)(dst + 2 * (size_t)n);
    memcpy(kk, k.data(), k.size() * 2);
    if (k.size() & 1) kk[k.size()] = 0;
}

// ---------------------------------------------------------------------------------------------------------------
// Sharding.  datago: get_data_slice_multirank (src/generator_files.rs:24-42) and
// hash_fn = DefaultHasher over the key (src/generator_wds.rs:50-54), i.e. SipHash-1-3 with a zero key over
// the key bytes followed by 0xFF.
// ---------------------------------------------------------------------------------------------------------------
static inline uint64_t rotl64(uint64_t x, int b) { return (x << b) | (x >> (64 - b)); }

uint64_t siphash13_str(const char* key, uint64_t len) {
    uint64_t v0 = 0x736f6d6570736575ULL, v1 = 0x646f72616e646f6dULL, v2 = 0x6c7967656e657261ULL, v3 = 0x7465646279746573ULL;
    auto sipround = [&]() {
        v0 += v1; v1 = rotl64(v1, 13); v1 ^= v0; v0 = rotl64(v0, 32);
        v2 += v3; v3 = rotl64(v3, 16); v3 ^= v2;
        v0 += v3; v3 = rotl64(v3, 21); v3 ^= v0;
        v2 += v1; v1 = rotl64(v1, 17); v1 ^= v2; v2 = rotl64(v2, 32);
    };
    const uint64_t total = len + 1;  // the 0xFF terminator `impl Hash for str` writes
    auto byte_at = [&](uint64_t i) -> uint64_t { return i < len ? (uint8_t)key[i] : 0xFFu; };
    uint64_t i = 0;
    for (; i + 8 <= total; i += 8) {
        uint64_t m = 0;
        for (int b = 0; b < 8; ++b) m |= byte_at(i + b) << (8 * b);
        v3 ^= m; sipround(); v0 ^= m;
    }
    uint64_t m = (total & 0xff) << 56;
    for (int b = 0; i + b < total; ++b) m |= byte_at(i + b) << (8 * b);
    v3 ^= m; sipround(); v0 ^= m;
    v2 ^= 0xff;
    sipround(); sipround(); sipround();
    return v0 ^ v1 ^ v2 ^ v3;
}

}  // namespace dg
