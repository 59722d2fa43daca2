// Separable Lanczos3 convolution passes on 8-bit interleaved images (1 or 3 channels), batched over images.
// Replaces the two fast_image_resize::Resizer::resize calls of datago's crop_and_resize
// (src/image_processing.rs:288-323): whole-image resize, then the centred crop (a copy for an integral offset,
// a 6-tap half-pixel shift along one axis otherwise).  Every pass rounds to 8 bits exactly as the CPU library does.
//
// HBM-bound byte work: one launch covers one pass of every image of a batch; a CTA owns one output tile.
#include <cstdint>

#include "kernels.h"

namespace dg {

__device__ __forceinline__ uint32_t owner_of_tile(const OwnerMap& m, uint32_t idx) {
    uint32_t o = __ldg(m.coarse + (idx >> m.shift));
    while (o + 1 < m.n && __ldg(m.first + o + 1) <= idx) ++o;
    return o;
}

__device__ __forceinline__ uint32_t clip8(int32_t v, uint32_t precision) {
    v >>= precision;
    return (uint32_t)min(max(v, 0), 255);
}

// ---- horizontal pass: one thread per output pixel ---------------------------------------------------------------
constexpr int kConvHThreads = kConvTileW * kConvTileH;

template <int C>
__device__ __forceinline__ void conv_h_pixel(const ConvPass& p, const uint32_t* tab, uint32_t x, uint32_t y) {
    const uint32_t t = p.t0 + x;
    const int32_t* start = reinterpret_cast<const int32_t*>(tab);
    const int32_t* size = start + p.tab_n;
    const int16_t* k = reinterpret_cast<const int16_t*>(size + p.tab_n) + t;
    const int32_t first = __ldg(start + t) - p.src_origin;
    const int32_t taps = __ldg(size + t);
    const uint8_t* s = p.src + (size_t)y * p.src_pitch + (size_t)first * C;
    int32_t acc[C];
#pragma unroll
    for (int c = 0; c < C; ++c) acc[c] = 1 << (p.precision - 1);
    for (int32_t i = 0; i < taps; ++i) {
        const int32_t kv = __ldg(k + (size_t)i * p.tab_n);
#pragma unroll
        for (int c = 0; c < C; ++c) acc[c] += kv * (int32_t)__ldg(s + i * C + c);
    }
    uint8_t* o = p.dst + (size_t)y * p.dst_pitch + (size_t)x * C;
#pragma unroll
    for (int c = 0; c < C; ++c) o[c] = (uint8_t)clip8(acc[c], p.precision);
}

__global__ void __launch_bounds__(kConvHThreads) k_conv_h(const ConvPass* passes, OwnerMap map, const uint32_t* tables) {
    const uint32_t pi = owner_of_tile(map, blockIdx.x);
    const ConvPass& p = passes[pi];
    const uint32_t tile = blockIdx.x - p.tile_first;
    const uint32_t ty = tile / p.tiles_x, tx = tile - ty * p.tiles_x;
    const uint32_t x = tx * kConvTileW + threadIdx.x % kConvTileW;
    const uint32_t y = ty * kConvTileH + threadIdx.x / kConvTileW;
    if (x >= p.out_w || y >= p.out_h) return;
    const uint32_t* tab = tables + p.tab_off;
    if (p.channels == 3) conv_h_pixel<3>(p, tab, x, y);
    else conv_h_pixel<1>(p, tab, x, y);
}

void launch_conv_h(const ConvPass* passes, OwnerMap map, const uint32_t* tables, cudaStream_t s) {
    if (map.total) k_conv_h<<<map.total, kConvHThreads, 0, s>>>(passes, map, tables);
}

// ---- vertical pass: one thread per 4 consecutive bytes of an output row ----------------------------------------------
constexpr int kConvVThreads = (kVTileBytes / 4) * kVTileH;

__global__ void __launch_bounds__(kConvVThreads) k_conv_v(const ConvPass* passes, OwnerMap map, const uint32_t* tables) {
    const uint32_t pi = owner_of_tile(map, blockIdx.x);
    const ConvPass& p = passes[pi];
    const uint32_t tile = blockIdx.x - p.tile_first;
    const uint32_t ty = tile / p.tiles_x, tx = tile - ty * p.tiles_x;
    const uint32_t row_bytes = p.out_w * p.channels;
    const uint32_t xb = tx * kVTileBytes + (threadIdx.x % (kVTileBytes / 4)) * 4;
    const uint32_t y = ty * kVTileH + threadIdx.x / (kVTileBytes / 4);
    if (xb >= row_bytes || y >= p.out_h) return;
    const uint32_t* tab = tables + p.tab_off;
    const uint32_t t = p.t0 + y;
    const int32_t* start = reinterpret_cast<const int32_t*>(tab);
    const int32_t* size = start + p.tab_n;
    const int16_t* k = reinterpret_cast<const int16_t*>(size + p.tab_n) + t;
    const int32_t first = __ldg(start + t) - p.src_origin;
    const int32_t taps = __ldg(size + t);
    const uint8_t* s = p.src + (size_t)first * p.src_pitch + xb;
    const int32_t half = 1 << (p.precision - 1);
    int32_t a0 = half, a1 = half, a2 = half, a3 = half;
    const uint32_t nb = min(4u, row_bytes - xb);
    const bool vec = nb == 4 && ((reinterpret_cast<uintptr_t>(s) | p.src_pitch) & 3u) == 0;
    if (vec) {
        for (int32_t i = 0; i < taps; ++i) {
            const int32_t kv = __ldg(k + (size_t)i * p.tab_n);
            const uint32_t v = __ldg(reinterpret_cast<const uint32_t*>(s + (size_t)i * p.src_pitch));
            a0 += kv * (int32_t)(v & 255u); a1 += kv * (int32_t)((v >> 8) & 255u);
            a2 += kv * (int32_t)((v >> 16) & 255u); a3 += kv * (int32_t)(v >> 24);
        }
    } else {
        for (int32_t i = 0; i < taps; ++i) {
            const int32_t kv = __ldg(k + (size_t)i * p.tab_n);
            const uint8_t* r = s + (size_t)i * p.src_pitch;
            a0 += kv * (int32_t)__ldg(r);
            if (nb > 1) a1 += kv * (int32_t)__ldg(r + 1);
            if (nb > 2) a2 += kv * (int32_t)__ldg(r + 2);
            if (nb > 3) a3 += kv * (int32_t)__ldg(r + 3);
        }
    }
    uint8_t* o = p.dst + (size_t)y * p.dst_pitch + xb;
    const uint32_t r0 = clip8(a0, p.precision), r1 = clip8(a1, p.precision), r2 = clip8(a2, p.precision), r3 = clip8(a3, p.precision);
    if (nb == 4 && ((reinterpret_cast<uintptr_t>(o)) & 3u) == 0) {
        *reinterpret_cast<uint32_t*>(o) = r0 | (r1 << 8) | (r2 << 16) | (r3 << 24);
    } else {
        o[0] = (uint8_t)r0;
        if (nb > 1) o[1] = (uint8_t)r1;
        if (nb > 2) o[2] = (uint8_t)r2;
        if (nb > 3) o[3] = (uint8_t)r3;
    }
}

void launch_conv_v(const ConvPass* passes, OwnerMap map, const uint32_t* tables, cudaStream_t s) {
    if (map.total) k_conv_v<<<map.total, kConvVThreads, 0, s>>>(passes, map, tables);
}

// ---- plain copies (identity payloads, integral crops without any filtering) ----------------------------------------
__global__ void __launch_bounds__(256) k_copy(const CopyJob* jobs, OwnerMap map) {
    const uint32_t ji = owner_of_tile(map, blockIdx.x);
    const CopyJob& j = jobs[ji];
    const uint64_t total = (uint64_t)j.row_bytes * j.rows;
    const uint64_t base = (uint64_t)(blockIdx.x - j.tile_first) * kCopyTileBytes;
    for (uint32_t i = threadIdx.x; i < kCopyTileBytes; i += 256) {
        const uint64_t b = base + i;
        if (b >= total) break;
        const uint32_t y = (uint32_t)(b / j.row_bytes), x = (uint32_t)(b - (uint64_t)y * j.row_bytes);
        j.dst[b] = __ldg(j.src + (size_t)y * j.src_pitch + x);
    }
}

void launch_copy(const CopyJob* jobs, OwnerMap map, cudaStream_t s) {
    if (map.total) k_copy<<<map.total, 256, 0, s>>>(jobs, map);
}

}  // namespace dg
