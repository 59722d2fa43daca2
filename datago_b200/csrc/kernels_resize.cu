// Separable Lanczos3 convolution passes on 8-bit interleaved images (1 or 3 channels), batched over images.
// Replaces the two fast_image_resize::Resizer::resize calls of datago's crop_and_resize
// (src/image_processing.rs:288-323): whole-image resize, then the centred crop (a copy for an integral offset,
// a 6-tap half-pixel shift along one axis otherwise).  Every pass rounds to 8 bits exactly as the CPU library does:
// int16 weights, int32 accumulation started at half an LSB, arithmetic shift, clamp.
//
// One launch covers one pass of every image of a wave; a CTA owns one output tile.  Two taps are applied per
// instruction: dp2a multiplies a pair of 16-bit weights with a pair of 8-bit samples and accumulates in 32 bits,
// which is exactly the reference arithmetic.
//   horizontal: one thread per output pixel column and 4 rows; windows are read as aligned words from global memory
//               (neighbouring lanes overlap almost completely, so L1 serves them) and realigned in registers.
//   vertical:   one thread per 16-byte column chunk and 8 output rows, 128-bit loads and stores; weights of the
//               tile's rows are staged in shared memory as ready-made pairs.
// Vertical passes over unaligned or unpadded rows take the plain 4-byte path.
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

__device__ __forceinline__ int32_t dp2a_lo(uint32_t weights, uint32_t samples, int32_t acc) {
    int32_t d;
    asm("dp2a.lo.s32.u32 %0, %1, %2, %3;" : "=r"(d) : "r"(weights), "r"(samples), "r"(acc));
    return d;
}
__device__ __forceinline__ int32_t dp2a_hi(uint32_t weights, uint32_t samples, int32_t acc) {
    int32_t d;
    asm("dp2a.hi.s32.u32 %0, %1, %2, %3;" : "=r"(d) : "r"(weights), "r"(samples), "r"(acc));
    return d;
}
__device__ __forceinline__ uint32_t pack_sat4(int32_t a, int32_t b, int32_t c, int32_t d) {  // a in the lowest byte
    uint32_t hi, r;
    asm("cvt.pack.sat.u8.s32.b32 %0, %1, %2, %3;" : "=r"(hi) : "r"(d), "r"(c), "r"(0));
    asm("cvt.pack.sat.u8.s32.b32 %0, %1, %2, %3;" : "=r"(r) : "r"(b), "r"(a), "r"(hi));
    return r;
}

struct Table {
    const int32_t* start;
    const int32_t* size;
    const int16_t* k;  // [tap][tab_n]
};
__device__ __forceinline__ Table table_of(const ConvPass& p, const uint32_t* tables) {
    Table t;
    t.start = reinterpret_cast<const int32_t*>(tables + p.tab_off);
    t.size = t.start + p.tab_n;
    t.k = reinterpret_cast<const int16_t*>(t.size + p.tab_n);
    return t;
}

// ---- horizontal pass ---------------------------------------------------------------------------------------------------
// One thread per output pixel column and kHRowsPerThread rows.  The window of an output pixel is taps * C consecutive
// bytes of a source row: it is fetched four taps at a time as aligned 32-bit words, realigned with funnel shifts, and
// the (tap, tap + 1) byte pairs of each channel are gathered with byte permutes and fed to dp2a.  Weights beyond a
// window are zero in the table, so the bytes read past it (at most 15) do not matter -- but they are read: sources
// inside the library's arenas have that much slack around them; for a source owned by the caller (GUARD) every word
// that is not entirely inside [guard_lo, guard_hi) is assembled from the bytes that are, the rest reading as zero.
constexpr int kHRowsPerThread = kConvTileH / 4;
constexpr int kConvHThreads = kConvTileW * 4;

template <bool GUARD>
__device__ __forceinline__ uint32_t load_word(const ConvPass& p, const uint32_t* w) {
    if (!GUARD) return __ldg(w);
    const uint8_t* b = reinterpret_cast<const uint8_t*>(w);
    if (b >= p.guard_lo && b + 4 <= p.guard_hi) return __ldg(w);
    uint32_t v = 0;
#pragma unroll
    for (int j = 0; j < 4; ++j)
        if (b + j >= p.guard_lo && b + j < p.guard_hi) v |= (uint32_t)__ldg(b + j) << (8 * j);
    return v;
}

template <int C, bool GUARD>
__device__ __forceinline__ void conv_h_rows(const ConvPass& p, const Table& tb, uint32_t x, uint32_t y0) {
    const uint32_t t = p.t0 + x;
    const int32_t first = __ldg(tb.start + t) - p.src_origin;
    const int32_t taps = __ldg(tb.size + t);
    const int16_t* k = tb.k + t;
    const uint32_t nrows = min((uint32_t)kHRowsPerThread, p.out_h - y0);
    const uint32_t* base[kHRowsPerThread];
    uint32_t shift[kHRowsPerThread];
    int32_t acc[kHRowsPerThread][C];
#pragma unroll
    for (int r = 0; r < kHRowsPerThread; ++r) {
        const uint8_t* g = p.src + (size_t)(y0 + min((uint32_t)r, nrows - 1)) * p.src_pitch + (size_t)first * C;
        const uint32_t m = (uint32_t)(reinterpret_cast<uintptr_t>(g) & 3u);
        base[r] = reinterpret_cast<const uint32_t*>(g - m);
        shift[r] = m * 8;
#pragma unroll
        for (int c = 0; c < C; ++c) acc[r][c] = 1 << (p.precision - 1);
    }
    for (int32_t i = 0; i < taps; i += 4) {
        // weights of taps i..i+3 as two pairs (entries past the window are zero; past the table they are not read)
        uint32_t kw[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) kw[j] = (uint32_t)(i + j) < p.window ? (uint16_t)__ldg(k + (size_t)(i + j) * p.tab_n) : 0u;
        const uint32_t k01 = kw[0] | (kw[1] << 16), k23 = kw[2] | (kw[3] << 16);
#pragma unroll
        for (int r = 0; r < kHRowsPerThread; ++r) {
            const uint32_t* w = base[r] + (i * C) / 4;  // i is a multiple of 4: i * C bytes is a whole number of words
            if (C == 3) {
                const uint32_t a0 = load_word<GUARD>(p, w), a1 = load_word<GUARD>(p, w + 1), a2 = load_word<GUARD>(p, w + 2), a3 = load_word<GUARD>(p, w + 3);
                const uint32_t w0 = __funnelshift_r(a0, a1, shift[r]), w1 = __funnelshift_r(a1, a2, shift[r]),
                               w2 = __funnelshift_r(a2, a3, shift[r]);
                // byte 3 * tap + channel
                acc[r][0] = dp2a_lo(k01, __byte_perm(w0, w0, 0x0030), acc[r][0]);
                acc[r][1] = dp2a_lo(k01, __byte_perm(w0, w1, 0x0041), acc[r][1]);
                acc[r][2] = dp2a_lo(k01, __byte_perm(w0, w1, 0x0052), acc[r][2]);
                acc[r][0] = dp2a_lo(k23, __byte_perm(w1, w2, 0x0052), acc[r][0]);
                acc[r][1] = dp2a_lo(k23, __byte_perm(w1, w2, 0x0063), acc[r][1]);
                acc[r][2] = dp2a_lo(k23, __byte_perm(w2, w2, 0x0030), acc[r][2]);
            } else {
                const uint32_t a0 = load_word<GUARD>(p, w), a1 = load_word<GUARD>(p, w + 1);
                const uint32_t w0 = __funnelshift_r(a0, a1, shift[r]);
                acc[r][0] = dp2a_hi(k23, w0, dp2a_lo(k01, w0, acc[r][0]));
            }
        }
    }
#pragma unroll
    for (int r = 0; r < kHRowsPerThread; ++r) {
        if ((uint32_t)r >= nrows) break;
        uint8_t* o = p.dst + (size_t)(y0 + r) * p.dst_pitch + (size_t)x * C;
#pragma unroll
        for (int c = 0; c < C; ++c) o[c] = (uint8_t)clip8(acc[r][c], p.precision);
    }
}

// ---- horizontal pass on the tensor cores -------------------------------------------------------------------------------
// A horizontal resize pass is a banded matrix product: out[row][j] = sum_k src[row][k] * Wt[k][j], with j the output byte
// (pixel x, channel c) and k the source byte of the same row; Wt[k][j] is the weight of source pixel k / C for output
// pixel x when k % C == c and zero otherwise.  The 16-bit weights are split into a signed high and an unsigned low
// byte, w = 256 hi + lo, so that the product runs on the 8-bit integer tensor-core path with 32-bit accumulation:
// out = 256 (src x hi) + (src x lo), which is exact -- the result equals the dp2a kernel's bit for bit.
//   CTA  = one strip of 64 output bytes x up to 512 rows of one pass; warp q owns output bytes 8q .. 8q+7 of the strip.
//   B    = the warp's slice of Wt (source bytes under its eight outputs, at most 256), both limbs, built once per CTA in
//          shared memory from the filter table and read as mma.m16n8k32 fragments;
//   A    = 32 source rows of the strip's band per chunk, brought in by 16-byte asynchronous copies into a ring of up to
//          four chunks (the planner only sends passes here whose source rows start on 16-byte boundaries), so the copies
//          of the next chunks are in flight while a chunk is multiplied; read with ldmatrix;
//   D    = two 16-row tiles per warp and chunk; merged, rounded, clamped, collected in shared memory and written out
//          as 16-byte pieces.
// The interleaved channel layout costs two thirds of the multiplies (zeros in Wt), which the tensor cores have to
// spare; in exchange the source needs no de-interleaving and the result is produced in its final byte order.
constexpr int kHMmaThreads = 256;
constexpr int kHMmaPitchB = (int)kHMmaMaxBand + 16;  // per output byte; + 16 spreads the eight rows of a fragment over the banks
constexpr int kHMmaChunk = 32;                       // rows per chunk (two mma row tiles)
constexpr int kHMmaRing = 45056;                     // bytes of the A ring: three chunks at a 4.5x reduction, one at the widest band
constexpr int kHMmaOutPitch = (int)kHMmaStrip + 16;

struct HMmaSmem {
    uint8_t B[kHMmaThreads / 32][2][8][kHMmaPitchB];
    uint8_t out[kHMmaChunk][kHMmaOutPitch];
    uint8_t A[kHMmaRing];
};
static_assert(kHMmaChunk * ((int)kHMmaMaxSpan + 32) <= kHMmaRing, "the ring must hold one chunk of the widest band");

__device__ __forceinline__ void mma_u8s8(int32_t (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k32.row.col.s32.u8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+r"(d[0]), "+r"(d[1]), "+r"(d[2]), "+r"(d[3]) : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ void mma_u8u8(int32_t (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k32.row.col.s32.u8.u8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+r"(d[0]), "+r"(d[1]), "+r"(d[2]), "+r"(d[3]) : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

__global__ void __launch_bounds__(kHMmaThreads, 2) k_conv_h_mma(const ConvPass* passes, OwnerMap map, const uint32_t* tables) {
    extern __shared__ __align__(16) unsigned char conv_h_smem[];
    HMmaSmem& sm = *reinterpret_cast<HMmaSmem*>(conv_h_smem);
    const ConvPass& p = passes[owner_of_tile(map, blockIdx.x)];
    const uint32_t tile = blockIdx.x - p.tile_first;
    const uint32_t ty = tile / p.tiles_x, tx = tile - ty * p.tiles_x;
    const Table tb = table_of(p, tables);
    const uint32_t lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const uint32_t C = p.channels, row_bytes = p.out_w * C;
    const uint32_t j0 = tx * kHMmaStrip;                          // first output byte of the strip
    const uint32_t jn0 = j0 + warp * 8;                           // ... of this warp's tile
    const uint32_t y_first = ty * kHMmaRows, y_end = min(p.out_h, y_first + kHMmaRows);
    // source byte range of the strip, in bytes from the start of a source row of the pass
    const uint32_t xs0 = j0 / C, xs1 = min(p.out_w - 1, (j0 + kHMmaStrip - 1) / C);
    const int32_t strip_lo = ((__ldg(tb.start + p.t0 + xs0) - p.src_origin) * (int32_t)C) & ~15;
    const int32_t strip_hi = (__ldg(tb.start + p.t0 + xs1) + __ldg(tb.size + p.t0 + xs1) - p.src_origin) * (int32_t)C;
    const uint32_t span16 = (uint32_t)(strip_hi - strip_lo + 15) >> 4;   // 16-byte pieces per staged row
    const uint32_t pitch_a = (span16 | 1u) * 16;                         // an odd number of pieces: ldmatrix rows hit different banks
    const uint32_t stage_bytes = kHMmaChunk * pitch_a;
    const uint32_t nstage = min(4u, (uint32_t)kHMmaRing / stage_bytes);  // >= 1 by the planner's span limit
    // ... and of this warp's eight output bytes (a warp past the end of the row only helps with the copies)
    const bool warp_active = jn0 < row_bytes;
    int32_t band_lo = strip_lo;
    uint32_t ksteps = 0;
    if (warp_active) {
        const uint32_t xw0 = jn0 / C, xw1 = min(p.out_w - 1, (jn0 + 7) / C);
        band_lo = ((__ldg(tb.start + p.t0 + xw0) - p.src_origin) * (int32_t)C) & ~15;
        const int32_t band_hi = (__ldg(tb.start + p.t0 + xw1) + __ldg(tb.size + p.t0 + xw1) - p.src_origin) * (int32_t)C;
        ksteps = (uint32_t)(band_hi - band_lo + 31) >> 5;
    }

    // queues the copies of chunk c (rows y_first + 32 c ...) into its ring slot; one commit group per call and thread
    const uint32_t nchunks = (y_end - y_first + kHMmaChunk - 1) / kHMmaChunk;
    auto queue_chunk = [&](uint32_t c) {
        if (c < nchunks) {
            uint8_t* slot = sm.A + (c % nstage) * stage_bytes;
#pragma unroll 1
            for (uint32_t r = warp; r < (uint32_t)kHMmaChunk; r += kHMmaThreads / 32) {
                const uint32_t y = min(y_first + c * kHMmaChunk + r, p.out_h - 1);  // rows past the end repeat the last one
                const uint8_t* src = p.src + (size_t)y * p.src_pitch + strip_lo;
                const uint32_t dst = (uint32_t)__cvta_generic_to_shared(slot + r * pitch_a);
                for (uint32_t v = lane; v < span16; v += 32)
                    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst + v * 16), "l"(src + v * 16) : "memory");
            }
        }
        asm volatile("cp.async.commit_group;" ::: "memory");
    };
    for (uint32_t c = 0; c + 1 < nstage; ++c) queue_chunk(c);

    // ---- B: zero, then scatter the weights of the warp's eight output bytes; lane l fills output byte l / 4, taps l % 4, + 4, ...
    {
        uint4* z = reinterpret_cast<uint4*>(&sm.B[warp][0][0][0]);
        for (uint32_t i = lane; i < sizeof(sm.B[0]) / 16; i += 32) z[i] = make_uint4(0, 0, 0, 0);
        __syncwarp();
        const uint32_t n = lane >> 2, j = jn0 + n;
        if (j < row_bytes) {
            const uint32_t x = j / C, c = j - x * C;
            const int32_t first = (__ldg(tb.start + p.t0 + x) - p.src_origin) * (int32_t)C + (int32_t)c - band_lo;
            const int32_t taps = __ldg(tb.size + p.t0 + x);
            const int16_t* k = tb.k + p.t0 + x;
#pragma unroll 4
            for (int32_t i = (int32_t)(lane & 3u); i < taps; i += 4) {
                const int32_t wv = __ldg(k + (size_t)i * p.tab_n);
                const uint32_t at = (uint32_t)(first + i * (int32_t)C);
                sm.B[warp][0][n][at] = (uint8_t)(wv >> 8);    // signed high byte
                sm.B[warp][1][n][at] = (uint8_t)(wv & 255);   // unsigned low byte
            }
        }
    }
    const uint32_t g = lane >> 2, t4 = lane & 3u;
    const int32_t half = 1 << (p.precision - 1);
    const bool dst16 = ((reinterpret_cast<uintptr_t>(p.dst) | p.dst_pitch) & 15u) == 0;
    const uint32_t a_off = (uint32_t)(band_lo - strip_lo);
    // ldmatrix: lanes 0-7 give the rows of tile rows 0-7 at k, lanes 8-15 rows 8-15 at k, 16-23 rows 0-7 at k + 16, ...
    const uint32_t a_lane = ((lane & 7u) + ((lane >> 3) & 1u) * 8) * pitch_a + a_off + (lane >> 4) * 16;
    const uint8_t* bh = &sm.B[warp][0][g][4 * t4];
    const uint8_t* bl = &sm.B[warp][1][g][4 * t4];

    for (uint32_t c = 0; c < nchunks; ++c) {
        queue_chunk(c + nstage - 1);  // into the slot the previous iteration finished with
        if (nstage == 4) asm volatile("cp.async.wait_group 3;" ::: "memory");
        else if (nstage == 3) asm volatile("cp.async.wait_group 2;" ::: "memory");
        else if (nstage == 2) asm volatile("cp.async.wait_group 1;" ::: "memory");
        else asm volatile("cp.async.wait_group 0;" ::: "memory");
        __syncthreads();  // chunk c has landed for every thread (first pass: B is complete as well)
        if (warp_active) {
            int32_t acc_hi[2][4], acc_lo[2][4];
#pragma unroll
            for (int mt = 0; mt < 2; ++mt)
#pragma unroll
                for (int i = 0; i < 4; ++i) { acc_hi[mt][i] = 0; acc_lo[mt][i] = half; }
            const uint32_t a_addr = (uint32_t)__cvta_generic_to_shared(sm.A + (c % nstage) * stage_bytes) + a_lane;
#pragma unroll 1
            for (uint32_t ks = 0; ks < ksteps; ++ks) {
                const uint32_t bh0 = *reinterpret_cast<const uint32_t*>(bh + ks * 32), bh1 = *reinterpret_cast<const uint32_t*>(bh + ks * 32 + 16);
                const uint32_t bl0 = *reinterpret_cast<const uint32_t*>(bl + ks * 32), bl1 = *reinterpret_cast<const uint32_t*>(bl + ks * 32 + 16);
#pragma unroll
                for (int mt = 0; mt < 2; ++mt) {
                    uint32_t a[4];
                    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
                                 : "=r"(a[0]), "=r"(a[1]), "=r"(a[2]), "=r"(a[3]) : "r"(a_addr + (uint32_t)mt * 16 * pitch_a + ks * 32));
                    mma_u8s8(acc_hi[mt], a, bh0, bh1);
                    mma_u8u8(acc_lo[mt], a, bl0, bl1);
                }
            }
            // ---- merge the limbs, round, clamp; accumulator i of a tile is row g + 8 (i / 2), output byte 2 t + i % 2
#pragma unroll
            for (int mt = 0; mt < 2; ++mt)
#pragma unroll
                for (int h = 0; h < 2; ++h) {
                    const uint32_t v0 = clip8(acc_hi[mt][2 * h] * 256 + acc_lo[mt][2 * h], p.precision);
                    const uint32_t v1 = clip8(acc_hi[mt][2 * h + 1] * 256 + acc_lo[mt][2 * h + 1], p.precision);
                    *reinterpret_cast<uint16_t*>(&sm.out[mt * 16 + g + 8 * h][warp * 8 + 2 * t4]) = (uint16_t)(v0 | (v1 << 8));
                }
        }
        __syncthreads();  // the out tile is complete; slot c % nstage is free for the copies the next iteration queues
        // ---- write the chunk out: thread i takes 16 bytes of row i / 4
        if (threadIdx.x < kHMmaChunk * (kHMmaStrip / 16)) {
            const uint32_t r = threadIdx.x >> 2, qd = threadIdx.x & 3u, y = y_first + c * kHMmaChunk + r, jb = j0 + qd * 16;
            if (y < y_end && jb < row_bytes) {
                uint8_t* o = p.dst + (size_t)y * p.dst_pitch + jb;
                const uint4 v = *reinterpret_cast<const uint4*>(&sm.out[r][qd * 16]);
                if (dst16 && jb + 16 <= row_bytes) {
                    *reinterpret_cast<uint4*>(o) = v;
                } else {
                    const uint32_t vw[4] = {v.x, v.y, v.z, v.w};
                    const uint32_t nb = min(16u, row_bytes - jb);
#pragma unroll
                    for (int wi = 0; wi < 4; ++wi)
#pragma unroll
                        for (int kb = 0; kb < 4; ++kb)
                            if ((uint32_t)(wi * 4 + kb) < nb) o[wi * 4 + kb] = (uint8_t)(vw[wi] >> (8 * kb));
                }
            }
        }
        // the out tile is rewritten only after the next iteration's first barrier
    }
}

__global__ void __launch_bounds__(kConvHThreads) k_conv_h(const ConvPass* passes, OwnerMap map, const uint32_t* tables, uint32_t first_tile) {
    const uint32_t tile_index = first_tile + blockIdx.x;
    const ConvPass& p = passes[owner_of_tile(map, tile_index)];
    const uint32_t tile = tile_index - p.tile_first;
    const uint32_t ty = tile / p.tiles_x, tx = tile - ty * p.tiles_x;
    const uint32_t x = tx * kConvTileW + threadIdx.x % kConvTileW;
    const uint32_t y0 = ty * kConvTileH + (threadIdx.x / kConvTileW) * kHRowsPerThread;
    if (x >= p.out_w || y0 >= p.out_h) return;
    const Table tb = table_of(p, tables);
    if (p.guard_hi) {
        if (p.channels == 3) conv_h_rows<3, true>(p, tb, x, y0);
        else conv_h_rows<1, true>(p, tb, x, y0);
    } else if (p.channels == 3) conv_h_rows<3, false>(p, tb, x, y0);
    else conv_h_rows<1, false>(p, tb, x, y0);
}

// Horizontal passes of one stage: the tensor-core passes come first in `passes` and own tiles [0, mma_tiles) of the map,
// the others the rest.
void launch_conv_h(const ConvPass* passes, OwnerMap map, const uint32_t* tables, uint32_t mma_tiles, cudaStream_t s) {
    if (!map.total) return;
    if (mma_tiles) {
        static bool configured[64] = {false};
        int dev = 0;
        cudaGetDevice(&dev);
        if (dev < 0 || dev >= 64) dev = 0;
        if (!configured[dev]) {
            cudaFuncSetAttribute(k_conv_h_mma, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)sizeof(HMmaSmem));
            configured[dev] = true;
        }
        k_conv_h_mma<<<mma_tiles, kHMmaThreads, sizeof(HMmaSmem), s>>>(passes, map, tables);
    }
    if (map.total > mma_tiles) k_conv_h<<<map.total - mma_tiles, kConvHThreads, 0, s>>>(passes, map, tables, mma_tiles);
}

// ---- vertical pass -----------------------------------------------------------------------------------------------------
constexpr int kConvVThreads = 256;
constexpr int kVFastCols = kVFastBytes / 16;          // 64 column chunks
constexpr int kVFastGroups = kConvVThreads / kVFastCols;  // 4 groups of rows
constexpr int kVRowsPerThread = kVFastRows / kVFastGroups;  // 8

__device__ __forceinline__ void conv_v_plain(const ConvPass& p, const Table& tb, uint32_t tx, uint32_t ty) {
    const uint32_t row_bytes = p.out_w * p.channels;
    const uint32_t xb = tx * kVTileBytes + (threadIdx.x % (kVTileBytes / 4)) * 4;
    const uint32_t y = ty * kVTileH + threadIdx.x / (kVTileBytes / 4);
    if (xb >= row_bytes || y >= p.out_h) return;
    const uint32_t t = p.t0 + y;
    const int16_t* k = tb.k + t;
    const int32_t first = __ldg(tb.start + t) - p.src_origin;
    const int32_t taps = __ldg(tb.size + t);
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

// 16-byte columns.  Source and destination rows are 16-byte aligned and padded, so the last chunk of a row may be
// read and written in full.
__device__ __forceinline__ void conv_v_vector(const ConvPass& p, const Table& tb, uint32_t tx, uint32_t ty,
                                              uint32_t (*s_k)[kVFastMaxWindow / 2], int32_t* s_first, int32_t* s_taps) {
    const uint32_t y0 = ty * kVFastRows;
    const uint32_t nrows = min((uint32_t)kVFastRows, p.out_h - y0);
    // stage start, size and paired weights of the tile's rows
    for (uint32_t i = threadIdx.x; i < nrows; i += kConvVThreads) {
        s_first[i] = __ldg(tb.start + p.t0 + y0 + i) - p.src_origin;
        s_taps[i] = __ldg(tb.size + p.t0 + y0 + i);
    }
    const uint32_t pairs = (p.window + 1) / 2;
    for (uint32_t i = threadIdx.x; i < nrows * pairs; i += kConvVThreads) {
        const uint32_t r = i / pairs, j = i - r * pairs;
        const int16_t* k = tb.k + p.t0 + y0 + r;
        const uint32_t lo = (uint16_t)__ldg(k + (size_t)(2 * j) * p.tab_n);
        const uint32_t hi = 2 * j + 1 < p.window ? (uint16_t)__ldg(k + (size_t)(2 * j + 1) * p.tab_n) : 0u;
        s_k[r][j] = lo | (hi << 16);
    }
    __syncthreads();
    const uint32_t col = threadIdx.x % kVFastCols, grp = threadIdx.x / kVFastCols;
    const uint32_t xb = tx * kVFastBytes + col * 16;
    if (xb >= p.out_w * p.channels) return;
    const int32_t half = 1 << (p.precision - 1);
#pragma unroll 1
    for (uint32_t rr = 0; rr < (uint32_t)kVRowsPerThread; ++rr) {
        const uint32_t r = grp * kVRowsPerThread + rr;
        if (r >= nrows) break;
        const int32_t taps = s_taps[r];
        const uint8_t* s = p.src + (size_t)s_first[r] * p.src_pitch + xb;
        int32_t acc[16];
#pragma unroll
        for (int i = 0; i < 16; ++i) acc[i] = half;
        for (int32_t i = 0; i < taps; i += 2) {
            const uint32_t kp = s_k[r][i >> 1];  // the weight after the last tap of an odd window is zero
            const uint4 a = __ldg(reinterpret_cast<const uint4*>(s + (size_t)i * p.src_pitch));
            const uint4 b = __ldg(reinterpret_cast<const uint4*>(s + (size_t)min(i + 1, taps - 1) * p.src_pitch));
            const uint32_t aw[4] = {a.x, a.y, a.z, a.w}, bw[4] = {b.x, b.y, b.z, b.w};
#pragma unroll
            for (int wq = 0; wq < 4; ++wq) {
                const uint32_t p01 = __byte_perm(aw[wq], bw[wq], 0x5140), p23 = __byte_perm(aw[wq], bw[wq], 0x7362);
                acc[4 * wq] = dp2a_lo(kp, p01, acc[4 * wq]);
                acc[4 * wq + 1] = dp2a_hi(kp, p01, acc[4 * wq + 1]);
                acc[4 * wq + 2] = dp2a_lo(kp, p23, acc[4 * wq + 2]);
                acc[4 * wq + 3] = dp2a_hi(kp, p23, acc[4 * wq + 3]);
            }
        }
        uint4 o;
        const uint32_t sh = p.precision;
        o.x = pack_sat4(acc[0] >> sh, acc[1] >> sh, acc[2] >> sh, acc[3] >> sh);
        o.y = pack_sat4(acc[4] >> sh, acc[5] >> sh, acc[6] >> sh, acc[7] >> sh);
        o.z = pack_sat4(acc[8] >> sh, acc[9] >> sh, acc[10] >> sh, acc[11] >> sh);
        o.w = pack_sat4(acc[12] >> sh, acc[13] >> sh, acc[14] >> sh, acc[15] >> sh);
        *reinterpret_cast<uint4*>(p.dst + (size_t)(y0 + r) * p.dst_pitch + xb) = o;
    }
}

__global__ void __launch_bounds__(kConvVThreads) k_conv_v(const ConvPass* passes, OwnerMap map, const uint32_t* tables) {
    __shared__ uint32_t s_k[kVFastRows][kVFastMaxWindow / 2];
    __shared__ int32_t s_first[kVFastRows], s_taps[kVFastRows];
    __shared__ uint32_t s_pass;
    if (threadIdx.x == 0) s_pass = owner_of_tile(map, blockIdx.x);
    __syncthreads();
    const ConvPass& p = passes[s_pass];
    const uint32_t tile = blockIdx.x - p.tile_first;
    const uint32_t ty = tile / p.tiles_x, tx = tile - ty * p.tiles_x;
    const Table tb = table_of(p, tables);
    if (p.fast) conv_v_vector(p, tb, tx, ty, s_k, s_first, s_taps);
    else conv_v_plain(p, tb, tx, ty);
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

// ---- convert_to_rgb8 (datago src/image_processing.rs:163-186) -------------------------------------------------------
// One thread per pixel, 2048 pixels per CTA.  Gray: the value in all three channels.  RGBA: source-over compositing on
// an opaque (128,128,128) background in f32 on values scaled to 0..1, scaled back by 255 and truncated -- each
// operation rounded once (the _rn intrinsics keep the compiler from fusing a multiply into an add), in the order the
// `image` crate's Pixel::blend uses, so that the result equals a CPU evaluation of the same expression bit for bit.
__global__ void __launch_bounds__(256) k_to_rgb8(const ToRgbJob* jobs, OwnerMap map) {
    const uint32_t ji = owner_of_tile(map, blockIdx.x);
    const ToRgbJob& j = jobs[ji];
    const uint32_t base = (blockIdx.x - j.tile_first) * kToRgbTilePx;
    for (uint32_t k = threadIdx.x; k < kToRgbTilePx; k += 256) {
        const uint32_t i = base + k;
        if (i >= j.npx) break;
        uint8_t* d = j.dst + (size_t)i * 3;
        if (j.channels <= 2) {
            const uint8_t v = __ldg(j.src + (size_t)i * j.channels);
            d[0] = v; d[1] = v; d[2] = v;
            continue;
        }
        const uint32_t px = __ldg(reinterpret_cast<const uint32_t*>(j.src) + i);  // RGBA rows are 4-byte aligned
        const uint32_t a = px >> 24;
        uint32_t c[3] = {px & 255u, (px >> 8) & 255u, (px >> 16) & 255u};
        if (a == 0) { c[0] = c[1] = c[2] = 128; }
        else if (a != 255) {
            const float max_t = 255.0f;
            const float bg_a = __fdiv_rn(255.0f, max_t), fg_a = __fdiv_rn((float)a, max_t);
            const float alpha_final = __fsub_rn(__fadd_rn(bg_a, fg_a), __fmul_rn(bg_a, fg_a));
            const float bg_pre = __fmul_rn(__fdiv_rn(128.0f, max_t), bg_a);
            const float keep = __fsub_rn(1.0f, fg_a);
#pragma unroll
            for (int ch = 0; ch < 3; ++ch) {
                const float fg_pre = __fmul_rn(__fdiv_rn((float)c[ch], max_t), fg_a);
                const float out_pre = __fadd_rn(fg_pre, __fmul_rn(bg_pre, keep));
                c[ch] = (uint32_t)__fmul_rn(max_t, __fdiv_rn(out_pre, alpha_final));  // float -> u32 truncates
            }
        }
        d[0] = (uint8_t)c[0]; d[1] = (uint8_t)c[1]; d[2] = (uint8_t)c[2];
    }
}

void launch_to_rgb8(const ToRgbJob* jobs, OwnerMap map, cudaStream_t s) {
    if (map.total) k_to_rgb8<<<map.total, 256, 0, s>>>(jobs, map);
}

}  // namespace dg
