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
#include <type_traits>

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
//   CTA  = one strip of 64 output bytes x up to 2048 rows of one pass; warp q of the first eight owns output bytes
//          8q .. 8q+7 of the strip, one thread of a ninth warp issues the copies.
//   B    = the warp's slice of Wt (source bytes under its eight outputs, at most 256), both limbs: every lane gathers its
//          mma.m16n8k32 fragments from the filter table once and keeps them in registers for all rows of the CTA;
//   A    = 32 source rows of the strip's band per chunk, brought in by one tensor-map copy (cp.async.bulk.tensor, box of
//          box_pieces * 16 bytes x 32 rows; the planner only sends passes here whose source rows start on 16-byte
//          boundaries) into a ring of up to eight chunks, so the copies of the next chunks are in flight while a chunk is
//          multiplied; read with ldmatrix;
//   D    = two 16-row tiles per warp and chunk; merged, rounded, saturated, collected in a 32 x 64 byte tile of shared
//          memory and written out as whole 64-byte row pieces (one store instruction covers four rows; eight-byte
//          stores of single tiles, 32 rows per instruction, cost a third more time).  The multiplying warps meet at one
//          named barrier per chunk for that; the copying warps only ever wait on the ring slots' barriers.
// The interleaved channel layout costs two thirds of the multiplies (zeros in Wt), which the tensor cores have to
// spare; in exchange the source needs no de-interleaving and the result is produced in its final byte order.
constexpr int kHMmaConsumers = 256;   // eight warps multiply
constexpr int kHMmaProducers = 32;    // one more warp, of which one thread issues the copies into the ring
constexpr int kHMmaThreads = kHMmaConsumers + kHMmaProducers;
constexpr int kHMmaChunk = 32;                       // rows per chunk (two mma row tiles)
#ifndef DG_HMMA_CTAS
#define DG_HMMA_CTAS 3
#endif
constexpr int kHMmaCtasPerSm = DG_HMMA_CTAS;
constexpr int kHMmaRing = kHMmaCtasPerSm == 3 ? 69632 : 98304;  // bytes of the A ring: the CTAs of an SM keep ~200 KB of source rows in flight
constexpr int kHMmaMaxStages = 8;
constexpr int kHMmaOutPitch = kHMmaStrip + 8;         // 18 words: the tiles' two-byte writes fall into different banks

struct HMmaSmem {
    uint8_t out[2][kHMmaChunk][kHMmaOutPitch];  // a chunk's output bytes, before they go out as 64-byte row pieces
    uint8_t A[kHMmaRing];
};
constexpr int kHMmaRingSlack = 64;
static_assert(2 * kHMmaChunk * ((int)kHMmaMaxSpan + 16) + kHMmaRingSlack <= kHMmaRing, "the ring must hold two chunks of the widest band");

// ldmatrix stays ordered after the wait on the ring slot (volatile, memory); the multiplies are pure register functions
// that the compiler may move between the loads
__device__ __forceinline__ void load_a(uint32_t (&a)[4], uint32_t addr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(a[0]), "=r"(a[1]), "=r"(a[2]), "=r"(a[3]) : "r"(addr) : "memory");
}
__device__ __forceinline__ void mma_u8s8(int32_t (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm("mma.sync.aligned.m16n8k32.row.col.s32.u8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+r"(d[0]), "+r"(d[1]), "+r"(d[2]), "+r"(d[3]) : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ void mma_u8u8(int32_t (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm("mma.sync.aligned.m16n8k32.row.col.s32.u8.u8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+r"(d[0]), "+r"(d[1]), "+r"(d[2]), "+r"(d[3]) : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

// mbarrier helpers: two barriers per ring slot, "filled" (the copies into it have landed) and "drained"
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {  // one arrival that also announces `bytes` of copies
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
// One box of a two-dimensional tensor map into shared memory; (x, y) in elements / rows, x * element size a multiple
// of 16 bytes.  The barrier receives the box's bytes as they land.
__device__ __forceinline__ void tensor_copy_2d(uint32_t dst, const void* map, int32_t x, int32_t y, uint32_t bar) {
    asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
                 ::"r"(dst), "l"(map), "r"(x), "r"(y), "r"(bar) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
    uint32_t done;
    // the last operand lets the hardware park the thread for up to that many nanoseconds instead of returning at once
    asm volatile("{\n .reg .pred p;\n mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n selp.u32 %0, 1, 0, p;\n}"
                 : "=r"(done) : "r"(bar), "r"(parity), "r"(2000u) : "memory");
    return done != 0;
}
constexpr uint32_t kHMmaWaitLimit = 1u << 20;  // waits of up to 2 us each on a ring slot's barrier before a CTA gives up on it

__global__ void __launch_bounds__(kHMmaThreads, kHMmaCtasPerSm) k_conv_h_mma(const ConvPass* passes, OwnerMap map, const uint32_t* tables,
                                                                unsigned int* timeouts) {
    extern __shared__ __align__(128) unsigned char conv_h_smem[];
    HMmaSmem& sm = *reinterpret_cast<HMmaSmem*>(conv_h_smem);
    __shared__ __align__(8) unsigned long long s_bar[2 * kHMmaMaxStages];  // per ring slot: "filled" (bytes arrived) and "drained" (all warps done reading)
    const ConvPass& pg = passes[owner_of_tile(map, blockIdx.x)];
    // everything the loops need from the descriptor, once (the asynchronous-copy statements below are memory barriers
    // for the compiler, which would otherwise fetch these fields again after each of them)
    uint8_t* const p_dst = pg.dst;
    const uint32_t dst_pitch = pg.dst_pitch, out_w = pg.out_w, out_h = pg.out_h, C = pg.channels;
    const uint32_t t0 = pg.t0, tab_n = pg.tab_n, precision = pg.precision, tiles_x = pg.tiles_x;
    const int32_t origin = pg.src_origin;
    const uint32_t tile = blockIdx.x - pg.tile_first;
    const Table tb = table_of(pg, tables);
    const uint32_t ty = tile / tiles_x, tx = tile - ty * tiles_x;
    const uint32_t lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const uint32_t row_bytes = out_w * C;
    const uint32_t j0 = tx * kHMmaStrip;                          // first output byte of the strip
    const uint32_t jn0 = j0 + warp * 8;                           // ... of this warp's tile
    const uint32_t y_first = ty * kHMmaRows, y_end = min(out_h, y_first + kHMmaRows);
    // first source byte of the strip, from the start of a source row of the pass (a multiple of 16)
    const uint32_t xs0 = j0 / C;
    const int32_t strip_lo = ((__ldg(tb.start + t0 + xs0) - origin) * (int32_t)C) & ~15;
    // staged rows: the box width of the pass's tensor map, an odd number of 16-byte pieces (ldmatrix rows then hit
    // different banks) that covers the widest strip of the pass
    const uint32_t pitch_a = pg.box_pieces * 16;
    const uint32_t stage_bytes = kHMmaChunk * pitch_a;
    // The last k step of a warp may read up to 47 bytes past the end of a staged row (they meet zero weights): the ring
    // keeps that much room behind its last slot.
    const uint32_t nstage = min((uint32_t)kHMmaMaxStages, (uint32_t)(kHMmaRing - kHMmaRingSlack) / stage_bytes);  // >= 2 by the planner's span limit
    // ... and of this warp's eight output bytes (a warp past the end of the row has no tile)
    const bool warp_active = jn0 < row_bytes;
    int32_t band_lo = strip_lo;
    uint32_t ksteps = 0;
    if (warp_active) {
        const uint32_t xw0 = jn0 / C, xw1 = min(out_w - 1, (jn0 + 7) / C);
        band_lo = ((__ldg(tb.start + t0 + xw0) - origin) * (int32_t)C) & ~15;
        const int32_t band_hi = (__ldg(tb.start + t0 + xw1) + __ldg(tb.size + t0 + xw1) - origin) * (int32_t)C;
        ksteps = (uint32_t)(band_hi - band_lo + 31) >> 5;
    }
    const uint32_t bar0 = (uint32_t)__cvta_generic_to_shared(&s_bar[0]);
    if (threadIdx.x == 0) {
        for (uint32_t i = 0; i < (uint32_t)kHMmaMaxStages; ++i) { mbar_init(bar0 + 8 * i, 1); mbar_init(bar0 + 8 * (kHMmaMaxStages + i), kHMmaConsumers / 32); }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();

    // Ring protocol.  Chunk c (rows y_first + 32 c ...) lives in slot c % nstage.  The copying thread announces the
    // box's bytes on the slot's "filled" barrier and issues one tensor-map copy, which reports to that barrier; a
    // multiplying warp waits for "filled", multiplies, and arrives on the slot's "drained" barrier, which the copying
    // thread waits for before it fills the slot again.  Every wait is bounded: a CTA that runs out of patience counts a
    // timeout (reported by the host) instead of hanging the GPU.
    const uint32_t nchunks = (y_end - y_first + kHMmaChunk - 1) / kHMmaChunk;
    const uint32_t a_base = (uint32_t)__cvta_generic_to_shared(sm.A);
    bool gave_up = false;
    auto wait_for = [&](uint32_t bar, uint32_t parity) {
        uint32_t polls = 0;
        while (!mbar_try_wait(bar, parity)) {
            if (++polls > kHMmaWaitLimit) { gave_up = true; break; }
        }
    };
    if (warp >= kHMmaConsumers / 32) {
        // ---- the copying thread
        if (lane != 0) return;
        const void* map = pg.tmap;
        // the descriptor sits in global memory that earlier batches may have used for other descriptors
        asm volatile("fence.proxy.tensormap::generic.acquire.gpu [%0], 128;" ::"l"(map) : "memory");
        const int32_t x_word = strip_lo >> 2;
        for (uint32_t c = 0; c < nchunks && !gave_up; ++c) {
            const uint32_t slot = c % nstage, use = c / nstage;
            if (use > 0) wait_for(bar0 + 8 * (kHMmaMaxStages + slot), (use - 1) & 1u);
            if (gave_up) break;
            mbar_expect_tx(bar0 + 8 * slot, stage_bytes);
            tensor_copy_2d(a_base + slot * stage_bytes, map, x_word, (int32_t)(y_first + c * kHMmaChunk), bar0 + 8 * slot);
        }
        // stay until every copy has landed: nothing may arrive in the shared memory of a CTA that has gone
        for (uint32_t c = nchunks > nstage ? nchunks - nstage : 0; c < nchunks; ++c) wait_for(bar0 + 8 * (c % nstage), (c / nstage) & 1u);
        if (gave_up) atomicAdd(timeouts, 1u);
        return;
    }

    const uint32_t g = lane >> 2, t4 = lane & 3u;
    const int32_t half = 1 << (precision - 1);
    const bool dst8 = ((reinterpret_cast<uintptr_t>(p_dst) | dst_pitch) & 7u) == 0;
    // ldmatrix: lanes 0-7 give the rows of tile rows 0-7 at k, lanes 8-15 rows 8-15 at k, 16-23 rows 0-7 at k + 16, ...
    const uint32_t a_lane = ((lane & 7u) + ((lane >> 3) & 1u) * 8) * pitch_a + (uint32_t)(band_lo - strip_lo) + (lane >> 4) * 16;
    // ---- B fragments, gathered straight from the filter table and kept in registers for all chunks.  A lane holds, for
    //      output byte g of the warp's tile and k step ks, source bytes 32 ks + 4 t .. + 3 and + 16 .. + 19 of the band;
    //      source byte kk carries tap (kk - first) / C of that output when that is a whole number inside the window.
    uint32_t bfr[8][4];
    {
        const uint32_t j = jn0 + g;
        const bool live = warp_active && j < row_bytes;
        const uint32_t x = live ? j / C : 0, ch = j - x * C;
        const int32_t first = live ? (__ldg(tb.start + t0 + x) - origin) * (int32_t)C + (int32_t)ch - band_lo : 0;
        const int32_t taps = live ? __ldg(tb.size + t0 + x) : 0;
        const int16_t* k = tb.k + t0 + x;
#pragma unroll
        for (int ks = 0; ks < 8; ++ks) {
            uint32_t hi[2] = {0, 0}, lo[2] = {0, 0};
            if ((uint32_t)ks < ksteps) {
#pragma unroll
                for (int hf = 0; hf < 2; ++hf)
#pragma unroll
                    for (int e = 0; e < 4; ++e) {
                        const int32_t d = 32 * ks + 16 * hf + 4 * (int32_t)t4 + e - first;
                        const int32_t i = C == 1 ? d : C == 3 ? d / 3 : d / (int32_t)C;
                        if (d >= 0 && i < taps && i * (int32_t)C == d) {
                            const int32_t wv = __ldg(k + (size_t)i * tab_n);
                            hi[hf] |= ((uint32_t)(wv >> 8) & 255u) << (8 * e);   // signed high byte
                            lo[hf] |= ((uint32_t)wv & 255u) << (8 * e);          // unsigned low byte
                        }
                    }
            }
            bfr[ks][0] = hi[0]; bfr[ks][1] = hi[1]; bfr[ks][2] = lo[0]; bfr[ks][3] = lo[1];
        }
    }
    // The chunk loop is compiled once per number of k steps, so that the multiplies of a chunk form one straight run
    // of loads and tensor-core instructions.
    auto consume = [&](auto ks_tag) {
    constexpr int KS = decltype(ks_tag)::value;
    for (uint32_t c = 0; c < nchunks; ++c) {
        const uint32_t slot = c % nstage;
        wait_for(bar0 + 8 * slot, (c / nstage) & 1u);  // chunk c is the (c / nstage)-th filling of its slot
        int32_t acc_hi[2][4], acc_lo[2][4];
#pragma unroll
        for (int mt = 0; mt < 2; ++mt)
#pragma unroll
            for (int i = 0; i < 4; ++i) { acc_hi[mt][i] = 0; acc_lo[mt][i] = half; }
        if (warp_active) {
            const uint32_t a_addr = a_base + slot * stage_bytes + a_lane;
            uint32_t a[2][2][4];  // [k step parity][row tile]
            load_a(a[0][0], a_addr);
            load_a(a[0][1], a_addr + 16 * pitch_a);
#pragma unroll
            for (int ks = 0; ks < KS; ++ks) {
                // the fragments of the next k step are requested before this step's multiplies are issued
                if (ks + 1 < KS) {
                    load_a(a[(ks + 1) & 1][0], a_addr + (ks + 1) * 32);
                    load_a(a[(ks + 1) & 1][1], a_addr + 16 * pitch_a + (ks + 1) * 32);
                }
#pragma unroll
                for (int mt = 0; mt < 2; ++mt) {
                    mma_u8s8(acc_hi[mt], a[ks & 1][mt], bfr[ks][0], bfr[ks][1]);
                    mma_u8u8(acc_lo[mt], a[ks & 1][mt], bfr[ks][2], bfr[ks][3]);
                }
            }
        }
        __syncwarp();
        if (lane == 0) mbar_arrive(bar0 + 8 * (kHMmaMaxStages + slot));  // this warp is done with the slot
        // ---- merge the limbs, round, saturate; accumulator i of a tile is row g + 8 (i / 2), output byte 2 t + i % 2.
        //      The chunk's 32 x 64 bytes are collected in shared memory (two buffers in turn, so that one barrier of the
        //      multiplying warps per chunk is enough) and leave as whole 64-byte row pieces, four rows per warp.
        uint8_t (*ob)[kHMmaOutPitch] = sm.out[c & 1];
        if (warp_active) {
#pragma unroll
            for (int mt = 0; mt < 2; ++mt)
#pragma unroll
                for (int h = 0; h < 2; ++h) {
                    const int32_t v0 = (acc_hi[mt][2 * h] * 256 + acc_lo[mt][2 * h]) >> precision;
                    const int32_t v1 = (acc_hi[mt][2 * h + 1] * 256 + acc_lo[mt][2 * h + 1]) >> precision;
                    uint32_t pk;
                    asm("cvt.pack.sat.u8.s32.b32 %0, %1, %2, %3;" : "=r"(pk) : "r"(v1), "r"(v0), "r"(0));
                    *reinterpret_cast<uint16_t*>(&ob[mt * 16 + g + 8 * h][warp * 8 + 2 * t4]) = (uint16_t)pk;
                }
        }
        asm volatile("bar.sync 1, %0;" ::"n"(kHMmaConsumers) : "memory");
        {
            const uint32_t row = warp * 4 + (lane >> 3), jb = j0 + (lane & 7u) * 8;
            const uint32_t y = y_first + c * kHMmaChunk + row;
            if (y < y_end && jb < row_bytes) {
                const uint2 v = *reinterpret_cast<const uint2*>(&ob[row][(lane & 7u) * 8]);
                uint8_t* o = p_dst + (size_t)y * dst_pitch + jb;
                if (dst8 && jb + 8 <= row_bytes) {
                    *reinterpret_cast<uint2*>(o) = v;
                } else {
                    const uint32_t nb = min(8u, row_bytes - jb);
#pragma unroll
                    for (int kb = 0; kb < 8; ++kb)
                        if ((uint32_t)kb < nb) o[kb] = (uint8_t)((kb < 4 ? v.x : v.y) >> (8 * (kb & 3)));
                }
            }
        }
    }
    };
    switch (ksteps) {
        case 1: consume(std::integral_constant<int, 1>{}); break;
        case 2: consume(std::integral_constant<int, 2>{}); break;
        case 3: consume(std::integral_constant<int, 3>{}); break;
        case 4: consume(std::integral_constant<int, 4>{}); break;
        case 5: consume(std::integral_constant<int, 5>{}); break;
        case 6: consume(std::integral_constant<int, 6>{}); break;
        case 7: consume(std::integral_constant<int, 7>{}); break;
        default: consume(std::integral_constant<int, 8>{}); break;
    }
    if (gave_up && lane == 0) atomicAdd(timeouts, 1u);
}

// Two- and four-channel images (alpha) that the tensor-core kernel cannot take: a plain loop, one tap at a time.
__device__ void conv_h_rows_any(const ConvPass& p, const Table& tb, uint32_t x, uint32_t y0) {
    const uint32_t t = p.t0 + x, C = p.channels;
    const int32_t first = __ldg(tb.start + t) - p.src_origin;
    const int32_t taps = __ldg(tb.size + t);
    const int16_t* k = tb.k + t;
    const uint32_t nrows = min((uint32_t)kHRowsPerThread, p.out_h - y0);
    for (uint32_t r = 0; r < nrows; ++r) {
        const uint8_t* g = p.src + (size_t)(y0 + r) * p.src_pitch + (size_t)first * C;
        int32_t acc[4] = {1 << (p.precision - 1), 1 << (p.precision - 1), 1 << (p.precision - 1), 1 << (p.precision - 1)};
        for (int32_t i = 0; i < taps; ++i) {
            const int32_t wv = __ldg(k + (size_t)i * p.tab_n);
            for (uint32_t c = 0; c < C; ++c) acc[c] += wv * (int32_t)__ldg(g + (size_t)i * C + c);
        }
        uint8_t* o = p.dst + (size_t)(y0 + r) * p.dst_pitch + (size_t)x * C;
        for (uint32_t c = 0; c < C; ++c) o[c] = (uint8_t)clip8(acc[c], p.precision);
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
    if (p.channels == 2 || p.channels == 4) { conv_h_rows_any(p, tb, x, y0); return; }
    if (p.guard_hi) {
        if (p.channels == 3) conv_h_rows<3, true>(p, tb, x, y0);
        else conv_h_rows<1, true>(p, tb, x, y0);
    } else if (p.channels == 3) conv_h_rows<3, false>(p, tb, x, y0);
    else conv_h_rows<1, false>(p, tb, x, y0);
}

// Counts CTAs of the tensor-core pass that gave up waiting for a copy (never expected; the counter exists so that a wait
// can be bounded without the failure going unnoticed).  One counter per device.
static __device__ unsigned int g_conv_timeouts;
static unsigned int* conv_timeouts() {
    static unsigned int* ptr[64] = {nullptr};
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev < 0 || dev >= 64) dev = 0;
    if (!ptr[dev]) cudaGetSymbolAddress(reinterpret_cast<void**>(&ptr[dev]), g_conv_timeouts);
    return ptr[dev];
}
unsigned int read_conv_timeouts(cudaStream_t s) {
    unsigned int v = 0;
    cudaMemcpyFromSymbolAsync(&v, g_conv_timeouts, sizeof v, 0, cudaMemcpyDeviceToHost, s);
    cudaStreamSynchronize(s);
    return v;
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
        k_conv_h_mma<<<mma_tiles, kHMmaThreads, sizeof(HMmaSmem), s>>>(passes, map, tables, conv_timeouts());
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

// ---- vertical pass on the tensor cores --------------------------------------------------------------------------------
// out[y][x] = sum_k w[y][k] * src[k][x] as a matrix product with the image's columns as the M dimension, the output rows
// as N and the source rows as K, on the same 8-bit path with the weights split into two limbs as in the horizontal pass.
//   CTA  = 64 output rows (warp q of the first eight owns rows 8q .. 8q+7) x up to 4096 bytes of the rows, walked in chunks
//          of 64 bytes (four tiles of 16 columns); one thread of a ninth warp issues the copies.
//   B    = the warp's weights (eight output rows x the source rows under them, at most 256), both limbs, gathered once
//          into registers.
//   A    = per chunk the source rows under the CTA's 64 output rows x 64 bytes, brought in by tensor-map copies with the
//          64-byte swizzle (boxes of at most 256 rows) into a ring.  The reduction runs over rows, which are not
//          contiguous in memory: ldmatrix.trans hands a lane the bytes (rows 2t, 2t+1) x (columns 2g, 2g+1) of each 8-row
//          group, and one byte permute per register turns two such words into four source rows of one column.  The k
//          slots of a fragment then hold rows {2t, 2t+1, 8+2t, 9+2t} (+16) of the 32-row step rather than 4t .. 4t+3;
//          the weights are gathered in the same order, so the product is the same.  With the swizzle the eight 16-byte
//          row pieces of an ldmatrix fall into different banks.
//   D    = 16 columns x 8 rows per tile: merged, rounded, saturated, collected per warp as 8 rows x 64 bytes in shared
//          memory and stored as 16 bytes per lane.
constexpr int kVMmaConsumers = 256, kVMmaThreads = kVMmaConsumers + 32;
constexpr int kVMmaChunk = 64;            // bytes of a row per chunk
constexpr int kVMmaRing = 98304;          // bytes of the ring: two CTAs per SM
constexpr int kVMmaRingSlack = 2048;      // a warp's last k step reads up to 31 rows past the staged ones (zero weights)
constexpr int kVMmaMaxStages = 8;
static_assert(2 * (int)kVMmaMaxSpan * kVMmaChunk + kVMmaRingSlack <= kVMmaRing, "the ring must hold two chunks of the tallest span");

struct VMmaSmem {
    uint8_t A[kVMmaRing];                                // first: slots start on 512-byte boundaries (swizzle pattern)
    uint8_t out[kVMmaConsumers / 32][8][kVMmaChunk + 16];  // per warp: a chunk's 8 x 64 output bytes (rows padded against bank conflicts)
};

__global__ void __launch_bounds__(kVMmaThreads, 2) k_conv_v_mma(const ConvPass* passes, OwnerMap map, const uint32_t* tables,
                                                                unsigned int* timeouts) {
    extern __shared__ __align__(1024) unsigned char conv_v_smem[];
    VMmaSmem& sm = *reinterpret_cast<VMmaSmem*>(conv_v_smem);
    __shared__ __align__(8) unsigned long long s_bar[2 * kVMmaMaxStages];
    const ConvPass& pg = passes[owner_of_tile(map, blockIdx.x)];
    uint8_t* const p_dst = pg.dst;
    const uint32_t dst_pitch = pg.dst_pitch, out_h = pg.out_h, row_bytes = pg.out_w * pg.channels;
    const uint32_t t0 = pg.t0, tab_n = pg.tab_n, precision = pg.precision, tiles_x = pg.tiles_x;
    const int32_t origin = pg.src_origin;
    const uint32_t box_rows = pg.box_pieces & 0xFFFFu, boxes = pg.box_pieces >> 16;
    const uint32_t tile = blockIdx.x - pg.tile_first;
    const Table tb = table_of(pg, tables);
    const uint32_t ty = tile / tiles_x, tx = tile - ty * tiles_x;
    const uint32_t lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const uint32_t y0 = ty * kVMmaRows, yw = y0 + warp * 8;
    const uint32_t x_first = tx * kVMmaCols, x_end = min(row_bytes, x_first + kVMmaCols);
    const uint32_t nchunks = (x_end - x_first + kVMmaChunk - 1) / kVMmaChunk;
    // first source row under the CTA's output rows (row 0 = the first row of the pass's source)
    const int32_t r_lo = __ldg(tb.start + t0 + y0) - origin;
    const uint32_t stage_bytes = box_rows * boxes * kVMmaChunk;
    const uint32_t nstage = min((uint32_t)kVMmaMaxStages, (uint32_t)(kVMmaRing - kVMmaRingSlack) / stage_bytes);  // >= 2 by the planner's span limit
    const bool warp_active = warp < kVMmaConsumers / 32 && yw < out_h;
    int32_t band_lo = 0;  // first staged row under the warp's output rows
    uint32_t ksteps = 0;
    if (warp_active) {
        const uint32_t yl = min(out_h - 1, yw + 7);
        band_lo = __ldg(tb.start + t0 + yw) - origin - r_lo;
        const int32_t band_hi = __ldg(tb.start + t0 + yl) + __ldg(tb.size + t0 + yl) - origin - r_lo;
        ksteps = (uint32_t)(band_hi - band_lo + 31) >> 5;
    }
    const uint32_t bar0 = (uint32_t)__cvta_generic_to_shared(&s_bar[0]);
    if (threadIdx.x == 0) {
        for (uint32_t i = 0; i < (uint32_t)kVMmaMaxStages; ++i) { mbar_init(bar0 + 8 * i, 1); mbar_init(bar0 + 8 * (kVMmaMaxStages + i), kVMmaConsumers / 32); }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();

    const uint32_t a_base = (uint32_t)__cvta_generic_to_shared(sm.A);
    bool gave_up = false;
    auto wait_for = [&](uint32_t bar, uint32_t parity) {
        uint32_t polls = 0;
        while (!mbar_try_wait(bar, parity)) {
            if (++polls > kHMmaWaitLimit) { gave_up = true; break; }
        }
    };
    if (warp >= kVMmaConsumers / 32) {
        // ---- the copying thread: per chunk `boxes` copies of box_rows rows x 64 bytes, one below the other
        if (lane != 0) return;
        const void* tmap = pg.tmap;
        asm volatile("fence.proxy.tensormap::generic.acquire.gpu [%0], 128;" ::"l"(tmap) : "memory");
        for (uint32_t c = 0; c < nchunks && !gave_up; ++c) {
            const uint32_t slot = c % nstage, use = c / nstage;
            if (use > 0) wait_for(bar0 + 8 * (kVMmaMaxStages + slot), (use - 1) & 1u);
            if (gave_up) break;
            mbar_expect_tx(bar0 + 8 * slot, stage_bytes);
            for (uint32_t bx = 0; bx < boxes; ++bx)
                tensor_copy_2d(a_base + slot * stage_bytes + bx * box_rows * kVMmaChunk, tmap, (int32_t)(x_first + c * kVMmaChunk),
                               r_lo + (int32_t)(bx * box_rows), bar0 + 8 * slot);
        }
        for (uint32_t c = nchunks > nstage ? nchunks - nstage : 0; c < nchunks; ++c) wait_for(bar0 + 8 * (c % nstage), (c / nstage) & 1u);
        if (gave_up) atomicAdd(timeouts, 1u);
        return;
    }

    const uint32_t g = lane >> 2, t4 = lane & 3u;
    const int32_t half = 1 << (precision - 1);
    // ---- B fragments: output row yw + g; byte e of a register is k slot 4 t + e, which holds staged row
    //      band_lo + 32 ks + 16 hf + {2t, 2t+1, 8+2t, 9+2t}[e]
    uint32_t bfr[8][4];
    {
        const uint32_t y = yw + g;
        const bool live = warp_active && y < out_h;
        const int32_t first = live ? __ldg(tb.start + t0 + y) - origin - r_lo - band_lo : 0;  // in rows of the warp's band
        const int32_t taps = live ? __ldg(tb.size + t0 + y) : 0;
        const int16_t* k = tb.k + t0 + y;
#pragma unroll
        for (int ks = 0; ks < 8; ++ks) {
            uint32_t hi[2] = {0, 0}, lo[2] = {0, 0};
            if ((uint32_t)ks < ksteps) {
#pragma unroll
                for (int hf = 0; hf < 2; ++hf)
#pragma unroll
                    for (int e = 0; e < 4; ++e) {
                        const int32_t i = 32 * ks + 16 * hf + 2 * (int32_t)t4 + (e & 1) + 8 * (e >> 1) - first;
                        if (i >= 0 && i < taps) {
                            const int32_t wv = __ldg(k + (size_t)i * tab_n);
                            hi[hf] |= ((uint32_t)(wv >> 8) & 255u) << (8 * e);   // signed high byte
                            lo[hf] |= ((uint32_t)wv & 255u) << (8 * e);          // unsigned low byte
                        }
                    }
            }
            bfr[ks][0] = hi[0]; bfr[ks][1] = hi[1]; bfr[ks][2] = lo[0]; bfr[ks][3] = lo[1];
        }
    }
    const uint32_t out_base = (uint32_t)__cvta_generic_to_shared(&sm.out[warp][0][0]);
    constexpr uint32_t kOutPitch = kVMmaChunk + 16;
    auto consume = [&](auto ks_tag) {
    constexpr int KS = decltype(ks_tag)::value;
    for (uint32_t c = 0; c < nchunks; ++c) {
        const uint32_t slot = c % nstage;
        wait_for(bar0 + 8 * slot, (c / nstage) & 1u);
        if (warp_active) {
            const uint32_t stage = a_base + slot * stage_bytes;
#pragma unroll
            for (int mt = 0; mt < 4; ++mt) {
                int32_t acc_hi[4] = {0, 0, 0, 0}, acc_lo[4] = {half, half, half, half};
#pragma unroll
                for (int ks = 0; ks < KS; ++ks) {
                    // lane i names staged row band_lo + 32 ks + i; its 16-byte piece mt sits at piece mt ^ (row / 2 % 4)
                    const uint32_t row = (uint32_t)band_lo + 32u * ks + lane;
                    uint32_t r[4];
                    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
                                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
                                 : "r"(stage + row * kVMmaChunk + 16u * ((uint32_t)mt ^ ((row >> 1) & 3u))) : "memory");
                    uint32_t a[4];
                    a[0] = __byte_perm(r[0], r[1], 0x6420);  // column 2g
                    a[1] = __byte_perm(r[0], r[1], 0x7531);  // column 2g + 1
                    a[2] = __byte_perm(r[2], r[3], 0x6420);
                    a[3] = __byte_perm(r[2], r[3], 0x7531);
                    mma_u8s8(acc_hi, a, bfr[ks][0], bfr[ks][1]);
                    mma_u8u8(acc_lo, a, bfr[ks][2], bfr[ks][3]);
                }
                // accumulators: (column 2g, row 2t), (column 2g, row 2t+1), (column 2g+1, row 2t), (column 2g+1, row 2t+1)
                int32_t v[4];
#pragma unroll
                for (int i = 0; i < 4; ++i) v[i] = (acc_hi[i] * 256 + acc_lo[i]) >> precision;
                uint32_t pk;
                asm("cvt.pack.sat.u8.s32.b32 %0, %1, %2, %3;" : "=r"(pk) : "r"(v[2]), "r"(v[0]), "r"(0));
                asm volatile("st.shared.u16 [%0], %1;" ::"r"(out_base + (2 * t4) * kOutPitch + 16 * mt + 2 * g), "h"((uint16_t)pk) : "memory");
                asm("cvt.pack.sat.u8.s32.b32 %0, %1, %2, %3;" : "=r"(pk) : "r"(v[3]), "r"(v[1]), "r"(0));
                asm volatile("st.shared.u16 [%0], %1;" ::"r"(out_base + (2 * t4 + 1) * kOutPitch + 16 * mt + 2 * g), "h"((uint16_t)pk) : "memory");
            }
        }
        __syncwarp();
        if (lane == 0) mbar_arrive(bar0 + 8 * (kVMmaMaxStages + slot));  // this warp is done with the slot
        if (warp_active) {
            const uint32_t row = lane >> 2, xb = x_first + c * kVMmaChunk + (lane & 3u) * 16;
            if (yw + row < out_h && xb < row_bytes)  // rows are padded to 16 bytes: the last piece of a row is stored in full
                *reinterpret_cast<uint4*>(p_dst + (size_t)(yw + row) * dst_pitch + xb) = *reinterpret_cast<const uint4*>(&sm.out[warp][row][(lane & 3u) * 16]);
        }
        __syncwarp();  // the warp's piece of shared memory is rewritten by the next chunk
    }
    };
    switch (ksteps) {
        case 1: consume(std::integral_constant<int, 1>{}); break;
        case 2: consume(std::integral_constant<int, 2>{}); break;
        case 3: consume(std::integral_constant<int, 3>{}); break;
        case 4: consume(std::integral_constant<int, 4>{}); break;
        case 5: consume(std::integral_constant<int, 5>{}); break;
        case 6: consume(std::integral_constant<int, 6>{}); break;
        case 7: consume(std::integral_constant<int, 7>{}); break;
        default: consume(std::integral_constant<int, 8>{}); break;
    }
    if (gave_up && lane == 0) atomicAdd(timeouts, 1u);
}

__global__ void __launch_bounds__(kConvVThreads) k_conv_v(const ConvPass* passes, OwnerMap map, const uint32_t* tables, uint32_t first_tile) {
    __shared__ uint32_t s_k[kVFastRows][kVFastMaxWindow / 2];
    __shared__ int32_t s_first[kVFastRows], s_taps[kVFastRows];
    __shared__ uint32_t s_pass;
    const uint32_t tile_index = first_tile + blockIdx.x;
    if (threadIdx.x == 0) s_pass = owner_of_tile(map, tile_index);
    __syncthreads();
    const ConvPass& p = passes[s_pass];
    const uint32_t tile = tile_index - p.tile_first;
    const uint32_t ty = tile / p.tiles_x, tx = tile - ty * p.tiles_x;
    const Table tb = table_of(p, tables);
    if (p.fast) conv_v_vector(p, tb, tx, ty, s_k, s_first, s_taps);
    else conv_v_plain(p, tb, tx, ty);
}

// Vertical passes of one stage: the tensor-core passes come first in `passes` and own tiles [0, mma_tiles) of the map.
void launch_conv_v(const ConvPass* passes, OwnerMap map, const uint32_t* tables, uint32_t mma_tiles, cudaStream_t s) {
    if (!map.total) return;
    if (mma_tiles) {
        static bool configured[64] = {false};
        int dev = 0;
        cudaGetDevice(&dev);
        if (dev < 0 || dev >= 64) dev = 0;
        if (!configured[dev]) {
            cudaFuncSetAttribute(k_conv_v_mma, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)sizeof(VMmaSmem));
            configured[dev] = true;
        }
        k_conv_v_mma<<<mma_tiles, kVMmaThreads, sizeof(VMmaSmem), s>>>(passes, map, tables, conv_timeouts());
    }
    if (map.total > mma_tiles) k_conv_v<<<map.total - mma_tiles, kConvVThreads, 0, s>>>(passes, map, tables, mma_tiles);
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

// ---- alpha pre-multiplication and division (what fast_image_resize does around a convolution of U8x2 / U8x4 images) ----
// multiply: colour = ((colour * alpha + 128) + ((colour * alpha + 128) >> 8)) >> 8
// divide:   colour = min(255, (colour * recip + 2^15) >> 16), recip = ((255 * 2^17) / alpha + 1) >> 1, 0 for alpha 0
__global__ void __launch_bounds__(256) k_alpha(const AlphaJob* jobs, OwnerMap map) {
    const AlphaJob& j = jobs[owner_of_tile(map, blockIdx.x)];
    const uint32_t base = (blockIdx.x - j.tile_first) * kAlphaTilePx, npx = j.width * j.rows, C = j.channels;
    for (uint32_t k = threadIdx.x; k < kAlphaTilePx; k += 256) {
        const uint32_t i = base + k;
        if (i >= npx) break;
        const uint32_t y = i / j.width, x = i - y * j.width;
        const uint8_t* s = j.src + (size_t)y * j.src_pitch + (size_t)x * C;
        uint8_t* d = j.dst + (size_t)y * j.dst_pitch + (size_t)x * C;
        const uint32_t a = s[C - 1];
        const uint32_t recip = a ? ((255u << 17) / a + 1u) >> 1 : 0u;
        for (uint32_t c = 0; c + 1 < C; ++c) {
            const uint32_t v = s[c];
            uint32_t r;
            if (j.divide) r = min(255u, (v * recip + (1u << 15)) >> 16);
            else { const uint32_t t = v * a + 128u; r = ((t >> 8) + t) >> 8; }
            d[c] = (uint8_t)r;
        }
        d[C - 1] = (uint8_t)a;
    }
}

void launch_alpha(const AlphaJob* jobs, OwnerMap map, cudaStream_t s) {
    if (map.total) k_alpha<<<map.total, 256, 0, s>>>(jobs, map);
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
