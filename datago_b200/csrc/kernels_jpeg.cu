// Baseline JPEG on sm_100a: byte unstuffing, Huffman entropy decode, dequantise + 8x8 integer IDCT,
// chroma upsampling + YCbCr->RGB.  Replaces the zune-jpeg decode datago reaches through
// image::load_from_memory (src/worker_wds.rs:45) / ImageReader::decode (src/worker_files.rs:14-16).
//
// All of it is integer / byte work bound by HBM traffic or by serial bit-parsing latency; no tensor cores.
#include <cstdint>
#include <cstdlib>

#include "kernels.h"

namespace dg {

// ---------------------------------------------------------------------------------------------------------------
// helpers
// ---------------------------------------------------------------------------------------------------------------
__device__ __forceinline__ uint32_t owner_of(const OwnerMap& m, uint32_t idx) {
    uint32_t o = __ldg(m.coarse + (idx >> m.shift));
    while (o + 1 < m.n && __ldg(m.first + o + 1) <= idx) ++o;
    return o;
}

__device__ const uint8_t kNatural[64] = {0,  1,  8,  16, 9,  2,  3,  10, 17, 24, 32, 25, 18, 11, 4,  5,
                                         12, 19, 26, 33, 40, 48, 41, 34, 27, 20, 13, 6,  7,  14, 21, 28,
                                         35, 42, 49, 56, 57, 50, 43, 36, 29, 22, 15, 23, 30, 37, 44, 51,
                                         58, 59, 52, 45, 38, 31, 39, 46, 53, 60, 61, 54, 47, 55, 62, 63};

// ---------------------------------------------------------------------------------------------------------------
// K0  unstuff: one CTA per image walks the entropy-coded segment in 4 KB steps, drops stuffed zeros (FF 00 -> FF),
//     fill bytes and RSTn markers, records where each restart segment starts in the compacted stream and stops at
//     the first other marker (EOI).  The compacted stream lets the entropy decoder load aligned 32-bit words.
//     The kept bytes of a step are collected in shared memory and leave as aligned 16-byte pieces (a thread's bytes land
//     at an arbitrary offset of the output, and single-byte stores to global memory cost a partial sector write each);
//     what does not fill a piece waits at the front of the buffer for the next step.
// ---------------------------------------------------------------------------------------------------------------
constexpr int kUnstuffThreads = 256;

__global__ void __launch_bounds__(kUnstuffThreads) k_unstuff(JpegWave w) {
    const JpegDesc& d = w.descs[blockIdx.x];
    const uint8_t* in = w.raw + d.raw_off;
    uint8_t* out = w.us + d.us_off;
    uint32_t* seg = w.seg_start + d.seg_off;
    const uint32_t len = d.raw_len;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;

    __shared__ uint32_t s_end;
    __shared__ uint32_t s_warp[kUnstuffThreads / 32];
    __shared__ __align__(16) uint8_t s_out[kUnstuffThreads * 16 + 16];  // a step's bytes behind at most 15 carried ones
    uint32_t kept = 0, nrst = 0;  // running totals, identical in every thread
    uint32_t flushed = 0;         // bytes already in global memory, a multiple of 16; kept - flushed wait in s_out
    if (tid == 0) seg[0] = 0;

    for (uint32_t base = 0; base < len; base += kUnstuffThreads * 16) {
        if (tid == 0) s_end = 0xFFFFFFFFu;
        __syncthreads();
        const uint32_t i0 = base + tid * 16;
        uint8_t b[18];
        {
            uint4 v = make_uint4(0, 0, 0, 0);
            if (i0 < len) v = __ldg(reinterpret_cast<const uint4*>(in + i0));  // blob slices are padded to 16 bytes with zeros
            const uint32_t ww[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
            for (int j = 0; j < 16; ++j) b[j + 1] = (uint8_t)(ww[j >> 2] >> (8 * (j & 3)));
            b[0] = (i0 > 0 && i0 <= len) ? __ldg(in + i0 - 1) : 0;
            b[17] = (i0 + 16 < len) ? __ldg(in + i0 + 16) : 0;
        }
        uint32_t keep = 0, rst = 0, term = 0xFFFFFFFFu;
#pragma unroll
        for (int j = 0; j < 16; ++j) {
            const uint32_t idx = i0 + j;
            if (idx >= len) break;
            const uint8_t cur = b[j + 1], pv = b[j], nx = b[j + 2];
            bool k = true;
            if (cur == 0xFF) {
                if (nx == 0x00) k = true;                      // data byte FF (its stuffed zero is dropped below)
                else if (nx == 0xFF) k = false;                // fill byte
                else if (nx >= 0xD0 && nx <= 0xD7) { k = false; rst |= 1u << j; }
                else { k = false; if (term == 0xFFFFFFFFu) term = idx; }  // any other marker ends the scan
            } else if (pv == 0xFF && (cur == 0x00 || (cur >= 0xD0 && cur <= 0xD7))) {
                k = false;
            }
            if (k) keep |= 1u << j;
        }
        if (term != 0xFFFFFFFFu) atomicMin(&s_end, term);
        __syncthreads();
        const uint32_t end = s_end;
        if (end != 0xFFFFFFFFu) {  // nothing at or after the terminating marker survives
            if (i0 >= end) { keep = 0; rst = 0; }
            else if (end - i0 < 16) { const uint32_t m = (1u << (end - i0)) - 1; keep &= m; rst &= m; }
        }
        // exclusive scan of (restart count << 16 | kept count) over the CTA
        const uint32_t mine = ((uint32_t)__popc(rst) << 16) | (uint32_t)__popc(keep);
        uint32_t inc = mine;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) { const uint32_t t = __shfl_up_sync(0xFFFFFFFFu, inc, o); if (lane >= o) inc += t; }
        if (lane == 31) s_warp[warp] = inc;
        __syncthreads();
        uint32_t wpre = 0, tot = 0;
#pragma unroll
        for (int i = 0; i < kUnstuffThreads / 32; ++i) { const uint32_t t = s_warp[i]; if (i < warp) wpre += t; tot += t; }
        const uint32_t excl = wpre + inc - mine;
        uint32_t pos = kept + (excl & 0xFFFFu), r = nrst + (excl >> 16);
#pragma unroll
        for (int j = 0; j < 16; ++j) {
            if (keep & (1u << j)) { s_out[pos - flushed] = b[j + 1]; ++pos; }
            if (rst & (1u << j)) { ++r; if (r < d.nseg) seg[r] = pos; }
        }
        kept += tot & 0xFFFFu;
        nrst += tot >> 16;
        __syncthreads();  // the step's bytes are in s_out
        const uint32_t pieces = (kept - flushed) >> 4, rem = (kept - flushed) & 15u;
        for (uint32_t t = tid; t < pieces; t += kUnstuffThreads)
            reinterpret_cast<uint4*>(out + flushed)[t] = reinterpret_cast<const uint4*>(s_out)[t];
        const uint8_t carried = (uint32_t)tid < rem ? s_out[pieces * 16 + tid] : (uint8_t)0;
        __syncthreads();  // ... and have been read: the rest moves to the front (the next step writes behind it, after
                          // its own first barrier)
        if ((uint32_t)tid < rem) s_out[tid] = carried;
        flushed += pieces * 16;
        if (end != 0xFFFFFFFFu) break;
    }
    __syncthreads();
    // the last bytes, and zeros behind them: the bit reader may look a few bytes past the end
    if ((uint32_t)tid < kept - flushed + 16) out[flushed + tid] = (uint32_t)tid < kept - flushed ? s_out[tid] : (uint8_t)0;
    if (tid == 0) {
        w.us_len[blockIdx.x] = kept;
        w.seg_found[blockIdx.x] = nrst + 1;
    }
}

void launch_unstuff(const JpegWave& w, cudaStream_t s) {
    if (w.n) k_unstuff<<<w.n, kUnstuffThreads, 0, s>>>(w);
}

// ---------------------------------------------------------------------------------------------------------------
// K1  Huffman entropy decode.
//
// The decoder state between two symbols is (bit position, slot), slot = 64 * block index + zig-zag index: every
// block owns exactly 64 slots, an AC run or an end-of-block only advances the slot.  Knowing the slot modulo the
// MCU size gives the component (hence the tables) and whether the next symbol is a DC or an AC code.
//
//  * images with restart intervals: one thread per restart segment; the segment's first MCU and the zero DC
//    predictors are known, so coefficients are written in a single pass.
//  * images without: the stream is cut into subsequences of kSubseqBits (2048) bits, one thread each.  Thread j decodes
//    from a guessed entry state, then re-decodes from the exit state of thread j-1 until entry(j) == exit(j-1)
//    for every j (Huffman streams re-synchronise after a few symbols, so this takes 2-3 rounds; the loop is
//    bounded by the thread count because thread j is final after round j).  A prefix sum over the slots and DC
//    differences of the subsequences then gives every thread its output position and DC predictors, and a last
//    pass writes the coefficients.  One CTA walks one image in chunks of as many subsequences as it has threads, carrying
//    the exact state across chunks, so no CTA ever waits on another.
// ---------------------------------------------------------------------------------------------------------------
struct HuffCtx {
    const char* base;  // tables are addressed as base + byte offset (shared memory or the global pool)
    uint32_t dc_off0, dc_off1, dc_off2, ac_off0, ac_off1, ac_off2;
    uint32_t luma_blocks;  // blocks of component 0 per MCU
    uint32_t mcu_slots;    // 64 * blocks per MCU
};

__device__ __forceinline__ uint32_t shr_clamp(uint32_t x, uint32_t n) {  // shift counts >= 32 give 0
    uint32_t r;
    asm("shr.b32 %0, %1, %2;" : "=r"(r) : "r"(x), "r"(n));
    return r;
}

// Codes longer than the fast table.  No search: the code length follows from six comparisons against the table's
// left-aligned limits (see HuffTable::limit), the symbol from the canonical offset of that length.  The lanes of a
// warp sit at unrelated places of their streams, so whenever one of them meets a long code all of them pay for this
// path: it has to be short.
template <bool WRITE>
__device__ __forceinline__ uint32_t huff_long_code(const HuffTable* t, uint32_t top, uint32_t& err) {
    const uint32_t v = top >> 16;
    const uint4 la = *reinterpret_cast<const uint4*>(&t->limit[0]);
    const uint4 lb = *reinterpret_cast<const uint4*>(&t->limit[4]);
    const uint32_t len = 10u + (v >= la.x) + (v >= la.y) + (v >= la.z) + (v >= la.w) + (v >= lb.x) + (v >= lb.y);
    if (v >= lb.z) { if (WRITE) err |= kStBadCode; return huff_pack(16, 0); }
    return huff_pack(len, t->vals[(int32_t)(v >> (16u - len)) + t->valoff[len]]);
}

// Decodes the symbols that start in [p, end_bit) while fewer than max_slots slots have been consumed.
// dc0..2: sums of DC differences (WRITE == false) or running DC predictors (WRITE == true).
// One code path for DC and AC symbols (selects instead of branches): the lanes of a warp are at unrelated places of
// their streams, so every branch taken by one lane is paid by all of them.
//
// Writing (WRITE == true).  Two-byte stores of single coefficients, every lane to another block, are what the decoders
// spent most of their time on (each is a partial write of a 32-byte sector, which the memory system completes by reading
// the sector first).  With ROWS > 0 a lane collects the first ROWS rows of its current block (ROWS * 16 bytes; the
// low-frequency corner, where nearly all coefficients of a sparse block are) in shared memory, buf[row * T + thread], and
// writes them out when the block ends: whole 32-byte sectors, two rows at a time, for the sectors that received a
// coefficient (the coefficient region is zero beforehand, so rows that are still zero may be written or skipped).
// Coefficients of later rows are stored one by one as before.  A block the span shares with a neighbouring span (a span
// of the speculative decoder starts and ends anywhere) is never written in rows: its first block, when the span begins
// inside it, is stored coefficient by coefficient, and so is what the buffer holds when the span ends inside a block.
// The buffer is all zero when the call begins and when it returns.
template <bool WRITE, int ROWS = 0, int T = 1>
__device__ __forceinline__ void decode_span(const uint32_t* __restrict__ words, const uint32_t nwords, uint32_t& p,
                                            const uint32_t end_bit, const uint32_t total_bits, uint32_t& slotmod,
                                            uint32_t& nslots, const uint32_t max_slots, int32_t& dc0, int32_t& dc1,
                                            int32_t& dc2, const HuffCtx& hc, int16_t* __restrict__ coef,
                                            const uint32_t slot_abs, const uint8_t* __restrict__ natural, uint32_t& err,
                                            uint4* buf = nullptr) {
    static_assert(ROWS % 2 == 0, "rows are written out as 32-byte sectors");
    auto word = [&](uint32_t i) -> uint32_t { return i < nwords ? __byte_perm(__ldg(words + i), 0, 0x0123) : 0u; };
    // a window of three stream words: the word fetched when the position crosses a word boundary is first needed one
    // boundary later, so its latency (the streams sit in global memory) stays off the symbol-to-symbol critical path
    uint32_t wi = p >> 5;
    uint32_t w0 = word(wi), w1 = word(wi + 1), w2 = word(wi + 2);
    uint32_t sectors = 0;                          // sectors of the buffer that hold a coefficient
    bool direct = (slotmod & 63u) != 0;            // the span begins inside a block
    const uint32_t buf_b = (WRITE && ROWS > 0) ? (uint32_t)__cvta_generic_to_shared(buf + threadIdx.x) : 0u;  // row 0 of this lane
    while (p < end_bit && nslots < max_slots) {
        const uint32_t top = __funnelshift_l(w1, w0, p & 31u);
        const uint32_t z = slotmod & 63u, c = slotmod >> 6;
        const bool isdc = z == 0;
        const uint32_t comp = c < hc.luma_blocks ? 0u : c - hc.luma_blocks + 1u;
        const uint32_t toff = isdc ? (comp == 0 ? hc.dc_off0 : comp == 1 ? hc.dc_off1 : hc.dc_off2)
                                   : (comp == 0 ? hc.ac_off0 : comp == 1 ? hc.ac_off1 : hc.ac_off2);
        const HuffTable* t = reinterpret_cast<const HuffTable*>(hc.base + toff);
        uint32_t e = t->lut[top >> (32 - kLutBits)];
        if (e == 0) e = huff_long_code<WRITE>(t, top, err);
        const uint32_t used = e & 63u, len = (e >> 6) & 31u, s = (e >> 11) & 15u, r = (e >> 15) & 15u;
        if (p + used > total_bits) { p = total_bits; break; }  // the stream ends inside this symbol
        const uint32_t raw = shr_clamp(top << len, 32u - s);   // the s extra bits (0 when s == 0)
        const int32_t v = (int32_t)raw - (int32_t)((shr_clamp(raw, s - 1u) ^ 1u) * ((1u << s) - 1u));  // T.81 EXTEND
        uint32_t adv = (s != 0u || r == 15u) ? r + 1u : 64u;   // coefficient after a run, ZRL, or end of block
        adv = isdc ? 1u : min(adv, 64u - z);
        const int32_t dv = isdc ? v : 0;
        dc0 += comp == 0 ? dv : 0;
        dc1 += comp == 1 ? dv : 0;
        dc2 += comp == 2 ? dv : 0;
        if (WRITE) {
            const uint32_t zz = isdc ? 0u : z + r;
            const int32_t val = isdc ? (comp == 0 ? dc0 : comp == 1 ? dc1 : dc2) : v;
            const bool has = isdc ? val != 0 : s != 0u;  // (a zero DC term needs no store: the region is zero beforehand)
            if (has && zz > 63u) err |= kStCoefRange;
            else if (has) {
                const uint32_t nat = natural[zz];
                int16_t* const block = coef + (size_t)(slot_abs + nslots - z);  // the slot of a DC code is 64 * its block
                if (ROWS == 0 || direct || nat >= 8u * ROWS) {
                    block[nat] = (int16_t)val;
                } else {
                    asm volatile("st.shared.u16 [%0], %1;" ::"r"(buf_b + (nat >> 3) * (uint32_t)(T * 16) + (nat & 7u) * 2u), "h"((uint16_t)val) : "memory");
                    sectors |= 1u << (nat >> 4);
                }
            }
            if (ROWS > 0 && !isdc && z + adv == 64u) {  // the block ends with this symbol
                if (sectors) {
                    uint4* const block = reinterpret_cast<uint4*>(coef + (size_t)(slot_abs + nslots - z));
#pragma unroll
                    for (int sc = 0; sc < ROWS / 2; ++sc)
                        if ((sectors >> sc) & 1u) {
                            uint4* const b0 = buf + (2 * sc) * T + threadIdx.x;
                            block[2 * sc] = b0[0];
                            block[2 * sc + 1] = b0[T];
                            b0[0] = make_uint4(0, 0, 0, 0);
                            b0[T] = make_uint4(0, 0, 0, 0);
                        }
                    sectors = 0;
                }
                direct = false;
            }
        }
        p += used;
        nslots += adv;
        slotmod += adv;
        if (slotmod >= hc.mcu_slots) slotmod -= hc.mcu_slots;
        const uint32_t nwi = p >> 5;
        if (nwi != wi) { w0 = w1; w1 = w2; w2 = word(nwi + 2); wi = nwi; }  // a symbol has at most 27 bits: one boundary at a time
    }
    if (WRITE && ROWS > 0 && sectors) {
        // the span ends inside a block that the next span continues: coefficient by coefficient
        int16_t* const block = coef + (size_t)(slot_abs + nslots - (slotmod & 63u));
#pragma unroll
        for (int row = 0; row < ROWS; ++row)
            if ((sectors >> (row >> 1)) & 1u) {
                uint4* const b0 = buf + row * T + threadIdx.x;
                const uint4 q = *b0;
                const uint32_t ww[4] = {q.x, q.y, q.z, q.w};
#pragma unroll
                for (int k = 0; k < 8; ++k) {
                    const uint32_t h = (ww[k >> 1] >> (16 * (k & 1))) & 0xFFFFu;
                    if (h) block[row * 8 + k] = (int16_t)h;
                }
                *b0 = make_uint4(0, 0, 0, 0);
            }
    }
}

// ---- restart-interval images: one thread per segment -----------------------------------------------------------
constexpr int kRestartThreads = 128;
constexpr uint32_t kRestartSharedTables = 8;  // a pool of at most this many Huffman tables is staged in shared memory
#ifndef DG_RESTART_BUF_ROWS
#define DG_RESTART_BUF_ROWS 4
#endif
#ifndef DG_RESTART_MIN_CTAS
#define DG_RESTART_MIN_CTAS 1
#endif
constexpr int kRestartBufRows = DG_RESTART_BUF_ROWS;  // rows of its current block a lane collects before writing them out

__global__ void __launch_bounds__(kRestartThreads, DG_RESTART_MIN_CTAS) k_huff_restart(JpegWave w) {
    __shared__ uint8_t s_nat[64];
    extern __shared__ __align__(16) unsigned char restart_smem[];
    // dynamic: the block buffers of the lanes (kRestartBufRows x 128 x 16 bytes), then the staged tables (when the pool is small)
    uint4* const s_buf = reinterpret_cast<uint4*>(restart_smem);
    HuffTable* const s_tab = reinterpret_cast<HuffTable*>(restart_smem + kRestartBufRows * kRestartThreads * 16);
    for (uint32_t i = threadIdx.x; i < (uint32_t)(kRestartBufRows * kRestartThreads); i += kRestartThreads) s_buf[i] = make_uint4(0, 0, 0, 0);
    if (threadIdx.x < 64) s_nat[threadIdx.x] = kNatural[threadIdx.x];
    // The segments of a CTA belong to several images, but files written by the same encoder share their tables and the
    // pool holds each distinct table once: a small pool is copied whole, so that the per-symbol table look-ups (on the
    // critical path of every lane) are shared-memory reads; a larger pool is read in place.
    const bool staged = w.n_huff <= kRestartSharedTables;
    if (staged) {
        const uint32_t words = w.n_huff * (uint32_t)(sizeof(HuffTable) / 4);
        const uint32_t* src = reinterpret_cast<const uint32_t*>(w.huff);
        uint32_t* dst = reinterpret_cast<uint32_t*>(&s_tab[0]);
        for (uint32_t i = threadIdx.x; i < words; i += kRestartThreads) dst[i] = __ldg(src + i);
    }
    __syncthreads();
    const uint32_t g = blockIdx.x * kRestartThreads + threadIdx.x;
    if (g >= w.restart_segs.total) return;
    const uint32_t r = owner_of(w.restart_segs, g);
    const uint32_t img = w.restart_list[r];
    const uint32_t k = g - w.restart_segs.first[r];
    const JpegDesc& d = w.descs[img];
    const uint32_t found = w.seg_found[img];
    if (k == 0 && found != d.nseg) atomicOr(w.status + d.item, kStBadMarker);
    if (k >= found) return;
    const uint32_t* seg = w.seg_start + d.seg_off;
    const uint32_t us_len = w.us_len[img];
    const uint32_t b0 = seg[k], b1 = (k + 1 < found && k + 1 < d.nseg) ? seg[k + 1] : us_len;
    const uint32_t mcus = d.mcux * d.mcuy;
    const uint32_t m0 = k * d.restart, m1 = min(m0 + d.restart, mcus);
    HuffCtx hc;
    hc.base = staged ? reinterpret_cast<const char*>(&s_tab[0]) : reinterpret_cast<const char*>(w.huff);
    hc.dc_off0 = d.dc_tab[0] * (uint32_t)sizeof(HuffTable); hc.ac_off0 = d.ac_tab[0] * (uint32_t)sizeof(HuffTable);
    hc.dc_off1 = d.dc_tab[1] * (uint32_t)sizeof(HuffTable); hc.ac_off1 = d.ac_tab[1] * (uint32_t)sizeof(HuffTable);
    hc.dc_off2 = d.dc_tab[2] * (uint32_t)sizeof(HuffTable); hc.ac_off2 = d.ac_tab[2] * (uint32_t)sizeof(HuffTable);
    hc.luma_blocks = d.hs * d.vs;
    hc.mcu_slots = d.bpm * 64u;
    uint32_t p = b0 * 8u, slotmod = 0, nslots = 0, err = 0;
    int32_t dc0 = 0, dc1 = 0, dc2 = 0;
    const uint32_t want = (m1 - m0) * hc.mcu_slots;
    decode_span<true, kRestartBufRows, kRestartThreads>(reinterpret_cast<const uint32_t*>(w.us + d.us_off), (us_len + 3) / 4 + 2, p, b1 * 8u,
                                                       b1 * 8u, slotmod, nslots, want, dc0, dc1, dc2, hc, w.coef + d.block_off * 64,
                                                       m0 * hc.mcu_slots, s_nat, err, s_buf);
    if (nslots < want) err |= kStTruncated;
    if (err) atomicOr(w.status + d.item, err);
}

// ---- images without restart markers: speculative subsequences, one CTA per image ---------------------------------
// Two CTA sizes: 256 threads when a launch has enough images to fill the GPU with them, 512 when it has not (few, large
// images: the launch then lasts as long as its longest image, whose chunks are walked one after the other, and a CTA
// twice as wide halves the number of chunks).
#ifndef DG_SPEC_THREADS
#define DG_SPEC_THREADS 256
#endif
#ifndef DG_SUBSEQ_BITS
#define DG_SUBSEQ_BITS 2048
#endif
#ifndef DG_SPEC_MIN_CTAS
#define DG_SPEC_MIN_CTAS 6
#endif
constexpr int kSpecThreads = DG_SPEC_THREADS;      // the narrow variant
constexpr int kSpecThreadsWide = 512, kSpecMinCtasWide = 3;
constexpr uint32_t kSpecWideBelow = 1024;         // images per launch below which the wide variant is used (DATAGO_B200_SPEC_WIDE_BELOW overrides)
constexpr uint32_t kSubseqBits = DG_SUBSEQ_BITS;

struct Scan4 { uint32_t n; int32_t a, b, c; };

// Per-subsequence state of the chunk being synchronised (shared memory).
template <int T>
struct SpecState {
    uint32_t entry_p[T], entry_sm[T];  // decoder state at the start of the subsequence
    uint32_t exit_p[T], exit_sm[T];    // ... after its last symbol
    uint32_t n[T];                     // slots consumed
    int32_t dc[3][T];                  // sums of DC differences per component
    uint32_t list[T];                  // subsequences to re-decode this round
    // The same after the first symbol that ends kSyncCheckBits or more into the subsequence: a re-decode from a
    // corrected entry state that arrives here in the state its predecessor had here has synchronised with it, and
    // the rest of the subsequence need not be decoded again.
    uint32_t ck_p[T], ck_sm[T], ck_n[T];
    int32_t ck_dc[3][T];
};
constexpr uint32_t kSyncCheckBits = 256;

template <int T>
struct SpecSmem {
    HuffTable tab[6];
    SpecState<T> st;
    Scan4 warp[T / 32];
    uint32_t wcount[T / 32];
    uint32_t carry_p, carry_slot;
    int32_t carry_dc[3];
    uint8_t nat[64];
};

template <int T, int MIN_CTAS>
__global__ void __launch_bounds__(T, MIN_CTAS) k_huff_spec(JpegWave w, uint32_t first) {
    const uint32_t img = w.spec_list[first + blockIdx.x];
    const JpegDesc& d = w.descs[img];
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;

    extern __shared__ __align__(16) unsigned char spec_smem[];
    SpecSmem<T>& sh = *reinterpret_cast<SpecSmem<T>*>(spec_smem);
    HuffTable (&s_tab)[6] = sh.tab;
    uint8_t (&s_nat)[64] = sh.nat;
    SpecState<T>& st = sh.st;
    Scan4 (&s_warp)[T / 32] = sh.warp;
    uint32_t (&s_wcount)[T / 32] = sh.wcount;
    uint32_t& s_carry_p = sh.carry_p;
    uint32_t& s_carry_slot = sh.carry_slot;
    int32_t (&s_carry_dc)[3] = sh.carry_dc;

    {   // stage the image's Huffman tables in shared memory (word copies)
        const uint32_t ids[6] = {d.dc_tab[0], d.dc_tab[1], d.dc_tab[2], d.ac_tab[0], d.ac_tab[1], d.ac_tab[2]};
        constexpr int kWords = sizeof(HuffTable) / 4;
        for (int t = 0; t < 6; ++t) {
            const uint32_t* src = reinterpret_cast<const uint32_t*>(w.huff + ids[t]);
            uint32_t* dst = reinterpret_cast<uint32_t*>(&s_tab[t]);
            for (int i = tid; i < kWords; i += T) dst[i] = __ldg(src + i);
        }
        if (tid < 64) s_nat[tid] = kNatural[tid];
        if (tid == 0) { s_carry_p = 0; s_carry_slot = 0; s_carry_dc[0] = s_carry_dc[1] = s_carry_dc[2] = 0; }
    }
    __syncthreads();
    HuffCtx hc;
    hc.base = reinterpret_cast<const char*>(&s_tab[0]);
    hc.dc_off0 = 0; hc.dc_off1 = sizeof(HuffTable); hc.dc_off2 = 2 * sizeof(HuffTable);
    hc.ac_off0 = 3 * sizeof(HuffTable); hc.ac_off1 = 4 * sizeof(HuffTable); hc.ac_off2 = 5 * sizeof(HuffTable);
    hc.luma_blocks = d.hs * d.vs;
    hc.mcu_slots = d.bpm * 64u;

    const uint32_t us_len = w.us_len[img];
    const uint32_t total_bits = us_len * 8u;
    const uint32_t total_slots = d.nblocks * 64u;
    const uint32_t nsub = (total_bits + kSubseqBits - 1) / kSubseqBits;
    const uint32_t* words = reinterpret_cast<const uint32_t*>(w.us + d.us_off);
    const uint32_t nwords = (us_len + 3) / 4 + 2;  // the unstuffed stream is followed by 16 zero bytes
    int16_t* coef = w.coef + d.block_off * 64;
    uint32_t err = 0;

    // decode subsequence j of the chunk from its recorded entry state and record exit state and sums
    auto decode_into_state = [&](uint32_t chunk, int j, bool first_time) {
        uint32_t p = st.entry_p[j], sm = st.entry_sm[j], n = 0, dummy = 0;
        int32_t a = 0, b = 0, c = 0;
        const uint32_t end_bit = min((chunk + j + 1) * kSubseqBits, total_bits);
        const uint32_t check_bit = min((chunk + j) * kSubseqBits + kSyncCheckBits, end_bit);
        decode_span<false>(words, nwords, p, check_bit, total_bits, sm, n, 0xFFFFFFFFu, a, b, c, hc, nullptr, 0, s_nat, dummy);
        if (!first_time && p == st.ck_p[j] && sm == st.ck_sm[j]) {
            // synchronised: from here on the previous decode of this subsequence stands; only the part before the
            // check point contributes differently to the slot count and the DC sums
            st.n[j] = n + (st.n[j] - st.ck_n[j]);
            st.dc[0][j] = a + (st.dc[0][j] - st.ck_dc[0][j]);
            st.dc[1][j] = b + (st.dc[1][j] - st.ck_dc[1][j]);
            st.dc[2][j] = c + (st.dc[2][j] - st.ck_dc[2][j]);
            st.ck_n[j] = n; st.ck_dc[0][j] = a; st.ck_dc[1][j] = b; st.ck_dc[2][j] = c;
            return;
        }
        st.ck_p[j] = p; st.ck_sm[j] = sm; st.ck_n[j] = n;
        st.ck_dc[0][j] = a; st.ck_dc[1][j] = b; st.ck_dc[2][j] = c;
        decode_span<false>(words, nwords, p, end_bit, total_bits, sm, n, 0xFFFFFFFFu, a, b, c, hc, nullptr, 0, s_nat, dummy);
        st.exit_p[j] = p; st.exit_sm[j] = sm; st.n[j] = n;
        st.dc[0][j] = a; st.dc[1][j] = b; st.dc[2][j] = c;
    };

    for (uint32_t chunk = 0; chunk < nsub; chunk += T) {
        const int cnt = (int)min((uint32_t)T, nsub - chunk);
        const bool active = tid < cnt;
        // entry state: exact for the first subsequence of the chunk, a guess (AC code of the first block) elsewhere
        st.entry_p[tid] = tid == 0 ? s_carry_p : (chunk + tid) * kSubseqBits;
        st.entry_sm[tid] = tid == 0 ? s_carry_slot % hc.mcu_slots : 1u;
        if (active) decode_into_state(chunk, tid, true);
        __syncthreads();
        uint32_t rounds = 1, decodes = (uint32_t)cnt;
        // Re-decode every subsequence whose entry state differs from its left neighbour's exit state until none
        // does.  After round r the first r subsequences are final, so the loop ends within cnt rounds.  The
        // subsequences to redo are compacted so that a late round with a handful of them occupies one warp.
        for (int round = 0; round <= T + 1; ++round) {
            bool need = false;
            if (active && tid > 0) {
                const uint32_t pp = st.exit_p[tid - 1], ps = st.exit_sm[tid - 1];
                need = pp != st.entry_p[tid] || ps != st.entry_sm[tid];
                if (need) { st.entry_p[tid] = pp; st.entry_sm[tid] = ps; }
            }
            const uint32_t ballot = __ballot_sync(0xFFFFFFFFu, need);
            if (lane == 0) s_wcount[warp] = __popc(ballot);
            __syncthreads();
            uint32_t before = 0, total = 0;
#pragma unroll
            for (int i = 0; i < T / 32; ++i) { const uint32_t v = s_wcount[i]; if (i < warp) before += v; total += v; }
            if (total == 0) break;
            if (need) st.list[before + __popc(ballot & ((1u << lane) - 1))] = (uint32_t)tid;
            __syncthreads();
            if ((uint32_t)tid < total) decode_into_state(chunk, (int)st.list[tid], false);
            ++rounds;
            decodes += total;
            __syncthreads();
            if (round == T + 1) err |= kStSyncLimit;
        }
        // exclusive prefix over (slots, DC sums) of the chunk
        Scan4 inc{active ? st.n[tid] : 0u, active ? st.dc[0][tid] : 0, active ? st.dc[1][tid] : 0, active ? st.dc[2][tid] : 0};
        const Scan4 mine = inc;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            const uint32_t tn = __shfl_up_sync(0xFFFFFFFFu, inc.n, o);
            const int32_t ta = __shfl_up_sync(0xFFFFFFFFu, inc.a, o), tb = __shfl_up_sync(0xFFFFFFFFu, inc.b, o),
                          tc = __shfl_up_sync(0xFFFFFFFFu, inc.c, o);
            if (lane >= o) { inc.n += tn; inc.a += ta; inc.b += tb; inc.c += tc; }
        }
        if (lane == 31) s_warp[warp] = inc;
        __syncthreads();
        Scan4 pre{0, 0, 0, 0}, tot{0, 0, 0, 0};
#pragma unroll
        for (int i = 0; i < T / 32; ++i) {
            const Scan4 t = s_warp[i];
            if (i < warp) { pre.n += t.n; pre.a += t.a; pre.b += t.b; pre.c += t.c; }
            tot.n += t.n; tot.a += t.a; tot.b += t.b; tot.c += t.c;
        }
        const uint32_t slot0 = s_carry_slot + pre.n + inc.n - mine.n;
        int32_t p0 = s_carry_dc[0] + pre.a + inc.a - mine.a, p1 = s_carry_dc[1] + pre.b + inc.b - mine.b,
                p2 = s_carry_dc[2] + pre.c + inc.c - mine.c;
        // write pass
        if (active && slot0 < total_slots) {
            uint32_t p = st.entry_p[tid], sm = st.entry_sm[tid], nn = 0;
            const uint32_t end_bit = min((chunk + tid + 1) * kSubseqBits, total_bits);
            decode_span<true>(words, nwords, p, end_bit, total_bits, sm, nn, total_slots - slot0, p0, p1, p2, hc, coef, slot0, s_nat, err);
        }
        __syncthreads();
        if (tid == 0) {
            atomicAdd(w.spec_stats, 1ull);
            atomicAdd(w.spec_stats + 1, (unsigned long long)rounds);
            atomicAdd(w.spec_stats + 2, (unsigned long long)decodes + (uint32_t)cnt);
            s_carry_p = st.exit_p[cnt - 1];
            s_carry_slot += tot.n;
            s_carry_dc[0] += tot.a; s_carry_dc[1] += tot.b; s_carry_dc[2] += tot.c;
        }
        __syncthreads();
    }
    if (tid == 0 && s_carry_slot < total_slots) err |= kStTruncated;
    if (err) atomicOr(w.status + d.item, err);
}

void launch_huff_restart(const JpegWave& w, cudaStream_t s) {
    if (w.restart_segs.total)
    {
        const size_t smem = (size_t)kRestartBufRows * kRestartThreads * 16 +
                            (w.n_huff <= kRestartSharedTables ? (size_t)w.n_huff * sizeof(HuffTable) : 0);
        k_huff_restart<<<(w.restart_segs.total + kRestartThreads - 1) / kRestartThreads, kRestartThreads, smem, s>>>(w);
    }
}

// Three CTA sizes.  A CTA walks its image chunk by chunk (T subsequences each), so the launch lasts as long as the
// longest image needs chunks: the first `n_huge` images of the list (the longest: more than 1024 subsequences) get
// 1024-thread CTAs, launched on `huge_stream` beside the rest.
constexpr int kSpecThreadsHuge = 1024;
template <int T, int MIN_CTAS>
static void launch_spec_variant(const JpegWave& w, uint32_t first, uint32_t count, cudaStream_t s) {
    static bool configured[64] = {false};
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev < 0 || dev >= 64) dev = 0;
    if (!configured[dev]) {
        cudaFuncSetAttribute(k_huff_spec<T, MIN_CTAS>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)sizeof(SpecSmem<T>));
        configured[dev] = true;
    }
    k_huff_spec<T, MIN_CTAS><<<count, T, sizeof(SpecSmem<T>), s>>>(w, first);
}

void launch_huff_spec(const JpegWave& w, uint32_t n_huge, cudaStream_t s, cudaStream_t huge_stream) {
    if (!w.n_spec) return;
    n_huge = min(n_huge, w.n_spec);
    if (n_huge) launch_spec_variant<kSpecThreadsHuge, 1>(w, 0, n_huge, huge_stream);
    const uint32_t rest = w.n_spec - n_huge;
    if (!rest) return;
    static const uint32_t wide_below = [] { const char* e = getenv("DATAGO_B200_SPEC_WIDE_BELOW"); return e ? (uint32_t)atoi(e) : kSpecWideBelow; }();
    if (rest < wide_below) launch_spec_variant<kSpecThreadsWide, kSpecMinCtasWide>(w, n_huge, rest, s);
    else launch_spec_variant<kSpecThreads, DG_SPEC_MIN_CTAS>(w, n_huge, rest, s);
}

// ---------------------------------------------------------------------------------------------------------------
// K2  dequantise + 8x8 inverse DCT (the 13-bit fixed-point "islow" factorisation: columns, round to 2 fractional
//     bits, rows, round, +128, clamp) for every block of a wave, written to 8-bit component planes.
//
//     The stage is bound by integer instruction issue, not by HBM, so the kernel is built to execute few
//     instructions: one thread per block (no exchange between lanes), dequantisation and 16-bit unpacking in one
//     dp2a per coefficient, rounding constants folded into the even part of each butterfly, saturating pack
//     instructions, a reduced butterfly when every block of the warp keeps its energy in the top-left 4x4, and a
//     constant fill when every block of the warp has nothing but a DC term.
//     All arithmetic is exact in 32-bit integers, so regrouping the butterflies cannot change a result.
// ---------------------------------------------------------------------------------------------------------------
constexpr int32_t F_0_298 = 2446, F_0_390 = 3196, F_0_541 = 4433, F_0_765 = 6270, F_0_899 = 7373, F_1_175 = 9633,
                  F_1_501 = 12299, F_1_847 = 15137, F_1_961 = 16069, F_2_053 = 16819, F_2_562 = 20995, F_3_072 = 25172;

// o[k] = (butterfly(x)[k] + RND) >> SHIFT
template <int32_t RND, int SHIFT>
__device__ __forceinline__ void idct8(int32_t x0, int32_t x1, int32_t x2, int32_t x3, int32_t x4, int32_t x5, int32_t x6,
                                      int32_t x7, int32_t (&o)[8]) {
    const int32_t z1e = (x2 + x6) * F_0_541;
    const int32_t t2 = z1e - x6 * F_1_847, t3 = z1e + x2 * F_0_765;
    const int32_t t0 = (x0 + x4) * 8192 + RND, t1 = (x0 - x4) * 8192 + RND;
    const int32_t t10 = t0 + t3, t13 = t0 - t3, t11 = t1 + t2, t12 = t1 - t2;
    int32_t z1 = x7 + x1, z2 = x5 + x3, z3 = x7 + x3, z4 = x5 + x1;
    const int32_t z5 = (z3 + z4) * F_1_175;
    z3 = z5 - z3 * F_1_961;
    z4 = z5 - z4 * F_0_390;
    z1 *= -F_0_899;
    z2 *= -F_2_562;
    const int32_t o0 = x7 * F_0_298 + z1 + z3, o1 = x5 * F_2_053 + z2 + z4, o2 = x3 * F_3_072 + z2 + z3,
                  o3 = x1 * F_1_501 + z1 + z4;
    o[0] = (t10 + o3) >> SHIFT; o[7] = (t10 - o3) >> SHIFT; o[1] = (t11 + o2) >> SHIFT; o[6] = (t11 - o2) >> SHIFT;
    o[2] = (t12 + o1) >> SHIFT; o[5] = (t12 - o1) >> SHIFT; o[3] = (t13 + o0) >> SHIFT; o[4] = (t13 - o0) >> SHIFT;
}

// The same butterfly with x4 = x5 = x6 = x7 = 0 (constants merged; exact because the arithmetic is a ring).
template <int32_t RND, int SHIFT>
__device__ __forceinline__ void idct8_lo4(int32_t x0, int32_t x1, int32_t x2, int32_t x3, int32_t (&o)[8]) {
    const int32_t t2 = x2 * F_0_541, t3 = x2 * (F_0_541 + F_0_765);
    const int32_t t0 = x0 * 8192 + RND;
    const int32_t t10 = t0 + t3, t13 = t0 - t3, t11 = t0 + t2, t12 = t0 - t2;
    const int32_t o0 = x1 * (F_1_175 - F_0_899) + x3 * (F_1_175 - F_1_961);
    const int32_t o1 = x1 * (F_1_175 - F_0_390) + x3 * (F_1_175 - F_2_562);
    const int32_t o2 = x1 * F_1_175 + x3 * (F_3_072 - F_2_562 - F_1_961 + F_1_175);
    const int32_t o3 = x1 * (F_1_501 - F_0_899 - F_0_390 + F_1_175) + x3 * F_1_175;
    o[0] = (t10 + o3) >> SHIFT; o[7] = (t10 - o3) >> SHIFT; o[1] = (t11 + o2) >> SHIFT; o[6] = (t11 - o2) >> SHIFT;
    o[2] = (t12 + o1) >> SHIFT; o[5] = (t12 - o1) >> SHIFT; o[3] = (t13 + o0) >> SHIFT; o[4] = (t13 - o0) >> SHIFT;
}

// ... and with x2 = x3 = 0 as well.
template <int32_t RND, int SHIFT>
__device__ __forceinline__ void idct8_lo2(int32_t x0, int32_t x1, int32_t (&o)[8]) {
    const int32_t t0 = x0 * 8192 + RND;
    const int32_t o0 = x1 * (F_1_175 - F_0_899), o1 = x1 * (F_1_175 - F_0_390), o2 = x1 * F_1_175,
                  o3 = x1 * (F_1_501 - F_0_899 - F_0_390 + F_1_175);
    o[0] = (t0 + o3) >> SHIFT; o[7] = (t0 - o3) >> SHIFT; o[1] = (t0 + o2) >> SHIFT; o[6] = (t0 - o2) >> SHIFT;
    o[2] = (t0 + o1) >> SHIFT; o[5] = (t0 - o1) >> SHIFT; o[3] = (t0 + o0) >> SHIFT; o[4] = (t0 - o0) >> SHIFT;
}

// packs sat_u8 of four ints into one word, first argument in the lowest byte
__device__ __forceinline__ uint32_t pack_sat_u8(int32_t a, int32_t b, int32_t c, int32_t d) {
    uint32_t hi, r;
    asm("cvt.pack.sat.u8.s32.b32 %0, %1, %2, %3;" : "=r"(hi) : "r"(d), "r"(c), "r"(0));
    asm("cvt.pack.sat.u8.s32.b32 %0, %1, %2, %3;" : "=r"(r) : "r"(b), "r"(a), "r"(hi));
    return r;
}

// coefficient pair (low half, high half of cw) times the two quantisers in bytes 0 and 3 of qw
__device__ __forceinline__ void dequant_pair(uint32_t cw, uint32_t qw, int32_t& lo, int32_t& hi) {
    asm("dp2a.lo.s32.u32 %0, %1, %2, 0;" : "=r"(lo) : "r"(cw), "r"(qw));
    asm("dp2a.hi.s32.u32 %0, %1, %2, 0;" : "=r"(hi) : "r"(cw), "r"(qw));
}

constexpr int32_t kRound1 = 1 << 10, kRound2 = (1 << 17) + (128 << 18);
constexpr int kIdctThreads = 128;

// How much of a block is non-zero decides how much of the butterfly is needed.
enum : int { kClsFull = 0, kCls4x4 = 1, kCls2x2 = 2, kClsDc = 3 };
__device__ __forceinline__ int block_class(const uint4 (&c)[8]) {
    const uint32_t hi_rows = c[4].x | c[4].y | c[4].z | c[4].w | c[5].x | c[5].y | c[5].z | c[5].w | c[6].x | c[6].y |
                             c[6].z | c[6].w | c[7].x | c[7].y | c[7].z | c[7].w;
    const uint32_t hi_cols = c[0].z | c[0].w | c[1].z | c[1].w | c[2].z | c[2].w | c[3].z | c[3].w;
    if (hi_rows | hi_cols) return kClsFull;
    if (c[0].y | c[1].y | c[2].x | c[2].y | c[3].x | c[3].y) return kCls4x4;
    return ((c[0].x >> 16) | c[1].x) ? kCls2x2 : kClsDc;
}

// Dequantise + inverse DCT of the calling lane's block; c = its coefficient rows (only the part class `cls` covers is
// read), qq = the quantiser rows in the dp2a layout.  emit(r, lo, hi) receives row r of the result as two words of
// four saturated samples.  cls must be the same for all lanes of the warp and no sparser than any lane's block.
template <class Emit>
__device__ __forceinline__ void idct_block(const uint4 (&c)[8], const uint4* __restrict__ qq, int cls, Emit&& emit) {
    if (cls == kClsDc) {
        // flat blocks: both passes reduce to shifts of the DC term
        int32_t lo, hi;
        dequant_pair(c[0].x, __ldg(reinterpret_cast<const uint32_t*>(qq)), lo, hi);
        const int32_t wsv = (lo * 8192 + kRound1) >> 11;
        const int32_t v = (wsv * 8192 + kRound2) >> 18;
        const uint32_t px4 = pack_sat_u8(v, v, v, v);
#pragma unroll
        for (int r = 0; r < 8; ++r) emit(r, px4, px4);
    } else if (cls == kCls2x2) {
        int32_t x[2][2], ws[8][2];
#pragma unroll
        for (int r = 0; r < 2; ++r) dequant_pair(c[r].x, __ldg(reinterpret_cast<const uint32_t*>(qq + r)), x[r][0], x[r][1]);
#pragma unroll
        for (int col = 0; col < 2; ++col) {
            int32_t o[8];
            idct8_lo2<kRound1, 11>(x[0][col], x[1][col], o);
#pragma unroll
            for (int r = 0; r < 8; ++r) ws[r][col] = o[r];
        }
#pragma unroll
        for (int r = 0; r < 8; ++r) {
            int32_t o[8];
            idct8_lo2<kRound2, 18>(ws[r][0], ws[r][1], o);
            emit(r, pack_sat_u8(o[0], o[1], o[2], o[3]), pack_sat_u8(o[4], o[5], o[6], o[7]));
        }
    } else if (cls == kCls4x4) {
        int32_t x[4][4], ws[8][4];
#pragma unroll
        for (int r = 0; r < 4; ++r) {
            const uint2 qv = __ldg(reinterpret_cast<const uint2*>(qq + r));
            dequant_pair(c[r].x, qv.x, x[r][0], x[r][1]);
            dequant_pair(c[r].y, qv.y, x[r][2], x[r][3]);
        }
#pragma unroll
        for (int col = 0; col < 4; ++col) {
            int32_t o[8];
            idct8_lo4<kRound1, 11>(x[0][col], x[1][col], x[2][col], x[3][col], o);
#pragma unroll
            for (int r = 0; r < 8; ++r) ws[r][col] = o[r];
        }
#pragma unroll
        for (int r = 0; r < 8; ++r) {
            int32_t o[8];
            idct8_lo4<kRound2, 18>(ws[r][0], ws[r][1], ws[r][2], ws[r][3], o);
            emit(r, pack_sat_u8(o[0], o[1], o[2], o[3]), pack_sat_u8(o[4], o[5], o[6], o[7]));
        }
    } else {
        int32_t ws[8][8];
#pragma unroll
        for (int r = 0; r < 8; ++r) {
            const uint4 qv = __ldg(qq + r);
            dequant_pair(c[r].x, qv.x, ws[r][0], ws[r][1]);
            dequant_pair(c[r].y, qv.y, ws[r][2], ws[r][3]);
            dequant_pair(c[r].z, qv.z, ws[r][4], ws[r][5]);
            dequant_pair(c[r].w, qv.w, ws[r][6], ws[r][7]);
        }
#pragma unroll
        for (int col = 0; col < 8; ++col) {
            int32_t o[8];
            idct8<kRound1, 11>(ws[0][col], ws[1][col], ws[2][col], ws[3][col], ws[4][col], ws[5][col], ws[6][col], ws[7][col], o);
#pragma unroll
            for (int r = 0; r < 8; ++r) ws[r][col] = o[r];
        }
#pragma unroll
        for (int r = 0; r < 8; ++r) {
            int32_t o[8];
            idct8<kRound2, 18>(ws[r][0], ws[r][1], ws[r][2], ws[r][3], ws[r][4], ws[r][5], ws[r][6], ws[r][7], o);
            emit(r, pack_sat_u8(o[0], o[1], o[2], o[3]), pack_sat_u8(o[4], o[5], o[6], o[7]));
        }
    }
}

// the class a whole warp can run: the least sparse of its lanes' classes
__device__ __forceinline__ int warp_class(int cls) { return (int)__reduce_min_sync(0xFFFFFFFFu, (unsigned)cls); }

#ifndef DG_IDCT_MIN_CTAS
#define DG_IDCT_MIN_CTAS 7
#endif
__global__ void __launch_bounds__(kIdctThreads, DG_IDCT_MIN_CTAS) k_idct(JpegWave w, uint32_t first, uint32_t count, bool rezero) {
    const uint32_t local = blockIdx.x * kIdctThreads + threadIdx.x;
    const bool valid = local < count;
    const uint32_t g = first + (valid ? local : 0);
    // A warp's 32 blocks are 4 KB of consecutive coefficients.  They are fetched with eight fully coalesced 16-byte
    // asynchronous copies per lane into shared memory (one chunk = one block row) while the descriptor look-ups run;
    // then every lane reads back the eight rows of its own block.  Row r of block b sits at chunk
    // b * 8 + (r ^ (b & 7)): copy-in and read-back both touch eight different 16-byte bank groups per quarter warp.
    // (One 16-byte load per lane and row straight from global memory makes every instruction touch 32 lines.)
    __shared__ __align__(16) uint4 s_coef[kIdctThreads / 32][256];
    const uint32_t lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    {
        const uint32_t warp_first = blockIdx.x * kIdctThreads + warp * 32;
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            const uint32_t chunk = i * 32 + lane, bb = chunk >> 3, r = chunk & 7;
            const uint32_t gb = first + min(warp_first + bb, count - 1);
            const uint32_t dst = (uint32_t)__cvta_generic_to_shared(&s_coef[warp][bb * 8 + (r ^ (bb & 7))]);
            const void* src = w.coef + (size_t)gb * 64 + r * 8;
            asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(src) : "memory");
        }
        asm volatile("cp.async.commit_group;" ::: "memory");
    }
    const uint32_t img = owner_of(w.blocks, g);
    const JpegDesc& d = w.descs[img];
    const uint32_t blk = g - (uint32_t)d.block_off;
    const uint32_t mcu = blk / d.bpm, k = blk - mcu * d.bpm;
    const uint32_t my = mcu / d.mcux, mx = mcu - my * d.mcux;
    const uint32_t luma = d.hs * d.vs;
    uint32_t comp, bx, by;
    if (k < luma) { comp = 0; const uint32_t ky = k / d.hs; bx = mx * d.hs + (k - ky * d.hs); by = my * d.vs + ky; }
    else { comp = k - luma + 1; bx = mx; by = my; }
    asm volatile("cp.async.wait_group 0;" ::: "memory");
    __syncwarp();
    uint4 c[8];
#pragma unroll
    for (int r = 0; r < 8; ++r) c[r] = s_coef[warp][lane * 8 + (r ^ (lane & 7))];
    if (rezero) {
        // zero the non-zero rows again, with the same lane <-> chunk assignment as the copy-in so that a warp's stores
        // fall into its contiguous 4 KB: lane l of step i owns row l % 8 of block 4 * i + l / 8
        uint32_t rowmask = 0;
#pragma unroll
        for (int r = 0; r < 8; ++r) rowmask |= ((c[r].x | c[r].y | c[r].z | c[r].w) != 0 ? 1u : 0u) << r;
        if (!valid) rowmask = 0;
        // base of the warp's 32 blocks, computed from the launch geometry (not from g: lanes past the end of the range
        // carry a stand-in g); blocks past the end have an empty mask, so nothing outside the range is written
        uint4* gwarp = reinterpret_cast<uint4*>(w.coef + (size_t)(first + blockIdx.x * kIdctThreads + warp * 32) * 64);
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            const uint32_t m = __shfl_sync(0xFFFFFFFFu, rowmask, i * 4 + (lane >> 3));
            if ((m >> (lane & 7)) & 1u) gwarp[i * 32 + lane] = make_uint4(0, 0, 0, 0);
        }
    }
    const uint4* qq = reinterpret_cast<const uint4*>(w.qt32 + (size_t)d.qt[comp] * 32);
    uint8_t* dst = w.planes + d.plane_off[comp] + (size_t)(by * 8) * d.plane_pitch[comp] + bx * 8;
    const uint32_t pitch = d.plane_pitch[comp];
    idct_block(c, qq, warp_class(block_class(c)), [&](int r, uint32_t lo, uint32_t hi) {
        if (valid) *reinterpret_cast<uint2*>(dst + (size_t)r * pitch) = make_uint2(lo, hi);
    });
}

void launch_idct(const JpegWave& w, uint32_t first, uint32_t count, bool rezero, cudaStream_t s) {
    if (count) k_idct<<<(count + kIdctThreads - 1) / kIdctThreads, kIdctThreads, 0, s>>>(w, first, count, rezero);
}

// ---------------------------------------------------------------------------------------------------------------
// K3  chroma upsampling + YCbCr -> RGB (16-bit fixed point constants 1.402, 0.34414, 0.71414, 1.772), interleaved
//     RGB8 out.  A CTA owns 256 pixels of two MCU rows, a thread 8 pixels of every eighth row of the tile.
//       4:2:0  triangle filter: every output sample is (9a + 3b + 3c + d + bias) >> 4 over its 2x2 chroma
//              neighbourhood -- one dp4a on bytes gathered from a shared-memory tile (1-sample halo, clamped to the
//              real plane extent, which is what the edge rules of the filter amount to);
//       4:4:4  and grayscale: straight from the planes;
//       other samplings and chroma planes at most two samples wide: a plain per-pixel path.
//     The +128 offsets and the rounding term are folded into one constant per channel; the luma byte is added with a
//     one-hot dp4a; results are saturated and packed four at a time.
// ---------------------------------------------------------------------------------------------------------------
constexpr int kColorThreads = 256;
constexpr int kCTileCols = kColorTileW / 2 + 8;  // 4 bytes of left margin (halo in the last one), halo + slack right

__device__ __forceinline__ uint32_t dp4a_u(uint32_t a, uint32_t b, uint32_t c) { return __dp4a(a, b, c); }

// 8 pixels: luma words y0, y1; chroma values cb[i] - 128, cr[i] - 128; out: 24 bytes.
// R = Y + ((91881 * (cr - 128) + 32768) >> 16) = (91881 * (cr - 128) + ((Y << 16) + 32768)) >> 16, and likewise for G and
// B: the luma byte is moved into bits 16..23 of a word that already carries the rounding term (one byte permute per
// pixel), so each channel is one multiply-add per chroma term and one shift.
__device__ __forceinline__ void ycc_to_rgb8(uint32_t y0, uint32_t y1, const int32_t (&cb)[8], const int32_t (&cr)[8], uint32_t (&out)[6]) {
#pragma unroll
    for (int h = 0; h < 2; ++h) {  // four pixels at a time keeps fewer values live
        const uint32_t yw = h ? y1 : y0;
        int32_t v[12];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const int32_t y16 = (int32_t)__byte_perm(yw, 0x00008000u, 0x7054u | ((uint32_t)i << 8));  // 0x00YY8000
            const int32_t b = cb[4 * h + i], r = cr[4 * h + i];
            v[3 * i] = (r * 91881 + y16) >> 16;
            v[3 * i + 1] = (b * -22554 + (r * -46802 + y16)) >> 16;
            v[3 * i + 2] = (b * 116130 + y16) >> 16;
        }
#pragma unroll
        for (int j = 0; j < 3; ++j) out[3 * h + j] = pack_sat_u8(v[4 * j], v[4 * j + 1], v[4 * j + 2], v[4 * j + 3]);
    }
}

__device__ __forceinline__ void store_rgb8(uint8_t* o, const uint32_t (&px)[6], int npx) {
    if (npx == 8 && (reinterpret_cast<uintptr_t>(o) & 7u) == 0) {
        uint2* o2 = reinterpret_cast<uint2*>(o);
        __stcs(o2, make_uint2(px[0], px[1])); __stcs(o2 + 1, make_uint2(px[2], px[3])); __stcs(o2 + 2, make_uint2(px[4], px[5]));
    } else {  // ragged right edge or an odd row start: byte by byte, the word index resolved at compile time
        const int nb = npx * 3;
#pragma unroll
        for (int wi = 0; wi < 6; ++wi)
#pragma unroll
            for (int k = 0; k < 4; ++k)
                if (wi * 4 + k < nb) o[wi * 4 + k] = (uint8_t)(px[wi] >> (8 * k));
    }
}

struct ChromaPlane {  // per-pixel path
    const uint8_t* p;
    uint32_t pitch;
    int dw, dh, hs, vs;
    __device__ __forceinline__ int px(int x, int y) const { return __ldg(p + (size_t)y * pitch + x); }
    __device__ __forceinline__ int colsum(int cx, int y) const {
        const int cy = y >> 1;
        int far = (y & 1) ? cy + 1 : cy - 1;
        far = min(max(far, 0), dh - 1);
        return 3 * px(cx, cy) + px(cx, far);
    }
    __device__ __forceinline__ int at(int x, int y) const {
        if (hs == 1 && vs == 1) return px(x, y);
        if (hs == 2 && dw <= 2) return px(x >> 1, vs == 2 ? y >> 1 : y);
        if (hs == 1) return (colsum(x, y) + ((y & 1) ? 2 : 1)) >> 2;
        const int cx = x >> 1;
        if (vs == 1) {
            const int t = px(cx, y);
            if (x & 1) return cx == dw - 1 ? t : (3 * t + px(cx + 1, y) + 2) >> 2;
            return cx == 0 ? t : (3 * t + px(cx - 1, y) + 1) >> 2;
        }
        const int t = colsum(cx, y);
        if (x & 1) return cx == dw - 1 ? (t * 4 + 7) >> 4 : (t * 3 + colsum(cx + 1, y) + 7) >> 4;
        return cx == 0 ? (t * 4 + 8) >> 4 : (t * 3 + colsum(cx - 1, y) + 8) >> 4;
    }
};

constexpr int kCTileRows = 8 * (int)kColorMcuRows + 2;  // chroma rows of a 4:2:0 tile plus one halo row above and below

// Chroma tile of a 4:2:0 image: rows cy0-1 .. cy0+32, columns cx0-4 .. cx0+131 as aligned words; s_c column = chroma column
// - cx0 + 4.  Coordinates are clamped to the real plane extent (dw x dh samples) and the first / last real column is
// replicated into the halo position, which is what the edge rules of the triangle filter amount to.
// Warp q loads tile rows q, q + 8, ... of both components; a lane loads word `lane` and, for two lanes, word 32 + lane.
// Two steps, both by every thread of the CTA (256), with a __syncthreads() after each: chroma_tile_fetch, chroma_tile_edges.
template <int ROWS>
__device__ __forceinline__ void chroma_tile_fetch(uint8_t (&s_c)[2][ROWS][kCTileCols], const JpegWave& w, const JpegDesc& d,
                                                  int tx, int ty, int dh) {
    constexpr int kCTileRows = ROWS;
    const int lane = threadIdx.x & 31, rowi = threadIdx.x >> 5;
    const int cx0 = tx * (int)(kColorTileW / 2), cy0 = ty * 8 * (int)kColorMcuRows;
    constexpr int kWords = kCTileCols / 4;  // 34
    const uint32_t cpitch = d.plane_pitch[1];
    const int wmax = (int)(cpitch / 4) - 1, w0 = cx0 / 4 - 1;
    const uint8_t* cb_base = w.planes + d.plane_off[1];
    const uint8_t* cr_base = w.planes + d.plane_off[2];
#pragma unroll
    for (int rr = 0; rr < (kCTileRows + 7) / 8; ++rr) {
        const int r = rowi + 8 * rr;
        if (r < kCTileRows) {
            const int gy = min(max(cy0 + r - 1, 0), dh - 1);
            const uint32_t* gb = reinterpret_cast<const uint32_t*>(cb_base + (size_t)gy * cpitch);
            const uint32_t* gr = reinterpret_cast<const uint32_t*>(cr_base + (size_t)gy * cpitch);
            uint32_t* sb = reinterpret_cast<uint32_t*>(s_c[0][r]);
            uint32_t* sr = reinterpret_cast<uint32_t*>(s_c[1][r]);
            const int g0 = min(max(w0 + lane, 0), wmax);
            sb[lane] = __ldg(gb + g0);
            sr[lane] = __ldg(gr + g0);
            if (lane < kWords - 32) {
                const int g1 = min(max(w0 + 32 + lane, 0), wmax);
                sb[32 + lane] = __ldg(gb + g1);
                sr[32 + lane] = __ldg(gr + g1);
            }
        }
    }
}

template <int ROWS>
__device__ __forceinline__ void chroma_tile_edges(uint8_t (&s_c)[2][ROWS][kCTileCols], int tx, int dw) {
    constexpr int kCTileRows = ROWS;
    const int cx0 = tx * (int)(kColorTileW / 2);
    if (threadIdx.x < 2 * kCTileRows) {
        const int comp = threadIdx.x / kCTileRows, r = threadIdx.x - comp * kCTileRows;
        if (cx0 == 0) s_c[comp][r][3] = s_c[comp][r][4];
        const int last = dw - 1 - cx0;  // tile-local index of the last real column
        if (last >= 0 && last < (int)(kColorTileW / 2)) s_c[comp][r][4 + last + 1] = s_c[comp][r][4 + last];
    }
}

__device__ __forceinline__ void load_chroma_tile(uint8_t (&s_c)[2][kCTileRows][kCTileCols], const JpegWave& w, const JpegDesc& d,
                                                 int tx, int ty, int dw, int dh) {
    chroma_tile_fetch(s_c, w, d, tx, ty, dh);
    __syncthreads();
    chroma_tile_edges(s_c, tx, dw);
    __syncthreads();
}

// Triangle upsampling of the chroma for 8 pixels of two output rows that read the same two chroma rows: row A has
// tile row p as its near row and p + 1 as its far row, row B the other way round (output rows 2j+1 and 2j+2 of the
// image).  cl = s_c column of the thread's first chroma sample (a word boundary).  Results are sample - 128.
template <bool WANT_A = true, bool WANT_B = true, int ROWS = kCTileRows>
__device__ __forceinline__ void chroma_pair(const uint8_t (&s_c)[2][ROWS][kCTileCols], int p, int cl, int32_t (&cbA)[8],
                                            int32_t (&crA)[8], int32_t (&cbB)[8], int32_t (&crB)[8]) {
    constexpr uint32_t kEvenA = 0x03090103u, kOddA = 0x01030309u;  // bytes: (near a, far a, near b, far b)
    constexpr uint32_t kEvenB = 0x09030301u, kOddB = 0x03010903u;  // the same bytes with near and far exchanged
    constexpr uint32_t kE = (uint32_t)(8 - 2048), kO = (uint32_t)(7 - 2048);  // rounding term minus 128 * 16
#pragma unroll
    for (int comp = 0; comp < 2; ++comp) {
        const uint32_t* nr = reinterpret_cast<const uint32_t*>(&s_c[comp][p][cl]);
        const uint32_t* fr = reinterpret_cast<const uint32_t*>(&s_c[comp][p + 1][cl]);
        const uint32_t Ln = nr[-1], Mn = nr[0], Nn = nr[1], Lf = fr[-1], Mf = fr[0], Nf = fr[1];
        const uint32_t I0 = __byte_perm(Mn, Mf, 0x5140), J = __byte_perm(Mn, Mf, 0x6251), I1 = __byte_perm(Mn, Mf, 0x7362);
        const uint32_t Lp = __byte_perm(__byte_perm(Ln, Lf, 0x0073), I0, 0x5410);  // (c-1, c)
        const uint32_t Rp = __byte_perm(I1, __byte_perm(Nn, Nf, 0x0040), 0x5432);  // (c+3, c+4)
        int32_t* da = comp ? crA : cbA;
        int32_t* db = comp ? crB : cbB;
        if (WANT_A) {
            da[0] = (int32_t)dp4a_u(Lp, kEvenA, kE) >> 4; da[1] = (int32_t)dp4a_u(I0, kOddA, kO) >> 4;
            da[2] = (int32_t)dp4a_u(I0, kEvenA, kE) >> 4; da[3] = (int32_t)dp4a_u(J, kOddA, kO) >> 4;
            da[4] = (int32_t)dp4a_u(J, kEvenA, kE) >> 4;  da[5] = (int32_t)dp4a_u(I1, kOddA, kO) >> 4;
            da[6] = (int32_t)dp4a_u(I1, kEvenA, kE) >> 4; da[7] = (int32_t)dp4a_u(Rp, kOddA, kO) >> 4;
        }
        if (WANT_B) {
            db[0] = (int32_t)dp4a_u(Lp, kEvenB, kE) >> 4; db[1] = (int32_t)dp4a_u(I0, kOddB, kO) >> 4;
            db[2] = (int32_t)dp4a_u(I0, kEvenB, kE) >> 4; db[3] = (int32_t)dp4a_u(J, kOddB, kO) >> 4;
            db[4] = (int32_t)dp4a_u(J, kEvenB, kE) >> 4;  db[5] = (int32_t)dp4a_u(I1, kOddB, kO) >> 4;
            db[6] = (int32_t)dp4a_u(I1, kEvenB, kE) >> 4; db[7] = (int32_t)dp4a_u(Rp, kOddB, kO) >> 4;
        }
    }
}

__global__ void __launch_bounds__(kColorThreads, 4) k_color(JpegWave w, uint32_t first_tile) {
    __shared__ __align__(16) uint8_t s_c[2][kCTileRows][kCTileCols];
    __shared__ uint32_t s_img;
    if (threadIdx.x == 0) s_img = owner_of(w.color_tiles, first_tile + blockIdx.x);
    __syncthreads();
    const uint32_t img = s_img;
    const JpegDesc& d = w.descs[img];
    const uint32_t tile = first_tile + blockIdx.x - w.color_tiles.first[img];
    const int W = (int)d.width, H = (int)d.height, hs = (int)d.hs, vs = (int)d.vs;
    const uint32_t tiles_x = (d.width + kColorTileW - 1) / kColorTileW;
    const uint32_t ty = tile / tiles_x, tx = tile - ty * tiles_x;
    const int lane = threadIdx.x & 31, rowi = threadIdx.x >> 5;  // 32 column groups x 8 rows
    const int x = (int)tx * (int)kColorTileW + lane * 8;
    const int y_base = (int)ty * 8 * vs * (int)kColorMcuRows;
    const int nsteps = vs * (int)kColorMcuRows;  // a thread converts rows rowi, rowi + 8, ... of the tile
    uint8_t* out = w.out + d.out_off;
    const uint8_t* yp = w.planes + d.plane_off[0];
    const uint32_t ypitch = d.plane_pitch[0];

    if (d.ncomp == 1) {  // grayscale: copy the real extent of the luma plane
        if (x >= W) return;
        const int npx = min(8, W - x);
        for (int k = 0; k < nsteps; ++k) {
            const int y = y_base + rowi + 8 * k;
            if (y >= H) break;
            const uint2 v = __ldg(reinterpret_cast<const uint2*>(yp + (size_t)y * ypitch + x));
            uint8_t* o = out + (size_t)y * d.out_pitch + x;
            if (npx == 8 && (reinterpret_cast<uintptr_t>(o) & 7u) == 0) __stcs(reinterpret_cast<uint2*>(o), v);
            else for (int i = 0; i < npx; ++i) o[i] = (uint8_t)((i < 4 ? v.x : v.y) >> (8 * (i & 3)));
        }
        return;
    }
    const int dw = (W + hs - 1) / hs, dh = (H + vs - 1) / vs;
    if (hs == 2 && vs == 2 && dw > 2) {
        load_chroma_tile(s_c, w, d, (int)tx, (int)ty, dw, dh);
        if (x >= W) return;
        const int cl = lane * 4 + 4;  // s_c column of this thread's first chroma sample (a word boundary)
        const int npx = min(8, W - x);
        // Output rows 2j+1 and 2j+2 read the same two chroma rows (j and j+1) with the near / far weights exchanged, so
        // the tile is shifted up by one row -- it covers rows 64 ty - 1 .. 64 ty + 62 -- and a thread converts such a
        // pair at a time: the byte gathering is done once, the second row only swaps the weights.
        const int y_first = (int)ty * 8 * 2 * (int)kColorMcuRows - 1;
        auto luma = [&](int y) -> uint2 {
            return (y >= 0 && y < H) ? __ldg(reinterpret_cast<const uint2*>(yp + (size_t)y * ypitch + x)) : make_uint2(0, 0);
        };
        uint2 nextA = luma(y_first + 2 * rowi), nextB = luma(y_first + 2 * rowi + 1);
#pragma unroll 1
        for (int m = 0; m < (int)kColorMcuRows; ++m) {
            const int p = rowi + 8 * m;  // pair index inside the tile = s_c row of the upper chroma row
            const int yA = y_first + 2 * p, yB = yA + 1;
            if (yA >= H) break;
            const uint2 ya = nextA, yb = nextB;
            if (m + 1 < (int)kColorMcuRows) { nextA = luma(yA + 16); nextB = luma(yB + 16); }  // next pair's luma in flight
            int32_t cbA[8], crA[8], cbB[8], crB[8];
            chroma_pair(s_c, p, cl, cbA, crA, cbB, crB);
            uint32_t px[6];
            if (yA >= 0) {
                ycc_to_rgb8(ya.x, ya.y, cbA, crA, px);
                store_rgb8(out + (size_t)yA * d.out_pitch + x * 3, px, npx);
            }
            if (yB < H) {
                ycc_to_rgb8(yb.x, yb.y, cbB, crB, px);
                store_rgb8(out + (size_t)yB * d.out_pitch + x * 3, px, npx);
            }
        }
        return;
    }
    if (x >= W) return;
    const int npx = min(8, W - x);
    if (hs == 1 && vs == 1) {
        for (int k = 0; k < nsteps; ++k) {
            const int y = y_base + rowi + 8 * k;
            if (y >= H) break;
            const uint2 b = __ldg(reinterpret_cast<const uint2*>(w.planes + d.plane_off[1] + (size_t)y * d.plane_pitch[1] + x));
            const uint2 r = __ldg(reinterpret_cast<const uint2*>(w.planes + d.plane_off[2] + (size_t)y * d.plane_pitch[2] + x));
            int32_t cbv[8], crv[8];
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                cbv[i] = (int32_t)(((i < 4 ? b.x : b.y) >> (8 * (i & 3))) & 255u) - 128;
                crv[i] = (int32_t)(((i < 4 ? r.x : r.y) >> (8 * (i & 3))) & 255u) - 128;
            }
            const uint2 yv = __ldg(reinterpret_cast<const uint2*>(yp + (size_t)y * ypitch + x));
            uint32_t px[6];
            ycc_to_rgb8(yv.x, yv.y, cbv, crv, px);
            store_rgb8(out + (size_t)y * d.out_pitch + x * 3, px, npx);
        }
        return;
    }
    // remaining samplings (4:2:2, 4:4:0, chroma planes at most two samples wide): one pixel at a time
    const ChromaPlane cbp{w.planes + d.plane_off[1], d.plane_pitch[1], dw, dh, hs, vs};
    const ChromaPlane crp{w.planes + d.plane_off[2], d.plane_pitch[2], dw, dh, hs, vs};
#pragma unroll 1
    for (int k = 0; k < nsteps; ++k) {
        const int y = y_base + rowi + 8 * k;
        if (y >= H) break;
#pragma unroll 1
        for (int i = 0; i < npx; ++i) {
            const int Y = __ldg(yp + (size_t)y * ypitch + x + i);
            const int cb = cbp.at(x + i, y) - 128, cr = crp.at(x + i, y) - 128;
            uint8_t* o = out + (size_t)y * d.out_pitch + (x + i) * 3;
            o[0] = (uint8_t)min(max(Y + ((91881 * cr + 32768) >> 16), 0), 255);
            o[1] = (uint8_t)min(max(Y + ((-22554 * cb - 46802 * cr + 32768) >> 16), 0), 255);
            o[2] = (uint8_t)min(max(Y + ((116130 * cb + 32768) >> 16), 0), 255);
        }
    }
}

void launch_color(const JpegWave& w, uint32_t first_tile, uint32_t count, cudaStream_t s) {
    if (count) k_color<<<count, kColorThreads, 0, s>>>(w, first_tile);
}

// ---------------------------------------------------------------------------------------------------------------
// Fused path for three-component 4:2:0 images (the common case): the luma samples never go to memory.
//   k_idct_chroma  IDCT of the Cb and Cr blocks only, into the chroma planes (0.5 bytes per pixel instead of 1.5);
//   k_luma_color   one CTA per 256 x 64 pixel tile (16 x 4 MCUs = 256 luma blocks, one per thread): luma coefficients
//                  staged with asynchronous copies, the chroma tile (with its halo, which is why chroma cannot be
//                  reconstructed tile by tile) loaded from the planes meanwhile, luma IDCT into shared memory, then
//                  upsampling and colour conversion from shared memory, RGB out.
// Traffic per pixel: 1 + 0.5 (chroma) + 2 + 0.5 + 3 (fused kernel) plus the zero write-back, against
// 3 + 1.5 + 1.5 + 3 for the two general kernels.
// ---------------------------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(kIdctThreads, DG_IDCT_MIN_CTAS) k_idct_chroma(JpegWave w, uint32_t first, uint32_t count, bool rezero) {
    const uint32_t local = blockIdx.x * kIdctThreads + threadIdx.x;
    const bool valid = local < count;
    const uint32_t q = first + min(local, count - 1);
    __shared__ __align__(16) uint4 s_coef[kIdctThreads / 32][256];
    const uint32_t lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const uint32_t o = owner_of(w.fused_chroma, q);
    const JpegDesc& d = w.descs[w.fused_first + o];
    const uint32_t ql = q - __ldg(w.fused_chroma.first + o);
    const uint32_t mcu = ql >> 1, which = ql & 1u;
    const uint32_t blk = (uint32_t)d.block_off + mcu * 6u + 4u + which;  // this lane's block in the coefficient array
    // Lanes 2j and 2j + 1 hold the Cb and Cr block of one MCU: 256 consecutive bytes.  Step i copies the eight rows of
    // blocks 4i .. 4i + 3 of the warp, lane l row l % 8 of block 4i + l / 8 (block addresses come from the owning lanes).
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        const uint32_t bb = i * 4 + (lane >> 3), r = lane & 7;
        const uint32_t gb = __shfl_sync(0xFFFFFFFFu, blk, bb);
        const uint32_t dst = (uint32_t)__cvta_generic_to_shared(&s_coef[warp][bb * 8 + (r ^ (bb & 7))]);
        const void* src = w.coef + (size_t)gb * 64 + r * 8;
        asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(src) : "memory");
    }
    asm volatile("cp.async.commit_group;" ::: "memory");
    const uint32_t my = mcu / d.mcux, mx = mcu - my * d.mcux;
    const uint32_t comp = 1u + which;
    const uint4* qq = reinterpret_cast<const uint4*>(w.qt32 + (size_t)d.qt[comp] * 32);
    const uint32_t pitch = d.plane_pitch[comp];
    uint8_t* dst = w.planes + d.plane_off[comp] + (size_t)(my * 8) * pitch + mx * 8;
    asm volatile("cp.async.wait_group 0;" ::: "memory");
    __syncwarp();
    uint4 c[8];
#pragma unroll
    for (int r = 0; r < 8; ++r) c[r] = s_coef[warp][lane * 8 + (r ^ (lane & 7))];
    if (rezero) {
        uint32_t rowmask = 0;
#pragma unroll
        for (int r = 0; r < 8; ++r) rowmask |= ((c[r].x | c[r].y | c[r].z | c[r].w) != 0 ? 1u : 0u) << r;
        if (!valid) rowmask = 0;  // lanes past the end stand in for the last block, which its own lane zeroes
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            const uint32_t src_lane = i * 4 + (lane >> 3);
            const uint32_t m = __shfl_sync(0xFFFFFFFFu, rowmask, src_lane);
            const uint32_t gb = __shfl_sync(0xFFFFFFFFu, blk, src_lane);
            if ((m >> (lane & 7)) & 1u) reinterpret_cast<uint4*>(w.coef + (size_t)gb * 64)[lane & 7] = make_uint4(0, 0, 0, 0);
        }
    }
    idct_block(c, qq, warp_class(block_class(c)), [&](int r, uint32_t lo, uint32_t hi) {
        if (valid) *reinterpret_cast<uint2*>(dst + (size_t)r * pitch) = make_uint2(lo, hi);
    });
}

void launch_idct_chroma(const JpegWave& w, uint32_t first, uint32_t count, bool rezero, cudaStream_t s) {
    if (count) k_idct_chroma<<<(count + kIdctThreads - 1) / kIdctThreads, kIdctThreads, 0, s>>>(w, first, count, rezero);
}

constexpr int kFusedThreads = 64 * (int)kFusedMcuRows;
constexpr int kFusedWarps = kFusedThreads / 32;
constexpr int kFTileRows = 8 * (int)kFusedMcuRows + 2;  // chroma rows of a tile plus one halo row above and below
constexpr int kLumaPitch = kColorTileW + 8;  // 8 * pitch = 64 (mod 128): the two block rows a half warp stores to fall into different banks
constexpr int kLumaRows = 16 * (int)kFusedMcuRows;

// What a CTA needs to know about one tile, gathered by one thread while the others work on the previous tile.
struct TileInfo {
    const int16_t* coef;   // first coefficient block of the image
    const uint8_t* cb;     // chroma planes
    const uint8_t* cr;
    uint8_t* out;          // decoded image
    const uint4* qq;       // luma quantiser rows (dp2a layout)
    uint32_t mcux, mcuy, width, height, cpitch, tx, ty, opitch;  // opitch: bytes per row of the decoded image
};

struct FusedSmem {
    uint4 coef[kFusedThreads / 32][256];          // staged luma coefficients of the tile being set up, 4 KB per warp
    uint8_t luma[kLumaRows][kLumaPitch];          // reconstructed luma tile
    uint8_t c[2][2][kFTileRows][kCTileCols];      // chroma tiles of this tile and of the next one
    TileInfo info[2];
    uint32_t count[kFusedThreads / 32];
    uint8_t perm[kFusedThreads], pcls[kFusedThreads];
};

__device__ __forceinline__ void fill_tile_info(TileInfo& t, const JpegWave& w, uint32_t tile_index) {
    const uint32_t o = owner_of(w.fused_tiles, tile_index);
    const JpegDesc& d = w.descs[w.fused_first + o];
    const uint32_t tile = tile_index - __ldg(w.fused_tiles.first + o);
    const uint32_t tiles_x = (d.width + kColorTileW - 1) / kColorTileW;
    t.ty = tile / tiles_x;
    t.tx = tile - t.ty * tiles_x;
    t.coef = w.coef + (size_t)d.block_off * 64;
    t.cb = w.planes + d.plane_off[1];
    t.cr = w.planes + d.plane_off[2];
    t.out = w.out + d.out_off;
    t.qq = reinterpret_cast<const uint4*>(w.qt32 + (size_t)d.qt[0] * 32);
    t.mcux = d.mcux; t.mcuy = d.mcuy; t.width = d.width; t.height = d.height; t.cpitch = d.plane_pitch[1];
    t.opitch = d.out_pitch;
}

// Queues the asynchronous copies of one tile's inputs (one commit group per thread).
//   luma coefficients: warp q owns MCU row q / 2 of the tile and MCUs 8 (q % 2) .. + 7 of it; step i copies the four luma
//     blocks of MCU i, 512 consecutive bytes, lane l row l % 8 of block l / 8 (into the XOR-swizzled layout the IDCT reads
//     back).  MCUs outside the image are replaced by the nearest one inside: their results land in tile positions no
//     output pixel reads.
//   chroma tile: rows cy0-1 .. cy0+8*rows, columns cx0-4 .. cx0+131 as aligned words, coordinates clamped to the plane.
__device__ __forceinline__ void queue_tile_copies(FusedSmem& sm, const TileInfo& t, int buf) {
    const uint32_t lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    {
        const uint32_t mrow = warp >> 1, half = warp & 1u;
        const uint32_t myc = min(t.ty * kFusedMcuRows + mrow, t.mcuy - 1), mx0 = t.tx * 16 + half * 8;
        const int16_t* row_base = t.coef + (size_t)myc * t.mcux * 384;
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            const uint32_t bb = i * 4 + (lane >> 3), r = lane & 7;
            const uint32_t mxc = min(mx0 + i, t.mcux - 1);
            const uint32_t dst = (uint32_t)__cvta_generic_to_shared(&sm.coef[warp][bb * 8 + (r ^ (bb & 7))]);
            const void* src = row_base + (size_t)mxc * 384 + lane * 8;
            asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(src) : "memory");
        }
    }
    {
        const int dh = ((int)t.height + 1) / 2;
        const int cx0 = (int)t.tx * (int)(kColorTileW / 2), cy0 = (int)t.ty * 8 * (int)kFusedMcuRows;
        constexpr int kWords = kCTileCols / 4;  // 34
        const int wmax = (int)(t.cpitch / 4) - 1, w0 = cx0 / 4 - 1;
        const int g0 = min(max(w0 + (int)lane, 0), wmax), g1 = min(max(w0 + 32 + (int)lane, 0), wmax);
#pragma unroll
        for (int rr = 0; rr < (kFTileRows + kFusedWarps - 1) / kFusedWarps; ++rr) {
            const int r = (int)warp + kFusedWarps * rr;
            if (r < kFTileRows) {
                const int gy = min(max(cy0 + r - 1, 0), dh - 1);
                const uint32_t* gb = reinterpret_cast<const uint32_t*>(t.cb + (size_t)gy * t.cpitch);
                const uint32_t* gr = reinterpret_cast<const uint32_t*>(t.cr + (size_t)gy * t.cpitch);
                const uint32_t sb = (uint32_t)__cvta_generic_to_shared(&sm.c[buf][0][r][0]);
                const uint32_t sr = (uint32_t)__cvta_generic_to_shared(&sm.c[buf][1][r][0]);
                asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(sb + lane * 4), "l"(gb + g0) : "memory");
                asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(sr + lane * 4), "l"(gr + g0) : "memory");
                if (lane < kWords - 32) {
                    asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(sb + (32 + lane) * 4), "l"(gb + g1) : "memory");
                    asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(sr + (32 + lane) * 4), "l"(gr + g1) : "memory");
                }
            }
        }
    }
    asm volatile("cp.async.commit_group;" ::: "memory");
}

// The full butterfly needs twice the registers of everything else in the fused kernel and runs for a few per cent of
// the blocks: it lives in a function of its own, so that it does not set the register count of the whole kernel.
__device__ __noinline__ void idct_full_to_tile(const uint4* rows, uint32_t swz, const uint4* qq, uint8_t* dst) {
    uint4 c[8];
#pragma unroll
    for (int r = 0; r < 8; ++r) c[r] = rows[r ^ swz];
    idct_block(c, qq, kClsFull, [&](int r, uint32_t lo, uint32_t hi) {
        *reinterpret_cast<uint2*>(dst + r * kLumaPitch) = make_uint2(lo, hi);
    });
}

// CTA b handles tiles b, b + gridDim.x, ...: while a tile is being converted, the inputs of the CTA's next tile (if the
// grid is smaller than the tile count) are already on their way into shared memory.
#ifndef DG_FUSED_MIN_CTAS
#define DG_FUSED_MIN_CTAS (12 / DG_FUSED_MCU_ROWS)
#endif
__global__ void __launch_bounds__(kFusedThreads, DG_FUSED_MIN_CTAS) k_luma_color(JpegWave w, uint32_t first_tile, uint32_t count, bool rezero) {
    extern __shared__ __align__(16) unsigned char smem_raw[];
    FusedSmem& sm = *reinterpret_cast<FusedSmem*>(smem_raw);
    const uint32_t lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const uint32_t mrow = warp >> 1, half = warp & 1u, mcu_local = lane >> 2;

    if (threadIdx.x == 0) fill_tile_info(sm.info[0], w, first_tile + blockIdx.x);
    __syncthreads();
    queue_tile_copies(sm, sm.info[0], 0);

    int cur = 0;
    for (uint32_t tile = blockIdx.x; tile < count; tile += gridDim.x, cur ^= 1) {
        const bool has_next = tile + gridDim.x < count;
        const TileInfo& t = sm.info[cur];  // read where needed: a copy in registers would not fit beside the butterfly
        const int W = (int)t.width, H = (int)t.height;

        // ---- this tile's inputs have been on their way since the previous tile was being reconstructed
        asm volatile("cp.async.wait_group 0;" ::: "memory");
        __syncwarp();  // the coefficients a warp reads were copied by its own lanes

        // ---- luma IDCT, one block per thread.  How much of the butterfly a block needs depends on where its non-zero
        //      coefficients end, and a warp runs the path its least sparse lane needs; so the tile's 256 blocks are first
        //      sorted by class (counting sort, classes of the lanes' own blocks) and thread i then reconstructs the i-th
        //      block of that order: all but at most three warps of the CTA are uniform.
        const uint32_t my = t.ty * kFusedMcuRows + mrow, mx0 = t.tx * 16 + half * 8;
        const bool valid = my < t.mcuy && mx0 + mcu_local < t.mcux;
        int cls;
        uint32_t ballot_mine;
        {
            uint4 c[8];
#pragma unroll
            for (int r = 0; r < 8; ++r) c[r] = sm.coef[warp][lane * 8 + (r ^ (lane & 7))];
            cls = block_class(c);
            if (rezero) {
                // the rows found non-zero are written back as zeros, which leaves the coefficient buffer clean for the next
                // wave that uses it; lane l of step i owns row l % 8 of block l / 8 of MCU i, as in the copy
                uint32_t rowmask = 0;
#pragma unroll
                for (int r = 0; r < 8; ++r) rowmask |= ((c[r].x | c[r].y | c[r].z | c[r].w) != 0 ? 1u : 0u) << r;
                if (!valid) rowmask = 0;  // a stand-in MCU belongs to other lanes (or another CTA, which may not have read it yet)
                int16_t* row_base = const_cast<int16_t*>(t.coef) + (size_t)min(my, t.mcuy - 1) * t.mcux * 384;
#pragma unroll
                for (int i = 0; i < 8; ++i) {
                    const uint32_t m = __shfl_sync(0xFFFFFFFFu, rowmask, i * 4 + (lane >> 3));
                    if ((m >> (lane & 7)) & 1u)
                        reinterpret_cast<uint4*>(row_base + (size_t)(mx0 + i) * 384)[lane] = make_uint4(0, 0, 0, 0);
                }
            }
        }
        {
            const uint32_t b0 = __ballot_sync(0xFFFFFFFFu, cls == 0), b1 = __ballot_sync(0xFFFFFFFFu, cls == 1),
                           b2 = __ballot_sync(0xFFFFFFFFu, cls == 2);
            if (lane == 0) sm.count[warp] = (uint32_t)__popc(b0) | ((uint32_t)__popc(b1) << 10) | ((uint32_t)__popc(b2) << 20);
            ballot_mine = cls == 0 ? b0 : cls == 1 ? b1 : cls == 2 ? b2 : ~(b0 | b1 | b2);
        }
        __syncthreads();  // class counts are in shared memory, and so is the chroma tile (every thread waited for its copies)
        // every thread has left the previous tile behind: its descriptor slot can take the next tile's
        if (threadIdx.x == 0 && has_next) fill_tile_info(sm.info[cur ^ 1], w, first_tile + tile + gridDim.x);
        {
            // per-class counts in 10-bit fields (a sum is at most 256; the fourth class is the rest): before this warp, in total
            uint32_t before = 0, total = 0;
#pragma unroll
            for (int i = 0; i < kFusedThreads / 32; ++i) { const uint32_t v = sm.count[i]; if (i < (int)warp) before += v; total += v; }
            const uint32_t t0 = total & 1023u, t1 = (total >> 10) & 1023u, t2 = total >> 20;
            const uint32_t p0 = before & 1023u, p1 = (before >> 10) & 1023u, p2 = before >> 20;
            uint32_t pos = cls == 0 ? p0 : cls == 1 ? t0 + p1 : cls == 2 ? t0 + t1 + p2 : t0 + t1 + t2 + (warp * 32u - p0 - p1 - p2);
            pos += __popc(ballot_mine & ((1u << lane) - 1u));
            sm.perm[pos & (kFusedThreads - 1)] = (uint8_t)threadIdx.x;
            sm.pcls[pos & (kFusedThreads - 1)] = (uint8_t)cls;
        }
        chroma_tile_edges(sm.c[cur], (int)t.tx, (W + 1) / 2);
        __syncthreads();
        {
            const uint32_t blk = sm.perm[threadIdx.x];
            const int wcls = warp_class((int)sm.pcls[threadIdx.x]);
            // where block blk was staged, and where it lies in the tile (from the lane / warp that staged it)
            const uint32_t bw = blk >> 5, bl = blk & 31u, swz = bl & 7u;
            const uint4* rows = &sm.coef[bw][bl * 8];
            const uint32_t bx = (bw & 1u) * 16 + (bl >> 2) * 2 + (bl & 1u), by = (bw >> 1) * 2 + ((bl >> 1) & 1u);
            uint8_t* dst = &sm.luma[by * 8][bx * 8];
            if (wcls == kClsFull) {
                idct_full_to_tile(rows, swz, t.qq, dst);
            } else {
                uint4 c[8];
                if (wcls == kCls4x4) {
#pragma unroll
                    for (int r = 0; r < 4; ++r) { const uint2 v = *reinterpret_cast<const uint2*>(&rows[r ^ swz]); c[r].x = v.x; c[r].y = v.y; }
                } else {
                    c[0].x = rows[0 ^ swz].x;
                    c[1].x = rows[1 ^ swz].x;
                }
                idct_block(c, t.qq, wcls, [&](int r, uint32_t lo, uint32_t hi) {
                    *reinterpret_cast<uint2*>(dst + r * kLumaPitch) = make_uint2(lo, hi);
                });
            }
        }
        __syncthreads();  // the luma tile is complete and the staged coefficients have all been consumed
        // the next tile's inputs travel while this tile is converted
        if (has_next) queue_tile_copies(sm, sm.info[cur ^ 1], cur ^ 1);

        // ---- upsampling + colour conversion.  Output rows 2j+1 and 2j+2 read the same two chroma rows with the near / far
        //      weights exchanged, so a thread converts such a pair at a time (pair p of the tile = tile rows 2p-1 and 2p,
        //      chroma tile rows p and p+1).  The tile's first row is the second half of pair 0 and its last row the first
        //      half of the pair after the last whole one: warp 0 converts those two halves in an extra step.
        const int x = (int)t.tx * (int)kColorTileW + (int)lane * 8;
        if (x < W) {
            const int npx = min(8, W - x);
            const int cl = (int)lane * 4 + 4;
            const int y0 = (int)t.ty * kLumaRows;
            // everything the loop needs from the tile record, once; x * 3 is a multiple of 8, so all rows of a thread are
            // 8-byte aligned when the image and its pitch are
            const uint32_t opitch = t.opitch;
            uint8_t* const obase = t.out + (size_t)x * 3;
            const bool wide = npx == 8 && ((reinterpret_cast<uintptr_t>(obase) | opitch) & 7u) == 0;
            auto store = [&](int y, const uint32_t (&px)[6]) {
                uint8_t* o = obase + (size_t)y * opitch;
                if (wide) {
                    uint2* o2 = reinterpret_cast<uint2*>(o);
                    __stcs(o2, make_uint2(px[0], px[1])); __stcs(o2 + 1, make_uint2(px[2], px[3])); __stcs(o2 + 2, make_uint2(px[4], px[5]));
                } else {
                    store_rgb8(o, px, npx);
                }
            };
#pragma unroll 1
            for (int m = 0; m <= kLumaRows / 2 / kFusedWarps; ++m) {
                const int p = (int)warp + kFusedWarps * m;
                if (p > kLumaRows / 2) break;
                const int yA = y0 + 2 * p - 1, yB = yA + 1;
                const bool doA = p > 0 && yA < H, doB = p < kLumaRows / 2 && yB < H;
                if (!doA && !doB) break;
                int32_t cbA[8], crA[8], cbB[8], crB[8];
                chroma_pair<true, true, kFTileRows>(sm.c[cur], p, cl, cbA, crA, cbB, crB);
                uint32_t px[6];
                if (doA) {
                    const uint2 ya = *reinterpret_cast<const uint2*>(&sm.luma[2 * p - 1][lane * 8]);
                    ycc_to_rgb8(ya.x, ya.y, cbA, crA, px);
                    store(yA, px);
                }
                if (doB) {
                    const uint2 yb = *reinterpret_cast<const uint2*>(&sm.luma[2 * p][lane * 8]);
                    ycc_to_rgb8(yb.x, yb.y, cbB, crB, px);
                    store(yB, px);
                }
            }
        }
        // The next iteration writes sm.luma, sm.c[cur] and sm.info[cur] only behind its first barrier, which every thread
        // reaches after this phase.
    }
}

void launch_luma_color(const JpegWave& w, uint32_t first_tile, uint32_t count, bool rezero, cudaStream_t s) {
    if (!count) return;
    // per device, once: the kernel's shared memory exceeds the default limit; the grid is sized from the SM count
    static int sm_count[64] = {0};
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev < 0 || dev >= 64) dev = 0;
    if (!sm_count[dev]) {
        int n = 0;
        cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev);
        cudaFuncSetAttribute(k_luma_color, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)sizeof(FusedSmem));
        sm_count[dev] = n > 0 ? n : 148;
    }
    // One CTA per tile.  The kernel also works as a persistent loop over tiles with the next tile's inputs prefetched
    // (any smaller grid), but measured slower that way: resident CTAs of this kernel then keep the other stream's
    // entropy decoders off the SMs for a whole launch, and the block scheduler already overlaps tiles across CTAs.
    // (A variant that read the coefficients with plain loads instead of staging them -- 27 KB of shared memory, four
    // to six CTAs per SM -- measured 15 to 30 % slower than this one at three.)
    const uint32_t grid = count;
    (void)sm_count;
    k_luma_color<<<grid, kFusedThreads, sizeof(FusedSmem), s>>>(w, first_tile, count, rezero);
}

}  // namespace dg
