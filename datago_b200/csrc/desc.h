// Descriptors shared by the host planner and the device kernels.  Plain structs, 8-byte aligned.
#pragma once
#include <stdint.h>

namespace dg {

constexpr int kLutBits = 9;  // Huffman fast-lookup width

// A decoded Huffman symbol as the entropy decoder wants it: code length, the number of extra bits s (low nibble of
// the symbol), the zero run r (high nibble; 0 for DC categories) and the total bits consumed.
//   bits 0-5: length + s   bits 6-10: length   bits 11-14: s   bits 15-18: r
#ifdef __CUDACC__
__host__ __device__
#endif
constexpr uint32_t huff_pack(uint32_t len, uint32_t sym) {
    return (len + (sym & 15u)) | (len << 6) | ((sym & 15u) << 11) | ((sym >> 4) << 15);
}

// One Huffman table (DC or AC) prepared for the device (T.81 Annex C code assignment).
struct alignas(16) HuffTable {
    // next 9 bits -> packed symbol (see huff_pack), 0 = the code is longer than 9 bits
    uint32_t lut[1 << kLutBits];
    // Codes longer than the fast table, without a search: limit[i] is the smallest 16-bit window (code bits left-aligned)
    // that does not start with a code of at most 10 + i bits, i = 0..6; canonical codes grow with their length, so the
    // length of the code at the head of window v is 10 + the number of i < 6 with v >= limit[i], and v >= limit[6]
    // means that no code matches.  limit[7] is unused.  (16-byte aligned: read as two vectors.)
    uint32_t limit[8];
    int32_t maxcode[18];          // [l], l = 1..16: largest code of length l, -1 if none; [17] = INT_MAX
    int32_t valoff[17];           // [l]: index of the first symbol of length l minus its first code
    uint8_t vals[256];
};

// Status bits a kernel may set for an image (ORed into status[item]).
enum : uint32_t {
    kStTruncated = 1u,   // entropy data ended before all blocks were decoded
    kStBadCode = 2u,     // a code that is not in the Huffman table
    kStBadMarker = 4u,   // restart markers missing / out of sequence
    kStSyncLimit = 8u,   // subsequence synchronisation hit its iteration cap
    kStCoefRange = 16u,  // coefficient index ran past the end of a block
};

// One baseline JPEG of a wave.
struct JpegDesc {
    uint64_t raw_off;       // entropy-coded segment inside the raw blob (16-byte aligned)
    uint64_t us_off;        // this image's slice of the unstuffed buffer (16-byte aligned, capacity raw_len + 32)
    uint64_t block_off;     // first 8x8 block in the coefficient buffer
    uint64_t plane_off[3];  // byte offset of each component plane (MCU-padded, pitch = plane_pitch)
    uint64_t out_off;       // byte offset of the decoded image (tightly packed HWC) in the decode target buffer
    uint32_t raw_len;
    uint32_t width, height;
    uint32_t mcux, mcuy;
    uint32_t ncomp, hs, vs, bpm;  // components, luma sampling factors, blocks per MCU
    uint32_t qt[3];               // quantisation table pool index per component
    uint32_t dc_tab[3], ac_tab[3];  // Huffman table pool index per component
    uint32_t restart;             // MCUs per restart interval, 0 = none
    uint32_t nseg;                // restart segments expected (1 when restart == 0)
    uint32_t seg_off;             // first entry of this image in the segment-start array
    uint32_t nblocks;
    uint32_t plane_pitch[3];
    uint32_t plane_rows[3];
    uint32_t item;                // index in the batch (status word, result)
    uint32_t out_pitch;           // bytes per row of the decoded image: width * channels for a payload, padded to 16 bytes
                                  // when a resize reads it (rows then start on 16-byte boundaries for asynchronous copies)
};

// One 1-D convolution pass over a region of one image (u8, 1 or 3 interleaved channels).
// horizontal: dst(x, y) = clip8((round + sum_i k[i][t0 + x] * src(start[t0 + x] - src_origin + i, y)) >> precision)
// vertical:   dst(x, y) = clip8((round + sum_i k[i][t0 + y] * src(x, start[t0 + y] - src_origin + i)) >> precision)
struct ConvPass {
    const uint8_t* src;  // first needed row (horizontal) / first needed column (vertical) already applied
    uint8_t* dst;
    uint32_t src_pitch, dst_pitch;  // bytes
    uint32_t out_w, out_h;          // produced region in pixels
    uint32_t channels;
    int32_t src_origin;             // coordinate, along the filtered axis, of element 0 of `src`
    uint32_t t0;                    // first table entry used
    uint32_t tab_n, window, precision;
    uint64_t tab_off;               // word offset in the table pool: start[tab_n] | size[tab_n] | int16 k[window][tab_n]
    uint32_t tile_first;            // first CTA tile of this pass in the launch (prefix sum)
    uint32_t tiles_x;               // tiles per row of tiles
    uint32_t fast;                  // vertical: 1 = the vectorised path applies; 2 (both directions) = the tensor-core path (see kernels_resize.cu)
    uint32_t box_pieces;            // tensor-core path, horizontal: 16-byte pieces per staged source row (odd), the width of the tensor map's
                                    // box; vertical: rows of a box | boxes per chunk << 16
    // Set when `src` is memory the library does not own (no slack behind it): the horizontal pass then loads no byte
    // outside [guard_lo, guard_hi).  Both null for sources inside the library's own padded arenas.
    const uint8_t* guard_lo;
    const uint8_t* guard_hi;
    // Tensor-core path: the CUtensorMap (128 opaque bytes, written by cuTensorMapEncodeTiled) of the pass's source; the
    // copying thread of a CTA hands its address to cp.async.bulk.tensor.  Horizontal: a two-dimensional array of 32-bit
    // words, box = box_pieces * 4 words x 32 rows; vertical: of bytes, box = 64 bytes x the rows of a box, 64-byte
    // swizzle.  Unused (zero) for every other pass.
    alignas(64) unsigned char tmap[128];
};
static_assert(sizeof(ConvPass) % 64 == 0, "passes are stored as an array: every tensor map must stay 64-byte aligned");

struct CopyJob {  // identity payloads / pitch removal
    const uint8_t* src;
    uint8_t* dst;
    uint32_t src_pitch, row_bytes, rows, tile_first;
};

// Alpha pre-multiplication / division around a convolution resize of an image with an alpha channel (2 = luma + alpha,
// 4 = RGBA): what fast_image_resize does inside Resizer::resize for such pixel types.
struct AlphaJob {
    const uint8_t* src;
    uint8_t* dst;            // may equal src
    uint32_t src_pitch, dst_pitch, width, rows, channels;  // width in pixels
    uint32_t divide;         // 0: colour = mul_div_255(colour, alpha); 1: colour = colour * recip(alpha), rounded and clipped
    uint32_t tile_first, pad;
};

struct ToRgbJob {  // convert_to_rgb8 of one payload: channels 1, 2 or 4 -> 3
    const uint8_t* src;
    uint8_t* dst;
    uint32_t npx, channels, tile_first, pad;
};

}  // namespace dg
