// Launch interface between the batch scheduler (api.cu) and the sm_100a kernels.
#pragma once
#include <cuda_runtime.h>

#include "desc.h"

namespace dg {

// Maps a flat work index (block, tile, segment) to its owner (image, pass): first[owner] <= idx < first[owner + 1].
// coarse[idx >> shift] is the owner of work item (idx >> shift) << shift, so the search is a short forward walk.
struct OwnerMap {
    const uint32_t* first;   // n + 1 entries
    const uint32_t* coarse;
    uint32_t n, shift, total;
};

struct JpegWave {
    const JpegDesc* descs;   // device, n images
    uint32_t n;
    const uint8_t* raw;      // compressed blob
    uint8_t* us;             // unstuffed streams
    uint32_t* us_len;        // [n] bytes of each unstuffed stream
    uint32_t* seg_start;     // restart-segment starts (bytes into the image's unstuffed stream)
    uint32_t* seg_found;     // [n] segments actually present
    int16_t* coef;           // [blocks][64], scan order, natural order inside a block
    uint8_t* planes;         // component planes after the IDCT
    uint8_t* out;            // decoded images
    uint32_t* status;        // [items of the batch]
    unsigned long long* spec_stats;  // [0] chunks, [1] synchronisation rounds, [2] subsequence decodes (all passes)
    const HuffTable* huff;   // table pool
    uint32_t n_huff;         // tables in the pool
    const uint32_t* qt32;    // quantisation pool, 32 words per table: word i holds q[2i] in byte 0 and q[2i+1] in byte 3
    // speculative (no restart marker) images and restart-interval images of this wave
    const uint32_t* spec_list; uint32_t n_spec;
    OwnerMap restart_segs;   // owner = index into restart_list
    const uint32_t* restart_list;
    OwnerMap blocks;         // owner = image
    OwnerMap color_tiles;    // owner = image
    // Images [fused_first, n) of the wave are three-component 4:2:0 images at least five pixels wide: they take the fused
    // path (chroma-only IDCT into planes, then one kernel for luma IDCT + upsampling + colour conversion) and are not
    // covered by `blocks` / `color_tiles`.  Owner o of these two maps is image fused_first + o.
    uint32_t fused_first;
    OwnerMap fused_chroma;   // flat index over the chroma blocks (Cb, Cr of MCU 0, Cb, Cr of MCU 1, ...)
    OwnerMap fused_tiles;    // colour tiles, color_tiles() per image
};

void launch_unstuff(const JpegWave& w, cudaStream_t s);
void launch_huff_restart(const JpegWave& w, cudaStream_t s);
// the first n_huge images of spec_list (longest first) have more than kSpecHugeBytes of entropy-coded data: they get the
// widest CTAs, on huge_stream, beside the others on s
constexpr uint32_t kSpecHugeBytes = 1024 * 2048 / 8, kSpecHugeMax = 64;
void launch_huff_spec(const JpegWave& w, uint32_t n_huge, cudaStream_t s, cudaStream_t huge_stream);
// blocks [first, first + count) of the wave / colour tiles [first, first + count): callers may launch them in groups of
// images (the planes written by the IDCT are then still in L2 when the colour kernel reads them) or once per wave
// rezero: the kernel writes zeros back over every coefficient row it found non-zero, which leaves the coefficient
// buffer all-zero again for the next wave that uses it (the entropy decoders only write non-zero coefficients)
void launch_idct(const JpegWave& w, uint32_t first, uint32_t count, bool rezero, cudaStream_t s);
void launch_color(const JpegWave& w, uint32_t first_tile, uint32_t count, cudaStream_t s);
// the fused path: chroma blocks [first, first + count) of fused_chroma, tiles [first, first + count) of fused_tiles
void launch_idct_chroma(const JpegWave& w, uint32_t first, uint32_t count, bool rezero, cudaStream_t s);
void launch_luma_color(const JpegWave& w, uint32_t first_tile, uint32_t count, bool rezero, cudaStream_t s);
// whether an image takes the fused path
inline bool fused_decode(uint32_t ncomp, uint32_t hs, uint32_t vs, uint32_t width) { return ncomp == 3 && hs == 2 && vs == 2 && width >= 5; }

// The colour kernel gives one CTA 256 pixels of four MCU rows.
constexpr uint32_t kColorTileW = 256, kColorMcuRows = 4;
inline uint32_t color_tiles(uint32_t width, uint32_t mcuy) {
    // one more row of tiles than the MCU rows need: the 4:2:0 path of the colour kernel shifts its tiles up by one pixel
    // row, so that every pair of output rows that shares its two chroma rows falls into one tile
    return ((width + kColorTileW - 1) / kColorTileW) * (mcuy / kColorMcuRows + 1);
}
#ifndef DG_FUSED_MCU_ROWS
#define DG_FUSED_MCU_ROWS 4
#endif
constexpr uint32_t kFusedMcuRows = DG_FUSED_MCU_ROWS;  // MCU rows of a tile of the fused kernel (64 threads per MCU row)
inline uint32_t fused_tiles(uint32_t width, uint32_t mcuy) {  // the fused kernel's tiles are aligned to MCU rows
    return ((width + kColorTileW - 1) / kColorTileW) * ((mcuy + kFusedMcuRows - 1) / kFusedMcuRows);
}

// ---- resize ---------------------------------------------------------------------------------------------------------
constexpr uint32_t kConvTileW = 64, kConvTileH = 16;    // horizontal pass: output pixels x rows per CTA
constexpr uint32_t kVTileBytes = 256, kVTileH = 4;      // vertical pass, plain path: output bytes x rows per CTA
constexpr uint32_t kVFastBytes = 1024, kVFastRows = 32; // vertical pass, vector path: 64 x 16-byte columns, 4 x 8 rows
constexpr uint32_t kVFastMaxWindow = 128;
// horizontal pass on the tensor cores (ConvPass::fast == 2): output bytes per strip x rows per CTA; limits of what a CTA
// can stage -- source bytes under one 8-byte output tile, and under a whole strip
constexpr uint32_t kHMmaStrip = 64, kHMmaRows = 2048, kHMmaMaxBand = 256, kHMmaMaxSpan = 1008;  // span: 63 pieces of 16 bytes = 252 words, inside the 256 elements a tensor-map box may have
// vertical pass on the tensor cores (ConvPass::fast == 2): output rows x bytes of a row per CTA; limits of what a CTA can
// stage -- source rows under the eight output rows of one warp, and under all rows of the CTA
constexpr uint32_t kVMmaRows = 64, kVMmaCols = 4096, kVMmaMaxBand = 256, kVMmaMaxSpan = 704;
inline uint32_t conv_tiles_x(const ConvPass& p, bool vertical) {
    if (!vertical && p.fast == 2) return (p.out_w * p.channels + kHMmaStrip - 1) / kHMmaStrip;
    if (vertical && p.fast == 2) return (p.out_w * p.channels + kVMmaCols - 1) / kVMmaCols;
    if (!vertical) return (p.out_w + kConvTileW - 1) / kConvTileW;
    const uint32_t row_bytes = p.out_w * p.channels;
    return p.fast ? (row_bytes + kVFastBytes - 1) / kVFastBytes : (row_bytes + kVTileBytes - 1) / kVTileBytes;
}
inline uint32_t conv_tiles(const ConvPass& p, bool vertical) {
    const uint32_t rows = !vertical ? (p.fast == 2 ? kHMmaRows : kConvTileH) : p.fast == 2 ? kVMmaRows : p.fast ? kVFastRows : kVTileH;
    return conv_tiles_x(p, vertical) * ((p.out_h + rows - 1) / rows);
}
constexpr uint32_t kCopyTileBytes = 4096;

// the passes that take the tensor-core kernel (fast == 2) come first in `passes` and own tiles [0, mma_tiles)
void launch_conv_h(const ConvPass* passes, OwnerMap map, const uint32_t* tables, uint32_t mma_tiles, cudaStream_t s);
// CTAs of the tensor-core horizontal pass that ran out of patience waiting for a copy since the library was loaded
unsigned int read_conv_timeouts(cudaStream_t s);
void launch_conv_v(const ConvPass* passes, OwnerMap map, const uint32_t* tables, uint32_t mma_tiles, cudaStream_t s);
void launch_copy(const CopyJob* jobs, OwnerMap map, cudaStream_t s);
constexpr uint32_t kAlphaTilePx = 2048;  // pixels per CTA of the alpha multiply / divide kernel
void launch_alpha(const AlphaJob* jobs, OwnerMap map, cudaStream_t s);
constexpr uint32_t kToRgbTilePx = 2048;  // pixels per CTA of the RGB8 conversion
void launch_to_rgb8(const ToRgbJob* jobs, OwnerMap map, cudaStream_t s);

}  // namespace dg
