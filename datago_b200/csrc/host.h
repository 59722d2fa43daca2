// Host-side planning: bucket table, crop geometry, filter tables, JPEG headers.
#pragma once
#include <cstdint>
#include <string>
#include <vector>

#include "../../include/datago_b200.h"
#include "desc.h"

namespace dg {

// ---- buckets (src/image_processing.rs:77-120, 188-252 of datago) -------------------------------------------------
struct BucketEntry {
    double ar;
    char key[16];
    uint32_t w, h;
};

struct Transform {
    std::vector<BucketEntry> buckets;  // sorted by ar
    int find(const char* key) const;
    int closest(int32_t w, int32_t h) const;
};

bool config_valid(const dg_image_config& c);
std::vector<std::pair<uint32_t, uint32_t>> image_size_list(const dg_image_config& c);
Transform make_transform(const dg_image_config& c);
void format_key(uint32_t w, uint32_t h, char out[16]);
// returns DG_OK or DG_E_UNKNOWN_KEY
int plan_geometry(const Transform& t, uint32_t w, uint32_t h, uint32_t channels, const char* forced_key, dg_plan* out);

// ---- Lanczos3 filter tables (the fast_image_resize coefficient rule) ----------------------------------------------
struct FilterTable {
    int n = 0, window = 0, precision = 0;
    std::vector<int32_t> start, size;
    std::vector<int16_t> k;  // [window][n]: tap-major so that neighbouring outputs read neighbouring words
    int first_in() const { return start[0]; }
    int last_in(int lo, int hi) const;  // one past the last input sample used by outputs [lo, hi)
    // start/size/k packed as 32-bit words, the layout ConvPass::tab_off points at
    size_t words() const { return (size_t)2 * n + ((size_t)window * n + 1) / 2; }
    void pack(uint32_t* dst) const;
};
FilterTable make_filter_table(int in_size, double in0, double in1, int out_size);

// ---- JPEG headers ----------------------------------------------------------------------------------------------------
struct JpegHeader {
    uint32_t width = 0, height = 0, ncomp = 0, hs = 1, vs = 1, mcux = 0, mcuy = 0, restart = 0;
    uint8_t comp_tq[3] = {0, 0, 0}, comp_td[3] = {0, 0, 0}, comp_ta[3] = {0, 0, 0};
    uint16_t qt[4][64];  // natural (row-major) order
    bool qt_set[4] = {false, false, false, false};
    struct RawHuff { bool set = false; uint8_t bits[17]; uint8_t vals[256]; int count = 0; } dc[4], ac[4];
    uint64_t scan_off = 0, scan_len = 0;
};
int parse_jpeg_header(const uint8_t* data, uint64_t len, JpegHeader& h);  // dg_status
bool build_huff_table(const JpegHeader::RawHuff& raw, HuffTable& out);
bool huff_lengths_valid(const JpegHeader::RawHuff& raw);  // what build_huff_table would accept, without building

// ---- errors ---------------------------------------------------------------------------------------------------------
// Stores msg as the calling thread's dg_last_error text and returns code.
int dg_set_error(int code, const char* msg);

// ---- sharding -------------------------------------------------------------------------------------------------------
uint64_t siphash13_str(const char* key, uint64_t len);

}  // namespace dg
