// JPEG marker-segment parser and Huffman table preparation (host).
// Stands in for what `image::ImageReader::decode()` / zune-jpeg reads before the entropy-coded data
// (datago call sites: src/worker_files.rs:14-16, src/worker_wds.rs:45, src/worker_http.rs:64).
// Only what the baseline path needs: SOF0/SOF1, 8-bit, 1 or 3 components, one interleaved scan.
#include <climits>
#include <cstring>

#include "host.h"

namespace dg {

namespace {

const uint8_t kZigzagToNatural[64] = {0,  1,  8,  16, 9,  2,  3,  10, 17, 24, 32, 25, 18, 11, 4,  5,
                                      12, 19, 26, 33, 40, 48, 41, 34, 27, 20, 13, 6,  7,  14, 21, 28,
                                      35, 42, 49, 56, 57, 50, 43, 36, 29, 22, 15, 23, 30, 37, 44, 51,
                                      58, 59, 52, 45, 38, 31, 39, 46, 53, 60, 61, 54, 47, 55, 62, 63};

struct Cursor {
    const uint8_t* p;
    uint64_t n, i;
    bool has(uint64_t k) const { return i + k <= n; }
    uint8_t u8() { return p[i++]; }
    uint32_t u16() { uint32_t v = ((uint32_t)p[i] << 8) | p[i + 1]; i += 2; return v; }
};

int read_dqt(Cursor seg, JpegHeader& h) {
    while (seg.has(1)) {
        const uint8_t pt = seg.u8();
        const int wide = pt >> 4, slot = pt & 15;
        if (slot > 3 || wide > 1) return DG_E_BAD_TABLE;
        if (!seg.has(wide ? 128 : 64)) return DG_E_TRUNCATED;
        for (int k = 0; k < 64; ++k) h.qt[slot][kZigzagToNatural[k]] = (uint16_t)(wide ? seg.u16() : seg.u8());
        h.qt_set[slot] = true;
    }
    return DG_OK;
}

int read_dht(Cursor seg, JpegHeader& h) {
    while (seg.has(1)) {
        const uint8_t tc_th = seg.u8();
        const int cls = tc_th >> 4, slot = tc_th & 15;
        if (cls > 1 || slot > 3) return DG_E_BAD_TABLE;
        if (!seg.has(16)) return DG_E_TRUNCATED;
        JpegHeader::RawHuff& t = cls ? h.ac[slot] : h.dc[slot];
        t.bits[0] = 0;
        t.count = 0;
        for (int l = 1; l <= 16; ++l) { t.bits[l] = seg.u8(); t.count += t.bits[l]; }
        if (t.count > 256) return DG_E_BAD_TABLE;
        if (!seg.has((uint64_t)t.count)) return DG_E_TRUNCATED;
        memset(t.vals, 0, sizeof t.vals);
        for (int k = 0; k < t.count; ++k) t.vals[k] = seg.u8();
        t.set = true;
    }
    return DG_OK;
}

int read_sof(Cursor seg, JpegHeader& h) {
    if (!seg.has(6)) return DG_E_TRUNCATED;
    if (seg.u8() != 8) return DG_E_UNSUPPORTED;  // sample precision
    h.height = seg.u16();
    h.width = seg.u16();
    h.ncomp = seg.u8();
    if (h.width == 0 || h.height == 0) return DG_E_UNSUPPORTED;
    if (h.ncomp != 1 && h.ncomp != 3) return DG_E_UNSUPPORTED;
    if (!seg.has(3ull * h.ncomp)) return DG_E_TRUNCATED;
    uint32_t hsamp[3], vsamp[3];
    for (uint32_t c = 0; c < h.ncomp; ++c) {
        seg.u8();  // component id: matched positionally against the scan header
        const uint8_t hv = seg.u8();
        hsamp[c] = hv >> 4;
        vsamp[c] = hv & 15;
        h.comp_tq[c] = seg.u8();
        if (h.comp_tq[c] > 3) return DG_E_BAD_TABLE;
    }
    if (h.ncomp == 1) {
        h.hs = h.vs = 1;  // a one-component scan is never interleaved: MCU = one block
    } else {
        if (hsamp[1] != 1 || vsamp[1] != 1 || hsamp[2] != 1 || vsamp[2] != 1) return DG_E_UNSUPPORTED;
        if (hsamp[0] < 1 || hsamp[0] > 2 || vsamp[0] < 1 || vsamp[0] > 2) return DG_E_UNSUPPORTED;
        h.hs = hsamp[0];
        h.vs = vsamp[0];
    }
    h.mcux = (h.width + 8 * h.hs - 1) / (8 * h.hs);
    h.mcuy = (h.height + 8 * h.vs - 1) / (8 * h.vs);
    return DG_OK;
}

}  // namespace

int parse_jpeg_header(const uint8_t* data, uint64_t len, JpegHeader& h) {
    if (!data || len < 4 || data[0] != 0xFF || data[1] != 0xD8) return DG_E_BAD_MARKER;
    uint64_t pos = 2;
    bool frame_seen = false;
    uint8_t frame_ids[3] = {0, 0, 0};
    for (;;) {
        if (pos + 2 > len) return DG_E_TRUNCATED;
        if (data[pos] != 0xFF) return DG_E_BAD_MARKER;
        while (pos < len && data[pos] == 0xFF) ++pos;  // optional fill bytes
        if (pos >= len) return DG_E_TRUNCATED;
        const uint8_t marker = data[pos++];
        if (marker == 0xD8 || marker == 0x01 || (marker >= 0xD0 && marker <= 0xD7)) continue;  // no payload
        if (marker == 0xD9) return DG_E_TRUNCATED;  // EOI before any scan
        if (pos + 2 > len) return DG_E_TRUNCATED;
        const uint64_t seglen = ((uint64_t)data[pos] << 8) | data[pos + 1];
        if (seglen < 2 || pos + seglen > len) return DG_E_TRUNCATED;
        Cursor seg{data + pos + 2, seglen - 2, 0};
        int rc = DG_OK;
        switch (marker) {
            case 0xDB: rc = read_dqt(seg, h); break;
            case 0xC4: rc = read_dht(seg, h); break;
            case 0xC0:
            case 0xC1:
                rc = read_sof(seg, h);
                if (rc == DG_OK) {
                    frame_seen = true;
                    for (uint32_t c = 0; c < h.ncomp; ++c) frame_ids[c] = data[pos + 2 + 6 + 3 * c];
                }
                break;
            case 0xDD:
                if (!seg.has(2)) return DG_E_TRUNCATED;
                h.restart = seg.u16();
                break;
            case 0xDA: {
                if (!frame_seen) return DG_E_BAD_MARKER;
                if (!seg.has(1)) return DG_E_TRUNCATED;
                const uint32_t ns = seg.u8();
                if (ns != h.ncomp) return DG_E_UNSUPPORTED;  // one interleaved scan only
                if (!seg.has(2ull * ns + 3)) return DG_E_TRUNCATED;
                for (uint32_t c = 0; c < ns; ++c) {
                    if (seg.u8() != frame_ids[c]) return DG_E_UNSUPPORTED;
                    const uint8_t tt = seg.u8();
                    h.comp_td[c] = tt >> 4;
                    h.comp_ta[c] = tt & 15;
                    if (h.comp_td[c] > 3 || h.comp_ta[c] > 3) return DG_E_BAD_TABLE;
                    if (!h.dc[h.comp_td[c]].set || !h.ac[h.comp_ta[c]].set || !h.qt_set[h.comp_tq[c]]) return DG_E_BAD_TABLE;
                }
                h.scan_off = pos + seglen;
                h.scan_len = len - h.scan_off;
                return DG_OK;
            }
            default:
                // SOF2.. (progressive, lossless, arithmetic) are not this path; DHT(C4), JPG(C8), DAC(CC) excluded
                if (marker >= 0xC2 && marker <= 0xCF && marker != 0xC4 && marker != 0xC8 && marker != 0xCC) return DG_E_UNSUPPORTED;
                break;  // APPn, COM, anything else: skipped
        }
        if (rc != DG_OK) return rc;
        pos += seglen;
    }
}

// Canonical code assignment (T.81 Annex C) into the device lookup form.
bool huff_lengths_valid(const JpegHeader::RawHuff& raw) {
    int code = 0;
    for (int l = 1; l <= 16; ++l) {
        if (code + raw.bits[l] > (1 << l)) return false;  // over-subscribed
        code = (code + raw.bits[l]) << 1;
    }
    return true;
}

bool build_huff_table(const JpegHeader::RawHuff& raw, HuffTable& out) {
    memset(&out, 0, sizeof out);
    memcpy(out.vals, raw.vals, 256);
    int code = 0, k = 0;
    for (int l = 1; l <= 16; ++l) {
        out.valoff[l] = k - code;
        if (raw.bits[l]) {
            if (code + raw.bits[l] > (1 << l)) return false;  // over-subscribed
            for (int j = 0; j < raw.bits[l]; ++j, ++k, ++code) {
                if (l <= kLutBits) {
                    const int span = 1 << (kLutBits - l);
                    for (int f = 0; f < span; ++f) out.lut[(code << (kLutBits - l)) | f] = huff_pack((uint32_t)l, raw.vals[k]);
                }
            }
            out.maxcode[l] = code - 1;
        } else {
            out.maxcode[l] = -1;
        }
        code <<= 1;
    }
    out.maxcode[17] = INT_MAX;
    // left-aligned end of the code space used by lengths <= l (the first code of the next length, shifted to 16 bits)
    uint32_t used = 0;  // in units of 2^-16 of the code space
    for (int l = 1; l <= 16; ++l) {
        used += (uint32_t)raw.bits[l] << (16 - l);
        if (l >= 10) out.limit[l - 10] = used;
    }
    out.limit[7] = 0xFFFFFFFFu;
    return true;
}

}  // namespace dg
