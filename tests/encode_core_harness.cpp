/* Host driver for the encoder rules in nwc_b200/csrc/nwc_encode_core.h (test infrastructure).
 *
 * The GPU encoder calls those rules from one thread per lane stream; this file calls the very same functions and sinks
 * from plain loops, so the stream walk, code emission, plane addressing and table construction can be compared with
 * the oracle on a machine without a GPU.  The kernels' own parts (thread indexing, warp scan, atomics) are not covered
 * here; the GPU tests cover them.
 */
#include <cstdint>
#include <cstring>
#include <vector>
#include "../nwc_b200/csrc/nwc_encode_core.h"

using namespace nwc;

extern "C" __attribute__((visibility("default")))
int64_t harness_encode(const void *w, uint64_t n, uint32_t K, int code, uint16_t *psym, uint32_t *bases, uint8_t *hdr,
                       uint8_t *data, uint64_t cap, uint8_t *low, uint32_t *lut) {
    if (!K || !n || n % K) return -1;
    const int type = type_of(code), layout = layout_of(code);
    const uint32_t M = (uint32_t)(n / K);
    const Geometry g(M, K, layout);
    unsigned long long hist[128] = {0};
    for (uint64_t i = 0; i < n; i++) {
        uint32_t sym, raw;
        if (type == kFp8) {
            const uint32_t b = static_cast<const uint8_t *>(w)[i];
            if (!(layout == 2 ? fp8_split_fixed(b, sym, raw) : fp8_split_prefix(b, sym, raw))) return -2;
        } else sym = (static_cast<const uint16_t *>(w)[i] >> 8) & 0x7Fu;
        hist[sym]++;
    }
    uint8_t rank_of[128];
    build_symbol_tables(hist, type, layout, psym, rank_of);
    build_table_words(psym, code, lut);
    const EncodeJob j{w, rank_of, type, layout, M, K};
    memset(low, 0, g.raw_plane_bytes(code));
    for (uint32_t b = 0; b < g.nb; b++)
        for (uint32_t L = 0; L < kLanes; L++) {
            CountSink s;
            if (layout == 2) { if (!encode_fixed_stream(j, g, b, L, s)) return -3; hdr[b * kLanes + L] = (uint8_t)s.exceptions; }
            else { encode_prefix_stream(j, g, b, L, s); const uint32_t words = (s.nbits + 31u) >> 5; if (words > 255u) return -1; hdr[b * kLanes + L] = (uint8_t)words; }
        }
    const uint32_t unit = layout == 2 ? (type == kFp8 ? 2u : 3u) : 4u;
    uint64_t pos = 0, end = 0;
    for (uint32_t b = 0; b < g.nb; b++) {
        uint32_t size = 0; for (uint32_t L = 0; L < kLanes; L++) size += hdr[b * kLanes + L];
        bases[b] = (uint32_t)pos; end = pos + (uint64_t)size * unit;
        pos += ((uint64_t)size * unit + 7u) & ~7ull;
    }
    if (end + 64 > cap) return -1;
    for (uint32_t b = 0; b < g.nb; b++) {
        uint32_t before = 0;
        for (uint32_t L = 0; L < kLanes; L++) {
            uint8_t *block = data + bases[b];
            if (layout == 2) { WriteSink s(g, type, nullptr, block + (uint64_t)before * unit, low); encode_fixed_stream(j, g, b, L, s); }
            else { WriteSink s(g, type, reinterpret_cast<uint32_t *>(block) + before, nullptr, low); encode_prefix_stream(j, g, b, L, s); s.flush(); }
            before += hdr[b * kLanes + L];
        }
    }
    if (layout == 0)
        for (uint32_t m = 0; m < M; m++) for (uint32_t c = 0; c < (g.K16 >> 4); c++) plane0_cell(j, g, m, c, low);
    return (int64_t)(pos + 64);
}

extern "C" __attribute__((visibility("default")))
int harness_layout(uint64_t M, uint32_t K, int code, uint64_t *out) {
    const Geometry g((uint32_t)M, K, layout_of(code));
    out[0] = g.nb; out[1] = g.raw_plane_bytes(code); out[2] = g.scratch_floats(); out[3] = g.K16;
    return 0;
}
