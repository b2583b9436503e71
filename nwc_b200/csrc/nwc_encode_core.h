/* Per-lane-stream encoding rules of the NWC formats, written once for host and device.
 *
 * The GPU encoder runs one thread per (block, lane) stream and calls these functions twice: first with a counting
 * sink (stream length -> header byte), then, after the block offsets are known, with a writing sink.  The same
 * functions compile as plain C++ so the index arithmetic can be exercised on a CPU without a device.
 *
 * Format rules restated from the reference's host encoder (csrc/nwc_ops.cu:135-173 fp8 symbol split, 175-243 layout
 * 2, 245-320 layouts 0 and 1).
 */
#pragma once
#include <cstdint>
#include <cstring>
#include "nwc_geometry.h"

namespace nwc {

constexpr uint32_t kFixedRanks = 7;        /* layout 2: ranks 0..6 are coded, 7 marks an exception */

/* fp8 e4m3 -> symbol of the prefix layouts (0..9) and 4-bit raw nibble; false for NaN */
NWC_HD bool fp8_split_prefix(uint32_t b, uint32_t &sym, uint32_t &nib) {
    const uint32_t e = (b >> 3) & 15u, m = b & 7u;
    if (e) { if (e == 15u && m == 7u) return false; sym = e >> 1; nib = ((e & 1u) << 3) | m; return true; }
    if (m >= 4u) { sym = 0u; nib = (m - 4u) << 1; }
    else if (m == 0u) { sym = 9u; nib = 0u; }
    else { sym = 8u; nib = m == 1u ? 0u : (m == 2u ? 8u : 12u); }
    return true;
}
/* fp8 e4m3 -> symbol of the fixed-width layout (0..19) and 3-bit field; false for NaN */
NWC_HD bool fp8_split_fixed(uint32_t b, uint32_t &sym, uint32_t &field) {
    const uint32_t e = (b >> 3) & 15u, m = b & 7u;
    if (e) { if (e == 15u && m == 7u) return false; sym = e; field = m; return true; }
    if (m >= 4u) { sym = 16u; field = (m - 4u) << 1; }
    else if (m >= 2u) { sym = 17u; field = (m - 2u) << 2; }
    else { sym = m == 1u ? 18u : 19u; field = 0u; }
    return true;
}
/* bf16 high byte (without sign) that a prefix-layout fp8 symbol decodes to */
NWC_HD uint32_t fp8_prefix_high(uint32_t sym) { return sym < 8u ? 60u + sym : (sym == 8u ? 59u : 0u); }
/* fixed-width layout: bf16 high byte and bit 7 of the low byte per fp8 symbol */
NWC_HD uint32_t fp8_fixed_high(uint32_t sym) {
    if (sym >= 1u && sym <= 15u) return 60u + (sym >> 1);
    return sym == 16u ? 60u : ((sym == 17u || sym == 18u) ? 59u : 0u);
}
NWC_HD uint32_t fp8_fixed_bit7(uint32_t sym) { return (sym >= 1u && sym <= 15u) ? ((sym & 1u) << 7) : (sym == 17u ? 0x80u : 0u); }

struct EncodeJob {
    const void *w;                 /* bf16 bits (uint16) or fp8 bytes, row-major M x K */
    const uint8_t *rank_of;        /* [128] rank of every symbol                        */
    int type, layout;
    uint32_t M, K;
};

/* (symbol | sign << 7, raw part) of one weight.  NaN cannot occur here: the histogram pass rejects it first. */
NWC_HD void classify(const EncodeJob &j, uint64_t index, uint32_t &high, uint32_t &raw) {
    if (j.type == kFp8) {
        const uint32_t b = static_cast<const uint8_t *>(j.w)[index];
        uint32_t s = 0, r = 0;
        if (j.layout == 2) fp8_split_fixed(b, s, r); else fp8_split_prefix(b, s, r);
        high = (b & 0x80u) | s; raw = r;
    } else {
        const uint32_t v = static_cast<const uint16_t *>(j.w)[index];
        high = v >> 8; raw = v & 0xFFu;
    }
}

/* weights a lane stream of block column cb codes */
NWC_HD uint32_t stream_weights(const Geometry &g, int layout, uint32_t cb) { return layout ? g.supers_in(cb) * 16u : 128u; }

NWC_HD void stream_position(const Geometry &g, int layout, uint32_t rb, uint32_t cb, uint32_t L, uint32_t i, uint32_t &row, uint32_t &col) {
    if (layout) { row = rb * 16u + frag_row(L, i & 15u); col = cb * kBlockCols + (i >> 4) * 32u + frag_col(L, i & 15u); }
    else { row = rb * 8u + (i >> 4); col = cb * kBlockCols + L * 16u + (i & 15u); }
}

/* Prefix layouts (0 and 1).  Sink interface:
 *   void bits(uint32_t value, int n)              append n bits, MSB first
 *   void raw1(uint64_t cell, uint32_t i, uint32_t raw)   layout 1 only: raw part of stream element i of plane cell
 * Returns nothing; the sink counts. */
template <class Sink>
NWC_HD void encode_prefix_stream(const EncodeJob &j, const Geometry &g, uint32_t b, uint32_t L, Sink &sink) {
    const uint32_t rb = b / g.CB, cb = b - rb * g.CB, n = stream_weights(g, j.layout, cb);
    const uint32_t max_rank = j.type == kFp8 ? 10u : 15u;
    const uint64_t slot0 = (uint64_t)rb * g.slots + cb * 16u;
    for (uint32_t i = 0; i < n; i++) {
        uint32_t row, col; stream_position(g, j.layout, rb, cb, L, i, row, col);
        if (row >= j.M || col >= j.K) { sink.bits(2u, 2); continue; }            /* filler: rank 0, sign 0 */
        uint32_t high, raw; classify(j, (uint64_t)row * j.K + col, high, raw);
        const uint32_t rank = j.rank_of[high & 0x7Fu];
        if (rank < max_rank) sink.bits(2u | (high >> 7), (int)rank + 2);         /* rank zeros, a one, the sign */
        else { sink.bits(1u, 16); sink.bits(high, 8); }                           /* escape: 15 zeros, a one, the byte */
        if (j.layout) sink.raw1((slot0 + (i >> 4)) * kLanes + L, i & 15u, raw);
    }
}

/* Fixed-width layout (2).  Sink interface:
 *   void nibble(uint64_t cell, uint32_t j, uint32_t value)     [sign | rank] of element j (0..15) of a plane cell
 *   void raw2(uint32_t rb, uint32_t cb, uint32_t sc, uint32_t L, uint64_t cell, uint32_t j, uint32_t raw)
 *   bool exception(uint32_t index, uint32_t b0, uint32_t b1)   false when the lane already holds 255 entries */
template <class Sink>
NWC_HD bool encode_fixed_stream(const EncodeJob &j, const Geometry &g, uint32_t b, uint32_t L, Sink &sink) {
    const uint32_t rb = b / g.CB, cb = b - rb * g.CB, n = stream_weights(g, 2, cb);
    const uint64_t slot0 = (uint64_t)rb * g.slots + cb * 16u;
    for (uint32_t i = 0; i < n; i++) {
        uint32_t row, col; stream_position(g, 2, rb, cb, L, i, row, col);
        if (row >= j.M || col >= j.K) continue;                                   /* filler: both planes stay 0 */
        const uint64_t index = (uint64_t)row * j.K + col;
        uint32_t high, raw; classify(j, index, high, raw);
        const uint32_t rank = j.rank_of[high & 0x7Fu];
        if (rank == kFixedRanks) {
            bool ok;
            if (j.type == kFp8) ok = sink.exception(i, static_cast<const uint8_t *>(j.w)[index], 0u);
            else { const uint32_t v = static_cast<const uint16_t *>(j.w)[index]; ok = sink.exception(i, v & 0xFFu, v >> 8); }
            if (!ok) return false;
            raw = 0u;
        }
        const uint64_t cell = (slot0 + (i >> 4)) * kLanes + L;
        sink.nibble(cell, i & 15u, ((high >> 7) << 3) | rank);
        sink.raw2(rb, cb, i >> 4, L, cell, i & 15u, raw);
    }
    return true;
}

/* byte offset inside the fp8 raw plane of layout 2 of the 32-bit word holding bit `3 * t` of a lane's 96-bit group */
NWC_HD uint64_t fixed_fp8_word(const Geometry &g, uint32_t rb, uint32_t cb, uint32_t sc, uint32_t L, uint32_t word) {
    const uint64_t pair = (uint64_t)rb * g.pair_slots + cb * 8u + (sc >> 1);
    return ((pair * 3u + word) * kLanes + L) * 4u;
}

/* Frequency order of the first nsym symbols: an in-place exchange pass that swaps whenever a later entry is strictly
   more frequent.  Ties resolve by this swap sequence, and the streams depend on it (reference: csrc/nwc_ops.cu:194,277). */
inline void frequency_order(const unsigned long long *hist, int nsym, int *order /* [128] */) {
    for (int i = 0; i < 128; i++) order[i] = i;
    for (int a = 0; a < nsym; a++)
        for (int b = a + 1; b < nsym; b++)
            if (hist[order[b]] > hist[order[a]]) { const int t = order[a]; order[a] = order[b]; order[b] = t; }
}

/* layout 0 raw plane: the 16 columns [16 c, 16 c + 16) of row m as one 16-byte (bf16 low bytes) or 8-byte (fp8 nibbles,
   interleaved so that one shift and one mask expand a word into four weight bytes) store */
NWC_HD void plane0_cell(const EncodeJob &j, const Geometry &g, uint32_t m, uint32_t c, uint8_t *low) {
    uint32_t out[4] = {0u, 0u, 0u, 0u};
    for (uint32_t k = 0; k < 16u; k++) {
        const uint32_t col = c * 16u + k;
        if (col >= j.K) break;
        uint32_t high, raw; classify(j, (uint64_t)m * j.K + col, high, raw);
        if (j.type == kFp8) { const uint32_t byte = (k & 3u) + ((k >> 3) << 2); out[byte >> 2] |= (raw << (((k >> 2) & 1u) ? 4u : 0u)) << (8u * (byte & 3u)); }
        else out[k >> 2] |= raw << (8u * (k & 3u));
    }
    uint32_t *dst = reinterpret_cast<uint32_t *>(j.type == kFp8 ? low + (uint64_t)m * (g.K16 >> 1) + c * 8u : low + (uint64_t)m * g.K16 + c * 16u);
    dst[0] = out[0]; dst[1] = out[1];
    if (j.type != kFp8) { dst[2] = out[2]; dst[3] = out[3]; }
}

/* ---- sinks --------------------------------------------------------------------------------------------------------- */
struct CountSink {
    uint32_t nbits = 0, exceptions = 0;
    NWC_HD void bits(uint32_t, int n) { nbits += (uint32_t)n; }
    NWC_HD void raw1(uint64_t, uint32_t, uint32_t) {}
    NWC_HD void nibble(uint64_t, uint32_t, uint32_t) {}
    NWC_HD void raw2(uint32_t, uint32_t, uint32_t, uint32_t, uint64_t, uint32_t, uint32_t) {}
    NWC_HD bool exception(uint32_t, uint32_t, uint32_t) { if (exceptions == 255u) return false; exceptions++; return true; }
};

struct WriteSink {
    const Geometry &g; int type;
    uint32_t *words; uint8_t *entries; uint8_t *low; uint8_t *raw_plane;
    uint64_t acc = 0; int held = 0; uint32_t exceptions = 0;
    NWC_HD WriteSink(const Geometry &g_, int type_, uint32_t *words_, uint8_t *entries_, uint8_t *low_)
        : g(g_), type(type_), words(words_), entries(entries_), low(low_), raw_plane(low_ + g_.nibble_plane_bytes()) {}
    NWC_HD void bits(uint32_t v, int n) {
        acc = (acc << n) | v; held += n;
        if (held >= 32) { *words++ = (uint32_t)(acc >> (held - 32)); held -= 32; }
    }
    NWC_HD void flush() { if (held) { *words++ = (uint32_t)(acc << (32 - held)); held = 0; } }
    NWC_HD void raw1(uint64_t cell, uint32_t i, uint32_t raw) {
        if (type == kFp8) low[cell * 8u + 4u * ((i >> 3) & 1u) + (i & 3u)] |= (uint8_t)(raw << (4u * ((i >> 2) & 1u)));
        else low[cell * 16u + i] = (uint8_t)raw;
    }
    NWC_HD void nibble(uint64_t cell, uint32_t j, uint32_t v) { low[cell * 8u + (j >> 1)] |= (uint8_t)(v << (4u * (j & 1u))); }
    NWC_HD void raw2(uint32_t rb, uint32_t cb, uint32_t sc, uint32_t L, uint64_t cell, uint32_t j, uint32_t raw) {
        if (type != kFp8) { raw_plane[cell * 16u + j] = (uint8_t)raw; return; }
        const uint32_t bit = 3u * (16u * (sc & 1u) + j), word = bit >> 5, sh = bit & 31u;
        uint32_t *p = reinterpret_cast<uint32_t *>(raw_plane + fixed_fp8_word(g, rb, cb, sc, L, word));
        *p |= raw << sh;
        if (sh > 29u) { uint32_t *p1 = reinterpret_cast<uint32_t *>(raw_plane + fixed_fp8_word(g, rb, cb, sc, L, word + 1u)); *p1 |= raw >> (32u - sh); }
    }
    NWC_HD bool exception(uint32_t index, uint32_t b0, uint32_t b1) {
        uint8_t *e = entries + (uint64_t)exceptions * (type == kFp8 ? 2u : 3u);
        e[0] = (uint8_t)index; e[1] = (uint8_t)b0;
        if (type != kFp8) e[2] = (uint8_t)b1;
        exceptions++;
        return true;
    }
};


/* ---- tables (host) --------------------------------------------------------------------------------------------------- */
inline uint32_t clz32(uint32_t x) { uint32_t n = 0; if (!x) return 32; while (!(x & 0x80000000u)) { x <<= 1; n++; } return n; }


/* Symbol table (psym) from the frequency order; returns the rank table for the device in rank_of[128]. */
inline void build_symbol_tables(const unsigned long long *hist, int type, int layout, uint16_t *psym, uint8_t *rank_of) {
    int order[128];
    const int nsym = type == kFp8 ? (layout == 2 ? 20 : 10) : 128;
    frequency_order(hist, nsym, order);
    for (uint32_t i = 0; i < kSymTableLen; i++) psym[i] = 0;
    if (layout == 2) {
        for (int r = 0; r < 128; r++) rank_of[order[r]] = (uint8_t)(r < (int)kFixedRanks ? r : (int)kFixedRanks);
        for (uint32_t r = 0; r < kFixedRanks; r++) {
            psym[r] = (uint16_t)(type == kFp8 ? fp8_fixed_high(order[r]) : order[r]);
            psym[8 + r] = (uint16_t)(type == kFp8 ? fp8_fixed_bit7(order[r]) : 0);
        }
    } else {
        for (int r = 0; r < 128; r++) rank_of[order[r]] = (uint8_t)r;
        for (uint32_t i = 0; i < 16; i++) psym[i] = (uint16_t)(type == kFp8 ? (i < 10 ? fp8_prefix_high(order[i]) : 0) : order[i]);
    }
}

inline void build_table_words(const uint16_t *psym, int code, uint32_t *lut) {
    if (layout_of(code) == 2) {
        memset(lut, 0, 4 * kTableWords);
        for (int r = 0; r < 8; r++) {
            lut[r >> 2] |= (uint32_t)(psym[r] & 0xFFu) << (8 * (r & 3));
            lut[2 + (r >> 2)] |= (uint32_t)(psym[8 + r] & 0xFFu) << (8 * (r & 3));
        }
        return;
    }
    const uint32_t max_rank = type_of(code) == kFp8 ? 10u : 15u;
    for (uint32_t pattern = 0; pattern < kTableWords; pattern++) {
        const uint32_t window = pattern << (32 - kPeekBits);
        uint32_t used = 0, found = 0, first = 0, byte[2] = {0, 0};
        while (found < 2 && used < kPeekBits) {
            const uint32_t rest = window << used, zeros = clz32(rest);
            if (zeros >= max_rank || zeros + 2 > kPeekBits - used) break;
            byte[found] = (((rest >> (30 - zeros)) & 1u) << 7) | (psym[zeros] & 0x7Fu);
            used += zeros + 2;
            if (!found) first = used;
            found++;
        }
        lut[pattern] = found == 2 ? (used | (byte[0] << 8) | (byte[1] << 16)) : (kEscape | (found ? first : 0u) | (byte[0] << 8) | (found << 24));
    }
    lut[0] = kEscape | ((psym[11] & 0x7Fu) << 8) | ((psym[12] & 0x7Fu) << 16);
    lut[1] = kEscape | ((psym[13] & 0x7Fu) << 8) | ((psym[14] & 0x7Fu) << 16);
}


}  // namespace nwc
