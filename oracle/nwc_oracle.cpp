/* CPU oracle for the NWC compressed-weight path.  TEST INFRASTRUCTURE ONLY.
 *
 * This file restates, in plain C++ on the CPU, the algorithms of the reference project's kernel library
 * (csrc/nwc_ops.cu) and of its pure-Python format decoder (tests/test_format_cpu.py).  Nothing in the shipped
 * library links, loads or calls it: it exists so that tests, the smoke check and the CPU-baseline leg of the
 * benchmark can compare the CUDA path against an independent implementation of the same format.
 *
 * Parity is pinned: the encoder below is checked byte for byte against the reference encoder compiled from its
 * own sources (oracle/_ref) and against SHA-256 known answers produced by that encoder; the decoder is checked
 * against outputs of the reference's Python decoder stored under tests/golden/.
 *
 * Reference lines each function follows (paths inside the reference project):
 *   geometry            csrc/nwc_ops.cu:87-126      (Shape, raw_bytes, nwc_layout)
 *   fp8 symbol split    csrc/nwc_ops.cu:135-173     (fp8_split, fp8_split2, fp8_hb2, fp8_lb2)
 *   prefix encoder      csrc/nwc_ops.cu:245-320     (nwc_encode, layouts 0 and 1)
 *   fixed-width encoder csrc/nwc_ops.cu:175-243     (encode2, layout 2)
 *   table builder       csrc/nwc_ops.cu:324-348     (nwc_build_tab)
 *   decoder, bf16       tests/test_format_cpu.py:14-111 (exp_of_rank, decode, decode2)
 *   decoder, fp8        csrc/nwc_ops.cu:135-173, 429-442, 615-619, 843-870 and docs/format.md:108-173
 *   finalize rounding   csrc/nwc_ops.cu:553-565     (kern_f32_to_bf16_bias)
 *   gather              csrc/nwc_ops.cu:568-601, 707-745, 985-1042 (output contract only)
 */
#include <cstdint>
#include <cstdlib>
#include <cstring>
#include <vector>
#include <algorithm>

#define ORACLE_API extern "C" __attribute__((visibility("default")))

namespace {

constexpr uint32_t kLanes = 32, kColsPerBlock = 512, kPeekBits = 12, kLutWords = 1u << kPeekBits;
constexpr uint32_t kMaxRankBf16 = 15, kMaxRankFp8 = 10, kMaxRankFixed = 7, kEscapeFlag = 1u << 30;
constexpr uint32_t kSymTableLen = 1024;

inline int elem_type(int code) { return code & 15; }
inline int elem_layout(int code) { return (code >> 4) & 15; }

/* Padded sizes of an M x K matrix in one of the three block layouts. */
struct Geometry {
    uint32_t M, K, rows, K16, Kp, CB, Mp, nb;
    uint32_t last_chunks;      /* coded 16-column chunks in the last column block          */
    uint32_t last_super;       /* 32-column super-chunks in the last column block          */
    uint32_t slots_per_group;  /* super-chunk slots per row group (layouts 1 and 2)        */
    uint32_t pairs_per_group;  /* pairs of super-chunks per row group (layout 2, fp8 raw)  */
    Geometry(uint32_t m, uint32_t k, int layout) : M(m), K(k) {
        rows = layout ? 16u : 8u;
        K16 = (K + 15u) / 16u * 16u;
        Kp = (K + kColsPerBlock - 1) / kColsPerBlock * kColsPerBlock;
        CB = Kp / kColsPerBlock;
        Mp = (M + rows - 1) / rows * rows;
        nb = (Mp / rows) * CB;
        last_chunks = (K16 - (CB - 1) * kColsPerBlock) / 16u;
        last_super = (last_chunks + 1) / 2;
        slots_per_group = 16u * (CB - 1) + last_super;
        pairs_per_group = 8u * (CB - 1) + (last_super + 1) / 2;
    }
    uint32_t chunks_in(uint32_t cb) const { return cb == CB - 1 ? last_chunks : 32u; }
    uint64_t nibble_plane_bytes() const { return (uint64_t)(Mp / 16u) * slots_per_group * kLanes * 8u; }
    uint64_t raw_plane_bytes(int code) const {
        const int t = elem_type(code), lay = elem_layout(code);
        if (lay == 2) {
            const uint64_t raw = t == 1 ? (uint64_t)(Mp / 16u) * pairs_per_group * 3u * kLanes * 4u
                                        : (uint64_t)(Mp / 16u) * slots_per_group * kLanes * 16u;
            return nibble_plane_bytes() + raw;
        }
        if (lay == 1) return (uint64_t)(Mp / 16u) * slots_per_group * kLanes * (t == 1 ? 8u : 16u);
        return t == 1 ? (uint64_t)M * (K16 / 2) : (uint64_t)M * K16;
    }
};

/* Position (row, column) inside a 16 x 32 super-chunk of element i (0..15) of lane L's stream: the order of two
   m16n8k16 A fragments. */
inline uint32_t frag_row(uint32_t L, uint32_t i) { return (L >> 2) + (((i >> 1) & 1u) << 3); }
inline uint32_t frag_col(uint32_t L, uint32_t i) { return ((L & 3u) << 3) + (((i >> 3) & 1u) << 2) + (((i >> 2) & 1u) << 1) + (i & 1u); }

/* ---- fp8 e4m3 helpers -------------------------------------------------------------------------------------- */
const uint8_t kFp8HighByte[10] = {60, 61, 62, 63, 64, 65, 66, 67, 59, 0};   /* bf16 high byte (no sign) per symbol */

/* prefix layouts: fp8 byte -> (symbol 0..9, 4-bit raw nibble). false on NaN. */
bool fp8_to_symbol(uint8_t b, uint8_t &sym, uint8_t &nib) {
    const uint32_t e = (b >> 3) & 15u, m = b & 7u;
    if (e) {
        if (e == 15 && m == 7) return false;
        sym = (uint8_t)(e >> 1); nib = (uint8_t)(((e & 1u) << 3) | m); return true;
    }
    if (m >= 4) { sym = 0; nib = (uint8_t)((m - 4) << 1); }
    else if (m == 0) { sym = 9; nib = 0; }
    else { sym = 8; nib = m == 1 ? 0 : (m == 2 ? 8 : 12); }
    return true;
}
/* fixed-width layout: fp8 byte -> (symbol 0..19, 3-bit field) */
bool fp8_to_symbol_fixed(uint8_t b, uint8_t &sym, uint8_t &field) {
    const uint32_t e = (b >> 3) & 15u, m = b & 7u;
    if (e) {
        if (e == 15 && m == 7) return false;
        sym = (uint8_t)e; field = (uint8_t)m; return true;
    }
    if (m >= 4) { sym = 16; field = (uint8_t)((m - 4) << 1); }
    else if (m >= 2) { sym = 17; field = (uint8_t)((m - 2) << 2); }
    else { sym = m == 1 ? 18 : 19; field = 0; }
    return true;
}
uint8_t fixed_fp8_high(int sym) {
    static const uint8_t t[20] = {0, 60, 61, 61, 62, 62, 63, 63, 64, 64, 65, 65, 66, 66, 67, 67, 60, 59, 59, 0};
    return t[sym];
}
uint8_t fixed_fp8_lowbit(int sym) { return (sym >= 1 && sym <= 15) ? (uint8_t)((sym & 1) << 7) : (uint8_t)(sym == 17 ? 0x80 : 0); }

/* fp8 e4m3 byte -> the same value as bf16 bits (exact) */
uint16_t fp8_to_bf16_bits(uint8_t b) {
    const uint32_t s = b >> 7, e = (b >> 3) & 15u, m = b & 7u;
    if (e) return (uint16_t)((s << 15) | ((e + 120u) << 7) | (m << 4));
    if (m == 0) return (uint16_t)(s << 15);
    /* subnormal m * 2^-9: normalise */
    uint32_t mm = m, ex = 127 - 9;
    int top = 2; while (!((mm >> top) & 1u)) top--;
    ex += top; mm = (mm << (3 - top)) & 7u;            /* 3 fraction bits after the leading one */
    return (uint16_t)((s << 15) | (ex << 7) | (mm << 4));
}

inline float bf16_bits_to_float(uint16_t h) { uint32_t u = (uint32_t)h << 16; float f; memcpy(&f, &u, 4); return f; }
inline uint16_t float_to_bf16_rne(float v) {
    uint32_t u; memcpy(&u, &v, 4);
    u += 0x7FFFu + ((u >> 16) & 1u);
    return (uint16_t)(u >> 16);
}

/* Frequency order of the first `nsym` symbols.  The reference orders them with an in-place exchange pass that swaps
   whenever a later entry is strictly more frequent; ties therefore resolve by that exact swap sequence, not by a stable
   sort, and the encoded streams depend on it. */
void frequency_order(const uint64_t *hist, int nsym, int *order /* [128] */) {
    for (int i = 0; i < 128; i++) order[i] = i;
    for (int a = 0; a < nsym; a++)
        for (int b = a + 1; b < nsym; b++)
            if (hist[order[b]] > hist[order[a]]) std::swap(order[a], order[b]);
}

/* MSB-first bit packer into 32-bit words */
struct BitPacker {
    std::vector<uint32_t> words; uint64_t acc = 0; int held = 0;
    void reset() { words.clear(); acc = 0; held = 0; }
    void put(uint32_t value, int nbits) {
        acc = (acc << nbits) | value; held += nbits;
        while (held >= 32) { words.push_back((uint32_t)(acc >> (held - 32))); held -= 32; }
    }
    void flush() { if (held) { words.push_back((uint32_t)(acc << (32 - held))); held = 0; } }
};

/* split weights into (symbol | sign<<7, raw part).  Returns false on fp8 NaN. */
bool split_planes(const void *w, uint64_t n, int type, bool fixed, std::vector<uint8_t> &high, std::vector<uint8_t> &raw) {
    high.resize(n); raw.resize(n);
    if (type == 1) {
        const uint8_t *p = (const uint8_t *)w;
        for (uint64_t i = 0; i < n; i++) {
            uint8_t s, r;
            if (!(fixed ? fp8_to_symbol_fixed(p[i], s, r) : fp8_to_symbol(p[i], s, r))) return false;
            high[i] = (uint8_t)((p[i] & 0x80u) | s); raw[i] = r;
        }
    } else {
        const uint16_t *p = (const uint16_t *)w;
        for (uint64_t i = 0; i < n; i++) { high[i] = (uint8_t)(p[i] >> 8); raw[i] = (uint8_t)p[i]; }
    }
    return true;
}

int64_t encode_fixed(const void *w, uint64_t n, uint32_t K, int type, uint16_t *psym, uint32_t *bases, uint8_t *hdr,
                     uint8_t *data, uint64_t cap, uint8_t *low) {
    const Geometry g((uint32_t)(n / K), K, 2);
    const int nsym = type == 1 ? 20 : 128, entry = type == 1 ? 2 : 3;
    std::vector<uint8_t> high, raw;
    if (!split_planes(w, n, type, true, high, raw)) return -2;
    uint64_t hist[128] = {0};
    for (uint64_t i = 0; i < n; i++) hist[high[i] & 0x7F]++;
    int order[128]; frequency_order(hist, nsym, order);
    uint8_t rank_of[128];
    for (int r = 0; r < 128; r++) rank_of[order[r]] = (uint8_t)std::min<int>(r, kMaxRankFixed);
    for (uint32_t i = 0; i < kSymTableLen; i++) psym[i] = 0;
    for (uint32_t r = 0; r < kMaxRankFixed; r++) {
        psym[r] = (uint16_t)(type == 1 ? fixed_fp8_high(order[r]) : order[r]);
        psym[8 + r] = (uint16_t)(type == 1 ? fixed_fp8_lowbit(order[r]) : 0);
    }
    const uint64_t nib_bytes = g.nibble_plane_bytes();
    memset(low, 0, g.raw_plane_bytes(type | 32));
    uint8_t *nib = low, *rawp = low + nib_bytes;
    uint64_t pos = 0;
    for (uint32_t b = 0; b < g.nb; b++) {
        const uint32_t rb = b / g.CB, cb = b % g.CB, nsc = (g.chunks_in(cb) + 1) / 2, slot0 = rb * g.slots_per_group + cb * 16;
        pos = (pos + 7) / 8 * 8;
        bases[b] = (uint32_t)pos;
        for (uint32_t L = 0; L < kLanes; L++) {
            uint32_t count = 0;
            for (uint32_t i = 0; i < nsc * 16; i++) {
                const uint32_t sc = i >> 4, j = i & 15;
                const uint32_t row = rb * 16 + frag_row(L, j), col = cb * kColsPerBlock + sc * 32 + frag_col(L, j);
                if (row >= g.M || col >= g.K) continue;
                const uint64_t wi = (uint64_t)row * K + col;
                const uint32_t sign = high[wi] >> 7, rank = rank_of[high[wi] & 0x7F];
                uint8_t value = raw[wi];
                if (rank == kMaxRankFixed) {
                    if (count == 255) return -3;
                    if (pos + (uint64_t)count * entry + entry + 64 > cap) return -1;
                    uint8_t *e = data + pos + (uint64_t)count * entry;
                    e[0] = (uint8_t)i;
                    if (type == 1) e[1] = ((const uint8_t *)w)[wi];
                    else { const uint16_t v = ((const uint16_t *)w)[wi]; e[1] = (uint8_t)v; e[2] = (uint8_t)(v >> 8); }
                    value = 0; count++;
                }
                const uint64_t cell = (uint64_t)(slot0 + sc) * kLanes + L;
                nib[cell * 8 + (j >> 1)] |= (uint8_t)(((sign << 3) | rank) << (4 * (j & 1)));
                if (type == 1) {
                    const uint32_t bit = 3 * (16 * (sc & 1) + j), word = bit >> 5, sh = bit & 31;
                    const uint64_t pair = (uint64_t)rb * g.pairs_per_group + cb * 8 + (sc >> 1);
                    uint8_t *p0 = rawp + ((pair * 3 + word) * kLanes + L) * 4;
                    uint32_t x; memcpy(&x, p0, 4); x |= (uint32_t)value << sh; memcpy(p0, &x, 4);
                    if (sh > 29) { uint8_t *p1 = p0 + kLanes * 4; memcpy(&x, p1, 4); x |= (uint32_t)value >> (32 - sh); memcpy(p1, &x, 4); }
                } else rawp[cell * 16 + j] = value;
            }
            hdr[(uint64_t)b * kLanes + L] = (uint8_t)count;
            pos += (uint64_t)count * entry;
        }
    }
    return (int64_t)((pos + 7) / 8 * 8 + 64);
}

int64_t encode_prefix(const void *w, uint64_t n, uint32_t K, int type, int layout, uint16_t *psym, uint32_t *bases,
                      uint8_t *hdr, uint8_t *data, uint64_t cap, uint8_t *low) {
    const Geometry g((uint32_t)(n / K), K, layout);
    const int nsym = type == 1 ? 10 : 128;
    const uint32_t max_rank = type == 1 ? kMaxRankFp8 : kMaxRankBf16;
    std::vector<uint8_t> high, raw;
    if (!split_planes(w, n, type, false, high, raw)) return -2;
    memset(low, 0, g.raw_plane_bytes(type | (layout << 4)));
    if (layout == 0) {
        for (uint32_t m = 0; m < g.M; m++)
            for (uint32_t k = 0; k < g.K; k++) {
                const uint8_t v = raw[(uint64_t)m * K + k];
                if (type == 1) {
                    const uint32_t j = k & 15;
                    low[(uint64_t)m * (g.K16 / 2) + (k / 16) * 8 + (j & 3) + ((j >> 3) << 2)] |= (uint8_t)(v << (((j >> 2) & 1) ? 4 : 0));
                } else low[(uint64_t)m * g.K16 + k] = v;
            }
    }
    uint64_t hist[128] = {0};
    for (uint64_t i = 0; i < n; i++) hist[high[i] & 0x7F]++;
    int order[128]; frequency_order(hist, nsym, order);
    uint8_t rank_of[128];
    for (int r = 0; r < 128; r++) rank_of[order[r]] = (uint8_t)r;
    for (uint32_t i = 0; i < kSymTableLen; i++) {
        uint16_t v = 0;
        if (i < 16) v = type == 1 ? (uint16_t)(i < 10 ? kFp8HighByte[order[i]] : 0) : (uint16_t)order[i];
        psym[i] = v;
    }
    BitPacker bp; uint64_t pos = 0;
    for (uint32_t b = 0; b < g.nb; b++) {
        const uint32_t rb = b / g.CB, cb = b % g.CB, nchunk = g.chunks_in(cb), slot0 = rb * g.slots_per_group + cb * 16;
        pos = (pos + 7) / 8 * 8;
        bases[b] = (uint32_t)pos;
        const uint32_t per_lane = layout ? ((nchunk + 1) / 2) * 16 : 128u;
        for (uint32_t L = 0; L < kLanes; L++) {
            bp.reset();
            for (uint32_t i = 0; i < per_lane; i++) {
                uint32_t row, col;
                if (layout) { row = rb * 16 + frag_row(L, i & 15); col = cb * kColsPerBlock + (i >> 4) * 32 + frag_col(L, i & 15); }
                else { row = rb * 8 + (i >> 4); col = cb * kColsPerBlock + L * 16 + (i & 15); }
                if (row >= g.M || col >= g.K) { bp.put(2, 2); continue; }
                const uint64_t wi = (uint64_t)row * K + col;
                const uint8_t h = high[wi]; const uint32_t rank = rank_of[h & 0x7F];
                if (rank < max_rank) { bp.put(1, (int)rank + 1); bp.put(h >> 7, 1); }
                else { bp.put(1, 16); bp.put(h, 8); }
                if (layout) {
                    const uint64_t cell = (uint64_t)(slot0 + (i >> 4)) * kLanes + L;
                    if (type == 1) low[cell * 8 + 4 * ((i >> 3) & 1) + (i & 3)] |= (uint8_t)(raw[wi] << (4 * ((i >> 2) & 1)));
                    else low[cell * 16 + (i & 15)] = raw[wi];
                }
            }
            bp.flush();
            const uint64_t nw = bp.words.size();
            if (nw > 255 || pos + 4 * nw + 64 > cap) return -1;
            hdr[(uint64_t)b * kLanes + L] = (uint8_t)nw;
            if (nw) memcpy(data + pos, bp.words.data(), 4 * nw);
            pos += 4 * nw;
        }
    }
    return (int64_t)((pos + 7) / 8 * 8 + 64);
}

uint32_t leading_zeros(uint32_t x) { return x ? (uint32_t)__builtin_clz(x) : 32u; }

/* ---- decoding ------------------------------------------------------------------------------------------------ */
/* symbol table of the prefix layouts, read back from the lookup table the way a loader without psym must */
void ranks_from_lut(const uint32_t *lut, uint8_t *sym_of_rank /* [16] */) {
    for (uint32_t r = 0; r < 11; r++) sym_of_rank[r] = (uint8_t)((lut[1u << (kPeekBits - 1 - r)] >> 8) & 0x7F);
    sym_of_rank[11] = (uint8_t)((lut[0] >> 8) & 0x7F); sym_of_rank[12] = (uint8_t)((lut[0] >> 16) & 0x7F);
    sym_of_rank[13] = (uint8_t)((lut[1] >> 8) & 0x7F); sym_of_rank[14] = (uint8_t)((lut[1] >> 16) & 0x7F);
    sym_of_rank[15] = 0;
}

/* MSB-first reader over little-endian 32-bit words */
struct BitReader {
    const uint8_t *p; uint64_t bitpos = 0;
    explicit BitReader(const uint8_t *start) : p(start) {}
    uint32_t bit() {
        uint32_t w; memcpy(&w, p + 4 * (bitpos >> 5), 4);
        const uint32_t v = (w >> (31 - (bitpos & 31))) & 1u; bitpos++; return v;
    }
    uint32_t bits(int n) { uint32_t v = 0; while (n--) v = (v << 1) | bit(); return v; }
};

/* one prefix-coded high byte (with sign) */
inline uint8_t read_high_byte(BitReader &r, const uint8_t *sym_of_rank, uint32_t max_rank, bool *filler_ok = nullptr) {
    uint32_t zeros = 0;
    while (r.bit() == 0) zeros++;
    if (zeros < max_rank) {
        const uint32_t s = r.bit();
        if (filler_ok) *filler_ok = (zeros == 0 && s == 0);
        return (uint8_t)((s << 7) | sym_of_rank[zeros]);
    }
    if (filler_ok) *filler_ok = false;
    return (uint8_t)r.bits(8);
}

/* Decode one block of a prefix layout into tile[rows][512] (bf16 bits); entries outside the matrix are left 0.
   Returns 0, or -4 if a filler position is not coded as rank 0 / sign 0. */
int decode_block_prefix(const Geometry &g, int type, int layout, const uint8_t *data, const uint32_t *bases,
                        const uint8_t *hdr, const uint8_t *sym_of_rank, const uint8_t *low, uint32_t b, uint16_t *tile) {
    const uint32_t rb = b / g.CB, cb = b % g.CB, nchunk = g.chunks_in(cb), slot0 = rb * g.slots_per_group + cb * 16;
    const uint32_t max_rank = type == 1 ? kMaxRankFp8 : kMaxRankBf16;
    const uint32_t per_lane = layout ? ((nchunk + 1) / 2) * 16 : 128u;
    uint64_t pos = bases[b];
    for (uint32_t L = 0; L < kLanes; L++) {
        BitReader r(data + pos);
        pos += 4ull * hdr[(uint64_t)b * kLanes + L];
        for (uint32_t i = 0; i < per_lane; i++) {
            uint32_t lr, lc;
            if (layout) { lr = frag_row(L, i & 15); lc = (i >> 4) * 32 + frag_col(L, i & 15); }
            else { lr = i >> 4; lc = L * 16 + (i & 15); }
            const uint32_t row = rb * g.rows + lr, col = cb * kColsPerBlock + lc;
            bool filler_ok = false;
            const uint8_t hb = read_high_byte(r, sym_of_rank, max_rank, &filler_ok);
            if (row >= g.M || col >= g.K) { if (!filler_ok) return -4; continue; }
            uint8_t lb;
            if (layout) {
                const uint64_t cell = (uint64_t)(slot0 + (i >> 4)) * kLanes + L;
                if (type == 1) lb = (uint8_t)(((low[cell * 8 + 4 * ((i >> 3) & 1) + (i & 3)] >> (4 * ((i >> 2) & 1))) & 15u) << 4);
                else lb = low[cell * 16 + (i & 15)];
            } else if (type == 1) {
                const uint32_t j = col & 15;
                const uint8_t byte = low[(uint64_t)row * (g.K16 / 2) + (col / 16) * 8 + (j & 3) + ((j >> 3) << 2)];
                lb = (uint8_t)(((byte >> (((j >> 2) & 1) ? 4 : 0)) & 15u) << 4);
            } else lb = low[(uint64_t)row * g.K16 + col];
            tile[lr * kColsPerBlock + lc] = (uint16_t)((hb << 8) | lb);
        }
    }
    return 0;
}

/* Decode one block of the fixed-width layout.  Returns 0, -4 on non-zero filler planes, -5 on a stray exception. */
int decode_block_fixed(const Geometry &g, int type, const uint8_t *data, const uint32_t *bases, const uint8_t *hdr,
                       const uint32_t *lut, const uint8_t *low, uint32_t b, uint16_t *tile) {
    const uint32_t rb = b / g.CB, cb = b % g.CB, nsc = (g.chunks_in(cb) + 1) / 2, slot0 = rb * g.slots_per_group + cb * 16;
    const int entry = type == 1 ? 2 : 3;
    const uint8_t *rawp = low + g.nibble_plane_bytes();
    uint8_t high_of[8], lowbit_of[8];
    for (int r = 0; r < 8; r++) { high_of[r] = (uint8_t)(lut[r >> 2] >> (8 * (r & 3))); lowbit_of[r] = (uint8_t)(lut[2 + (r >> 2)] >> (8 * (r & 3))); }
    uint64_t pos = bases[b];
    for (uint32_t L = 0; L < kLanes; L++) {
        const uint32_t count = hdr[(uint64_t)b * kLanes + L];
        const uint8_t *exc = data + pos; pos += (uint64_t)count * entry;
        uint32_t used = 0;
        for (uint32_t i = 0; i < nsc * 16; i++) {
            const uint32_t sc = i >> 4, j = i & 15, lr = frag_row(L, j), lc = sc * 32 + frag_col(L, j);
            const uint32_t row = rb * 16 + lr, col = cb * kColsPerBlock + lc;
            const uint64_t cell = (uint64_t)(slot0 + sc) * kLanes + L;
            const uint32_t nibble = (low[cell * 8 + (j >> 1)] >> (4 * (j & 1))) & 15u;
            uint32_t rawv;
            if (type == 1) {
                const uint32_t bit = 3 * (16 * (sc & 1) + j), word = bit >> 5, sh = bit & 31;
                const uint64_t pair = (uint64_t)rb * g.pairs_per_group + cb * 8 + (sc >> 1);
                const uint8_t *p0 = rawp + ((pair * 3 + word) * kLanes + L) * 4;
                uint32_t x0, x1 = 0; memcpy(&x0, p0, 4);
                if (sh > 29) memcpy(&x1, p0 + kLanes * 4, 4);
                rawv = (uint32_t)((((uint64_t)x1 << 32) | x0) >> sh) & 7u;
            } else rawv = rawp[cell * 16 + j];
            if (row >= g.M || col >= g.K) { if (nibble || rawv) return -4; continue; }
            const uint32_t sign = nibble >> 3, rank = nibble & 7u;
            uint16_t v;
            if (rank < kMaxRankFixed) {
                if (type == 1) v = (uint16_t)((((sign << 7) | high_of[rank]) << 8) | lowbit_of[rank] | (rawv << 4));
                else v = (uint16_t)((((sign << 7) | high_of[rank]) << 8) | rawv);
            } else {
                /* the lane's exception entries are in stream order; find the one carrying index i */
                const uint8_t *e = nullptr;
                for (uint32_t k = 0; k < count; k++) if (exc[k * entry] == (uint8_t)i) { e = exc + k * entry; break; }
                if (!e || rawv) return -5;
                v = type == 1 ? fp8_to_bf16_bits(e[1]) : (uint16_t)(e[1] | (e[2] << 8));
                used++;
            }
            tile[lr * kColsPerBlock + lc] = v;
        }
        if (used != count) return -5;
    }
    return 0;
}

int decode_block(const Geometry &g, int code, const uint8_t *data, const uint32_t *bases, const uint8_t *hdr,
                 const uint32_t *lut, const uint8_t *sym_of_rank, const uint8_t *low, uint32_t b, uint16_t *tile) {
    const int type = elem_type(code), layout = elem_layout(code);
    if (layout == 2) return decode_block_fixed(g, type, data, bases, hdr, lut, low, b, tile);
    return decode_block_prefix(g, type, layout, data, bases, hdr, sym_of_rank, low, b, tile);
}

}  // namespace

/* ================================================== exports ================================================== */

/* [blocks, raw-plane bytes, scratch floats, K16]; 0 or -1 */
ORACLE_API int nwo_layout(uint64_t M, uint32_t K, int code, uint64_t *out) {
    if (!M || !K || M > 0xFFFFFFFFull) return -1;
    const Geometry g((uint32_t)M, K, elem_layout(code));
    out[0] = g.nb; out[1] = g.raw_plane_bytes(code); out[2] = (uint64_t)g.Mp * g.CB; out[3] = g.K16;
    return 0;
}

/* Host encoder: same outputs and return codes as the reference's nwc_encode (data length incl. 64 bytes of slack,
   -1 shape / capacity / over-long stream, -2 fp8 NaN, -3 more than 255 exceptions in a lane of layout 2). */
ORACLE_API int64_t nwo_encode(const void *w, uint64_t n, uint32_t K, int code, uint16_t *freq, uint16_t *psym,
                              uint32_t *bases, uint8_t *hdr, uint8_t *data, uint64_t cap, uint8_t *low) {
    if (!K || n % K || n / K > 0xFFFFFFFFull) return -1;
    for (uint32_t i = 0; i < kSymTableLen; i++) freq[i] = 0;
    const int type = elem_type(code), layout = elem_layout(code);
    if (layout == 2) return encode_fixed(w, n, K, type, psym, bases, hdr, data, cap, low);
    return encode_prefix(w, n, K, type, layout, psym, bases, hdr, data, cap, low);
}

/* 4096-word decoder table from the symbol table */
ORACLE_API void nwo_build_tab(const uint16_t *psym, int code, uint32_t *lut) {
    if (elem_layout(code) == 2) {
        memset(lut, 0, 4 * kLutWords);
        for (int r = 0; r < 8; r++) {
            lut[r >> 2] |= (uint32_t)(psym[r] & 0xFFu) << (8 * (r & 3));
            lut[2 + (r >> 2)] |= (uint32_t)(psym[8 + r] & 0xFFu) << (8 * (r & 3));
        }
        return;
    }
    const uint32_t max_rank = elem_type(code) == 1 ? kMaxRankFp8 : kMaxRankBf16;
    for (uint32_t pattern = 0; pattern < kLutWords; pattern++) {
        const uint32_t window = pattern << (32 - kPeekBits);
        uint32_t used = 0, found = 0, first_len = 0, byte[2] = {0, 0};
        while (found < 2 && used < kPeekBits) {
            const uint32_t rest = window << used, zeros = leading_zeros(rest);
            if (zeros >= max_rank || zeros + 2 > kPeekBits - used) break;
            const uint32_t sign = (rest >> (30 - zeros)) & 1u;
            byte[found] = (sign << 7) | (psym[zeros] & 0x7Fu);
            used += zeros + 2;
            if (!found) first_len = used;
            found++;
        }
        lut[pattern] = found == 2 ? (used | (byte[0] << 8) | (byte[1] << 16))
                                  : (kEscapeFlag | (found ? first_len : 0u) | (byte[0] << 8) | (found << 24));
    }
    lut[0] = kEscapeFlag | ((psym[11] & 0x7Fu) << 8) | ((psym[12] & 0x7Fu) << 16);
    lut[1] = kEscapeFlag | ((psym[13] & 0x7Fu) << 8) | ((psym[14] & 0x7Fu) << 16);
}

/* Full matrix -> bf16 bits, row-major with row stride K16 (columns K..K16-1 are written as 0).
   fp8 matrices come back as the unscaled fp8 values in bf16.  0 ok, <0 format violation. */
ORACLE_API int nwo_decode(const uint8_t *data, const uint32_t *bases, const uint8_t *hdr, const uint32_t *lut,
                          const uint8_t *low, uint64_t M, uint32_t K, int code, uint16_t *out, int threads) {
    const Geometry g((uint32_t)M, K, elem_layout(code));
    uint8_t sym_of_rank[16]; ranks_from_lut(lut, sym_of_rank);
    int rc = 0;
    (void)threads;
#pragma omp parallel for schedule(dynamic, 16) num_threads(threads > 0 ? threads : 1)
    for (int64_t b = 0; b < (int64_t)g.nb; b++) {
        std::vector<uint16_t> tile(g.rows * kColsPerBlock, 0);
        const int r = decode_block(g, code, data, bases, hdr, lut, sym_of_rank, low, (uint32_t)b, tile.data());
        if (r) {
#pragma omp critical
            rc = r;
            continue;
        }
        const uint32_t rb = (uint32_t)b / g.CB, cb = (uint32_t)b % g.CB;
        for (uint32_t lr = 0; lr < g.rows; lr++) {
            const uint32_t row = rb * g.rows + lr; if (row >= g.M) break;
            for (uint32_t lc = 0; lc < kColsPerBlock; lc++) {
                const uint32_t col = cb * kColsPerBlock + lc; if (col >= g.K16) break;
                out[(uint64_t)row * g.K16 + col] = col < g.K ? tile[lr * kColsPerBlock + lc] : 0;
            }
        }
    }
    return rc;
}

/* y32[i] = sum_k W[i,k] * x[k], fp32 accumulation in ascending k, decoded block by block (the fused CPU path that the
   benchmark times).  x fp32[K]. */
ORACLE_API int nwo_matvec_f32(const uint8_t *data, const uint32_t *bases, const uint8_t *hdr, const uint32_t *lut,
                              const uint8_t *low, const float *x, uint64_t M, uint32_t K, int code, float *y, int threads) {
    const Geometry g((uint32_t)M, K, elem_layout(code));
    uint8_t sym_of_rank[16]; ranks_from_lut(lut, sym_of_rank);
    int rc = 0;
    const int64_t groups = g.Mp / g.rows;
#pragma omp parallel for schedule(dynamic, 4) num_threads(threads > 0 ? threads : 1)
    for (int64_t rb = 0; rb < groups; rb++) {
        std::vector<uint16_t> tile(g.rows * kColsPerBlock);
        float acc[16] = {0};
        for (uint32_t cb = 0; cb < g.CB; cb++) {
            std::fill(tile.begin(), tile.end(), 0);
            const int r = decode_block(g, code, data, bases, hdr, lut, sym_of_rank, low, (uint32_t)rb * g.CB + cb, tile.data());
            if (r) {
#pragma omp critical
                rc = r;
                break;
            }
            const uint32_t ncol = std::min(kColsPerBlock, g.K - cb * kColsPerBlock);
            for (uint32_t lr = 0; lr < g.rows; lr++) {
                float s = acc[lr];
                const uint16_t *t = tile.data() + lr * kColsPerBlock; const float *xv = x + cb * kColsPerBlock;
                for (uint32_t c = 0; c < ncol; c++) s += bf16_bits_to_float(t[c]) * xv[c];
                acc[lr] = s;
            }
        }
        for (uint32_t lr = 0; lr < g.rows; lr++) { const uint64_t row = (uint64_t)rb * g.rows + lr; if (row < g.M) y[row] = acc[lr]; }
    }
    return rc;
}

/* y[i] = bf16_rne(y32[i] * scale[i] + bias[i]) with the reference's hand-rolled rounding (no NaN handling) */
ORACLE_API void nwo_finalize(const float *y32, const uint16_t *bias, const float *scale, uint64_t M, uint16_t *y) {
    for (uint64_t i = 0; i < M; i++) {
        float v = y32[i];
        if (scale) v *= scale[i];
        if (bias) v += bf16_bits_to_float(bias[i]);
        y[i] = float_to_bf16_rne(v);
    }
}

/* rows ids[] -> out[n_ids][K16]; ids outside [0, M) leave their output row untouched */
ORACLE_API int nwo_gather(const uint8_t *data, const uint32_t *bases, const uint8_t *hdr, const uint32_t *lut,
                          const uint8_t *low, const int64_t *ids, uint32_t n_ids, uint64_t M, uint32_t K, int code, uint16_t *out) {
    const Geometry g((uint32_t)M, K, elem_layout(code));
    uint8_t sym_of_rank[16]; ranks_from_lut(lut, sym_of_rank);
    std::vector<uint16_t> tile(g.rows * kColsPerBlock);
    for (uint32_t t = 0; t < n_ids; t++) {
        const int64_t id = ids[t];
        if (id < 0 || id >= (int64_t)g.M) continue;
        const uint32_t rb = (uint32_t)id / g.rows, lr = (uint32_t)id % g.rows;
        for (uint32_t cb = 0; cb < g.CB; cb++) {
            std::fill(tile.begin(), tile.end(), 0);
            const int r = decode_block(g, code, data, bases, hdr, lut, sym_of_rank, low, rb * g.CB + cb, tile.data());
            if (r) return r;
            for (uint32_t lc = 0; lc < kColsPerBlock; lc++) {
                const uint32_t col = cb * kColsPerBlock + lc; if (col >= g.K16) break;
                out[(uint64_t)t * g.K16 + col] = col < g.K ? tile[lr * kColsPerBlock + lc] : 0;
            }
        }
    }
    return 0;
}

/* fp8 e4m3 bytes -> bf16 bits of the same values (used to check fp8 dequantisation) */
ORACLE_API void nwo_fp8_to_bf16(const uint8_t *src, uint64_t n, uint16_t *dst) { for (uint64_t i = 0; i < n; i++) dst[i] = fp8_to_bf16_bits(src[i]); }

/* Plain uncompressed fp8 weight-only matvec (the "native fp8" comparison): y = bf16(scale[i] * sum_k fp8[i,k] x[k]) */
ORACLE_API void nwo_ref_fp8(const uint8_t *w, const float *scale, const float *x, uint64_t M, uint32_t K, uint16_t *y) {
    for (uint64_t i = 0; i < M; i++) {
        float s = 0.f;
        for (uint32_t k = 0; k < K; k++) s += bf16_bits_to_float(fp8_to_bf16_bits(w[i * K + k])) * x[k];
        y[i] = float_to_bf16_rne(s * scale[i]);
    }
}
