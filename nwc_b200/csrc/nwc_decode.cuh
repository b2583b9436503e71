/* Device-side building blocks of the NWC decoders (sm_100a).
 *
 *   BitWindow      64-bit MSB-first window over a lane's little-endian 32-bit stream words.  Semantics follow the
 *                  reference decoder (csrc/nwc_ops.cu:351-393): `mark` is 2^(empty bits) and rotates with every
 *                  consume; a wrap-around of the rotation means "32 or fewer valid bits left", and the pre-loaded
 *                  next word is then dropped right behind the valid bits with one 64-bit multiply-add.
 *   quad()         the decoder step of this library: TWO 12-bit table look-ups (four symbols) are resolved from the
 *                  high word alone and the window is advanced ONCE by their summed length.  Only when one of the two
 *                  entries is flagged does the lane fall back to pair-at-a-time decoding with the reference's
 *                  per-pair rules (table entry, then count-leading-zeros, then the 24-bit escape).
 *   FixedTables    layout 2: rank -> high byte by PRMT, sign bits moved with one more PRMT.
 *   mma_bf16       m16n8k16 bf16 x bf16 -> fp32: the accumulate step of every matvec kernel here.  A batch-1
 *                  matvec has one right-hand column, so the instruction is used as a wide dot-product engine
 *                  (8 or 16 useful fp32 sums per issue), not as a GEMM tile; tcgen05 / TMEM would add a TMEM round
 *                  trip per 16 weights for no gain at N = 1.
 */
#pragma once
#include <cstdint>
#include <cuda_runtime.h>
#include "nwc_geometry.h"

namespace nwc {

constexpr uint32_t kMaxRankBf16 = 15, kMaxRankFp8 = 10;

__device__ __forceinline__ uint32_t lds32(uint32_t addr) { uint32_t v; asm volatile("ld.shared.u32 %0, [%1];" : "=r"(v) : "r"(addr)); return v; }
__device__ __forceinline__ uint32_t ldg_stream32(const uint32_t *p) { uint32_t v; asm volatile("ld.global.nc.u32 %0, [%1];" : "=r"(v) : "l"(p)); return v; }
__device__ __forceinline__ uint4 ldg_stream128(const void *p) {
    uint4 v; asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p)); return v;
}
__device__ __forceinline__ uint2 ldg_stream64(const void *p) {
    uint2 v; asm volatile("ld.global.nc.L1::no_allocate.v2.u32 {%0,%1}, [%2];" : "=r"(v.x), "=r"(v.y) : "l"(p)); return v;
}
__device__ __forceinline__ uint32_t prmt(uint32_t a, uint32_t b, uint32_t sel) { uint32_t r; asm("prmt.b32 %0, %1, %2, %3;" : "=r"(r) : "r"(a), "r"(b), "r"(sel)); return r; }
__device__ __forceinline__ void prefetch_l2(const void *p) { asm volatile("prefetch.global.L2 [%0];" ::"l"(p)); }

/* byte offset into the 4096-word table of the 12 leading bits of `word` */
__device__ __forceinline__ uint32_t peek_offset(uint32_t word) { return (word >> 18) & 0x3FFCu; }

/* Decoder tables of one CTA in shared memory: [4096 table words][16 bytes symbol-of-rank]. */
constexpr uint32_t kTableSmemBytes = 4u * kTableWords + 16u;

/* Copies the on-disk table into shared memory and rebuilds symbol-of-rank from it: ranks 0..10 from the entries whose
   pattern is "r zeros, a one", ranks 11..14 from entries 0 and 1 (reference: csrc/nwc_ops.cu:407-415). */
__device__ __forceinline__ void stage_tables(uint32_t *smem, const uint32_t *__restrict__ lut, uint32_t tid, uint32_t nthreads) {
    for (uint32_t i = tid; i < kTableWords / 4; i += nthreads) reinterpret_cast<uint4 *>(smem)[i] = __ldg(reinterpret_cast<const uint4 *>(lut) + i);
    if (tid < 16) {
        uint32_t e = 0, shift = 8;
        if (tid < 11) e = __ldg(lut + (1u << (kPeekBits - 1 - tid)));
        else if (tid < 15) { e = __ldg(lut + ((tid - 11) >> 1)); shift = (tid & 1) ? 8 : 16; }
        reinterpret_cast<uint8_t *>(smem + kTableWords)[tid] = (uint8_t)((e >> shift) & 0x7Fu);
    }
    __syncthreads();
}

template <uint32_t MAX_RANK>
struct BitWindow {
    uint32_t hi, lo, next, mark;
    const uint32_t *src;

    __device__ __forceinline__ void open(const uint32_t *words) {
        hi = ldg_stream32(words); lo = ldg_stream32(words + 1); next = ldg_stream32(words + 2);
        mark = 1u; src = words + 3;
    }
    /* drop the `c & 31` leading bits and top the window up */
    __device__ __forceinline__ void consume(uint32_t c) {
        const uint32_t before = mark;
        const uint32_t nhi = __funnelshift_l(lo, hi, c), nlo = __funnelshift_l(0u, lo, c);
        mark = __funnelshift_l(before, before, c);
        const bool refill = mark < before;
        const uint64_t shifted = ((uint64_t)nhi << 32) | nlo;
        const uint64_t merged = (uint64_t)next * (refill ? mark : 0u) + shifted;
        hi = (uint32_t)(merged >> 32); lo = (uint32_t)merged;
        if (refill) { next = ldg_stream32(src); src++; }
    }
    /* one symbol by counting leading zeros: unary rank + sign, or the 24-bit escape (bf16 only) */
    __device__ __forceinline__ uint32_t one(const uint8_t *sym_of_rank) {
        const uint32_t h = hi, zeros = min((uint32_t)__clz((int)h), 15u);
        if (MAX_RANK == kMaxRankFp8 || zeros < MAX_RANK) {
            const uint32_t sign = (h >> (30u - zeros)) & 1u, b = (sign << 7) | sym_of_rank[zeros];
            consume(zeros + 2u);
            return b;
        }
        consume(16u);
        const uint32_t b = hi >> 24;
        consume(8u);
        return b;
    }
    /* two symbols with a window advance of their own: [. | byte0 | byte1 | .] */
    __device__ __forceinline__ uint32_t pair(uint32_t table, const uint8_t *sym_of_rank) {
        const uint32_t e = lds32(table + peek_offset(hi));
        if (e < kEscape) { consume(e); return e; }
        uint32_t b0 = (e >> 8) & 0xFFu;
        if (e & (1u << 24)) consume(e); else b0 = one(sym_of_rank);
        const uint32_t b1 = one(sym_of_rank);
        return (b0 << 8) | (b1 << 16);
    }
    /* four symbols: e01 and e23 carry the high bytes in bytes 1 and 2 */
    __device__ __forceinline__ void quad(uint32_t table, const uint8_t *sym_of_rank, uint32_t &e01, uint32_t &e23) {
        const uint32_t a = lds32(table + peek_offset(hi));
        const uint32_t b = lds32(table + peek_offset(__funnelshift_l(0u, hi, a)));
        if (((a | b) & kEscape) == 0u) { consume(a + b); e01 = a; e23 = b; }
        else { e01 = pair(table, sym_of_rank); e23 = pair(table, sym_of_rank); }
    }
};

/* two bf16 weights in one register: low half = [raw byte r0 | high byte from entry byte 1], high half = [raw byte r0+1 |
   entry byte 2]; FIRST is the index (0 or 2) of the first raw byte inside `raw` */
template <int FIRST>
__device__ __forceinline__ uint32_t weave(uint32_t raw, uint32_t entry) {
    return prmt(raw, entry, FIRST == 0 ? 0x6150u : 0x6352u);
}

/* fp8 raw words: 8 stored bytes hold 16 nibbles; after expansion word w, byte b is (nibble of weight 4w + b) << 4 */
__device__ __forceinline__ uint4 expand_nibbles(uint2 v) {
    return make_uint4((v.x << 4) & 0xF0F0F0F0u, v.x & 0xF0F0F0F0u, (v.y << 4) & 0xF0F0F0F0u, v.y & 0xF0F0F0F0u);
}

__device__ __forceinline__ void mma_bf16(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3]) : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

/* (x1, x0) -> bf16x2 with x0 in the low half, round to nearest even */
__device__ __forceinline__ uint32_t pack_bf16x2(float x1, float x0) { uint32_t r; asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(x1), "f"(x0)); return r; }
/* fp32 pair -> leading bf16x2 part and the bf16x2 of what rounding left over: hi + lo carries ~16 mantissa bits */
__device__ __forceinline__ void split_bf16x2(float x0, float x1, uint32_t &hi, uint32_t &lo) {
    hi = pack_bf16x2(x1, x0);
    lo = pack_bf16x2(x1 - __uint_as_float(hi & 0xFFFF0000u), x0 - __uint_as_float(hi << 16));
}
__device__ __forceinline__ uint16_t bf16_round(float v) {          /* the reference's finalize rounding (no NaN case) */
    uint32_t u = __float_as_uint(v); u += 0x7FFFu + ((u >> 16) & 1u); return (uint16_t)(u >> 16);
}
/* round to nearest even, NaN kept: activations (unlike weights) may overflow */
__device__ __forceinline__ uint16_t bf16_round_nan(float v) {
    uint32_t u = __float_as_uint(v);
    if ((u & 0x7FFFFFFFu) > 0x7F800000u) return (uint16_t)((u >> 16) | 0x40u);
    u += 0x7FFFu + ((u >> 16) & 1u);
    return (uint16_t)(u >> 16);
}
__device__ __forceinline__ float bf16_to_float(uint16_t h) { return __uint_as_float((uint32_t)h << 16); }

/* fp8 e4m3 byte -> fp32 */
__device__ __forceinline__ float fp8_to_float(uint32_t b) {
    const uint32_t s = b >> 7, e = (b >> 3) & 15u, m = b & 7u;
    const float v = e ? __uint_as_float(((e + 120u) << 23) | (m << 20)) : (float)m * 0.001953125f;
    return s ? -v : v;
}

/* ---- layout 2 ------------------------------------------------------------------------------------------------- */
struct FixedTables {
    uint32_t high_lo, high_hi;     /* high byte of rank 0..3 / 4..7 (rank 7 = exception = 0) */
    uint32_t bit7_lo, bit7_hi;     /* fp8: bit 7 of the low byte per rank                     */
    __device__ __forceinline__ void load(const uint32_t *__restrict__ lut) {
        high_lo = __ldg(lut); high_hi = __ldg(lut + 1); bit7_lo = __ldg(lut + 2); bit7_hi = __ldg(lut + 3);
    }
};

/* Four weights from the 16-bit half `HALF` of a nibble word ([sign | rank] per nibble) and their four low bytes:
   out01 / out23 are bf16x2 registers.  `shifted` is `nibbles << 4`, shared by both halves of a word. */
template <int ELEM, int HALF>
__device__ __forceinline__ void fixed_group(const FixedTables &t, uint32_t nibbles, uint32_t shifted, uint32_t lowbytes,
                                            uint32_t &out01, uint32_t &out23) {
    const uint32_t sel = (HALF ? (nibbles >> 16) : nibbles) & 0x7777u;
    const uint32_t signs = prmt(nibbles, shifted, HALF ? 0x3726u : 0x1504u);      /* bit 7 of byte i = sign of weight i */
    const uint32_t high = prmt(t.high_lo, t.high_hi, sel) | (signs & 0x80808080u);
    if (ELEM == kFp8) lowbytes |= prmt(t.bit7_lo, t.bit7_hi, sel);
    out01 = prmt(lowbytes, high, 0x5140u);
    out23 = prmt(lowbytes, high, 0x7362u);
}

/* fp8 layout 2: bits [12g, 12g+12) of the 96-bit little-endian integer (w2:w1:w0): four 3-bit fields (in the low 12 bits
   of the result) */
template <int G>
__device__ __forceinline__ uint32_t field12(uint32_t w0, uint32_t w1, uint32_t w2) {
    constexpr int bit = 12 * G, word = bit >> 5, sh = bit & 31;
    const uint32_t a = word == 0 ? w0 : (word == 1 ? w1 : w2), b = word == 0 ? w1 : (word == 1 ? w2 : 0u);
    return __funnelshift_r(a, b, sh);                            /* bits 12.. are not the field's: spread_fields masks */
}
/* four 3-bit fields (low 12 bits of f, anything above is ignored) -> four bytes (field << 4) */
__device__ __forceinline__ uint32_t spread_fields(uint32_t f) {
    /* two doubling steps (fields 2, 3 to the upper half, then fields 1 and 3 to their bytes): 7 instructions instead of 11 */
    const uint32_t t = (f & 0x03Fu) | ((f & 0xFC0u) << 10);
    return ((t & 0x00070007u) | ((t & 0x00380038u) << 5)) << 4;
}

/* Half a super-chunk of layout 2 (eight weights of one lane, one mma's A fragment).  `word` holds the eight
   [sign | rank] nibbles; the low bytes come from two raw words (bf16) or, for fp8, from the 12-bit field groups G and
   G + 1 of the lane's 96-bit group (f2:f1:f0). */
template <int ELEM, int G>
__device__ __forceinline__ void fixed_half(const FixedTables &t, uint32_t word, uint32_t raw0, uint32_t raw1, uint32_t f0, uint32_t f1, uint32_t f2,
                                           uint32_t &a0, uint32_t &a1, uint32_t &a2, uint32_t &a3) {
    if (ELEM == kFp8) { raw0 = spread_fields(field12<G>(f0, f1, f2)); raw1 = spread_fields(field12<G + 1>(f0, f1, f2)); }
    const uint32_t shifted = word << 4;
    fixed_group<ELEM, 0>(t, word, shifted, raw0, a0, a1);
    fixed_group<ELEM, 1>(t, word, shifted, raw1, a2, a3);
}

/* exclusive prefix sum of one value per lane; `total` receives the warp sum */
__device__ __forceinline__ uint32_t warp_exclusive_sum(uint32_t v, uint32_t lane, uint32_t &total) {
    uint32_t s = v;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) { const uint32_t t = __shfl_up_sync(0xffffffffu, s, o); if (lane >= (uint32_t)o) s += t; }
    total = __shfl_sync(0xffffffffu, s, 31);
    return s - v;
}

}  // namespace nwc
