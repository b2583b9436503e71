/* Segment kernels of the NWC decode engine (sm_100a): fused batch-1 matvec, dequantisation, fp32 test matvec.
 *
 * Work decomposition.  A matrix is a grid of row groups (8 or 16 rows) x column blocks (512 columns).  The unit a
 * warp owns is a SEGMENT: a run of consecutive column blocks of one row group.  Inside a segment the warp decodes
 * block after block and keeps its fp32 row sums in registers, so a row group that fits one segment is written to
 * y as bf16 directly (scale, bias and rounding fused) with no scratch traffic and no second kernel.  Only matrices
 * with too few row groups to fill the GPU are split along K; those write one fp32 partial per (row, split) and a
 * small finalize kernel adds them in a fixed order, so results are deterministic in every configuration.
 *
 * Arithmetic.  Decoded weights are assembled as bf16x2 registers and multiplied with x by mma.sync m16n8k16
 * (bf16 in, fp32 accumulate) in all three layouts:
 *   - layouts 1 and 2 store their streams in A-fragment order, every lane of a quad holds the same rows, so x enters
 *     as a B fragment whose eight columns are identical and lanes q == 0 end up with the sums of rows r and r + 8;
 *   - layout 0 gives every lane 16 columns of 8 rows.  Two rows at a time are fed as the (row r, row r + 8) halves of
 *     the A fragment and the lane's own x values as its B columns; the diagonal D[r][r] (and D[r + 8][r]) then holds
 *     the quad's dot products of the two rows, which one lane per quad parks in shared memory until the block's
 *     eight rows are complete.
 *   x in fp32 (layout 0 and the fp32 test path) is split into a bf16x2 head and a bf16x2 remainder, two mma each, so
 *   the product keeps ~16 mantissa bits of x.
 *
 * Interfaces replaced (reference: csrc/nwc_ops.cu): kern_block 446-550, kern_block1 632-703, kern_block2 884-981,
 * kern_f32_to_bf16_bias 553-565.
 */
#include <cstdlib>
#include <mutex>
#include <cooperative_groups.h>
#include "nwc_decode.cuh"
#include "nwc_async.cuh"
#include "nwc_launch.h"

namespace nwc {

constexpr int kModeLinear = 0, kModeDequant = 1, kModeAtomic = 2;

/* ---- x fragments ------------------------------------------------------------------------------------------------ */
/* eight consecutive x values as four bf16x2 registers (head) and, for fp32 x, four remainder registers */
template <bool FP32>
struct XFrag8 {
    uint32_t head[4], tail[4];
    __device__ __forceinline__ void load(const void *x, uint32_t col) {
        if (FP32) {
            const float4 a = __ldg(reinterpret_cast<const float4 *>(static_cast<const float *>(x) + col));
            const float4 b = __ldg(reinterpret_cast<const float4 *>(static_cast<const float *>(x) + col + 4));
            split_bf16x2(a.x, a.y, head[0], tail[0]); split_bf16x2(a.z, a.w, head[1], tail[1]);
            split_bf16x2(b.x, b.y, head[2], tail[2]); split_bf16x2(b.z, b.w, head[3], tail[3]);
        } else {
            const uint4 v = __ldg(reinterpret_cast<const uint4 *>(static_cast<const uint16_t *>(x) + col));
            head[0] = v.x; head[1] = v.y; head[2] = v.z; head[3] = v.w;
        }
    }
    /* eight bf16 values from a vector staged in shared memory (bf16 only) */
    __device__ __forceinline__ void load_shared(uint32_t addr) {
        const uint4 v = lds128(addr);
        head[0] = v.x; head[1] = v.y; head[2] = v.z; head[3] = v.w;
    }
    __device__ __forceinline__ void zero() {
#pragma unroll
        for (int i = 0; i < 4; i++) { head[i] = 0u; tail[i] = 0u; }
    }
};

/* ---- output of a finished row ------------------------------------------------------------------------------------- */
template <int MODE>
__device__ __forceinline__ void emit_row(const SegmentArgs &a, uint32_t row, uint32_t split, float v) {
    if (MODE == kModeAtomic) { if (row < a.M) atomicAdd(a.y32 + row, v); return; }
    if (a.splits > 1) { a.y32[(uint64_t)row * a.splits + split] = v; return; }          /* scratch covers padded rows */
    if (row >= a.M) return;
    if (a.scale) v *= __ldg(a.scale + row);
    if (a.bias) v += bf16_to_float(__ldg(a.bias + row));
    a.y[row] = bf16_round(v);
}

/* ---- layout 0 ----------------------------------------------------------------------------------------------------- */
template <int ELEM>
__device__ __forceinline__ uint4 raw_row16(const uint8_t *p, bool ok) {
    if (!ok) return make_uint4(0u, 0u, 0u, 0u);
    if (ELEM == kFp8) return expand_nibbles(ldg_stream64(p));
    return ldg_stream128(p);
}

template <int ELEM, int MODE, bool XF32>
__device__ __forceinline__ void segment_layout0(const SegmentArgs &a, const Geometry &g, uint32_t rb, uint32_t cb0, uint32_t cb1,
                                                uint32_t split, uint32_t lane, uint32_t table, const uint8_t *sym, float *stash) {
    constexpr uint32_t MR = ELEM == kFp8 ? kMaxRankFp8 : kMaxRankBf16;
    const uint32_t r = lane >> 2, q = lane & 3u, row0 = rb * 8u;
    const uint32_t stride = ELEM == kFp8 ? (g.K16 >> 1) : g.K16;
    const bool diag = q == (r >> 1);
    float row_sum = 0.f;                                         /* lanes 0..7: row row0 + lane */
    for (uint32_t cb = cb0; cb < cb1; cb++) {
        const uint32_t b = rb * g.CB + cb, col0 = cb * kBlockCols + lane * 16u;
        const bool col_ok = col0 < g.K16;
        uint32_t total;
        const uint32_t words = __ldg(a.hdr + (uint64_t)b * kLanes + lane), before = warp_exclusive_sum(words, lane, total);
        const uint8_t *stream = a.data + __ldg(a.bases + b);
        if (lane * 32u < total) prefetch_l2(stream + lane * 128u);
        BitWindow<MR> W; W.open(reinterpret_cast<const uint32_t *>(stream) + before);

        XFrag8<XF32> xa, xb;                                    /* columns 0..7 and 8..15 of the lane */
        if (MODE != kModeDequant) {
            if (col_ok) { xa.load(a.x, col0); xb.load(a.x, col0 + 8u); } else { xa.zero(); xb.zero(); }
        }
        const uint8_t *rawp = a.low + (uint64_t)row0 * stride + (ELEM == kFp8 ? (col0 >> 1) : col0);
        uint4 nextA = raw_row16<ELEM>(rawp, col_ok && row0 < g.M), nextB = raw_row16<ELEM>(rawp + stride, col_ok && row0 + 1u < g.M);
#pragma unroll 1
        for (uint32_t rp = 0; rp < 4u; rp++) {
            const uint4 rawA = nextA, rawB = nextB;
            const uint32_t rowA = row0 + 2u * rp;
            if (rp < 3u) {
                nextA = raw_row16<ELEM>(rawp + (uint64_t)(2u * rp + 2u) * stride, col_ok && rowA + 2u < g.M);
                nextB = raw_row16<ELEM>(rawp + (uint64_t)(2u * rp + 3u) * stride, col_ok && rowA + 3u < g.M);
            }
            const uint32_t wa[4] = {rawA.x, rawA.y, rawA.z, rawA.w}, wb[4] = {rawB.x, rawB.y, rawB.z, rawB.w};
            uint32_t pa[8];
#pragma unroll
            for (int k = 0; k < 4; k++) {
                uint32_t e01, e23; W.quad(table, sym, e01, e23);
                pa[2 * k] = weave<0>(wa[k], e01); pa[2 * k + 1] = weave<2>(wa[k], e23);
            }
            if (MODE == kModeDequant) {
                if (col_ok && rowA < g.M) {
                    uint4 *o = reinterpret_cast<uint4 *>(a.out + (uint64_t)rowA * g.K16 + col0);
                    o[0] = make_uint4(pa[0], pa[1], pa[2], pa[3]); o[1] = make_uint4(pa[4], pa[5], pa[6], pa[7]);
                }
            }
            float d[4] = {0.f, 0.f, 0.f, 0.f};
            uint32_t pb[8];
#pragma unroll
            for (int k = 0; k < 4; k++) {
                uint32_t e01, e23; W.quad(table, sym, e01, e23);
                pb[2 * k] = weave<0>(wb[k], e01); pb[2 * k + 1] = weave<2>(wb[k], e23);
                if (MODE != kModeDequant) {
                    const XFrag8<XF32> &xf = k < 2 ? xa : xb;
                    const int w = 2 * (k & 1);
                    mma_bf16(d, pa[2 * k], pb[2 * k], pa[2 * k + 1], pb[2 * k + 1], xf.head[w], xf.head[w + 1]);
                    if (XF32) mma_bf16(d, pa[2 * k], pb[2 * k], pa[2 * k + 1], pb[2 * k + 1], xf.tail[w], xf.tail[w + 1]);
                }
            }
            if (MODE == kModeDequant) {
                if (col_ok && rowA + 1u < g.M) {
                    uint4 *o = reinterpret_cast<uint4 *>(a.out + (uint64_t)(rowA + 1u) * g.K16 + col0);
                    o[0] = make_uint4(pb[0], pb[1], pb[2], pb[3]); o[1] = make_uint4(pb[4], pb[5], pb[6], pb[7]);
                }
            } else if (diag) {                                   /* D[r][r] and D[r+8][r] live in this lane */
                stash[(2u * rp) * 8u + r] = (r & 1u) ? d[1] : d[0];
                stash[(2u * rp + 1u) * 8u + r] = (r & 1u) ? d[3] : d[2];
            }
        }
        if (MODE != kModeDequant) {
            __syncwarp();
            if (lane < 8u) {
                const float4 s0 = *reinterpret_cast<const float4 *>(stash + lane * 8u), s1 = *reinterpret_cast<const float4 *>(stash + lane * 8u + 4u);
                row_sum += ((s0.x + s0.y) + (s0.z + s0.w)) + ((s1.x + s1.y) + (s1.z + s1.w));
            }
            __syncwarp();
        }
    }
    if (MODE != kModeDequant && lane < 8u) emit_row<MODE>(a, row0 + lane, split, row_sum);
}

/* ---- layout 1 ----------------------------------------------------------------------------------------------------- */
template <int MODE>
__device__ __forceinline__ void store_fragment(const SegmentArgs &a, const Geometry &g, uint32_t row0, uint32_t r, uint32_t col,
                                               uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3) {
    if (col >= g.K16) return;                                    /* filler half of the last super-chunk */
    uint16_t *o = a.out + (uint64_t)(row0 + r) * g.K16 + col;
    if (row0 + r < g.M) *reinterpret_cast<uint2 *>(o) = make_uint2(a0, a2);
    if (row0 + r + 8u < g.M) *reinterpret_cast<uint2 *>(o + (uint64_t)8u * g.K16) = make_uint2(a1, a3);
}

template <int ELEM, int MODE, bool XF32>
__device__ __forceinline__ void segment_layout1(const SegmentArgs &a, const Geometry &g, uint32_t rb, uint32_t cb0, uint32_t cb1,
                                                uint32_t split, uint32_t lane, uint32_t table, const uint8_t *sym) {
    constexpr uint32_t MR = ELEM == kFp8 ? kMaxRankFp8 : kMaxRankBf16;
    constexpr uint32_t RB = ELEM == kFp8 ? 8u : 16u;             /* raw bytes per lane and super-chunk */
    const uint32_t r = lane >> 2, q = lane & 3u, row0 = rb * 16u;
    float d[4] = {0.f, 0.f, 0.f, 0.f};
    for (uint32_t cb = cb0; cb < cb1; cb++) {
        const uint32_t b = rb * g.CB + cb, nsc = g.supers_in(cb);
        uint32_t total;
        const uint32_t words = __ldg(a.hdr + (uint64_t)b * kLanes + lane), before = warp_exclusive_sum(words, lane, total);
        const uint8_t *stream = a.data + __ldg(a.bases + b);
        if (lane * 32u < total) prefetch_l2(stream + lane * 128u);
        BitWindow<MR> W; W.open(reinterpret_cast<const uint32_t *>(stream) + before);
        const uint8_t *rp = a.low + ((uint64_t)(rb * g.slots + cb * 16u) * kLanes + lane) * RB;
        uint4 ahead = ELEM == kFp8 ? expand_nibbles(ldg_stream64(rp)) : ldg_stream128(rp);
#pragma unroll 1
        for (uint32_t sc = 0; sc < nsc; sc++) {
            const uint4 cw = ahead;
            rp += kLanes * RB;                                   /* one slot ahead, unguarded: the plane carries 512 B of slack */
            ahead = ELEM == kFp8 ? expand_nibbles(ldg_stream64(rp)) : ldg_stream128(rp);
            const uint32_t kc = cb * kBlockCols + sc * 32u + 8u * q;
            XFrag8<XF32> xf;
            if (MODE != kModeDequant) xf.load(a.x, kc);
            const uint32_t c[4] = {cw.x, cw.y, cw.z, cw.w};
#pragma unroll
            for (int h = 0; h < 2; h++) {
                uint32_t e0, e1, e2, e3;
                W.quad(table, sym, e0, e1); W.quad(table, sym, e2, e3);
                const uint32_t a0 = weave<0>(c[2 * h], e0), a1 = weave<2>(c[2 * h], e1), a2 = weave<0>(c[2 * h + 1], e2), a3 = weave<2>(c[2 * h + 1], e3);
                if (MODE == kModeDequant) store_fragment<MODE>(a, g, row0, r, kc + 4u * h, a0, a1, a2, a3);
                else {
                    mma_bf16(d, a0, a1, a2, a3, xf.head[2 * h], xf.head[2 * h + 1]);
                    if (XF32) mma_bf16(d, a0, a1, a2, a3, xf.tail[2 * h], xf.tail[2 * h + 1]);
                }
            }
        }
    }
    if (MODE != kModeDequant && q == 0u) { emit_row<MODE>(a, row0 + r, split, d[0]); emit_row<MODE>(a, row0 + r + 8u, split, d[2]); }
}

/* ---- layout 2 ----------------------------------------------------------------------------------------------------- */
template <int ELEM, int MODE, bool XF32, int SC_PARITY>
__device__ __forceinline__ void fixed_super_chunk(const SegmentArgs &a, const Geometry &g, const FixedTables &t, uint2 nib, uint4 raw,
                                                  uint32_t f0, uint32_t f1, uint32_t f2, uint32_t row0, uint32_t r, uint32_t kc, float (&d)[4]) {
    XFrag8<XF32> xf;
    if (MODE != kModeDequant) xf.load(a.x, kc);
    const uint32_t c[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
    for (int h = 0; h < 2; h++) {
        uint32_t a0, a1, a2, a3;
        if (h == 0) fixed_half<ELEM, 4 * SC_PARITY>(t, nib.x, c[0], c[1], f0, f1, f2, a0, a1, a2, a3);
        else fixed_half<ELEM, 4 * SC_PARITY + 2>(t, nib.y, c[2], c[3], f0, f1, f2, a0, a1, a2, a3);
        if (MODE == kModeDequant) store_fragment<MODE>(a, g, row0, r, kc + 4u * h, a0, a1, a2, a3);
        else {
            mma_bf16(d, a0, a1, a2, a3, xf.head[2 * h], xf.head[2 * h + 1]);
            if (XF32) mma_bf16(d, a0, a1, a2, a3, xf.tail[2 * h], xf.tail[2 * h + 1]);
        }
    }
}

template <int ELEM, int MODE, bool XF32>
__device__ __forceinline__ void segment_layout2(const SegmentArgs &a, const Geometry &g, uint32_t rb, uint32_t cb0, uint32_t cb1,
                                                uint32_t split, uint32_t lane) {
    constexpr uint32_t ES = ELEM == kFp8 ? 2u : 3u;              /* bytes per exception entry */
    const uint32_t r = lane >> 2, q = lane & 3u, row0 = rb * 16u;
    FixedTables t; t.load(a.lut);
    const uint8_t *raw_plane = a.low + g.nibble_plane_bytes();
    float d[4] = {0.f, 0.f, 0.f, 0.f}, ex_lo = 0.f, ex_hi = 0.f;
    for (uint32_t cb = cb0; cb < cb1; cb++) {
        const uint32_t b = rb * g.CB + cb, nsc = g.supers_in(cb), slot0 = rb * g.slots + cb * 16u;
        const uint8_t *np = a.low + ((uint64_t)slot0 * kLanes + lane) * 8u;
        const uint32_t kbase = cb * kBlockCols + 8u * q;
        if (ELEM == kFp8) {
            const uint8_t *fp = raw_plane + (((uint64_t)rb * g.pair_slots + cb * 8u) * 3u * kLanes + lane) * 4u;
#pragma unroll 1
            for (uint32_t sc = 0; sc < nsc; sc += 2u) {
                const uint32_t f0 = ldg_stream32(reinterpret_cast<const uint32_t *>(fp)), f1 = ldg_stream32(reinterpret_cast<const uint32_t *>(fp + kLanes * 4u)),
                               f2 = ldg_stream32(reinterpret_cast<const uint32_t *>(fp + 2u * kLanes * 4u));
                fp += 3u * kLanes * 4u;
                const uint2 n0 = ldg_stream64(np);
                fixed_super_chunk<ELEM, MODE, XF32, 0>(a, g, t, n0, make_uint4(0u, 0u, 0u, 0u), f0, f1, f2, row0, r, kbase + sc * 32u, d);
                if (sc + 1u < nsc) {
                    const uint2 n1 = ldg_stream64(np + kLanes * 8u);
                    fixed_super_chunk<ELEM, MODE, XF32, 1>(a, g, t, n1, make_uint4(0u, 0u, 0u, 0u), f0, f1, f2, row0, r, kbase + (sc + 1u) * 32u, d);
                }
                np += 2u * kLanes * 8u;
            }
        } else {
            const uint8_t *rp = raw_plane + ((uint64_t)slot0 * kLanes + lane) * 16u;
            uint2 nib_ahead = ldg_stream64(np); uint4 raw_ahead = ldg_stream128(rp);
#pragma unroll 1
            for (uint32_t sc = 0; sc < nsc; sc++) {
                const uint2 nib = nib_ahead; const uint4 raw = raw_ahead;
                np += kLanes * 8u; rp += kLanes * 16u;           /* one slot ahead: covered by the plane's slack */
                nib_ahead = ldg_stream64(np); raw_ahead = ldg_stream128(rp);
                fixed_super_chunk<ELEM, MODE, XF32, 0>(a, g, t, nib, raw, 0u, 0u, 0u, row0, r, kbase + sc * 32u, d);
            }
        }
        /* exceptions of this lane: (stream index, value) entries; their plane entries decoded to +-0 above */
        uint32_t total;
        const uint32_t count = __ldg(a.hdr + (uint64_t)b * kLanes + lane), before = warp_exclusive_sum(count, lane, total);
        if (total) {
            const uint8_t *ep = a.data + __ldg(a.bases + b) + (uint64_t)before * ES;
            for (uint32_t k = 0; k < count; k++, ep += ES) {
                const uint32_t i = ep[0], j = i & 15u, col = cb * kBlockCols + (i >> 4) * 32u + frag_col(lane, j), upper = (j >> 1) & 1u;
                const float w = ELEM == kFp8 ? fp8_to_float(ep[1]) : __uint_as_float(((uint32_t)ep[1] | ((uint32_t)ep[2] << 8)) << 16);
                if (MODE == kModeDequant) { a.out[(uint64_t)(row0 + r + 8u * upper) * g.K16 + col] = (uint16_t)(__float_as_uint(w) >> 16); continue; }
                const float xv = XF32 ? __ldg(static_cast<const float *>(a.x) + col) : bf16_to_float(__ldg(static_cast<const uint16_t *>(a.x) + col));
                if (upper) ex_hi = fmaf(w, xv, ex_hi); else ex_lo = fmaf(w, xv, ex_lo);
            }
        }
    }
    if (MODE != kModeDequant) {
        ex_lo += __shfl_xor_sync(0xffffffffu, ex_lo, 1); ex_lo += __shfl_xor_sync(0xffffffffu, ex_lo, 2);
        ex_hi += __shfl_xor_sync(0xffffffffu, ex_hi, 1); ex_hi += __shfl_xor_sync(0xffffffffu, ex_hi, 2);
        if (q == 0u) { emit_row<MODE>(a, row0 + r, split, d[0] + ex_lo); emit_row<MODE>(a, row0 + r + 8u, split, d[2] + ex_hi); }
    }
}

/* ---- activation vector of a token matvec, built in shared memory --------------------------------------------------- */
/* x (bf16, `cols` values, zero beyond K) comes from one of three sources: a plain vector, the residual stream
   (h_out = h_in + delta, x = RMSNorm(h_out) * w) or a fused gate/up vector (x = silu(gate) * up), with the rounding
   steps of the separate kernels in nwc_model.cu.  Every CTA builds its own copy; CTA 0 writes h_out.  K % 8 == 0 takes
   16-byte vectors (the entry point checks the pointers), other K one value at a time. */
__device__ __forceinline__ float bf16_rt(float v) { return bf16_to_float(bf16_round_nan(v)); }
__device__ __forceinline__ float bf16_lo(uint32_t pair) { return __uint_as_float(pair << 16); }
__device__ __forceinline__ float bf16_hi(uint32_t pair) { return __uint_as_float(pair & 0xFFFF0000u); }
__device__ __forceinline__ uint32_t bf16_pack(float lo, float hi) { return (uint32_t)bf16_round_nan(lo) | ((uint32_t)bf16_round_nan(hi) << 16); }
__device__ __forceinline__ void sts128(uint32_t addr, uint4 v) { asm volatile("st.shared.v4.u32 [%0], {%1,%2,%3,%4};" ::"r"(addr), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w) : "memory"); }

__host__ __device__ __forceinline__ bool norm_like(int mode) { return mode == kInputNorm || mode == kInputPeerNorm; }

__device__ __forceinline__ unsigned long long global_timer_ns() { unsigned long long t; asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t)); return t; }
__device__ __forceinline__ uint4 ld_volatile128(const void *p) {                 /* never from L1: peers rewrite these addresses every other call */
    uint4 v;
    asm volatile("ld.volatile.global.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
    return v;
}

/* kInputPeerNorm: the call number that the words of push slot `in.slot` must carry = this rank's own push count for
   the slot (all ranks make the same sequence of calls; the own push finished before this kernel passed its dependency
   wait). */
__device__ __forceinline__ uint32_t expected_push(const FusedInput &in) {
    return *reinterpret_cast<const volatile uint32_t *>(&reinterpret_cast<const CommControl *>(in.comm)->push_epoch[in.slot]);
}
/* Eight rows of rank r's partial = four 8-byte words {two rows, call number} = two 16-byte loads, repeated until all four
   words carry the expected call number (they normally do at the first look).  Bounded by the global timer: ok = false
   when it runs out. */
__device__ __forceinline__ uint4 pushed_chunk(const uint8_t *words, uint32_t epoch, unsigned long long timeout_ns, bool &ok) {
    uint4 a = ld_volatile128(words), b = ld_volatile128(words + 16);
    auto fresh = [&]() { return (int32_t)(a.y - epoch) >= 0 && (int32_t)(a.w - epoch) >= 0 && (int32_t)(b.y - epoch) >= 0 && (int32_t)(b.w - epoch) >= 0; };
    if (!fresh()) {
        const unsigned long long t0 = global_timer_ns();
        do {
            if (global_timer_ns() - t0 > timeout_ns) { ok = false; break; }
            a = ld_volatile128(words); b = ld_volatile128(words + 16);
        } while (!fresh());
    }
    return make_uint4(a.x, a.z, b.x, b.z);
}

/* two fp32 values -> bf16x2 (first value in the low half), round to nearest even in hardware */
__device__ __forceinline__ uint32_t cvt_pair(float lo, float hi) { return pack_bf16x2(hi, lo); }

/* RMSNorm weights of the chunks a thread owns, kept in registers across the dependency wait */
constexpr uint32_t kNormRegChunks = 4;
struct NormWeights { uint4 w[kNormRegChunks]; bool in_regs; };

/* Before the dependency wait: the RMSNorm weight (a constant).  Vectors of up to kNormRegChunks * 8 * THREADS values stay in
   the registers of the threads that will normalise those chunks (no shared-memory round trip, nothing to wait for before
   griddepcontrol.wait returns); longer ones go to shared memory. */
template <uint32_t THREADS>
__device__ __forceinline__ void stage_norm_weight(const FusedInput &in, uint32_t K, uint16_t *nw, NormWeights &nr) {
    nr.in_regs = false;
    if (!norm_like(in.mode) || (K & 7u) != 0u) return;
    const uint32_t live = K >> 3;
    if (live <= kNormRegChunks * THREADS) {
        nr.in_regs = true;
#pragma unroll
        for (uint32_t i = 0; i < kNormRegChunks; i++) {
            const uint32_t c = threadIdx.x + i * THREADS;
            nr.w[i] = c < live ? __ldg(reinterpret_cast<const uint4 *>(in.norm_w) + c) : make_uint4(0u, 0u, 0u, 0u);
        }
        return;
    }
    const uint32_t nw_addr = smem_addr(nw);
    for (uint32_t c = threadIdx.x; c < live; c += THREADS) sts128(nw_addr + c * 16u, __ldg(reinterpret_cast<const uint4 *>(in.norm_w) + c));
}

/* eight values of h_in + delta (delta = a local vector, or the sum of the ranks' pushed partials in rank order), rounded to
   bf16 as the residual stream is: four bf16x2 words; *ss gets the sum of their squares in element order */
__device__ __forceinline__ void residual_chunk(const FusedInput &in, bool peer, uint32_t epoch, uint32_t K, uint32_t c, uint32_t (&out)[4], float &ss, bool &ok) {
    const uint4 h = *(reinterpret_cast<const uint4 *>(in.h_in) + c);
    const uint32_t hw[4] = {h.x, h.y, h.z, h.w};
    if (peer) {                                                  /* all loads in flight before the first add */
        uint4 part[kCommMaxRanks];
#pragma unroll
        for (uint32_t r = 0; r < kCommMaxRanks; r++)
            part[r] = r < in.world ? pushed_chunk(in.comm + comm_push_offset(K, in.slot, r) + (uint64_t)c * 32u, epoch, in.timeout_ns, ok) : make_uint4(0u, 0u, 0u, 0u);
        float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
#pragma unroll
        for (uint32_t r = 0; r < kCommMaxRanks; r++) {
            if (r < in.world) {
                const uint32_t pw[4] = {part[r].x, part[r].y, part[r].z, part[r].w};
#pragma unroll
                for (int k = 0; k < 4; k++) { acc[2 * k] += bf16_lo(pw[k]); acc[2 * k + 1] += bf16_hi(pw[k]); }
            }
        }
#pragma unroll
        for (int k = 0; k < 4; k++) {
            const uint32_t d = cvt_pair(acc[2 * k], acc[2 * k + 1]);               /* the sum is a bf16 vector, like a local delta */
            out[k] = cvt_pair(bf16_lo(hw[k]) + bf16_lo(d), bf16_hi(hw[k]) + bf16_hi(d));
        }
    } else if (in.delta) {
        const uint4 d = *(reinterpret_cast<const uint4 *>(in.delta) + c);
        const uint32_t dw[4] = {d.x, d.y, d.z, d.w};
#pragma unroll
        for (int k = 0; k < 4; k++) out[k] = cvt_pair(bf16_lo(hw[k]) + bf16_lo(dw[k]), bf16_hi(hw[k]) + bf16_hi(dw[k]));
    } else {
#pragma unroll
        for (int k = 0; k < 4; k++) out[k] = hw[k];
    }
#pragma unroll
    for (int k = 0; k < 4; k++) { const float v0 = bf16_lo(out[k]), v1 = bf16_hi(out[k]); ss += v0 * v0; ss += v1 * v1; }
}

/* x = bf16(weight * bf16(h * inv)) for eight values */
__device__ __forceinline__ uint4 normalised_chunk(const uint32_t (&h)[4], uint4 weight, float inv) {
    const uint32_t ww[4] = {weight.x, weight.y, weight.z, weight.w};
    uint32_t o[4];
#pragma unroll
    for (int k = 0; k < 4; k++) {
        const uint32_t n = cvt_pair(bf16_lo(h[k]) * inv, bf16_hi(h[k]) * inv);
        o[k] = cvt_pair(bf16_lo(ww[k]) * bf16_lo(n), bf16_hi(ww[k]) * bf16_hi(n));
    }
    return make_uint4(o[0], o[1], o[2], o[3]);
}

/* distributed shared memory of a thread-block cluster */
__device__ __forceinline__ uint32_t cluster_addr(uint32_t local, uint32_t cta) {
    uint32_t r;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(local), "r"(cta));
    return r;
}
__device__ __forceinline__ void cluster_sts128(uint32_t addr, uint4 v) {
    asm volatile("st.shared::cluster.v4.u32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w) : "memory");
}
__device__ __forceinline__ void cluster_sts64(uint32_t addr, float a, float b) {
    asm volatile("st.shared::cluster.v2.f32 [%0], {%1, %2};" ::"r"(addr), "f"(a), "f"(b) : "memory");
}
__device__ __forceinline__ void cluster_arrive() { asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory"); }
__device__ __forceinline__ void cluster_wait() { asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory"); }

/* kInputPeerNorm when the launch runs clusters of `ctas` CTAs (FusedInput::share).  Every CTA of a launch needs the whole
   vector h = h_in + the ranks' partials, and with one CTA per SM every SM would pull world x 4 K bytes out of L2 for it:
   at 8 ranks that is 38 MB per launch from the same few lines, 7 to 8 us.  Here CTA `rank` of a cluster adds up chunks
   [rank, rank + 1) * live / ctas only and stores the sums, and its warps' sums of squares, into the shared memory of
   every CTA of the cluster; after one cluster barrier each CTA normalises its own copy.  The caller has made every
   thread arrive at the cluster barrier once (at the kernel's top): the wait for that arrival, after the loads, is what
   guarantees that the other CTAs run before their shared memory is written.  cl: ctas * THREADS / 32 pairs of floats
   {sum of squares, 1 = all of the warp's words arrived}.  Needs the RMSNorm weight in registers (nr.in_regs) and
   live % ctas == 0.  The sum of squares is added in another order than build_activation adds it (lane-strided, then a
   butterfly), the same one in every CTA of every rank.  Ends with __syncthreads(). */
template <uint32_t THREADS>
__device__ __forceinline__ void build_activation_shared(const FusedInput &in, uint32_t K, uint32_t cols, uint16_t *xs, float *cl, const NormWeights &nr,
                                                        uint32_t ctas, uint32_t rank, bool first_cluster) {
    const uint32_t tid = threadIdx.x, lane = tid & 31u, warp = tid >> 5;
    const uint32_t xs_addr = smem_addr(xs), cl_addr = smem_addr(cl), chunks = cols >> 3, live = K >> 3, per = live / ctas;
    const uint32_t epoch = expected_push(in);
    const bool write_h = first_cluster && in.h_out != nullptr;
    bool ok = true;
    float ss = 0.f;
    uint32_t held[kNormRegChunks][4];
#pragma unroll
    for (uint32_t i = 0; i < kNormRegChunks; i++) {
        const uint32_t j = tid + i * THREADS;
        if (j < per) {
            const uint32_t c = rank * per + j;
            residual_chunk(in, true, epoch, K, c, held[i], ss, ok);
            if (write_h) *(reinterpret_cast<uint4 *>(in.h_out) + c) = make_uint4(held[i][0], held[i][1], held[i][2], held[i][3]);
        }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
    const bool warp_ok = __all_sync(0xffffffffu, ok);
    cluster_wait();                                              /* every CTA of the cluster has started */
#pragma unroll
    for (uint32_t i = 0; i < kNormRegChunks; i++) {
        const uint32_t j = tid + i * THREADS;
        if (j < per) {
            const uint32_t at = xs_addr + (rank * per + j) * 16u;
            const uint4 v = make_uint4(held[i][0], held[i][1], held[i][2], held[i][3]);
            for (uint32_t r = 0; r < ctas; r++) cluster_sts128(cluster_addr(at, r), v);
        }
    }
    if (lane == 0)
        for (uint32_t r = 0; r < ctas; r++) cluster_sts64(cluster_addr(cl_addr + (rank * (THREADS / 32u) + warp) * 8u, r), ss, warp_ok ? 1.f : 0.f);
    __syncwarp();
    cluster_arrive();
    cluster_wait();
    float tot = 0.f;
    bool good = true;
    for (uint32_t e = lane; e < ctas * (THREADS / 32u); e += 32u) {
        const float2 v = *reinterpret_cast<const float2 *>(cl + 2u * e);
        tot += v.x;
        good = good && v.y != 0.f;
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) tot += __shfl_xor_sync(0xffffffffu, tot, o);
    if (!__all_sync(0xffffffffu, good)) {                        /* a rank is missing (every CTA of the cluster sees it): poison x */
        if (tid == 0) atomicExch(&g_kernel_status, kStatusPeerTimeout);
        for (uint32_t c = tid; c < chunks; c += THREADS) sts128(xs_addr + c * 16u, make_uint4(0x7FC07FC0u, 0x7FC07FC0u, 0x7FC07FC0u, 0x7FC07FC0u));
        __syncthreads();
        return;
    }
    const float inv = rsqrtf(tot / (float)K + in.eps);
#pragma unroll
    for (uint32_t i = 0; i < kNormRegChunks; i++) {
        const uint32_t c = tid + i * THREADS;
        if (c < live) {
            const uint4 v = lds128(xs_addr + c * 16u);
            const uint32_t vw[4] = {v.x, v.y, v.z, v.w};
            sts128(xs_addr + c * 16u, normalised_chunk(vw, nr.w[i], inv));
        }
    }
    for (uint32_t c = live + tid; c < chunks; c += THREADS) sts128(xs_addr + c * 16u, make_uint4(0u, 0u, 0u, 0u));
    __syncthreads();
}

/* after the dependency wait; ends with __syncthreads().  scal: THREADS / 32 floats of shared memory. */
template <uint32_t THREADS>
__device__ __forceinline__ void build_activation(const FusedInput &in, const void *x, uint32_t K, uint32_t cols, uint16_t *xs, uint16_t *nw, float *scal,
                                                 const NormWeights &nr) {
    const uint32_t tid = threadIdx.x, lane = tid & 31u, warp = tid >> 5;
    const uint32_t xs_addr = smem_addr(xs), nw_addr = smem_addr(nw), chunks = cols >> 3, live = K >> 3;   /* chunks of eight values */
    const bool vec = (K & 7u) == 0u;
    if (norm_like(in.mode)) {
        const bool peer = in.mode == kInputPeerNorm;             /* (the entry point admits this mode only with K % 8 == 0) */
        const uint32_t epoch = peer ? expected_push(in) : 0u;
        bool ok = true;
        const bool write_h = blockIdx.x == 0 && in.h_out != nullptr;
        float ss = 0.f;
        uint32_t held[kNormRegChunks][4];                        /* register path: the thread's chunks of h_out */
        if (vec && nr.in_regs) {
#pragma unroll
            for (uint32_t i = 0; i < kNormRegChunks; i++) {
                const uint32_t c = tid + i * THREADS;
                if (c < live) {
                    residual_chunk(in, peer, epoch, K, c, held[i], ss, ok);
                    if (write_h) *(reinterpret_cast<uint4 *>(in.h_out) + c) = make_uint4(held[i][0], held[i][1], held[i][2], held[i][3]);
                }
            }
        } else if (vec) {
            for (uint32_t c = tid; c < live; c += THREADS) {
                uint32_t o[4];
                residual_chunk(in, peer, epoch, K, c, o, ss, ok);
                if (write_h) *(reinterpret_cast<uint4 *>(in.h_out) + c) = make_uint4(o[0], o[1], o[2], o[3]);
                sts128(xs_addr + c * 16u, make_uint4(o[0], o[1], o[2], o[3]));
            }
        } else {
            for (uint32_t i = tid; i < K; i += THREADS) {
                float v = bf16_to_float(in.h_in[i]);
                if (in.delta) v = bf16_rt(v + bf16_to_float(in.delta[i]));
                if (write_h) in.h_out[i] = bf16_round_nan(v);
                xs[i] = bf16_round_nan(v);
                ss += v * v;
            }
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
        if (lane == 0) scal[warp] = ss;
        if (!__syncthreads_and(ok)) {                            /* a rank is missing: poison x so that nothing downstream looks valid */
            if (tid == 0) atomicExch(&g_kernel_status, kStatusPeerTimeout);
            for (uint32_t c = tid; c < chunks; c += THREADS) sts128(xs_addr + c * 16u, make_uint4(0x7FC07FC0u, 0x7FC07FC0u, 0x7FC07FC0u, 0x7FC07FC0u));
            __syncthreads();
            return;
        }
        float tot = 0.f;
        for (uint32_t i = 0; i < THREADS / 32u; i++) tot += scal[i];
        const float inv = rsqrtf(tot / (float)K + in.eps);
        if (vec && nr.in_regs) {
#pragma unroll
            for (uint32_t i = 0; i < kNormRegChunks; i++) {
                const uint32_t c = tid + i * THREADS;
                if (c < live) sts128(xs_addr + c * 16u, normalised_chunk(held[i], nr.w[i], inv));
            }
            for (uint32_t c = live + tid; c < chunks; c += THREADS) sts128(xs_addr + c * 16u, make_uint4(0u, 0u, 0u, 0u));
        } else if (vec) {
            for (uint32_t c = tid; c < chunks; c += THREADS) {   /* each thread re-reads the chunks it wrote itself */
                uint4 o = make_uint4(0u, 0u, 0u, 0u);
                if (c < live) {
                    const uint4 v = lds128(xs_addr + c * 16u);
                    const uint32_t vw[4] = {v.x, v.y, v.z, v.w};
                    o = normalised_chunk(vw, lds128(nw_addr + c * 16u), inv);
                }
                sts128(xs_addr + c * 16u, o);
            }
        } else {
            for (uint32_t i = tid; i < cols; i += THREADS)
                xs[i] = i < K ? bf16_round_nan(bf16_to_float(in.norm_w[i]) * bf16_rt(bf16_to_float(xs[i]) * inv)) : (uint16_t)0;
        }
    } else if (in.mode == kInputSwiglu) {
        if (vec) {                                               /* eight values per step; exponentials and quotients by the fast hardware paths */
            const uint4 *gate = reinterpret_cast<const uint4 *>(in.gate_up), *up = reinterpret_cast<const uint4 *>(in.gate_up + K);
#pragma unroll 2
            for (uint32_t c = tid; c < chunks; c += THREADS) {
                uint4 o = make_uint4(0u, 0u, 0u, 0u);
                if (c < live) {
                    const uint4 gv = gate[c], uv = up[c];
                    const uint32_t gw[4] = {gv.x, gv.y, gv.z, gv.w}, uw[4] = {uv.x, uv.y, uv.z, uv.w};
                    uint32_t ow[4];
#pragma unroll
                    for (int k = 0; k < 4; k++) {
                        const float g0 = bf16_lo(gw[k]), g1 = bf16_hi(gw[k]);
                        const uint32_t act = cvt_pair(__fdividef(g0, 1.f + __expf(-g0)), __fdividef(g1, 1.f + __expf(-g1)));
                        ow[k] = cvt_pair(bf16_lo(act) * bf16_lo(uw[k]), bf16_hi(act) * bf16_hi(uw[k]));
                    }
                    o = make_uint4(ow[0], ow[1], ow[2], ow[3]);
                }
                sts128(xs_addr + c * 16u, o);
            }
        } else {
            for (uint32_t i = tid; i < cols; i += THREADS) {
                uint16_t v = 0;
                if (i < K) { const float gt = bf16_to_float(in.gate_up[i]), up = bf16_to_float(in.gate_up[K + i]); v = bf16_round_nan(bf16_rt(gt / (1.f + __expf(-gt))) * up); }
                xs[i] = v;
            }
        }
    } else if (vec) {
        for (uint32_t c = tid; c < chunks; c += THREADS)
            sts128(xs_addr + c * 16u, c < live ? *(reinterpret_cast<const uint4 *>(x) + c) : make_uint4(0u, 0u, 0u, 0u));
    } else {
        for (uint32_t i = tid; i < cols; i += THREADS) xs[i] = i < K ? static_cast<const uint16_t *>(x)[i] : (uint16_t)0;
    }
    __syncthreads();
}

/* ---- layout 2, token path, bf16: planes streamed through a per-warp ring of bulk copies ------------------------------ */
/* Work split.  The matrix is one flat sequence of super-chunk slots (row-group-major; both planes are contiguous in that
   order).  Every CTA of the grid (one per SM) takes a contiguous run of slots and its warps split that run evenly.  A
   warp writes a row group it covers alone straight to the output; the row groups it shares with other warps of the CTA
   (at most its first and its last one) are added up in shared memory in warp order.  The CTA runs are whole row groups
   when that leaves little imbalance (one launch, bf16 y written here); otherwise they are equal runs of slots, a row
   group cut by a CTA boundary gets one fp32 partial per CTA in the caller's scratch and finalize_flat_kernel adds them.
   Data path.  A stage holds kRingSlots slots of both planes (256 B of nibbles and 512 B of low bytes per slot, each slot
   lane-contiguous) and every warp keeps kRingStages stages in flight.  Measured on B200 (4096 x 4096 up to
   151936 x 2560): 16 warps with 6-slot stages beat 32 warps with 2- or 3-slot stages and 8 warps with 12-slot stages,
   because the per-stage work (barrier wait, refill, bulk-copy operands) is issue-slot cost, not hidden latency. */
constexpr uint32_t kRingThreads = 512, kRingSlots = 6, kRingStages = 2, kRingCtasPerSm = 1;
constexpr uint32_t kRingStageBytes = kRingSlots * (256u + 512u);
constexpr uint32_t kRingWarpBytes = kRingStages * kRingStageBytes;
constexpr uint32_t kRingBarrierBytes = (kRingThreads / 32u) * kRingStages * 8u;
constexpr uint32_t kRingMaxSmem = 232448u;                       /* 227 KB opt-in limit of a CTA */
/* shared memory of the layout-2 ring kernel: x (32 columns per slot, bf16), the barriers, then the per-warp rings */
__host__ __device__ static inline uint32_t ring_x_bytes(const Geometry &g) { return (g.slots * 64u + 127u) & ~127u; }
static inline uint32_t ring_smem_bytes(const Geometry &g, int input_mode = kInputPlain) { return (norm_like(input_mode) ? 2u : 1u) * ring_x_bytes(g) + 2u * (kRingThreads / 32u) * 68u + 256u + kRingBarrierBytes + (kRingThreads / 32u) * kRingWarpBytes; }

/* CTAs of the layout-2 ring kernel the launcher plans for: kRingCtasPerSm per SM while that many fit an SM's shared memory
   side by side (each CTA also costs the SM 1 KB of bookkeeping), otherwise one per SM */
/* the layout-2 ring kernel covers bf16, and fp8 matrices whose row groups hold an even number of slots (K % 64 in [1, 32] is
   the exception: its last pair would straddle two row groups) */
static inline bool ring_covers(int code, const Geometry &g, int input_mode) {
    if (layout_of(code) != 2 || ring_smem_bytes(g, input_mode) > kRingMaxSmem || (uint64_t)g.groups * g.slots >= (1ull << 31)) return false;
    return type_of(code) == kBf16 || (g.slots & 1u) == 0u;
}
static inline int ring_ctas(const Geometry &g, int input_mode, int sms) {
    const uint32_t per_cta = ring_smem_bytes(g, input_mode) + 1024u;
    return sms * (int)(per_cta * kRingCtasPerSm <= 233472u ? kRingCtasPerSm : 1u);
}

/* n / d for 32-bit n and a divisor fixed on the host: one multiply-high, one add, one shift (the kernels' index
   arithmetic sits on the critical path of launches that last a few microseconds; a hardware-less 64-bit division costs
   hundreds of cycles there).  m = ceil(2^(32 + s) / d) - 2^32 with s = ceil(log2 d). */
struct FastDiv {
    uint32_t d, m, s;
    void set(uint32_t divisor) {
        d = divisor ? divisor : 1u;
        s = 0; while ((1ull << s) < d) s++;
        m = (uint32_t)((((1ull << (32u + s)) + d - 1u) / d) - (1ull << 32));
    }
    __host__ __device__ __forceinline__ uint32_t div(uint32_t n) const {
#if defined(__CUDA_ARCH__)
        return (uint32_t)(((uint64_t)__umulhi(n, m) + n) >> s);
#else
        return (uint32_t)(((((uint64_t)n * m) >> 32) + n) >> s);
#endif
    }
};

/* Contiguous runs of `chunks` pieces of work for `warps` workers: chunks = q * warps + r, worker w owns q + (w < r) chunks
   starting at chunk w * q + min(w, r).  All counts fit 32 bits (the launchers check). */
struct FlatPlan {
    uint32_t units_per_group;   /* slots (layout 2; fp8: slot pairs) or blocks (layouts 0, 1) per row group             */
    uint32_t grain;             /* run boundaries are multiples of this many units (a whole row group when CB == 1)      */
    uint32_t chunks;            /* total units / grain                                                                 */
    uint32_t warps;             /* workers that take part                                                               */
    uint32_t parts;             /* row stride of the partial sums = most workers that can share a row group             */
    uint32_t direct;            /* 1: no row group is cut, workers write y themselves                                    */
    uint32_t fix;               /* 1 (layout 2 ring kernel, direct == 0): a cut row group is completed inside the kernel by
                                   the CTA that arrives last at the group's counter, no finalize launch                   */
    uint32_t q, r;
    FastDiv by_grain, by_q, by_q1, by_group;
    void finish() { q = chunks / warps; r = chunks % warps; by_grain.set(grain); by_q.set(q); by_q1.set(q + 1u); by_group.set(units_per_group); }
    __host__ __device__ __forceinline__ uint32_t start(uint32_t w) const { return (w * q + (w < r ? w : r)) * grain; }
    /* the worker whose run holds unit u */
    __host__ __device__ __forceinline__ uint32_t owner(uint32_t u) const {
        const uint32_t c = by_grain.div(u), split = r * (q + 1u);
        return c < split ? by_q1.div(c) : r + by_q.div(c - split);
    }
    /* the row group that holds unit u */
    __host__ __device__ __forceinline__ uint32_t group_of(uint32_t u) const { return by_group.div(u); }
};

__device__ __forceinline__ void emit_flat(const SegmentArgs &a, const FlatPlan &p, uint32_t row, uint32_t part, float v) {
    if (!p.direct) { a.y32[(uint64_t)row * p.parts + part] = v; return; }
    if (row >= a.M) return;
    if (a.scale) v *= __ldg(a.scale + row);
    if (a.bias) v += bf16_to_float(__ldg(a.bias + row));
    a.y[row] = bf16_round(v);
}

/* Equal runs per CTA cut row groups.  Entry i: the 16 row sums (fp32 bits) of the part of its FIRST row group that CTA i
   holds when that group began in an earlier CTA's run; kCutEmpty (a NaN pattern no sum is allowed to keep) = nothing
   there.  Written by CTA i, read and emptied by the CTA where the group begins; empty between kernels.  One set per
   device, so launches that use such plans must be in stream order on their device. */
constexpr uint32_t kFixCounters = 1024;                          /* most CTAs of such a launch */
constexpr uint32_t kCutEmpty = 0xFFFFFFFFu;
constexpr unsigned long long kCutWaitNs = 2000000000ull;         /* longest wait for another CTA's part */
static __device__ unsigned int g_cut_part[kFixCounters][16];

/* The 16 finished rows of row group `grp`, one per lane of a half-warp (`sub` = lane & 15 = row inside the group, `mask`
   = the 16 lanes, all of which make this call): scale, bias and bf16 rounding as the reference's finalize step, then
   either the local y or, for a row-parallel matrix of a tensor-parallel group, the push slot of EVERY rank's exchange
   buffer (plain 4-byte stores over NVLink, two rows each; the flag that publishes them is raised at the kernel's end). */
__device__ __forceinline__ void emit_group(const SegmentArgs &a, uint32_t grp, uint32_t sub, float v, uint32_t mask, uint32_t push_call) {
    const uint32_t row = grp * 16u + sub;
    const bool live = row < a.M;
    if (live && a.scale) v *= __ldg(a.scale + row);
    if (live && a.bias) v += bf16_to_float(__ldg(a.bias + row));
    const uint32_t h = live ? (uint32_t)bf16_round_nan(v) : 0u;        /* (the reference's rounding for every finite value; NaN stays NaN) */
    if (a.push.world == 0u) { if (live) a.y[row] = (uint16_t)h; return; }
    const uint32_t pair = h | (__shfl_down_sync(mask, h, 1) << 16);
    if ((sub & 1u) == 0u && live) {
        const uint64_t off = comm_push_offset(a.push.H, a.push.slot, a.push.rank) + (uint64_t)(row >> 1) * 8u;
#pragma unroll
        for (uint32_t p = 0; p < kCommMaxRanks; p++)
            if (p < a.push.world) asm volatile("st.volatile.global.v2.u32 [%0], {%1, %2};" ::"l"(a.push.buf[p] + off), "r"(pair), "r"(push_call) : "memory");
    }
}

/* Exceptions of one block (column block cb) for this lane: sum of value * x over the lane's `count` entries at `ep`, split
   by fragment half.  Called once per 16 slots, so it stays out of line to keep the slot loop short. */
template <int ELEM>
__device__ __noinline__ float2 ring_exceptions(uint32_t count, const uint8_t *__restrict__ ep, uint32_t xs, uint32_t cb, uint32_t lane) {
    constexpr uint32_t ES = ELEM == kFp8 ? 2u : 3u;              /* bytes per entry: stream index, then the fp8 byte or the bf16 value */
    float lo = 0.f, hi = 0.f;
    if (__any_sync(0xffffffffu, count != 0u)) {
        for (uint32_t k = 0; k < count; k++, ep += ES) {
            const uint32_t i = ep[0], jj = i & 15u, col = cb * kBlockCols + (i >> 4) * 32u + frag_col(lane, jj);
            const float wv = ELEM == kFp8 ? fp8_to_float(ep[1]) : __uint_as_float(((uint32_t)ep[1] | ((uint32_t)ep[2] << 8)) << 16);
            uint16_t xb;
            asm volatile("ld.shared.u16 %0, [%1];" : "=h"(xb) : "r"(xs + col * 2u));
            const float xv = bf16_to_float(xb);
            if ((jj >> 1) & 1u) hi = fmaf(wv, xv, hi); else lo = fmaf(wv, xv, lo);
        }
    }
    return make_float2(lo, hi);
}

/* What the ring kernel that FOLLOWS this launch on the stream reads first: its plan and the two planes of its matrix.
   A kernel boundary leaves HBM idle for a few microseconds (the last CTAs' reductions, the SMs' hand-over, the first
   copies' latency); weights do not depend on the activations, so every warp, once its own last copy is under way, asks
   L2 for the bytes that the same warp of the next launch will request first.  They travel during the boundary and the
   next launch's ring fills from L2.  nib == null: nothing known about the next launch. */
struct NextFill {
    const uint8_t *nib, *raw;
    FlatPlan plan;
    uint32_t blocks;            /* CTAs of the next launch                    */
    uint32_t cluster_shift;     /* log2 of its cluster size                    */
    uint32_t nib_unit, raw_unit;/* bytes of a unit in the two planes           */
    uint32_t units;             /* most units per warp worth fetching ahead    */
    uint32_t pooled;            /* 1: the next launch's warps draw stages from their CTA's pool; its first 2 x 16 stages are the start of the CTA's run */
};
__device__ __forceinline__ void l2_prefetch(const uint8_t *p, uint32_t bytes) {
    asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;" ::"l"(p), "r"(bytes) : "memory");
}
/* one lane per warp: the first units of warp `warp` of every CTA of the next launch that maps to this CTA */
__device__ __forceinline__ void prefetch_next_fill(const NextFill &nx, uint32_t warp) {
    if (nx.nib == nullptr) return;
    for (uint32_t b = blockIdx.x; b < nx.blocks; b += gridDim.x) {
        const uint32_t cl = b >> nx.cluster_shift, rank = b & ((1u << nx.cluster_shift) - 1u);
        const uint32_t k0 = nx.plan.start(cl), k1 = nx.plan.start(cl + 1u);
        const uint32_t c0 = k0 + (((k1 - k0) * rank) >> nx.cluster_shift), c1 = k0 + (((k1 - k0) * (rank + 1u)) >> nx.cluster_shift);
        const uint32_t cn = c1 - c0;
        uint32_t w0 = cn * warp / (kRingThreads / 32u), w1 = cn * (warp + 1u) / (kRingThreads / 32u);
        if (nx.pooled) { w0 = min(warp * nx.units, cn); w1 = cn; }
        const uint32_t n = min(w1 - w0, nx.units);
        if (n) {
            l2_prefetch(nx.nib + (uint64_t)(c0 + w0) * nx.nib_unit, n * nx.nib_unit);
            l2_prefetch(nx.raw + (uint64_t)(c0 + w0) * nx.raw_unit, n * nx.raw_unit);
        }
    }
}

/* Shared memory behind the rings: what each warp contributes to row groups it shares with other warps of its CTA.
   A warp's run is contiguous, so only its first and its last row group can be shared: entry 2 * warp is the first one
   ("head"), entry 2 * warp + 1 the last one ("tail", used only when it differs from the head's group). */
constexpr uint32_t kRingEntries = 2u * (kRingThreads / 32u);
constexpr uint32_t kRingShareBytes = kRingEntries * 4u + kRingEntries * 16u * 4u;
constexpr uint32_t kNoGroup = 0xFFFFFFFFu;

/* ELEM = fp8: the raw plane holds 3-bit fields, 96 bits per lane and PAIR of slots (384 B per pair), so the unit of all
   counting below is a pair of slots; the launcher takes this kernel only when every row group has an even number of slots. */
/* SHARE: the instance that is launched when FusedInput::share is set (a kernel of its own so that the cluster's code
   costs the other launches nothing).
   Everything else - the four input modes, whole and cut row groups, local and pushed output - is deliberately ONE
   instance per element type.  Instances per input mode, and instances with the cut-group, cluster and push code compiled
   out for plans of whole row groups, were built and measured on B200 against this one on the same box: each of them is
   faster when it runs back to back with itself (6144 x 2560: 8.15 against 8.65 us; 57344 x 8192: 112.4 against 115.0 us),
   but a decode step alternates between them and comes out slower (Qwen3-4B 428 against 439 tokens/s, Llama-3-70B shapes
   50.4 against 50.8, two GPUs 82 against 87): a launch whose code the previous launch left in the instruction caches
   starts faster than a shorter kernel that has to be fetched. */
template <int ELEM, bool SHARE>
__global__ void __launch_bounds__(kRingThreads, kRingCtasPerSm) ring_kernel_layout2(const SegmentArgs a, const FlatPlan plan, const FusedInput in, const NextFill nx) {
    constexpr uint32_t U = ELEM == kFp8 ? 2u : 1u;               /* slots per unit                                  */
    constexpr uint32_t kUnits = kRingSlots / U;                  /* units per stage                                 */
    constexpr uint32_t kNibUnit = 256u * U, kRawUnit = ELEM == kFp8 ? 384u : 512u;      /* bytes of a unit in the two planes */
    constexpr uint32_t kBlockUnits = 16u / U;                    /* units per 512-column block                      */
    static_assert(kRingSlots % U == 0u, "a stage holds whole units");
    extern __shared__ __align__(128) uint8_t ring_smem[];
    const uint32_t lane = threadIdx.x & 31u, warp = threadIdx.x >> 5;
    const Geometry g(a.M, a.K, 2);
    /* shared memory: x | RMSNorm weight (kInputNorm only) | shared row groups | reduction scratch | barriers | rings */
    const uint32_t xs = smem_addr(ring_smem), x_bytes = ring_x_bytes(g), front = norm_like(in.mode) ? 2u * x_bytes : x_bytes;
    uint32_t *share_group = reinterpret_cast<uint32_t *>(ring_smem + front);
    float *share_value = reinterpret_cast<float *>(ring_smem + front + kRingEntries * 4u);
    float *scal = reinterpret_cast<float *>(ring_smem + front + kRingShareBytes);
    /* what this CTA contributes to row groups it shares with other CTAs of its cluster: entry 0 its first group, entry 1 its last */
    uint32_t *cta_group = reinterpret_cast<uint32_t *>(ring_smem + front + kRingShareBytes + 64u);
    float *cta_value = reinterpret_cast<float *>(ring_smem + front + kRingShareBytes + 128u);
    const uint32_t bars = xs + front + kRingShareBytes + 256u + warp * (kRingStages * 8u);
    const uint32_t ring = xs + front + kRingShareBytes + 256u + kRingBarrierBytes + warp * kRingWarpBytes;
    /* The plan's runs belong to clusters (a cluster of one CTA unless the launch says otherwise); the CTAs of a cluster
       split the cluster's run evenly, then the warps split the CTA's run. */
    namespace cg = cooperative_groups;
    cg::cluster_group cluster = cg::this_cluster();
    /* (a cluster that exists only to share the pushed partials, FusedInput::share bit 1, is invisible to the plan) */
    const uint32_t real_ctas = cluster.num_blocks(), real_rank = cluster.block_rank();
    const bool share_only = SHARE && (in.share & 2u) != 0u;
    const uint32_t cluster_ctas = share_only ? 1u : real_ctas, cta_rank = share_only ? 0u : real_rank, cluster_id = blockIdx.x / cluster_ctas;
    if (SHARE) cluster_arrive();                                 /* "this CTA runs": waited for before the first store into its shared memory */
    const uint32_t k0 = plan.start(cluster_id), k1 = plan.start(cluster_id + 1u), cluster_shift = (uint32_t)__ffs((int)cluster_ctas) - 1u;   /* clusters of 1, 2, 4 or 8 */
    const uint32_t c0 = k0 + (((k1 - k0) * cta_rank) >> cluster_shift), c1 = k0 + (((k1 - k0) * (cta_rank + 1u)) >> cluster_shift);
    const uint32_t cn = c1 - c0, w0 = cn * warp / (kRingThreads / 32u), w1 = cn * (warp + 1u) / (kRingThreads / 32u);
    const uint32_t u0 = c0 + w0;
    const uint32_t count = w1 - w0, n_stage = (count + kUnits - 1u) / kUnits;
    const uint8_t *nib_next = a.low + (uint64_t)u0 * kNibUnit, *raw_next = a.low + g.nibble_plane_bytes() + (uint64_t)u0 * kRawUnit;
    uint32_t left = count;                                       /* units not yet requested */
    if (lane == 0) {
        for (uint32_t b = 0; b < kRingStages; b++) mbar_init(bars + b * 8u, 1u);
        mbar_init_fence();
        for (uint32_t b = 0; b < kRingStages && left; b++) {     /* fill the ring before anything else */
            const uint32_t n = min(kUnits, left), dst = ring + b * kRingStageBytes;
            mbar_expect(bars + b * 8u, n * (kNibUnit + kRawUnit));
            bulk_load(dst, nib_next, n * kNibUnit, bars + b * 8u);
            bulk_load(dst + kRingSlots * 256u, raw_next, n * kRawUnit, bars + b * 8u);
            nib_next += n * kNibUnit; raw_next += n * kRawUnit; left -= n;
        }
    }
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    FixedTables t; t.load(a.lut);
    const uint32_t slots = g.slots / U;                          /* units per row group */
    uint32_t rb = plan.group_of(u0), s = u0 - rb * slots;         /* row group and unit inside it */
    /* exception count of this lane and data offset of the next block to start in this run, fetched one block ahead */
    /* Exception lists, three blocks deep so that no warp ever waits for memory at a block boundary: `ahead` = exception
       count and data offset of the block after next (loads in flight), `next` = the next block to start in this run, its
       count and the address of this lane's first entry, already pulled towards L1. */
    constexpr uint32_t kEntryBytes = ELEM == kFp8 ? 2u : 3u;
    uint32_t next_block = rb * g.CB + ((s + kBlockUnits - 1u) / kBlockUnits), next_count = 0, ahead_count = 0, ahead_base = 0;
    const uint8_t *next_entries = a.data;
    auto load_ahead = [&](uint32_t b) {
        ahead_count = 0; ahead_base = 0;
        if (b < g.nb) { ahead_count = __ldg(a.hdr + (uint64_t)b * kLanes + lane); ahead_base = __ldg(a.bases + b); }
    };
    auto promote = [&]() {                                       /* ahead -> next: where this lane's entries start, and fetch them */
        uint32_t total;
        const uint32_t before = warp_exclusive_sum(ahead_count, lane, total);
        next_count = ahead_count;
        next_entries = a.data + ahead_base + (uint64_t)before * kEntryBytes;
        if (next_count) asm volatile("prefetch.global.L1 [%0];" ::"l"(next_entries));
    };
    load_ahead(next_block);
    /* The weights do not depend on the kernel before this one, the activation vector does.  It is built in shared
       memory, zero beyond K (the last slot may cover columns past K16). */
    NormWeights norm_regs;
    stage_norm_weight<kRingThreads>(in, a.K, reinterpret_cast<uint16_t *>(ring_smem + x_bytes), norm_regs);
    if (threadIdx.x < kRingEntries) share_group[threadIdx.x] = kNoGroup;
    if (threadIdx.x < 2u) cta_group[threadIdx.x] = kNoGroup;
    asm volatile("griddepcontrol.wait;" ::: "memory");
    /* tensor-parallel output: the call number that this launch's words carry = this rank's pushes to the slot so far + 1
       (read by every CTA before any CTA can finish; the last CTA to finish counts the push) */
    const uint32_t push_call = a.push.world ? *reinterpret_cast<const volatile uint32_t *>(&reinterpret_cast<const CommControl *>(a.push.buf[a.push.rank])->push_epoch[a.push.slot]) + 1u : 0u;
    promote(); load_ahead(next_block + 1u);                      /* the first block's entries travel while x is built */
    if (SHARE)                                                   /* (the RMSNorm weight is in registers: its place in shared memory holds the cluster's scalars) */
        build_activation_shared<kRingThreads>(in, a.K, x_bytes >> 1, reinterpret_cast<uint16_t *>(ring_smem), reinterpret_cast<float *>(ring_smem + x_bytes), norm_regs,
                                              real_ctas, real_rank, blockIdx.x < real_ctas);
    else
        build_activation<kRingThreads>(in, a.x, a.K, x_bytes >> 1, reinterpret_cast<uint16_t *>(ring_smem), reinterpret_cast<uint16_t *>(ring_smem + x_bytes), scal, norm_regs);
    const uint32_t lane8 = lane * 8u, lane16 = kRingSlots * 256u + lane * (ELEM == kFp8 ? 4u : 16u), xq = xs + (lane & 3u) * 16u;
    uint32_t seg_first = s, entry = 2u * warp;                   /* first slot of the current segment; where a shared one goes */
    float d[4] = {0.f, 0.f, 0.f, 0.f}, ex_lo = 0.f, ex_hi = 0.f;
    /* the segment [seg_first, s) of row group rb is complete */
    auto flush = [&]() {
        ex_lo += __shfl_xor_sync(0xffffffffu, ex_lo, 1); ex_lo += __shfl_xor_sync(0xffffffffu, ex_lo, 2);
        ex_hi += __shfl_xor_sync(0xffffffffu, ex_hi, 1); ex_hi += __shfl_xor_sync(0xffffffffu, ex_hi, 2);
        const float lo = d[0] + ex_lo, hi = d[2] + ex_hi;
        const uint32_t r = lane >> 2;
        if (seg_first == 0u && s == slots) {                     /* a whole row group: nobody else adds to it */
            if (plan.direct || plan.fix) {                       /* final: row i of the group to lane i < 16, from the quad leader that holds it */
                const uint32_t src = (lane & 7u) << 2;
                const float vlo = __shfl_sync(0xffffffffu, lo, src), vhi = __shfl_sync(0xffffffffu, hi, src);
                if (lane < 16u) emit_group(a, rb, lane, (lane & 8u) ? vhi : vlo, 0x0000FFFFu, push_call);
            } else if ((lane & 3u) == 0u) {
                const uint32_t part = cluster_id - plan.owner(rb * slots);
                emit_flat(a, plan, rb * 16u + r, part, lo); emit_flat(a, plan, rb * 16u + r + 8u, part, hi);
            }
        } else {
            if ((lane & 3u) == 0u) { share_value[entry * 16u + r] = lo; share_value[entry * 16u + r + 8u] = hi; }
            if (lane == 0) share_group[entry] = rb;
            entry = 2u * warp + 1u;
        }
        d[0] = d[1] = d[2] = d[3] = 0.f; ex_lo = ex_hi = 0.f;
    };
    uint32_t buf = 0, parity = 0, todo = count;
    bool hinted = false;                                         /* the next launch's first bytes are on their way to L2 */
#pragma unroll 1
    for (uint32_t st = 0; st < n_stage; st++) {
        const uint32_t bar = bars + buf * 8u, src = ring + buf * kRingStageBytes;
        if (!mbar_wait(bar, parity)) {                           /* gave up (status word set): let copies already issued land, then stop */
            for (uint32_t b = 0; b < kRingStages; b++) for (uint32_t i = 0; i < 64u && !mbar_poll(bars + b * 8u, parity ^ (b < buf ? 1u : 0u)); i++) {}
            break;
        }
        /* one unit: per slot 16 weights per lane against 32 columns of x (fp8: two slots that share one 96-bit field group) */
        auto slot = [&](uint32_t j, uint32_t column_unit) {
            uint32_t a0, a1, a2, a3;
            if (ELEM == kFp8) {
                const uint32_t f0 = lds32(src + j * 384u + lane16), f1 = lds32(src + j * 384u + 128u + lane16), f2 = lds32(src + j * 384u + 256u + lane16);
                const uint2 n0 = lds64(src + (2u * j) * 256u + lane8), n1 = lds64(src + (2u * j + 1u) * 256u + lane8);
                const uint4 x0 = lds128(xq + (2u * column_unit) * 64u), x1 = lds128(xq + (2u * column_unit + 1u) * 64u);
                fixed_half<kFp8, 0>(t, n0.x, 0u, 0u, f0, f1, f2, a0, a1, a2, a3); mma_bf16(d, a0, a1, a2, a3, x0.x, x0.y);
                fixed_half<kFp8, 2>(t, n0.y, 0u, 0u, f0, f1, f2, a0, a1, a2, a3); mma_bf16(d, a0, a1, a2, a3, x0.z, x0.w);
                fixed_half<kFp8, 4>(t, n1.x, 0u, 0u, f0, f1, f2, a0, a1, a2, a3); mma_bf16(d, a0, a1, a2, a3, x1.x, x1.y);
                fixed_half<kFp8, 6>(t, n1.y, 0u, 0u, f0, f1, f2, a0, a1, a2, a3); mma_bf16(d, a0, a1, a2, a3, x1.z, x1.w);
            } else {
                const uint2 nib = lds64(src + j * 256u + lane8);
                const uint4 raw = lds128(src + j * 512u + lane16);
                const uint4 xv = lds128(xq + column_unit * 64u);
                fixed_half<kBf16, 0>(t, nib.x, raw.x, raw.y, 0u, 0u, 0u, a0, a1, a2, a3);
                mma_bf16(d, a0, a1, a2, a3, xv.x, xv.y);
                fixed_half<kBf16, 2>(t, nib.y, raw.z, raw.w, 0u, 0u, 0u, a0, a1, a2, a3);
                mma_bf16(d, a0, a1, a2, a3, xv.z, xv.w);
            }
        };
        /* the block whose first unit is f starts here: this warp adds the block's exceptions */
        auto exceptions = [&](uint32_t f) {
            const float2 e = ring_exceptions<ELEM>(next_count, next_entries, xs, f / kBlockUnits, lane);
            ex_lo += e.x; ex_hi += e.y;
            next_block++;
            promote(); load_ahead(next_block + 1u);
        };
        if (todo >= kUnits && s + kUnits <= slots) {             /* a full stage inside one row group: no per-unit checks */
#pragma unroll
            for (uint32_t j = 0; j < kUnits; j++) slot(j, s + j);
            const uint32_t to_block = (0u - s) & (kBlockUnits - 1u);      /* units from s to the next first unit of a block */
            if (to_block < kUnits) exceptions(s + to_block);
            s += kUnits;
            if (s == slots) { flush(); s = 0; seg_first = 0; rb++; }
        } else {
            const uint32_t n = min(todo, kUnits);
#pragma unroll 1
            for (uint32_t j = 0; j < n; j++) {
                slot(j, s);
                if ((s & (kBlockUnits - 1u)) == 0u) exceptions(s);
                if (++s == slots) { flush(); s = 0; seg_first = 0; rb++; }
            }
        }
        todo -= min(todo, kUnits);
        __syncwarp();
        if (lane == 0) {
            if (left) {                                          /* refill the stage just read */
                const uint32_t n = min(kUnits, left);
                async_proxy_fence();
                mbar_expect(bar, n * (kNibUnit + kRawUnit));
                bulk_load(src, nib_next, n * kNibUnit, bar);
                bulk_load(src + kRingSlots * 256u, raw_next, n * kRawUnit, bar);
                nib_next += n * kNibUnit; raw_next += n * kRawUnit; left -= n;
            } else if (!hinted) { prefetch_next_fill(nx, warp); hinted = true; }      /* this warp's last copy is under way */
        }
        if (++buf == kRingStages) { buf = 0; parity ^= 1u; }
    }
    if (lane == 0 && !hinted) prefetch_next_fill(nx, warp);
    if (s != seg_first) flush();
    __syncthreads();
    /* Shared row groups: entries of one group are adjacent in entry order.  The first entry of each group adds the
       others in that order (so the sum does not depend on timing).  The result is final when this CTA's run holds the
       whole group (or the plan keeps per-cluster partials anyway); otherwise it is this CTA's share of a group that
       other CTAs of the cluster also hold, and goes to the cluster-level entries. */
    {
        const uint32_t e = threadIdx.x >> 4, row = threadIdx.x & 15u, grp = share_group[e];
        bool leader = grp != kNoGroup;
        for (uint32_t p = e; leader && p-- > 0u;) { const uint32_t gp = share_group[p]; if (gp == grp) leader = false; else if (gp != kNoGroup) break; }
        if (leader) {
            float v = share_value[e * 16u + row];
            for (uint32_t n = e + 1u; n < kRingEntries; n++) {
                const uint32_t gn = share_group[n];
                if (gn == grp) v += share_value[n * 16u + row]; else if (gn != kNoGroup) break;
            }
            const uint32_t g0 = grp * slots;
            const bool inside = g0 >= c0 && g0 + slots <= c1;
            const uint32_t half_mask = 0xFFFFu << (threadIdx.x & 16u);
            if (plan.direct ? (cluster_ctas == 1u || inside) : (plan.fix && inside)) emit_group(a, grp, row, v, half_mask, push_call);
            else if (plan.fix) {
                /* Equal runs: a row group cut by run boundaries.  A CTA whose run holds a later part of it leaves that part
                   in its own entry of g_cut_part; the CTA where the group begins adds the later parts in CTA order (so the
                   sum does not depend on timing), writes the rows and empties the entries again.  One trip through L2 after
                   the last CTA's loop, no counter. */
                if (g0 < c0) {
                    uint32_t w = __float_as_uint(v);
                    if (w == kCutEmpty) w = 0x7FC00000u;             /* (another NaN) */
                    *reinterpret_cast<volatile unsigned int *>(&g_cut_part[blockIdx.x][row]) = w;
                } else {
                    const uint32_t holders = plan.owner(g0 + slots - 1u) - blockIdx.x;
                    const unsigned long long t0 = global_timer_ns();
                    bool ok = true;
                    for (uint32_t h = 1; h <= holders && ok; h++) {
                        volatile unsigned int *theirs = &g_cut_part[blockIdx.x + h][row];
                        uint32_t w = *theirs;
                        while (w == kCutEmpty) {
                            if (global_timer_ns() - t0 > kCutWaitNs) { ok = false; break; }
                            w = *theirs;
                        }
                        if (ok) { v += __uint_as_float(w); *theirs = kCutEmpty; }
                    }
                    if (!ok) { atomicExch(&g_kernel_status, kStatusWaitTimeout); v = __uint_as_float(0x7FC00000u); }
                    emit_group(a, grp, row, v, half_mask, push_call);
                }
            }
            else if (cluster_ctas == 1u) emit_flat(a, plan, grp * 16u + row, cluster_id - plan.owner(g0), v);      /* one fp32 partial per CTA */
            else {
                const uint32_t which = g0 < c0 ? 0u : 1u;            /* the group began before this CTA's run: its first group */
                cta_value[which * 16u + row] = v;
                if (row == 0u) cta_group[which] = grp;
            }
        }
    }
    if (cluster_ctas > 1u) {                                        /* same again one level up, through distributed shared memory */
        cluster.sync();
        if (threadIdx.x < 32u) {
            const uint32_t which = threadIdx.x >> 4, row = threadIdx.x & 15u, grp = cta_group[which];
            /* this CTA is the first of its cluster to hold the group unless the group began before its run */
            if (grp != kNoGroup && !(grp * slots < c0 && cta_rank > 0u)) {
                float v = cta_value[which * 16u + row];
                for (uint32_t r = cta_rank + 1u; r < cluster_ctas; r++) {        /* later CTAs hold it as their first group, in rank order */
                    const uint32_t theirs = cluster.map_shared_rank(cta_group, r)[0];
                    if (theirs == grp) v += cluster.map_shared_rank(cta_value, r)[row];
                    else if (theirs != kNoGroup) break;          /* (no entry: an empty run, or one that starts on a group boundary) */
                }
                emit_group(a, grp, row, v, 0xFFFFu << (threadIdx.x & 16u), push_call);
            }
        }
        cluster.sync();                                             /* nobody leaves while its shared memory may still be read */
    }
    /* Tensor-parallel output: the words this launch stored carry their own call number, nothing has to be published; the
       CTA that finishes last counts the push (every CTA read the count before any CTA could get here). */
    if (a.push.world && threadIdx.x == 0) {
        CommControl *own = reinterpret_cast<CommControl *>(a.push.buf[a.push.rank]);
        if (atomicAdd(&own->push_done, 1u) == gridDim.x - 1u) {
            own->push_done = 0u;
            volatile uint32_t *count = &own->push_epoch[a.push.slot];
            *count = *count + 1u;
        }
    }
}

/* ---- layout 2, token path, second form: the warps of a CTA draw their stages from one pool ---------------------------
   Measured on B200 with the kernel above (every warp owns one contiguous run of its CTA's units): the 16 warps of a CTA,
   with equal runs, finish 10 % of the loop time apart (10 us of 100 on 57344 x 8192), and a warp that has finished leaves
   its ring empty while its CTA waits for the slowest one.  Here the CTA's run is a sequence of stages (kUnits units, never
   across a row-group boundary); a warp that has a ring buffer free takes the next stage from a shared-memory counter, so
   all warps end within one stage of each other whatever their speeds were.
   The result must not depend on which warp took which stage: every stage leaves its own partial sums (16 rows, fp32) in
   shared memory, and the warp that completes a row group's last stage adds the group's stage partials in stage order.
   Runs are equal per CTA (they may cut row groups).  A CTA works front to back, so the part of a row group that began in
   an earlier CTA's run is complete EARLY in this CTA's run: it is published then (g_cut_part, one entry per CTA), and
   the CTA where the group began adds the later CTAs' parts, in CTA order, when its own part is complete at the end of its
   run: no counter, no second launch, and normally no wait. */
struct PoolShape {
    uint32_t stages_per_group;  /* S = ceil(units per row group / units per stage)                     */
    uint32_t group_slots;       /* G: row groups whose stage partials shared memory holds at once (2, 4, 8 or 16) */
    uint32_t group_shift;       /* log2 G                                                                          */
    FastDiv by_stages;
};
constexpr uint32_t kPoolCtrlBytes = 256u;                        /* next stage | 15 spare words | 16 arrival counts | 16 generations | 16 floats for the prologue */

static inline uint32_t pool_units(int elem) { return elem == kFp8 ? kRingSlots / 2u : kRingSlots; }
static inline PoolShape make_pool_shape(const Geometry &g, int elem) {
    PoolShape ps;
    const uint32_t units = elem == kFp8 ? g.slots / 2u : g.slots, per = pool_units(elem);
    ps.stages_per_group = (units + per - 1u) / per;
    const uint32_t S = ps.stages_per_group;
    ps.group_shift = S >= 96u ? 1u : (S >= 24u ? 2u : (S >= 12u ? 3u : 4u));       /* more than the 16 warps' three stages each can span */
    ps.group_slots = 1u << ps.group_shift;
    ps.by_stages.set(S);
    return ps;
}
static inline uint32_t pool_smem_bytes(const Geometry &g, int elem, int input_mode) {
    const PoolShape ps = make_pool_shape(g, elem);
    return (norm_like(input_mode) ? 2u : 1u) * ring_x_bytes(g) + ps.group_slots * ps.stages_per_group * 64u + kPoolCtrlBytes + kRingBarrierBytes + (kRingThreads / 32u) * kRingWarpBytes;
}
/* at least 6 stages per row group (the stage partials of the groups in flight must fit their 16 slots) */
static inline bool pool_covers(int code, const Geometry &g, int input_mode) {
    if (!ring_covers(code, g, input_mode)) return false;
    return make_pool_shape(g, type_of(code)).stages_per_group >= 6u && pool_smem_bytes(g, type_of(code), input_mode) <= kRingMaxSmem;
}

template <int ELEM>
__global__ void __launch_bounds__(kRingThreads, 1) pool_kernel_layout2(const SegmentArgs a, const FlatPlan plan, const FusedInput in, const NextFill nx, const PoolShape ps) {
    constexpr uint32_t U = ELEM == kFp8 ? 2u : 1u;
    constexpr uint32_t kUnits = kRingSlots / U;
    constexpr uint32_t kNibUnit = 256u * U, kRawUnit = ELEM == kFp8 ? 384u : 512u;
    constexpr uint32_t kBlockUnits = 16u / U;
    constexpr uint32_t kNone = 0xFFFFFFFFu;
    static_assert(kRingStages == 2u, "the loop below alternates between two ring buffers");
    extern __shared__ __align__(128) uint8_t ring_smem[];
    const uint32_t lane = threadIdx.x & 31u, warp = threadIdx.x >> 5;
    const Geometry g(a.M, a.K, 2);
    /* shared memory: x | RMSNorm weight (norm modes) | stage partials | control words | barriers | rings */
    const uint32_t xs = smem_addr(ring_smem), x_bytes = ring_x_bytes(g), front = norm_like(in.mode) ? 2u * x_bytes : x_bytes;
    const uint32_t S = ps.stages_per_group, G = ps.group_slots, part_bytes = G * S * 64u;
    float *part = reinterpret_cast<float *>(ring_smem + front);
    volatile uint32_t *ctrl = reinterpret_cast<volatile uint32_t *>(ring_smem + front + part_bytes);
    uint32_t *next_stage = reinterpret_cast<uint32_t *>(ring_smem + front + part_bytes);
    uint32_t *arrived = reinterpret_cast<uint32_t *>(ring_smem + front + part_bytes) + 16;
    volatile uint32_t *generation = ctrl + 32;
    float *scal = reinterpret_cast<float *>(ring_smem + front + part_bytes + 192u);
    const uint32_t bars = xs + front + part_bytes + kPoolCtrlBytes + warp * (kRingStages * 8u);
    const uint32_t ring = xs + front + part_bytes + kPoolCtrlBytes + kRingBarrierBytes + warp * kRingWarpBytes;
    /* this CTA's run of units and its stages: the rest of the row group the run starts in, whole row groups, the start of a last one */
    const uint32_t slots = g.slots / U;
    const uint32_t c0 = plan.start(blockIdx.x), c1 = plan.start(blockIdx.x + 1u), cn = c1 - c0;
    const uint32_t grp0 = plan.group_of(c0), off0 = c0 - grp0 * slots;
    const uint32_t n0 = min(slots - off0, cn), S0 = (n0 + kUnits - 1u) / kUnits;
    const uint32_t rest = cn - n0, whole = plan.group_of(rest), tail = rest - whole * slots;
    const uint32_t n_stages = S0 + whole * S + (tail + kUnits - 1u) / kUnits;
    const uint8_t *raw_plane = a.low + g.nibble_plane_bytes();
    /* stage t: row group (counted from the run's first), stage inside the group's part, first unit inside the row group, units */
    struct Stage { uint32_t gi, index, first, count, stages; };
    auto describe = [&](uint32_t t) {
        Stage s;
        uint32_t end;
        if (t < S0) { s.gi = 0u; s.index = t; s.first = off0 + t * kUnits; end = off0 + n0; s.stages = S0; }
        else {
            const uint32_t r = t - S0, q = ps.by_stages.div(r);
            s.gi = 1u + q; s.index = r - q * S; s.first = s.index * kUnits;
            end = q < whole ? slots : tail; s.stages = q < whole ? S : (tail + kUnits - 1u) / kUnits;
        }
        s.count = min(kUnits, end - s.first);
        return s;
    };
    /* the block (if any) whose first unit lies in the stage: units from the stage's start to it, or kNone */
    auto block_start = [&](const Stage &s) { const uint32_t d = (0u - s.first) & (kBlockUnits - 1u); return d < s.count ? d : kNone; };
    constexpr uint32_t kEntryBytes = ELEM == kFp8 ? 2u : 3u;
    /* ring buffer b holds stage T[b]; exception count of this lane and data offset of the block that starts in it */
    uint32_t T0 = warp < n_stages ? warp : kNone, T1 = warp + kRingThreads / 32u < n_stages ? warp + kRingThreads / 32u : kNone;
    uint32_t EC0 = 0, EC1 = 0, EB0 = 0, EB1 = 0, EP0 = 0, EP1 = 0;
    auto issue = [&](uint32_t b, uint32_t t, uint32_t &ec, uint32_t &eb) {
        const Stage s = describe(t);
        const uint32_t u = (grp0 + s.gi) * slots + s.first;
        if (lane == 0) {
            const uint32_t bar = bars + b * 8u, dst = ring + b * kRingStageBytes;
            mbar_expect(bar, s.count * (kNibUnit + kRawUnit));
            bulk_load(dst, a.low + (uint64_t)u * kNibUnit, s.count * kNibUnit, bar);
            bulk_load(dst + kRingSlots * 256u, raw_plane + (uint64_t)u * kRawUnit, s.count * kRawUnit, bar);
        }
        const uint32_t d = block_start(s);
        ec = 0u; eb = 0u;
        if (d != kNone) {
            const uint32_t blk = (grp0 + s.gi) * g.CB + (s.first + d) / kBlockUnits;
            ec = __ldg(a.hdr + (uint64_t)blk * kLanes + lane); eb = __ldg(a.bases + blk);
        }
    };
    /* where this lane's entries of that block start (offset into data), and pull them towards L1 */
    auto promote = [&](uint32_t ec, uint32_t eb, uint32_t &ep) {
        uint32_t total;
        const uint32_t before = warp_exclusive_sum(ec, lane, total);
        ep = eb + before * kEntryBytes;
        if (ec) asm volatile("prefetch.global.L1 [%0];" ::"l"(a.data + ep));
    };
    if (lane == 0) {
        for (uint32_t b = 0; b < kRingStages; b++) mbar_init(bars + b * 8u, 1u);
        mbar_init_fence();
    }
    __syncwarp();
    if (T0 != kNone) issue(0u, T0, EC0, EB0);                    /* fill the ring before anything else */
    if (T1 != kNone) issue(1u, T1, EC1, EB1);
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    FixedTables t; t.load(a.lut);
    NormWeights norm_regs;
    stage_norm_weight<kRingThreads>(in, a.K, reinterpret_cast<uint16_t *>(ring_smem + x_bytes), norm_regs);
    if (threadIdx.x < 48u) ctrl[threadIdx.x] = threadIdx.x == 0u ? 2u * (kRingThreads / 32u) : 0u;      /* (visible after build_activation's barrier) */
    asm volatile("griddepcontrol.wait;" ::: "memory");
    const uint32_t push_call = a.push.world ? *reinterpret_cast<const volatile uint32_t *>(&reinterpret_cast<const CommControl *>(a.push.buf[a.push.rank])->push_epoch[a.push.slot]) + 1u : 0u;
    promote(EC0, EB0, EP0); promote(EC1, EB1, EP1);
    build_activation<kRingThreads>(in, a.x, a.K, x_bytes >> 1, reinterpret_cast<uint16_t *>(ring_smem), reinterpret_cast<uint16_t *>(ring_smem + x_bytes), scal, norm_regs);
    const uint32_t lane8 = lane * 8u, lane16 = kRingSlots * 256u + lane * (ELEM == kFp8 ? 4u : 16u), xq = xs + (lane & 3u) * 16u;
    bool hinted = false, failed = false;
    uint32_t parity = 0;
    /* One stage out of ring buffer b.  other_*: the other buffer's block, whose entries are pulled towards L1 at the end. */
    auto consume = [&](uint32_t b, uint32_t &T, uint32_t &ec, uint32_t &eb, uint32_t &ep, uint32_t other_T, uint32_t other_ec, uint32_t other_eb, uint32_t &other_ep) {
        const uint32_t bar = bars + b * 8u, src = ring + b * kRingStageBytes;
        if (!mbar_wait(bar, parity)) { failed = true; return; }
        const Stage s = describe(T);
        float d[4] = {0.f, 0.f, 0.f, 0.f};
        auto slot = [&](uint32_t j, uint32_t column_unit) {
            uint32_t a0, a1, a2, a3;
            if (ELEM == kFp8) {
                const uint32_t f0 = lds32(src + j * 384u + lane16), f1 = lds32(src + j * 384u + 128u + lane16), f2 = lds32(src + j * 384u + 256u + lane16);
                const uint2 n0v = lds64(src + (2u * j) * 256u + lane8), n1v = lds64(src + (2u * j + 1u) * 256u + lane8);
                const uint4 x0 = lds128(xq + (2u * column_unit) * 64u), x1 = lds128(xq + (2u * column_unit + 1u) * 64u);
                fixed_half<kFp8, 0>(t, n0v.x, 0u, 0u, f0, f1, f2, a0, a1, a2, a3); mma_bf16(d, a0, a1, a2, a3, x0.x, x0.y);
                fixed_half<kFp8, 2>(t, n0v.y, 0u, 0u, f0, f1, f2, a0, a1, a2, a3); mma_bf16(d, a0, a1, a2, a3, x0.z, x0.w);
                fixed_half<kFp8, 4>(t, n1v.x, 0u, 0u, f0, f1, f2, a0, a1, a2, a3); mma_bf16(d, a0, a1, a2, a3, x1.x, x1.y);
                fixed_half<kFp8, 6>(t, n1v.y, 0u, 0u, f0, f1, f2, a0, a1, a2, a3); mma_bf16(d, a0, a1, a2, a3, x1.z, x1.w);
            } else {
                const uint2 nib = lds64(src + j * 256u + lane8);
                const uint4 raw = lds128(src + j * 512u + lane16);
                const uint4 xv = lds128(xq + column_unit * 64u);
                fixed_half<kBf16, 0>(t, nib.x, raw.x, raw.y, 0u, 0u, 0u, a0, a1, a2, a3);
                mma_bf16(d, a0, a1, a2, a3, xv.x, xv.y);
                fixed_half<kBf16, 2>(t, nib.y, raw.z, raw.w, 0u, 0u, 0u, a0, a1, a2, a3);
                mma_bf16(d, a0, a1, a2, a3, xv.z, xv.w);
            }
        };
        if (s.count == kUnits) {
#pragma unroll
            for (uint32_t j = 0; j < kUnits; j++) slot(j, s.first + j);
        } else {
#pragma unroll 1
            for (uint32_t j = 0; j < s.count; j++) slot(j, s.first + j);
        }
        __syncwarp();
        /* the buffer is read: draw the next stage and send for it before the bookkeeping below */
        uint32_t fresh = 0u;
        if (lane == 0) { fresh = atomicAdd(next_stage, 1u); async_proxy_fence(); }
        fresh = __shfl_sync(0xffffffffu, fresh, 0);
        const uint32_t mine_ec = ec, mine_ep = ep;
        if (fresh < n_stages) { T = fresh; issue(b, fresh, ec, eb); }
        else {
            T = kNone;
            if (!hinted) { if (lane == 0) prefetch_next_fill(nx, warp); hinted = true; }      /* this warp sends for nothing more */
        }
        float lo = d[0], hi = d[2];
        const uint32_t bs = block_start(s);
        if (bs != kNone) {                                       /* a block starts in this stage: its exceptions belong to the stage */
            float2 e = ring_exceptions<ELEM>(mine_ec, a.data + mine_ep, xs, (s.first + bs) / kBlockUnits, lane);
            e.x += __shfl_xor_sync(0xffffffffu, e.x, 1); e.x += __shfl_xor_sync(0xffffffffu, e.x, 2);
            e.y += __shfl_xor_sync(0xffffffffu, e.y, 1); e.y += __shfl_xor_sync(0xffffffffu, e.y, 2);
            lo += e.x; hi += e.y;
        }
        /* the stage's 16 row sums go to the slot of its row group; the slot is free once the group that used it before is added up */
        const uint32_t gslot = s.gi & (G - 1u), turn = s.gi >> ps.group_shift;
        {
            uint32_t polls = 0;
            while (generation[gslot] != turn && ++polls < kWaitPolls) {}
            if (!__all_sync(0xffffffffu, polls < kWaitPolls)) { atomicExch(&g_kernel_status, kStatusWaitTimeout); failed = true; return; }
        }
        float *mine = part + (gslot * S + s.index) * 16u;
        if ((lane & 3u) == 0u) { mine[lane >> 2] = lo; mine[(lane >> 2) + 8u] = hi; }
        __syncwarp();
        uint32_t last = 0u;
        if (lane == 0) { __threadfence_block(); last = atomicAdd(arrived + gslot, 1u) + 1u == s.stages ? 1u : 0u; }
        last = __shfl_sync(0xffffffffu, last, 0);
        if (other_T != kNone) promote(other_ec, other_eb, other_ep);
        else if (T != kNone) promote(ec, eb, ep);
        if (!last) return;
        /* this warp completed the row group's part: add its stage partials in stage order (two interleaved chains, then the two) */
        __threadfence_block();
        const uint32_t row = lane & 15u, half = lane >> 4;
        const float *p = part + gslot * S * 16u + row;
        float v = 0.f;
        for (uint32_t i = half; i < s.stages; i += 2u) v += p[i * 16u];
        v += __shfl_down_sync(0xffffffffu, v, 16);
        __syncwarp();
        if (lane == 0) { arrived[gslot] = 0u; __threadfence_block(); generation[gslot] = turn + 1u; }
        const uint32_t grp = grp0 + s.gi, g_first = grp * slots;
        const bool begins_here = g_first >= c0, ends_here = g_first + slots <= c1;
        if (begins_here && ends_here) { if (lane < 16u) emit_group(a, grp, row, v, 0x0000FFFFu, push_call); return; }
        if (!begins_here) {                                      /* the group began in an earlier CTA's run: leave this part for that CTA */
            if (lane < 16u) {
                uint32_t w = __float_as_uint(v);
                if (w == kCutEmpty) w = 0x7FC00000u;            /* (another NaN) */
                *reinterpret_cast<volatile unsigned int *>(&g_cut_part[blockIdx.x][row]) = w;
            }
            return;
        }
        /* the group begins here and goes on in later CTAs: add their parts in CTA order */
        const uint32_t holders = plan.owner(g_first + slots - 1u) - blockIdx.x;
        bool ok = true;
        if (lane < 16u) {
            const unsigned long long t0 = global_timer_ns();
            for (uint32_t h = 1; h <= holders && ok; h++) {
                volatile unsigned int *src_word = &g_cut_part[blockIdx.x + h][row];
                uint32_t w = *src_word;
                while (w == kCutEmpty) {
                    if (global_timer_ns() - t0 > kCutWaitNs) { ok = false; break; }
                    w = *src_word;
                }
                if (ok) { v += __uint_as_float(w); *src_word = kCutEmpty; }
            }
        }
        if (!__all_sync(0xffffffffu, ok)) { atomicExch(&g_kernel_status, kStatusWaitTimeout); v = __uint_as_float(0x7FC00000u); }
        if (lane < 16u) emit_group(a, grp, row, v, 0x0000FFFFu, push_call);
    };
#pragma unroll 1
    while ((T0 != kNone || T1 != kNone) && !failed) {
        if (T0 != kNone) consume(0u, T0, EC0, EB0, EP0, T1, EC1, EB1, EP1);
        if (T1 != kNone && !failed) consume(1u, T1, EC1, EB1, EP1, T0, EC0, EB0, EP0);
        parity ^= 1u;
    }
    if (failed) {                                                /* gave up (status word set): let copies already issued land before the CTA leaves */
        for (uint32_t b = 0; b < kRingStages; b++) for (uint32_t i = 0; i < 64u && !mbar_poll(bars + b * 8u, parity); i++) {}
    }
    if (lane == 0 && !hinted) prefetch_next_fill(nx, warp);
    /* Tensor-parallel output: the words this launch stored carry their own call number, nothing has to be published; the
       CTA that finishes last counts the push (every CTA read the count before any CTA could get here). */
    if (a.push.world && threadIdx.x == 0) {
        CommControl *own = reinterpret_cast<CommControl *>(a.push.buf[a.push.rank]);
        if (atomicAdd(&own->push_done, 1u) == gridDim.x - 1u) {
            own->push_done = 0u;
            volatile uint32_t *count = &own->push_epoch[a.push.slot];
            *count = *count + 1u;
        }
    }
}

/* y[i] = bf16((sum of the partials of the warps that shared row i's row group, in warp order) * scale[i] + bias[i]) */
__global__ void finalize_flat_kernel(const float *__restrict__ partial, const uint16_t *__restrict__ bias, const float *__restrict__ scale,
                                     uint16_t *__restrict__ y, uint32_t M, uint32_t rows, const FlatPlan plan) {
    const uint32_t i = blockIdx.x * blockDim.x + threadIdx.x;
    asm volatile("griddepcontrol.wait;" ::: "memory");
    if (i >= M) return;
    const uint32_t first_unit = (i / rows) * plan.units_per_group;
    const uint32_t n = plan.owner(first_unit + plan.units_per_group - 1u) - plan.owner(first_unit) + 1u;
    float v = 0.f;
    for (uint32_t p = 0; p < n; p++) v += partial[(uint64_t)i * plan.parts + p];
    if (scale) v *= scale[i];
    if (bias) v += bf16_to_float(bias[i]);
    y[i] = bf16_round(v);
}

/* Equal contiguous runs (they differ by at most one grain) for up to `warps` warps.  Fewer warps take part when the
   warps that could share one row group would not fit the caller's scratch (CB floats per row); with a single column
   block no row group may be cut at all. */
static void make_flat_plan(const Geometry &g, uint32_t units_per_group, uint64_t warps, FlatPlan &p, bool whole_groups = false) {
    const uint64_t total = (uint64_t)g.groups * units_per_group;
    p.units_per_group = units_per_group;
    p.grain = g.CB == 1u || whole_groups ? units_per_group : 1u;
    p.chunks = (uint32_t)(total / p.grain);
    uint64_t use = warps < p.chunks ? warps : p.chunks;
    if (p.grain == 1u && g.CB > 1u) {
        const uint64_t need = (units_per_group - 1u) / (g.CB - 1u) + 1u;       /* shortest run that keeps parts <= CB */
        if (total / use < need) use = total / need ? total / need : 1u;
    }
    p.warps = (uint32_t)use;
    p.direct = p.grain % units_per_group == 0u ? 1u : 0u;
    p.fix = 0u;
    p.parts = p.direct ? 1u : (uint32_t)((units_per_group - 1u) / (total / use)) + 2u;
    if (p.parts > g.CB) p.parts = g.CB;                                        /* bound above guarantees the true count fits */
    p.finish();
}

/* Layout 2: the plan's "warps" are CTAs (the 32 warps of a CTA split its run evenly and add up in shared memory).
   Whole row groups per CTA need no second launch but leave some CTAs one group short; equal runs of slots keep every
   CTA busy to the end but need the finalize launch; measured on B200 that second launch and its kernel boundary cost
   4 to 5 us, the time one CTA streams about kFinalizeSlots slots. */
constexpr uint64_t kFinalizeSlots = 256;
/* How many clusters of 2 / 4 / 8 CTAs of the layout-2 kernel one device runs at once (a cluster needs its SMs inside one
   GPC, so fewer SMs are usable the larger the cluster); asked from the runtime once per device. */
constexpr uint64_t kClusterSlots = 128;                          /* measured: a cluster launch pays off only beyond this many slots saved per CTA */
struct ClusterRoom { int count[4]; };                            /* index = log2(cluster size); [0] = SM count */
static ClusterRoom cluster_room(int sms);
/* The runs of the plan belong to clusters of `cluster` CTAs.  Candidates: whole row groups per CTA (cluster 1), whole row
   groups per cluster of 2, 4 or 8 CTAs that split them (one launch each, bf16 y written by the kernel; the larger the
   cluster the finer the split but the fewer SMs), or equal runs of slots per CTA with per-CTA partials and the finalize
   launch.  Cost = slots the busiest CTA streams, plus what the extra synchronisation or launch is worth in slots. */
/* With allow_fix the equal runs need no second launch: the parts of a cut row group meet in the CTA where the group
   begins (FlatPlan::fix, g_cut_part), which costs one trip through L2 after the last CTA's loop: about 1 us, the time a
   CTA streams kFixSlots slots.
   Cost of a candidate = what its busiest CTA streams, except that CTAs which finish early leave their share of the HBM
   bandwidth to the others, so only half of the imbalance counts, plus what the extra synchronisation or launch is worth. */
constexpr uint64_t kFixSlots = 96;
static bool g_disable_ring = false, g_disable_fixup = false;     /* A/B switches of the tests (set_ring_kernels, set_fixup_plans) */
static void make_cta_plan_layout2(const Geometry &g0, int elem, int sms, FlatPlan &p, uint32_t &cluster, bool allow_fix = false) {
    Geometry g = g0;
    if (elem == kFp8) g.slots >>= 1;                              /* fp8: the kernel counts in pairs of slots; the slot-based costs below scale alike */
    const uint64_t total = (uint64_t)g.groups * g.slots;
    const ClusterRoom room = cluster_room(sms);
    if (sms > (int)kFixCounters || g_disable_fixup) allow_fix = false;
    const uint64_t even = (total + (uint64_t)sms - 1u) / (uint64_t)sms;       /* slots per CTA if all were equally loaded */
    uint64_t best = even + (allow_fix ? kFixSlots : kFinalizeSlots);
    uint32_t best_cluster = 0;                                   /* 0 = equal runs (+ fix-up or finalize) */
    for (uint32_t lg = 0; lg < 4u; lg++) {
        const uint64_t clusters = lg == 0u ? (uint64_t)sms : (uint64_t)room.count[lg];
        if (!clusters) continue;
        const uint64_t use = clusters < g.groups ? clusters : g.groups;
        const uint64_t busiest = (((g.groups + use - 1u) / use) * g.slots + (1u << lg) - 1u) / (1u << lg);
        const uint64_t cost = (busiest + (even < busiest ? even : busiest) + 1u) / 2u + (lg ? kClusterSlots : 0u);
        if (cost < best) { best = cost; best_cluster = 1u << lg; }
    }
    cluster = best_cluster ? best_cluster : 1u;
    if (best_cluster == 0u) {                                     /* (a single column block forces whole groups) */
        make_flat_plan(g, g.slots, (uint64_t)sms, p, false);
        if (!p.direct) { p.fix = allow_fix ? 1u : 0u; return; }
        cluster = 1u;
    }
    make_flat_plan(g, g.slots, cluster == 1u ? (uint64_t)sms : (uint64_t)room.count[cluster == 2u ? 1 : (cluster == 4u ? 2 : 3)], p, true);
}

/* Off unless switched on (set_pool_kernels): measured on B200 the pool's bookkeeping per stage (+30 % warp instructions)
   costs more than the even finish gains - 263 against 242 us on 128256 x 8192, 122 against 116 us on 57344 x 8192. */
static bool g_disable_pool = true;
void set_pool_kernels(bool on) { g_disable_pool = !on; }

/* Plan of the layout-2 token matvec for a matrix the ring kernels cover.  pool: the kernel whose warps draw stages from a
   pool runs it - equal runs per CTA when the caller allows cut row groups (they are completed inside that kernel), else
   whole row groups per CTA when that plan needs neither a cluster nor a second launch. */
static void choose_ring_plan(int code, const Geometry &g, int input_mode, int sms, bool allow_fix, FlatPlan &plan, uint32_t &cluster, bool &pool) {
    const int elem = type_of(code);
    pool = !g_disable_pool && sms <= (int)kFixCounters && pool_covers(code, g, input_mode);
    if (pool && allow_fix && !g_disable_fixup) {
        Geometry gu = g;
        if (elem == kFp8) gu.slots >>= 1;
        make_flat_plan(gu, gu.slots, (uint64_t)sms, plan, false);
        if (!plan.direct) plan.fix = 1u;
        cluster = 1u;
        return;
    }
    make_cta_plan_layout2(g, elem, ring_ctas(g, input_mode, sms), plan, cluster, allow_fix);
    pool = pool && plan.direct && cluster == 1u;
}

/* kInputPeerNorm: from this many ranks on, the ring kernel's launch is made of clusters that share the sum of the pushed
   partials (build_activation_shared); 0 = never, the default.  Measured on B200 with 8192 values per partial and the same
   kernel before and after: every CTA adding up all of them costs 2.3 / 4.4 / 8.4 us at 2 / 4 / 8 ranks, the clusters
   2.2 / 3.0 / 4.4 us.  In the decode loop of the Llama-3-70B shapes on 2 / 4 / 8 GPUs the clusters nevertheless lose:
   79.4 / 119.1 / 155.2 against 87.0 / 131.0 / 168.8 tokens/s, 3 to 7 us per cluster launch, with clusters of 2 as with
   clusters of 4 - a cluster launch that follows a kernel of single CTAs does not start on the SMs that kernel frees one by
   one, so the overlap that the dependent launch buys (about 4.5 us per boundary) is lost. */
static int g_share_min_world = 0;
void set_peer_sharing(int min_world) { g_share_min_world = min_world; }

/* Decides FusedInput::share for a launch of the layout-2 ring kernel whose plan and cluster size have been chosen: a plan
   that runs clusters anyway shares inside them; a plan of single CTAs is made again for the CTAs that clusters of 4 (else
   2) can occupy at once, if those are nearly all of the device and the plan still wants single CTAs. */
static uint32_t choose_peer_sharing(int code, const Geometry &g, const FusedInput &in, int sms, bool allow_fix, FlatPlan &plan, uint32_t &cluster) {
    const uint32_t live = g.K >> 3;
    if (in.mode != kInputPeerNorm || g_share_min_world <= 0 || (int)in.world < g_share_min_world) return 0u;
    if ((g.K & 7u) != 0u || g.K < 1024u || live > kNormRegChunks * kRingThreads) return 0u;
    if (cluster > 1u) return live % cluster == 0u ? 1u : 0u;
    const ClusterRoom room = cluster_room(sms);
    for (uint32_t lg = 2; lg >= 1u; lg--) {
        const uint32_t size = 1u << lg, ctas = (uint32_t)room.count[lg] * size;
        if (live % size != 0u || (uint64_t)ctas * 100u < (uint64_t)sms * 97u || ctas > (uint32_t)sms) continue;
        FlatPlan p;
        uint32_t c = 1u;
        make_cta_plan_layout2(g, type_of(code), (int)ctas, p, c, allow_fix);
        if (c != 1u || p.warps % size != 0u || p.direct != plan.direct || p.fix != plan.fix) continue;     /* (same number of launches either way) */
        plan = p;
        cluster = size;
        return 3u;
    }
    return 0u;
}

/* ---- layouts 0 and 1, token path: lane streams staged in shared memory by bulk copies -------------------------------- */
/* Same flat work split as above with the block (32 lane streams) as the unit.  A warp's run of blocks is one contiguous
   span of `data`; the stream of block n + 1 is copied into the warp's second stage while block n is decoded, so the
   bit windows refill from shared memory with 32-bit addresses and no lane ever waits for a 4-byte global load.  Raw
   rows still come straight from global memory (coalesced 512 B per row and warp, two rows ahead).
   A block whose stream does not fit a stage (escape-heavy data) is decoded through the global-memory window instead. */
constexpr uint32_t kPrefixThreads = 1024, kPrefixStageBytes = 2560, kPrefixWarpBytes = 2u * kPrefixStageBytes + 256u + 16u;
constexpr uint32_t kPrefixSmemBytes = 16416u + (kPrefixThreads / 32u) * kPrefixWarpBytes;

/* bit window over a stream staged in shared memory; table look-ups form their address with one shift and one IMAD */
template <uint32_t MAX_RANK>
struct SmemWindow {
    uint32_t hi, lo, next, mark, src;
    /* the three opening loads are volatile so they stay behind the wait on the stage's barrier; every later load
       depends on them */
    __device__ __forceinline__ void open(uint32_t addr) { hi = lds32(addr); lo = lds32(addr + 4u); next = lds32(addr + 8u); mark = 1u; src = addr + 12u; }
    /* Drop c & 31 bits.  One fixed instruction sequence: three funnel shifts, the wrap test of the rotating fill mark,
       two 32-bit multiply-adds that drop `next` behind the valid bits, and a predicated reload. */
    __device__ __forceinline__ void consume(uint32_t c) {
        asm("{\n\t"
            ".reg .pred p;\n\t"
            ".reg .b32 nh, nl, nm, mh;\n\t"
            "shf.l.wrap.b32 nh, %1, %0, %5;\n\t"
            "shf.l.wrap.b32 nl, 0, %1, %5;\n\t"
            "shf.l.wrap.b32 nm, %3, %3, %5;\n\t"
            "setp.lt.u32 p, nm, %3;\n\t"
            "selp.u32 mh, nm, 0, p;\n\t"
            "mad.lo.u32 %1, %2, mh, nl;\n\t"          /* on a refill nl is 0, otherwise mh is 0: no carry into the high word */
            "mad.hi.u32 %0, %2, mh, nh;\n\t"
            "mov.u32 %3, nm;\n\t"
            "@p ld.shared.u32 %2, [%4];\n\t"
            "@p add.u32 %4, %4, 4;\n\t"
            "}" : "+r"(hi), "+r"(lo), "+r"(next), "+r"(mark), "+r"(src) : "r"(c));
    }
    __device__ __forceinline__ uint32_t look(uint32_t word, uint32_t table, uint32_t four) const {
        uint32_t e;
        asm("{\n\t.reg .b32 i, a;\n\tshr.u32 i, %1, 20;\n\tmad.lo.u32 a, i, %2, %3;\n\tld.shared.u32 %0, [a];\n\t}" : "=r"(e) : "r"(word), "r"(four), "r"(table));
        return e;
    }
    __device__ __forceinline__ uint32_t one(uint32_t sym) {
        const uint32_t h = hi, zeros = min((uint32_t)__clz((int)h), 15u);
        if (MAX_RANK == kMaxRankFp8 || zeros < MAX_RANK) {
            uint32_t s8; asm volatile("ld.shared.u8 %0, [%1];" : "=r"(s8) : "r"(sym + zeros));
            const uint32_t b = (((h >> (30u - zeros)) & 1u) << 7) | s8;
            consume(zeros + 2u);
            return b;
        }
        consume(16u);
        const uint32_t b = hi >> 24;
        consume(8u);
        return b;
    }
    __device__ __forceinline__ uint32_t pair(uint32_t table, uint32_t sym, uint32_t four) {
        const uint32_t e = look(hi, table, four);
        if (e < kEscape) { consume(e); return e; }
        uint32_t b0 = (e >> 8) & 0xFFu;
        if (e & (1u << 24)) consume(e); else b0 = one(sym);
        const uint32_t b1 = one(sym);
        return (b0 << 8) | (b1 << 16);
    }
    /* Four symbols.  Both look-ups and the single advance are straight-line code; a lane that meets a flagged entry
       decodes pair by pair in a side branch (advancing its window itself) and joins the common advance with a shift
       of zero. */
    __device__ __forceinline__ void quad(uint32_t table, uint32_t sym, uint32_t four, uint32_t &e01, uint32_t &e23) {
        uint32_t a = look(hi, table, four);
        uint32_t b = look(__funnelshift_l(0u, hi, a), table, four);
        uint32_t c = a + b;
        if (((a | b) & kEscape) != 0u) { a = pair(table, sym, four); b = pair(table, sym, four); c = 0u; }
        consume(c);
        e01 = a; e23 = b;
    }
};
/* the global-memory window behind the same interface (oversize blocks) */
template <uint32_t MAX_RANK>
struct GlobalWindow : BitWindow<MAX_RANK> {
    const uint8_t *sym_ptr;
    __device__ __forceinline__ void quad(uint32_t table, uint32_t, uint32_t, uint32_t &e01, uint32_t &e23) { BitWindow<MAX_RANK>::quad(table, sym_ptr, e01, e23); }
};

/* One layout-0 block: 8 rows x 16 columns per lane.  Even rows enter the mma as the "row r" half of the A fragment, odd
   rows as the "row r + 8" half (both rows meet the same columns of x); after two rows the diagonal of D holds the lane
   quads' dot products. */
/* the low bytes of the first two rows of a lane's 8 x 16 cell of block (rb, cb): constants, so a caller may fetch them early */
template <int ELEM>
__device__ __forceinline__ void first_raw_rows(const SegmentArgs &a, const Geometry &g, uint32_t rb, uint32_t cb, uint32_t lane, uint4 &raw0, uint4 &raw1) {
    const uint32_t row0 = rb * 8u, col0 = cb * kBlockCols + lane * 16u, stride = ELEM == kFp8 ? (g.K16 >> 1) : g.K16;
    const bool col_ok = col0 < g.K16;
    const uint8_t *rawp = a.low + (uint64_t)row0 * stride + (ELEM == kFp8 ? (col0 >> 1) : col0);
    raw0 = raw_row16<ELEM>(rawp, col_ok && row0 < g.M); raw1 = raw_row16<ELEM>(rawp + stride, col_ok && row0 + 1u < g.M);
}

template <class WIN, int ELEM, bool XF32>
__device__ __forceinline__ float prefix_block_layout0(WIN &W, const SegmentArgs &a, const Geometry &g, uint32_t rb, uint32_t cb, uint32_t lane,
                                                      uint32_t table, uint32_t sym, uint32_t four, float *stash, uint32_t xs = 0u, const uint4 *early_rows = nullptr) {
    const uint32_t r = lane >> 2, q = lane & 3u, row0 = rb * 8u, col0 = cb * kBlockCols + lane * 16u;
    const uint32_t stride = ELEM == kFp8 ? (g.K16 >> 1) : g.K16;
    const bool col_ok = col0 < g.K16, diag = q == (r >> 1);
    XFrag8<XF32> xa, xb;
    if (!col_ok) { xa.zero(); xb.zero(); }
    else if (!XF32 && xs) { xa.load_shared(xs + col0 * 2u); xb.load_shared(xs + col0 * 2u + 16u); }     /* x staged by the CTA */
    else { xa.load(a.x, col0); xb.load(a.x, col0 + 8u); }
    const uint8_t *rawp = a.low + (uint64_t)row0 * stride + (ELEM == kFp8 ? (col0 >> 1) : col0);
    uint4 raw0, raw1;
    if (early_rows) { raw0 = early_rows[0]; raw1 = early_rows[1]; }
    else { raw0 = raw_row16<ELEM>(rawp, col_ok && row0 < g.M); raw1 = raw_row16<ELEM>(rawp + stride, col_ok && row0 + 1u < g.M); }
#pragma unroll 1
    for (uint32_t rp = 0; rp < 4u; rp++) {
        const uint4 rawA = raw0, rawB = raw1;
        if (rp < 3u) {
            raw0 = raw_row16<ELEM>(rawp + (uint64_t)(2u * rp + 2u) * stride, col_ok && row0 + 2u * rp + 2u < g.M);
            raw1 = raw_row16<ELEM>(rawp + (uint64_t)(2u * rp + 3u) * stride, col_ok && row0 + 2u * rp + 3u < g.M);
        }
        float d[4] = {0.f, 0.f, 0.f, 0.f};
        const uint32_t wa[4] = {rawA.x, rawA.y, rawA.z, rawA.w}, wb[4] = {rawB.x, rawB.y, rawB.z, rawB.w};
        /* the even row's fragments wait in registers until the odd row is decoded: one mma then takes both rows */
        uint32_t even0[4], even1[4];
#pragma unroll
        for (int k = 0; k < 4; k++) {
            uint32_t e01, e23; W.quad(table, sym, four, e01, e23);
            even0[k] = weave<0>(wa[k], e01); even1[k] = weave<2>(wa[k], e23);
        }
#pragma unroll
        for (int k = 0; k < 4; k++) {
            uint32_t e01, e23; W.quad(table, sym, four, e01, e23);
            const XFrag8<XF32> &xf = k < 2 ? xa : xb;
            const int w = 2 * (k & 1);
            const uint32_t p0 = weave<0>(wb[k], e01), p1 = weave<2>(wb[k], e23);
            mma_bf16(d, even0[k], p0, even1[k], p1, xf.head[w], xf.head[w + 1]);
            if (XF32) mma_bf16(d, even0[k], p0, even1[k], p1, xf.tail[w], xf.tail[w + 1]);
        }
        if (diag) {
            stash[(2u * rp) * 8u + r] = (r & 1u) ? d[1] : d[0];
            stash[(2u * rp + 1u) * 8u + r] = (r & 1u) ? d[3] : d[2];
        }
    }
    __syncwarp();
    float sum = 0.f;
    if (lane < 8u) {
        const float4 s0 = *reinterpret_cast<const float4 *>(stash + lane * 8u), s1 = *reinterpret_cast<const float4 *>(stash + lane * 8u + 4u);
        sum = ((s0.x + s0.y) + (s0.z + s0.w)) + ((s1.x + s1.y) + (s1.z + s1.w));
    }
    __syncwarp();
    return sum;
}

/* One layout-1 block (16 rows x 512 columns, stored in A-fragment order): `nsc` super-chunks of 16 weights per lane, raw
   low bytes one slot ahead from the plane, the sums stay in the mma accumulators d (rows r and r + 8 of lane group r). */
template <class WIN, int ELEM>
__device__ __forceinline__ void prefix_block_layout1(WIN &W, const SegmentArgs &a, const Geometry &g, uint32_t rb, uint32_t cb, uint32_t lane,
                                                     uint32_t table, uint32_t sym, uint32_t four, float (&d)[4], uint32_t xs = 0u) {
    constexpr uint32_t RB = ELEM == kFp8 ? 8u : 16u;             /* raw bytes per lane and super-chunk */
    const uint32_t q = lane & 3u, nsc = g.supers_in(cb);
    const uint8_t *rp = a.low + ((uint64_t)(rb * g.slots + cb * 16u) * kLanes + lane) * RB;
    uint4 ahead = ELEM == kFp8 ? expand_nibbles(ldg_stream64(rp)) : ldg_stream128(rp);
#pragma unroll 1
    for (uint32_t sc = 0; sc < nsc; sc++) {
        const uint4 cw = ahead;
        rp += kLanes * RB;                                       /* one slot ahead, unguarded: the plane carries 512 B of slack */
        ahead = ELEM == kFp8 ? expand_nibbles(ldg_stream64(rp)) : ldg_stream128(rp);
        XFrag8<false> xf;
        if (xs) xf.load_shared(xs + (cb * kBlockCols + sc * 32u + 8u * q) * 2u);           /* x staged by the CTA */
        else xf.load(a.x, cb * kBlockCols + sc * 32u + 8u * q);
        const uint32_t c[4] = {cw.x, cw.y, cw.z, cw.w};
#pragma unroll
        for (int h = 0; h < 2; h++) {
            uint32_t e0, e1, e2, e3;
            W.quad(table, sym, four, e0, e1); W.quad(table, sym, four, e2, e3);
            mma_bf16(d, weave<0>(c[2 * h], e0), weave<2>(c[2 * h], e1), weave<0>(c[2 * h + 1], e2), weave<2>(c[2 * h + 1], e3), xf.head[2 * h], xf.head[2 * h + 1]);
        }
    }
    __syncwarp();                                                /* all lanes are done with the stage that held this block */
}

/* in.mode != kInputPlain (bf16 x only): the CTA builds the activation vector itself in shared memory behind the rings
   (RMSNorm of the residual stream or SwiGLU of a gate/up vector, as in the layout-2 kernel), so nwc_linear_fused needs no
   prologue launch; the launcher takes this form only when the vector and the norm weights' registers suffice. */
template <int LAYOUT, int ELEM, bool XF32, uint32_t THREADS, uint32_t STAGE>
__device__ __forceinline__ void prefix_ring_body(const SegmentArgs &a, const FlatPlan &plan, const uint32_t four, const FusedInput &in) {
    constexpr uint32_t kWarpBytes = 2u * STAGE + 256u + 16u;
    constexpr uint32_t MR = ELEM == kFp8 ? kMaxRankFp8 : kMaxRankBf16;
    extern __shared__ __align__(128) uint8_t ring_smem[];
    uint32_t *tables = reinterpret_cast<uint32_t *>(ring_smem);
    stage_tables(tables, a.lut, threadIdx.x, THREADS);
    uint32_t xs_addr = 0u;
    if (!XF32 && in.mode != kInputPlain) {                       /* (uniform over the grid; before any warp leaves: it ends with a CTA barrier) */
        const Geometry gx(a.M, a.K, LAYOUT);
        uint8_t *behind = ring_smem + 16416u + (THREADS / 32u) * kWarpBytes;
        float *scal = reinterpret_cast<float *>(behind);
        uint16_t *xs = reinterpret_cast<uint16_t *>(behind + 128u);
        NormWeights norm_regs;
        stage_norm_weight<THREADS>(in, a.K, xs, norm_regs);     /* (the weights fit the registers: the launcher checked) */
        build_activation<THREADS>(in, a.x, a.K, (gx.K16 + 31u) & ~31u, xs, xs, scal, norm_regs);      /* zero up to the end of the last 32-column slot (layout 1 reads whole slots) */
        xs_addr = smem_addr(xs);
    }
    const uint32_t lane = threadIdx.x & 31u, warp = threadIdx.x >> 5;
    const uint32_t table = smem_addr(tables), sym = table + 4u * kTableWords;
    uint8_t *mine = ring_smem + 16416u + warp * kWarpBytes;
    const uint32_t stages = smem_addr(mine), bars = stages + 2u * STAGE + 256u;
    float *stash = reinterpret_cast<float *>(mine + 2u * STAGE);
    const Geometry g(a.M, a.K, LAYOUT);
    const uint32_t w = warp * gridDim.x + blockIdx.x;           /* interleaved: a short plan still spreads over all SMs */
    if (w >= plan.warps) return;
    const uint32_t b0 = plan.start(w), b1 = plan.start(w + 1u);
    if (lane == 0) { mbar_init(bars, 1u); mbar_init(bars + 8u, 1u); mbar_init_fence(); }
    __syncwarp();
    /* byte span of block b inside data: [start, start + bytes), rounded out to 16; bytes == 0 means "does not fit a stage" */
    auto span = [&](uint32_t b, uint32_t words_of_b, uint32_t &start, uint32_t &bytes) {
        const uint32_t base = __ldg(a.bases + b);
        uint32_t len;
        if (b + 1u < g.nb) len = __ldg(a.bases + b + 1u) - base;
        else { uint32_t t; warp_exclusive_sum(words_of_b, lane, t); len = 4u * t; }
        start = base & ~15u;
        bytes = (base + len + 16u - start + 15u) & ~15u;          /* + 16: the windows read up to three words past a stream */
        if (bytes > STAGE) bytes = 0u;
    };
    auto issue = [&](uint32_t b, uint32_t words_of_b) {
        uint32_t start, bytes; span(b, words_of_b, start, bytes);
        if (bytes && lane == 0) {
            const uint32_t buf = (b - b0) & 1u;
            async_proxy_fence();
            mbar_expect(bars + buf * 8u, bytes);
            bulk_load(stages + buf * STAGE, a.data + start, bytes, bars + buf * 8u);
        }
    };
    uint32_t words = __ldg(a.hdr + (uint64_t)b0 * kLanes + lane);
    uint32_t words_next = b0 + 1u < b1 ? __ldg(a.hdr + (uint64_t)(b0 + 1u) * kLanes + lane) : 0u;
    issue(b0, words);
    if (b0 + 1u < b1) issue(b0 + 1u, words_next);
    uint32_t rb = b0 / g.CB, cb = b0 - rb * g.CB, phase_bits = 0;
    float row_sum = 0.f, d[4] = {0.f, 0.f, 0.f, 0.f};     /* layout 0: the 8 row sums in lanes 0..7; layout 1: mma accumulators */
    for (uint32_t b = b0; b < b1; b++) {
        const uint32_t words_after = b + 2u < b1 ? __ldg(a.hdr + (uint64_t)(b + 2u) * kLanes + lane) : 0u;
        uint32_t start, bytes, total; span(b, words, start, bytes);
        const uint32_t before = warp_exclusive_sum(words, lane, total), buf = (b - b0) & 1u, base = __ldg(a.bases + b);
        if (bytes) {
            if (!mbar_wait(bars + buf * 8u, (phase_bits >> buf) & 1u)) {
                for (uint32_t i = 0; i < 64u && !mbar_poll(bars + (buf ^ 1u) * 8u, (phase_bits >> (buf ^ 1u)) & 1u); i++) {}
                return;
            }
            phase_bits ^= 1u << buf;
            SmemWindow<MR> W; W.open(stages + buf * STAGE + (base - start) + 4u * before);
            if (LAYOUT == 0) row_sum += prefix_block_layout0<SmemWindow<MR>, ELEM, XF32>(W, a, g, rb, cb, lane, table, sym, four, stash, xs_addr);
            else prefix_block_layout1<SmemWindow<MR>, ELEM>(W, a, g, rb, cb, lane, table, sym, four, d, xs_addr);
        } else {
            GlobalWindow<MR> W; W.sym_ptr = reinterpret_cast<const uint8_t *>(tables + kTableWords);
            W.open(reinterpret_cast<const uint32_t *>(a.data + base) + before);
            if (LAYOUT == 0) row_sum += prefix_block_layout0<GlobalWindow<MR>, ELEM, XF32>(W, a, g, rb, cb, lane, table, sym, four, stash, xs_addr);
            else prefix_block_layout1<GlobalWindow<MR>, ELEM>(W, a, g, rb, cb, lane, table, sym, four, d, xs_addr);
        }
        if (b + 2u < b1) issue(b + 2u, words_after);              /* the stage just decoded is free again (all lanes passed the block's last __syncwarp) */
        words = words_next; words_next = words_after;
        if (++cb == g.CB || b + 1u == b1) {                       /* the warp's share of this row group is complete */
            const uint32_t part = w - plan.owner(rb * g.CB);
            if (LAYOUT == 0) { if (lane < 8u) emit_flat(a, plan, rb * 8u + lane, part, row_sum); }
            else if ((lane & 3u) == 0u) { emit_flat(a, plan, rb * 16u + (lane >> 2), part, d[0]); emit_flat(a, plan, rb * 16u + (lane >> 2) + 8u, part, d[2]); }
            row_sum = 0.f; d[0] = d[1] = d[2] = d[3] = 0.f;
            if (cb == g.CB) { cb = 0; rb++; }
        }
    }
}

template <int ELEM, bool XF32>
__global__ void __launch_bounds__(kPrefixThreads, 1) prefix_ring_kernel_layout0(const SegmentArgs a, const FlatPlan plan, const uint32_t four, const FusedInput in) {
    prefix_ring_body<0, ELEM, XF32, kPrefixThreads, kPrefixStageBytes>(a, plan, four, in);
}
/* layout 1: a block is 16 x 512 (twice the stream), so half as many warps with stages twice as large; x is bf16 */
constexpr uint32_t kPrefix1Threads = 512, kPrefix1StageBytes = 4608;
constexpr uint32_t kPrefix1SmemBytes = 16416u + (kPrefix1Threads / 32u) * (2u * kPrefix1StageBytes + 256u + 16u);
/* shared memory behind the rings when the kernel builds x itself: 128 bytes of reduction scratch + the vector */
static inline size_t prefix_fused_bytes(const Geometry &g) { return 128u + (size_t)((g.K16 + 31u) & ~31u) * 2u; }
/* the layout 0 / 1 ring kernel can build x for this matrix: the vector fits behind the rings and the RMSNorm weights fit the
   registers of the threads that normalise them (or K is not a multiple of 8: the scalar path reads them from memory) */
static inline bool prefix_ring_fuses(int code, const Geometry &g, int input_mode) {
    const int layout = layout_of(code);
    if (layout > 1 || input_mode == kInputPlain || input_mode == kInputPeerNorm) return false;
    const uint32_t threads = layout == 0 ? kPrefixThreads : kPrefix1Threads;
    const size_t rings = layout == 0 ? kPrefixSmemBytes : kPrefix1SmemBytes;
    if (rings + prefix_fused_bytes(g) > kRingMaxSmem) return false;
    return (g.K & 7u) != 0u || (g.K >> 3) <= kNormRegChunks * threads;
}
template <int ELEM>
__global__ void __launch_bounds__(kPrefix1Threads, 1) prefix_ring_kernel_layout1(const SegmentArgs a, const FlatPlan plan, const uint32_t four, const FusedInput in) {
    prefix_ring_body<1, ELEM, false, kPrefix1Threads, kPrefix1StageBytes>(a, plan, four, in);
}

/* ---- layout 0, small matrices of the decode step: one launch, activation prologue fused ------------------------------ */
/* A decoder layer's matrices hold at most one block per resident warp on a B200, so their cost is launch latency plus
   the serial decode of one block, and every extra launch (norm, activation, finalize) costs as much as the matvec.
   Here a CTA of 8 warps owns whole row groups: the warps of a row group split its column blocks, add their row sums
   through shared memory in warp order and write bf16 y themselves.  The activation vector is built once per CTA in
   shared memory, optionally from the residual stream (h_out = h_in + delta, x = RMSNorm(h_out) * w) or from a fused
   gate/up vector (x = silu(gate) * up), with the rounding steps of the separate kernels in nwc_model.cu.
   Everything that does not depend on the previous kernel (table staging) runs before griddepcontrol.wait, so with
   programmatic dependent launch it overlaps the predecessor's tail. */
constexpr uint32_t kSmallThreads = 256, kSmallWarps = kSmallThreads / 32u;
/* warps that share one row group: the smallest power of two that covers its column blocks (at most the CTA) */
__host__ __device__ static inline uint32_t small_group_warps(uint32_t CB) { return CB > 4u ? 8u : (CB > 2u ? 4u : (CB > 1u ? 2u : 1u)); }

constexpr uint32_t kSmallResident = 2;      /* CTAs of the small kernel per SM the register budget is set for */
template <int ELEM>
__global__ void __launch_bounds__(kSmallThreads, kSmallResident) small_kernel_layout0(const SegmentArgs a, const FusedInput in, const uint32_t four) {
    constexpr uint32_t MR = ELEM == kFp8 ? kMaxRankFp8 : kMaxRankBf16;
    extern __shared__ __align__(128) uint8_t small_smem[];
    uint32_t *tables = reinterpret_cast<uint32_t *>(small_smem);
    float *stash_all = reinterpret_cast<float *>(small_smem + 16416u);                 /* [8 warps][64] */
    float *red = stash_all + kSmallWarps * 64u;                                         /* [8 warps][8 rows] */
    float *scal = red + kSmallWarps * 8u;                                               /* [8] block reduction scratch */
    uint8_t *stage_all = reinterpret_cast<uint8_t *>(scal + 8u);                        /* [8 warps][2][kPrefixStageBytes] lane streams of a block */
    uint64_t *bar_all = reinterpret_cast<uint64_t *>(stage_all + kSmallWarps * 2u * kPrefixStageBytes);
    uint16_t *xs = reinterpret_cast<uint16_t *>(bar_all + 2u * kSmallWarps);            /* [K16] activation vector */
    const uint32_t lane = threadIdx.x & 31u, warp = threadIdx.x >> 5, tid = threadIdx.x;
    const Geometry g(a.M, a.K, 0);
    uint16_t *nw = xs + g.K16;                                                         /* [K16] RMSNorm weight (kInputNorm only) */
    const uint32_t stage0 = smem_addr(stage_all) + warp * 2u * kPrefixStageBytes, bar0 = smem_addr(bar_all) + warp * 16u;
    if (lane == 0) { mbar_init(bar0, 1u); mbar_init(bar0 + 8u, 1u); mbar_init_fence(); }
    __syncwarp();
    /* byte span of block b inside data, rounded out to 16 bytes, and the bulk copy of it into stage `which` of this
       warp; returns 0 (no copy) when the stream does not fit the stage */
    auto fetch = [&](uint32_t b, uint32_t words_of_b, uint32_t which, uint32_t &start) -> uint32_t {
        const uint32_t base = __ldg(a.bases + b);
        uint32_t len;
        if (b + 1u < g.nb) len = __ldg(a.bases + b + 1u) - base;
        else { uint32_t t; warp_exclusive_sum(words_of_b, lane, t); len = 4u * t; }
        start = base & ~15u;
        uint32_t bytes = (base + len + 16u - start + 15u) & ~15u;
        if (bytes > kPrefixStageBytes) bytes = 0u;
        if (bytes && lane == 0) { async_proxy_fence(); mbar_expect(bar0 + 8u * which, bytes); bulk_load(stage0 + which * kPrefixStageBytes, a.data + start, bytes, bar0 + 8u * which); }
        return bytes;
    };
    /* warps per row group and row groups per CTA pass; warp j of a row group takes column blocks j, j + wg, ... */
    const uint32_t wg = small_group_warps(g.CB), per_pass = kSmallWarps / wg;
    const uint32_t my_group = warp / wg, j = warp - my_group * wg, passes = (g.groups + per_pass - 1u) / per_pass;
    /* this warp's blocks in the order it decodes them: (pass, cb) -> the next one, false after the last */
    auto settle = [&](uint32_t &pass, uint32_t &cb) -> bool {
        while (pass < passes) {
            if (pass * per_pass + my_group < g.groups && cb < g.CB) return true;
            pass += gridDim.x; cb = j;
        }
        return false;
    };
    /* the stream of the block after the current one is always in flight: issued before the current block is decoded */
    struct Ahead { uint32_t pass, cb, b, words, start, bytes; bool valid; } next;
    auto prefetch_block = [&](uint32_t pass, uint32_t cb, uint32_t which) {
        next.pass = pass; next.cb = cb; next.valid = settle(next.pass, next.cb);
        if (!next.valid) return;
        const uint32_t rb = next.pass * per_pass + my_group;
        next.b = rb * g.CB + next.cb;
        next.words = __ldg(a.hdr + (uint64_t)next.b * kLanes + lane);
        next.bytes = fetch(next.b, next.words, which, next.start);
        const uint32_t stride = ELEM == kFp8 ? (g.K16 >> 1) : g.K16, row = rb * 8u + (lane >> 2), off = next.cb * (ELEM == kFp8 ? 256u : 512u) + (lane & 3u) * 128u;
        if (row < g.M && off < stride) prefetch_l2(a.low + (uint64_t)row * stride + off);
    };
    /* the weights do not depend on the kernel before this one: start the copy of this warp's first stream and pull its
       raw rows towards L2 before anything else, so that both overlap the table staging, the wait and the prologue */
    prefetch_block(blockIdx.x, j, 0u);
    /* the first two raw rows of that block as well: the decode loop then starts without a trip to L2 */
    uint4 early_rows[2] = {make_uint4(0u, 0u, 0u, 0u), make_uint4(0u, 0u, 0u, 0u)};
    const uint32_t early_block = next.valid ? next.b : 0xFFFFFFFFu;
    if (next.valid) first_raw_rows<ELEM>(a, g, next.pass * per_pass + my_group, next.cb, lane, early_rows[0], early_rows[1]);
    stage_tables(tables, a.lut, tid, kSmallThreads);
    NormWeights norm_regs;
    stage_norm_weight<kSmallThreads>(in, a.K, nw, norm_regs);
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    asm volatile("griddepcontrol.wait;" ::: "memory");
    build_activation<kSmallThreads>(in, a.x, a.K, g.K16, xs, nw, scal, norm_regs);
    const uint32_t xs_addr = smem_addr(xs);
    const uint32_t table = smem_addr(tables), sym = table + 4u * kTableWords;
    float *stash = stash_all + warp * 64u;
    uint32_t phases = 0, which = 0;                              /* parity per stage; the stage that holds the current block */
    for (uint32_t pass = blockIdx.x; pass < passes; pass += gridDim.x) {
        const uint32_t rb = pass * per_pass + my_group;
        float row_sum = 0.f;
        if (rb < g.groups) {
            for (uint32_t cb = j; cb < g.CB; cb += wg) {
                const Ahead cur = next;                           /* by construction (pass, cb) == (cur.pass, cur.cb) */
                prefetch_block(pass, cb + wg, which ^ 1u);
                uint32_t total;
                const uint32_t before = warp_exclusive_sum(cur.words, lane, total), base = __ldg(a.bases + cur.b);
                if (cur.bytes) {
                    const bool landed = mbar_wait(bar0 + 8u * which, (phases >> which) & 1u);    /* on a timeout the status word is set and the block is skipped; the CTA's barriers below still need this warp */
                    phases ^= 1u << which;
                    if (landed) {
                        SmemWindow<MR> W; W.open(stage0 + which * kPrefixStageBytes + (base - cur.start) + 4u * before);
                        row_sum += prefix_block_layout0<SmemWindow<MR>, ELEM, false>(W, a, g, rb, cb, lane, table, sym, four, stash, xs_addr,
                                                                                     cur.b == early_block ? early_rows : nullptr);
                    }
                } else {
                    GlobalWindow<MR> W; W.sym_ptr = reinterpret_cast<const uint8_t *>(tables + kTableWords);
                    W.open(reinterpret_cast<const uint32_t *>(a.data + base) + before);
                    row_sum += prefix_block_layout0<GlobalWindow<MR>, ELEM, false>(W, a, g, rb, cb, lane, table, sym, four, stash, xs_addr);
                }
                which ^= 1u;
            }
        }
        if (lane < 8u) red[warp * 8u + lane] = row_sum;
        __syncthreads();
        if (j == 0u && lane < 8u && rb < g.groups) {
            float v = 0.f;
            for (uint32_t k = 0; k < wg; k++) v += red[(warp + k) * 8u + lane];
            const uint32_t row = rb * 8u + lane;
            if (row < a.M) {
                if (a.scale) v *= __ldg(a.scale + row);
                if (a.bias) v += bf16_to_float(__ldg(a.bias + row));
                a.y[row] = bf16_round(v);
            }
        }
        __syncthreads();
    }
}

/* ---- layout 0, small matrices, four warps per block --------------------------------------------------------------- */
/* A lane's stream of a layout-0 block is 128 symbols that only one lane can walk from bit 0: 32 dependent four-symbol
   steps, about 5 us, whatever the GPU.  The side table breaks that chain: for every block and lane it holds the bit
   position at which rows 2, 4 and 6 begin (3 x 32 x 2 bytes per block; built once when a matrix is loaded, never stored in
   checkpoints).  A TEAM of four warps then decodes one block, warp r the row pair (2r, 2r + 1): eight dependent steps
   instead of 32.  A CTA is two teams; the teams of a CTA split the column blocks of the row group(s) they own and add up
   through shared memory; the block's stream is copied once per team (double-buffered bulk copies, one mbarrier per stage,
   a 128-thread named barrier frees a stage for its next copy). */
constexpr uint32_t kSplitThreads = 256, kSplitTeams = 2, kSplitTeamWarps = 4;
constexpr uint32_t kSideBytesPerBlock = 3u * kLanes * 2u;

/* one thread per lane stream: walk 96 symbols with the code's length rule (r zeros, a one, the sign: r + 2 bits; bf16
   ranks beyond 14: 24 bits) and record the bit positions after 32, 64 and 96 symbols */
template <int ELEM>
__global__ void side_table_kernel(const uint8_t *__restrict__ data, const uint32_t *__restrict__ bases, const uint8_t *__restrict__ hdr, uint16_t *__restrict__ side, uint32_t nb) {
    constexpr uint32_t MR = ELEM == kFp8 ? kMaxRankFp8 : kMaxRankBf16;
    const uint32_t lane = threadIdx.x & 31u, b = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (b >= nb) return;
    uint32_t total;
    const uint32_t words = __ldg(hdr + (uint64_t)b * kLanes + lane), before = warp_exclusive_sum(words, lane, total);
    const uint32_t *stream = reinterpret_cast<const uint32_t *>(data + __ldg(bases + b)) + before;
    uint32_t pos = 0;
    for (uint32_t part = 0; part < 3u; part++) {
        for (uint32_t i = 0; i < 32u; i++) {
            const uint32_t w = pos >> 5, v = __funnelshift_l(__ldg(stream + w + 1u), __ldg(stream + w), pos & 31u);
            const uint32_t zeros = min((uint32_t)__clz((int)v), 15u);
            pos += (ELEM == kFp8 || zeros < MR) ? zeros + 2u : 24u;
        }
        side[((uint64_t)b * 3u + part) * kLanes + lane] = (uint16_t)pos;
    }
}

/* rows (2 rp, 2 rp + 1) of one block for this warp: returns the quad partial sums through `stash` (16 floats), lane 0 / 1 then
   hold the sums of the even / odd row over the block's 512 columns */
template <class WIN, int ELEM>
__device__ __forceinline__ float split_row_pair(WIN &W, const SegmentArgs &a, const Geometry &g, uint32_t rb, uint32_t cb, uint32_t rp, uint32_t lane,
                                                uint32_t table, uint32_t sym, uint32_t four, float *stash, uint32_t xs) {
    const uint32_t r = lane >> 2, q = lane & 3u, row0 = rb * 8u + 2u * rp, col0 = cb * kBlockCols + lane * 16u;
    const uint32_t stride = ELEM == kFp8 ? (g.K16 >> 1) : g.K16;
    const bool col_ok = col0 < g.K16, diag = q == (r >> 1);
    XFrag8<false> xa, xb;
    if (!col_ok) { xa.zero(); xb.zero(); } else { xa.load_shared(xs + col0 * 2u); xb.load_shared(xs + col0 * 2u + 16u); }
    const uint8_t *rawp = a.low + (uint64_t)row0 * stride + (ELEM == kFp8 ? (col0 >> 1) : col0);
    const uint4 rawA = raw_row16<ELEM>(rawp, col_ok && row0 < g.M), rawB = raw_row16<ELEM>(rawp + stride, col_ok && row0 + 1u < g.M);
    float d[4] = {0.f, 0.f, 0.f, 0.f};
    const uint32_t wa[4] = {rawA.x, rawA.y, rawA.z, rawA.w}, wb[4] = {rawB.x, rawB.y, rawB.z, rawB.w};
    uint32_t even0[4], even1[4];
#pragma unroll
    for (int k = 0; k < 4; k++) {
        uint32_t e01, e23; W.quad(table, sym, four, e01, e23);
        even0[k] = weave<0>(wa[k], e01); even1[k] = weave<2>(wa[k], e23);
    }
#pragma unroll
    for (int k = 0; k < 4; k++) {
        uint32_t e01, e23; W.quad(table, sym, four, e01, e23);
        const XFrag8<false> &xf = k < 2 ? xa : xb;
        const int w = 2 * (k & 1);
        mma_bf16(d, even0[k], weave<0>(wb[k], e01), even1[k], weave<2>(wb[k], e23), xf.head[w], xf.head[w + 1]);
    }
    if (diag) { stash[r] = (r & 1u) ? d[1] : d[0]; stash[8u + r] = (r & 1u) ? d[3] : d[2]; }
    __syncwarp();
    float sum = 0.f;
    if (lane < 2u) {
        const float4 s0 = *reinterpret_cast<const float4 *>(stash + lane * 8u), s1 = *reinterpret_cast<const float4 *>(stash + lane * 8u + 4u);
        sum = ((s0.x + s0.y) + (s0.z + s0.w)) + ((s1.x + s1.y) + (s1.z + s1.w));
    }
    __syncwarp();
    return sum;
}

template <int ELEM>
__global__ void __launch_bounds__(kSplitThreads, 3) small_split_kernel_layout0(const SegmentArgs a, const FusedInput in, const uint32_t four, const uint16_t *__restrict__ side) {
    constexpr uint32_t MR = ELEM == kFp8 ? kMaxRankFp8 : kMaxRankBf16;
    extern __shared__ __align__(128) uint8_t small_smem[];
    uint32_t *tables = reinterpret_cast<uint32_t *>(small_smem);
    float *stash_all = reinterpret_cast<float *>(small_smem + 16416u);                 /* [8 warps][16] */
    float *red = stash_all + 8u * 16u;                                                  /* [2 teams][8 rows] */
    float *scal = red + kSplitTeams * 8u;                                               /* [8] block reduction scratch */
    uint8_t *stage_all = reinterpret_cast<uint8_t *>(scal + 8u);                        /* [2 teams][2][kPrefixStageBytes] */
    uint64_t *bar_all = reinterpret_cast<uint64_t *>(stage_all + kSplitTeams * 2u * kPrefixStageBytes);
    uint16_t *xs = reinterpret_cast<uint16_t *>(bar_all + 2u * kSplitTeams);            /* [K16] activation vector */
    const uint32_t lane = threadIdx.x & 31u, warp = threadIdx.x >> 5, tid = threadIdx.x;
    const uint32_t team = warp >> 2, rp = warp & 3u;                                    /* this warp's team and row pair */
    const Geometry g(a.M, a.K, 0);
    uint16_t *nw = xs + g.K16;
    const uint32_t stage0 = smem_addr(stage_all) + team * 2u * kPrefixStageBytes, bar0 = smem_addr(bar_all) + team * 16u;
    if (rp == 0u && lane == 0) { mbar_init(bar0, 1u); mbar_init(bar0 + 8u, 1u); mbar_init_fence(); }
    /* teams per row group: both teams share a row group with several column blocks, else each takes its own row group */
    const uint32_t share = g.CB > 1u ? kSplitTeams : 1u, per_pass = kSplitTeams / share;
    const uint32_t my_group = team / share, j = team - my_group * share, passes = (g.groups + per_pass - 1u) / per_pass;
    /* the team's blocks in decode order; (pass, cb) -> next valid one */
    auto settle = [&](uint32_t &pass, uint32_t &cb) -> bool {
        while (pass < passes) {
            if (pass * per_pass + my_group < g.groups && cb < g.CB) return true;
            pass += gridDim.x; cb = j;
        }
        return false;
    };
    struct Ahead { uint32_t pass, cb, b, words, start, bytes, bit; bool valid; } next;
    /* metadata of the team's block after (pass, cb) - header, offsets and this lane's side-table entry, all loads in flight
       one block ahead - and, by the team's first lane, the bulk copy of its stream into stage `which`; every warp of the
       team runs this with the same arguments */
    auto prefetch_block = [&](uint32_t pass, uint32_t cb, uint32_t which) {
        next.pass = pass; next.cb = cb; next.valid = settle(next.pass, next.cb);
        if (!next.valid) return;
        const uint32_t rb = next.pass * per_pass + my_group;
        next.b = rb * g.CB + next.cb;
        next.words = __ldg(a.hdr + (uint64_t)next.b * kLanes + lane);
        next.bit = rp ? (uint32_t)__ldg(side + ((uint64_t)next.b * 3u + (rp - 1u)) * kLanes + lane) : 0u;     /* where this lane's row pair starts */
        const uint32_t base = __ldg(a.bases + next.b);
        uint32_t len;
        if (next.b + 1u < g.nb) len = __ldg(a.bases + next.b + 1u) - base;
        else { uint32_t t; warp_exclusive_sum(next.words, lane, t); len = 4u * t; }
        next.start = base & ~15u;
        next.bytes = (base + len + 16u - next.start + 15u) & ~15u;
        if (next.bytes > kPrefixStageBytes) next.bytes = 0u;
        if (next.bytes && rp == 0u && lane == 0) {
            async_proxy_fence(); mbar_expect(bar0 + 8u * which, next.bytes);
            bulk_load(stage0 + which * kPrefixStageBytes, a.data + next.start, next.bytes, bar0 + 8u * which);
        }
        const uint32_t stride = ELEM == kFp8 ? (g.K16 >> 1) : g.K16, row = rb * 8u + 2u * rp + (lane >> 4), off = next.cb * (ELEM == kFp8 ? 256u : 512u) + (lane & 15u) * 32u;
        if (row < g.M && off < stride) prefetch_l2(a.low + (uint64_t)row * stride + off);
    };
    __syncthreads();                                                                     /* barriers initialised before anyone arms them */
    prefetch_block(blockIdx.x, j, 0u);
    stage_tables(tables, a.lut, tid, kSplitThreads);
    NormWeights norm_regs;
    stage_norm_weight<kSplitThreads>(in, a.K, nw, norm_regs);
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    asm volatile("griddepcontrol.wait;" ::: "memory");
    build_activation<kSplitThreads>(in, a.x, a.K, g.K16, xs, nw, scal, norm_regs);
    const uint32_t xs_addr = smem_addr(xs), table = smem_addr(tables), sym = table + 4u * kTableWords;
    float *stash = stash_all + warp * 16u;
    uint32_t phases = 0, which = 0;
    for (uint32_t pass = blockIdx.x; pass < passes; pass += gridDim.x) {
        const uint32_t rb = pass * per_pass + my_group;
        float row_sum = 0.f;                                     /* lanes 0, 1: rows rb * 8 + 2 rp + lane */
        if (rb < g.groups) {
            for (uint32_t cb = j; cb < g.CB; cb += share) {
                const Ahead cur = next;
                /* the other stage held the block before this one: every warp of the team must be done with it */
                asm volatile("bar.sync %0, %1;" ::"r"(1u + team), "r"(kSplitTeamWarps * 32u) : "memory");
                prefetch_block(pass, cb + share, which ^ 1u);
                uint32_t total;
                const uint32_t before = warp_exclusive_sum(cur.words, lane, total), base = __ldg(a.bases + cur.b);
                const uint32_t bit = cur.bit;
                if (cur.bytes) {
                    const bool landed = mbar_wait(bar0 + 8u * which, (phases >> which) & 1u);
                    phases ^= 1u << which;
                    if (landed) {
                        SmemWindow<MR> W; W.open(stage0 + which * kPrefixStageBytes + (base - cur.start) + 4u * (before + (bit >> 5)));
                        W.consume(bit & 31u);
                        row_sum += split_row_pair<SmemWindow<MR>, ELEM>(W, a, g, rb, cb, rp, lane, table, sym, four, stash, xs_addr);
                    }
                } else {
                    GlobalWindow<MR> W; W.sym_ptr = reinterpret_cast<const uint8_t *>(tables + kTableWords);
                    W.open(reinterpret_cast<const uint32_t *>(a.data + base) + before + (bit >> 5));
                    W.consume(bit & 31u);
                    row_sum += split_row_pair<GlobalWindow<MR>, ELEM>(W, a, g, rb, cb, rp, lane, table, sym, four, stash, xs_addr);
                }
                which ^= 1u;
            }
        }
        if (lane < 2u) red[team * 8u + 2u * rp + lane] = row_sum;
        __syncthreads();
        if (j == 0u && rp == 0u && lane < 8u && rb < g.groups) {
            float v = 0.f;
            for (uint32_t k = 0; k < share; k++) v += red[(team + k) * 8u + lane];
            const uint32_t row = rb * 8u + lane;
            if (row < a.M) {
                if (a.scale) v *= __ldg(a.scale + row);
                if (a.bias) v += bf16_to_float(__ldg(a.bias + row));
                a.y[row] = bf16_round(v);
            }
        }
        __syncthreads();
    }
}

/* ---- the persistent segment kernel -------------------------------------------------------------------------------- */
template <int LAYOUT, int ELEM, int MODE, bool XF32>
__global__ void __launch_bounds__(kSegmentThreads, 1) segment_kernel(const SegmentArgs a) {
    extern __shared__ __align__(16) uint32_t smem[];
    const uint32_t lane = threadIdx.x & 31u, warp = threadIdx.x >> 5;
    uint32_t table = 0; const uint8_t *sym = nullptr; float *stash = nullptr;
    if (LAYOUT != 2) {
        stage_tables(smem, a.lut, threadIdx.x, kSegmentThreads);
        table = (uint32_t)__cvta_generic_to_shared(smem);
        sym = reinterpret_cast<const uint8_t *>(smem + kTableWords);
        stash = reinterpret_cast<float *>(smem + kTableWords + 4) + warp * 64u;
    }
    const Geometry g(a.M, a.K, LAYOUT);
    const uint32_t items = g.groups * a.splits, stride = gridDim.x * (kSegmentThreads / 32u);
    for (uint32_t item = blockIdx.x * (kSegmentThreads / 32u) + warp; item < items; item += stride) {
        const uint32_t rb = item / a.splits, split = item - rb * a.splits;
        const uint32_t cb0 = (uint32_t)((uint64_t)split * g.CB / a.splits), cb1 = (uint32_t)((uint64_t)(split + 1u) * g.CB / a.splits);
        if (LAYOUT == 0) segment_layout0<ELEM, MODE, XF32>(a, g, rb, cb0, cb1, split, lane, table, sym, stash);
        else if (LAYOUT == 1) segment_layout1<ELEM, MODE, XF32>(a, g, rb, cb0, cb1, split, lane, table, sym);
        else segment_layout2<ELEM, MODE, XF32>(a, g, rb, cb0, cb1, split, lane);
    }
}

/* y[i] = bf16(sum of the row's partials in split order * scale[i] + bias[i]) (reference: csrc/nwc_ops.cu:553-565) */
__global__ void finalize_kernel(const float *__restrict__ partial, const uint16_t *__restrict__ bias, const float *__restrict__ scale,
                                uint16_t *__restrict__ y, uint32_t M, uint32_t splits) {
    const uint32_t i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= M) return;
    float v = 0.f;
    for (uint32_t s = 0; s < splits; s++) v += partial[(uint64_t)i * splits + s];
    if (scale) v *= scale[i];
    if (bias) v += bf16_to_float(bias[i]);
    y[i] = bf16_round(v);
}

template <int LAYOUT, int ELEM>
static cudaError_t launch_modes(int mode, int grid, size_t smem, cudaStream_t st, const SegmentArgs &a) {
    /* x is fp32 on the fp32 test path (all layouts) and on layout 0's token path unless the caller passes bf16 */
    if (mode == kModeDequant) segment_kernel<LAYOUT, ELEM, kModeDequant, false><<<grid, kSegmentThreads, smem, st>>>(a);
    else if (mode == kModeAtomic) segment_kernel<LAYOUT, ELEM, kModeAtomic, true><<<grid, kSegmentThreads, smem, st>>>(a);
    else if (LAYOUT == 0 && !a.x_bf16) segment_kernel<LAYOUT, ELEM, kModeLinear, true><<<grid, kSegmentThreads, smem, st>>>(a);
    else segment_kernel<LAYOUT, ELEM, kModeLinear, false><<<grid, kSegmentThreads, smem, st>>>(a);
    return cudaGetLastError();
}

/* number of K splits: one segment per row group when there are enough row groups to give every resident warp work,
   otherwise the fewest splits (at most one per column block) that reach two segments per warp */
static bool g_dependent_launch = false;
void set_dependent_launch(bool on) { g_dependent_launch = on; }
bool dependent_launch() { return g_dependent_launch; }

/* kernel launch that may start before its stream predecessor has finished (the kernel orders itself with
   griddepcontrol.wait) when dependent launch is switched on */
template <class... Params, class... Args>
static cudaError_t launch_cluster_kernel(void (*kernel)(Params...), uint32_t cluster, dim3 grid, dim3 block, size_t smem, cudaStream_t st, Args... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid; cfg.blockDim = block; cfg.dynamicSmemBytes = smem; cfg.stream = st;
    cudaLaunchAttribute attr[2];
    unsigned n = 0;
    if (cluster > 1u) { attr[n].id = cudaLaunchAttributeClusterDimension; attr[n].val.clusterDim.x = cluster; attr[n].val.clusterDim.y = 1; attr[n].val.clusterDim.z = 1; n++; }
    if (g_dependent_launch) { attr[n].id = cudaLaunchAttributeProgrammaticStreamSerialization; attr[n].val.programmaticStreamSerializationAllowed = 1; n++; }
    cfg.attrs = attr; cfg.numAttrs = n;
    return cudaLaunchKernelEx(&cfg, kernel, static_cast<Params>(args)...);
}
template <class... Params, class... Args>
static cudaError_t launch_kernel(void (*kernel)(Params...), dim3 grid, dim3 block, size_t smem, cudaStream_t st, Args... args) {
    return launch_cluster_kernel(kernel, 1u, grid, block, smem, st, args...);
}

constexpr uint32_t kSmallFixedSmem = 16416u + kSmallWarps * 64u * 4u + kSmallWarps * 8u * 4u + 32u + kSmallWarps * 2u * kPrefixStageBytes + kSmallWarps * 16u;
constexpr uint32_t kSplitFixedSmem = 16416u + 8u * 16u * 4u + kSplitTeams * 8u * 4u + 32u + kSplitTeams * 2u * kPrefixStageBytes + kSplitTeams * 16u;
cudaError_t launch_small_layout0(int code, int sms, cudaStream_t st, const SegmentArgs &a, const FusedInput &in, const uint16_t *side) {
    const Geometry g(a.M, a.K, 0);
    if (side) {                                                   /* four warps per block along the side table */
        const uint32_t share = g.CB > 1u ? kSplitTeams : 1u, passes = (g.groups + kSplitTeams / share - 1u) / (kSplitTeams / share);
        const uint32_t grid = passes < 3u * (uint32_t)sms ? passes : 3u * (uint32_t)sms;      /* one resident wave (measured: fewer, longer-running CTAs are slower); CTAs loop over further passes */
        const size_t smem = kSplitFixedSmem + (size_t)g.K16 * (norm_like(in.mode) ? 4u : 2u);
        if (type_of(code) == kFp8) return launch_kernel(small_split_kernel_layout0<kFp8>, dim3(grid), dim3(kSplitThreads), smem, st, a, in, 4u, side);
        return launch_kernel(small_split_kernel_layout0<kBf16>, dim3(grid), dim3(kSplitThreads), smem, st, a, in, 4u, side);
    }
    const uint32_t wg = small_group_warps(g.CB), per_pass = kSmallWarps / wg;
    const uint32_t passes = (g.groups + per_pass - 1u) / per_pass;
    const uint32_t grid = passes < 4u * (uint32_t)sms ? passes : 4u * (uint32_t)sms;
    const size_t smem = kSmallFixedSmem + (size_t)g.K16 * (norm_like(in.mode) ? 4u : 2u);
    if (type_of(code) == kFp8) return launch_kernel(small_kernel_layout0<kFp8>, dim3(grid), dim3(kSmallThreads), smem, st, a, in, 4u);
    return launch_kernel(small_kernel_layout0<kBf16>, dim3(grid), dim3(kSmallThreads), smem, st, a, in, 4u);
}

void set_ring_kernels(bool on) { g_disable_ring = !on; }
void set_fixup_plans(bool on) { g_disable_fixup = !on; }
int read_kernel_status(bool clear) {
    int v = 0;
    if (cudaMemcpyFromSymbol(&v, g_kernel_status, sizeof(int)) != cudaSuccess) return -1;
    if (clear && v) { const int z = 0; cudaMemcpyToSymbol(g_kernel_status, &z, sizeof(int)); }
    return v;
}

uint32_t choose_splits(const Geometry &g, int mode, int code, int sms) {
    if (mode == kModeDequant) return g.CB;                       /* no sums: finest grain */
    (void)code;
    const uint64_t warps = (uint64_t)sms * (kSegmentThreads / 32u);
    if (g.groups >= 2u * warps || g.CB == 1u) return 1u;
    const uint64_t want = (2u * warps + g.groups - 1u) / g.groups;
    return (uint32_t)(want < g.CB ? want : g.CB);
}

/* kernels the token path launches for an M x K matrix (automatic splits) */
int count_token_launches(int code, int sms, uint32_t M, uint32_t K, bool allow_fix) {
    const int layout = layout_of(code), elem = type_of(code);
    const Geometry g(M, K, layout);
    FlatPlan plan;
    if (!g_disable_ring && layout == 0) { make_flat_plan(g, g.CB, (uint64_t)sms * (kPrefixThreads / 32u), plan); return plan.direct ? 1 : 2; }
    if (!g_disable_ring && layout == 1) { make_flat_plan(g, g.CB, (uint64_t)sms * (kPrefix1Threads / 32u), plan); return plan.direct ? 1 : 2; }
    if (!g_disable_ring && ring_covers(code, g, kInputPlain)) { uint32_t cluster; bool pool; choose_ring_plan(code, g, kInputPlain, sms, allow_fix, plan, cluster, pool); return plan.direct || plan.fix ? 1 : 2; }
    return choose_splits(g, kModeLinear, code, sms) > 1 ? 2 : 1;
}

/* Layout 0, a matrix of at most two blocks per resident warp: the single-launch small-matrix kernel, or the prologue
   kernel + the large-matrix ring kernel + finalize?  Both are bound by the serial walk of a block (about 5.5 us on B200).
   The small kernel gives a row group to a team of up to 8 warps and runs its row groups in rounds of 2 CTAs per SM, so a
   matrix of many column blocks (2560 x 9728: 19 blocks per group, 320 groups) walks 3 blocks per warp in each of 2 rounds
   (35 us measured) where the ring kernel's 32 warps per SM walk 2 (22 us + the prologue launch); matrices of few column
   blocks are faster on the small kernel (4096 x 1024: 8 against 16 us).  Measured fixed costs: 4 us and 14 us. */
bool small_layout0_preferred(uint32_t M, uint32_t K, int sms, int input_mode) {
    const Geometry g(M, K, 0);
    const uint32_t wg = small_group_warps(g.CB), per_pass = kSmallWarps / wg, passes = (g.groups + per_pass - 1u) / per_pass;
    const uint32_t rounds = (passes + 2u * (uint32_t)sms - 1u) / (2u * (uint32_t)sms), walks = (g.CB + wg - 1u) / wg;
    const uint32_t small_cost = 55u * walks * rounds + 40u;                                               /* tenths of a microsecond */
    const uint32_t ring_cost = 55u * ((g.nb + 32u * (uint32_t)sms - 1u) / (32u * (uint32_t)sms)) + 140u + (input_mode != kInputPlain ? 35u : 0u);
    return g_disable_ring || small_cost <= ring_cost;
}

/* the token path of this matrix builds its activation vector itself (nwc_linear_fused needs no prologue launch) */
bool token_path_fuses_input(int code, uint32_t M, uint32_t K, int input_mode) {
    const Geometry g(M, K, layout_of(code));
    if (g_disable_ring) return false;
    return layout_of(code) == 2 ? ring_covers(code, g, input_mode) : prefix_ring_fuses(code, g, input_mode);
}

static uint32_t g_next_fill_stages = kRingStages;
void set_next_fill_stages(uint32_t stages) { g_next_fill_stages = stages; }

/* the ring kernel's view of the launch that follows (all zero when that launch is unknown or takes another kernel) */
static NextFill make_next_fill(const NextMatrix *next, int sms) {
    NextFill nx{};
    if (!next || !next->low || g_next_fill_stages == 0u || g_disable_ring || next->M == 0u || next->K == 0u) return nx;
    const Geometry g(next->M, next->K, layout_of(next->code));
    if (!ring_covers(next->code, g, next->input_mode)) return nx;
    const int elem = type_of(next->code);
    uint32_t cluster;
    bool pool;
    choose_ring_plan(next->code, g, next->input_mode, sms, next->fixup != 0u, nx.plan, cluster, pool);
    nx.pooled = pool ? 1u : 0u;
    const uint32_t U = elem == kFp8 ? 2u : 1u;
    nx.nib = next->low; nx.raw = next->low + g.nibble_plane_bytes();
    nx.blocks = nx.plan.warps * cluster;
    nx.cluster_shift = cluster == 8u ? 3u : (cluster == 4u ? 2u : (cluster == 2u ? 1u : 0u));
    nx.nib_unit = 256u * U; nx.raw_unit = elem == kFp8 ? 384u : 512u;
    nx.units = g_next_fill_stages * (kRingSlots / U);
    return nx;
}

cudaError_t launch_segments(int mode, int code, int sms, cudaStream_t st, SegmentArgs a, const FusedInput *input, const NextMatrix *next) {
    const int layout = layout_of(code), elem = type_of(code);
    const Geometry g(a.M, a.K, layout);
    a.splits_forced = a.splits;
    if (a.splits == 0) a.splits = choose_splits(g, mode, code, sms);
    const uint32_t warps_per_cta = kSegmentThreads / 32u;
    const uint64_t items = (uint64_t)g.groups * a.splits;
    int grid = (int)((items + warps_per_cta - 1) / warps_per_cta);
    if (grid > sms) grid = sms;
    const size_t smem = layout == 2 ? 0 : kTableSmemBytes + (size_t)warps_per_cta * 64u * sizeof(float);
    cudaError_t err;
    FlatPlan plan;
    FusedInput fin{kInputPlain, nullptr, nullptr, nullptr, nullptr, 0.f, nullptr, nullptr, 0u, 0u, 0ull};
    if (input && a.x_bf16 && prefix_ring_fuses(code, g, input->mode)) fin = *input;       /* the layout 0 / 1 ring kernels build x themselves */
    const size_t fused_bytes = fin.mode != kInputPlain ? prefix_fused_bytes(g) : 0u;
    if (layout == 0 && mode == kModeLinear && !g_disable_ring && a.splits_forced == 0) {
        make_flat_plan(g, g.CB, (uint64_t)sms * (kPrefixThreads / 32u), plan);
        const int rgrid = (int)(plan.warps < (uint32_t)sms ? plan.warps : (uint32_t)sms);
        const size_t rsmem = kPrefixSmemBytes + fused_bytes;
        if (elem == kFp8) { if (a.x_bf16) prefix_ring_kernel_layout0<kFp8, false><<<rgrid, kPrefixThreads, rsmem, st>>>(a, plan, 4u, fin); else prefix_ring_kernel_layout0<kFp8, true><<<rgrid, kPrefixThreads, rsmem, st>>>(a, plan, 4u, fin); }
        else { if (a.x_bf16) prefix_ring_kernel_layout0<kBf16, false><<<rgrid, kPrefixThreads, rsmem, st>>>(a, plan, 4u, fin); else prefix_ring_kernel_layout0<kBf16, true><<<rgrid, kPrefixThreads, rsmem, st>>>(a, plan, 4u, fin); }
        err = cudaGetLastError();
        if (err == cudaSuccess && !plan.direct) {
            finalize_flat_kernel<<<(a.M + 255u) / 256u, 256, 0, st>>>(a.y32, a.bias, a.scale, a.y, a.M, g.rows, plan);
            err = cudaGetLastError();
        }
        return err;
    }
    if (layout == 1 && mode == kModeLinear && !g_disable_ring && a.splits_forced == 0) {
        make_flat_plan(g, g.CB, (uint64_t)sms * (kPrefix1Threads / 32u), plan);
        const int rgrid = (int)(plan.warps < (uint32_t)sms ? plan.warps : (uint32_t)sms);
        if (elem == kFp8) prefix_ring_kernel_layout1<kFp8><<<rgrid, kPrefix1Threads, kPrefix1SmemBytes + fused_bytes, st>>>(a, plan, 4u, fin);
        else prefix_ring_kernel_layout1<kBf16><<<rgrid, kPrefix1Threads, kPrefix1SmemBytes + fused_bytes, st>>>(a, plan, 4u, fin);
        err = cudaGetLastError();
        if (err == cudaSuccess && !plan.direct) {
            finalize_flat_kernel<<<(a.M + 255u) / 256u, 256, 0, st>>>(a.y32, a.bias, a.scale, a.y, a.M, g.rows, plan);
            err = cudaGetLastError();
        }
        return err;
    }
    FusedInput in{kInputPlain, nullptr, nullptr, nullptr, nullptr, 0.f, nullptr, nullptr, 0u, 0u, 0ull};
    if (input) in = *input;
    if (mode == kModeLinear && !g_disable_ring && a.splits_forced == 0 && ring_covers(code, g, in.mode)) {
        uint32_t cluster;
        bool pool;
        choose_ring_plan(code, g, in.mode, sms, a.fixup != 0u, plan, cluster, pool);
        const NextFill nx = make_next_fill(next, sms);
        if (pool) {
            const PoolShape ps = make_pool_shape(g, elem);
            const size_t smem = pool_smem_bytes(g, elem, in.mode);
            return elem == kFp8 ? launch_kernel(pool_kernel_layout2<kFp8>, dim3(plan.warps), dim3(kRingThreads), smem, st, a, plan, in, nx, ps)
                                : launch_kernel(pool_kernel_layout2<kBf16>, dim3(plan.warps), dim3(kRingThreads), smem, st, a, plan, in, nx, ps);
        }
        in.share = choose_peer_sharing(code, g, in, sms, a.fixup != 0u, plan, cluster);
        if (in.share & 2u) {                                     /* clusters of CTAs that each own a run of the plan */
            err = elem == kFp8 ? launch_cluster_kernel(ring_kernel_layout2<kFp8, true>, cluster, dim3(plan.warps), dim3(kRingThreads), ring_smem_bytes(g, in.mode), st, a, plan, in, nx)
                               : launch_cluster_kernel(ring_kernel_layout2<kBf16, true>, cluster, dim3(plan.warps), dim3(kRingThreads), ring_smem_bytes(g, in.mode), st, a, plan, in, nx);
            if (err == cudaSuccess && !plan.direct && !plan.fix)
                err = launch_kernel(finalize_flat_kernel, dim3((a.M + 255u) / 256u), dim3(256), 0, st, a.y32, a.bias, a.scale, a.y, a.M, g.rows, plan);
            return err;
        }
        if (in.share)                                            /* the plan's own clusters share the partials as well */
            err = elem == kFp8 ? launch_cluster_kernel(ring_kernel_layout2<kFp8, true>, cluster, dim3(plan.warps * cluster), dim3(kRingThreads), ring_smem_bytes(g, in.mode), st, a, plan, in, nx)
                               : launch_cluster_kernel(ring_kernel_layout2<kBf16, true>, cluster, dim3(plan.warps * cluster), dim3(kRingThreads), ring_smem_bytes(g, in.mode), st, a, plan, in, nx);
        else
            err = elem == kFp8 ? launch_cluster_kernel(ring_kernel_layout2<kFp8, false>, cluster, dim3(plan.warps * cluster), dim3(kRingThreads), ring_smem_bytes(g, in.mode), st, a, plan, in, nx)
                               : launch_cluster_kernel(ring_kernel_layout2<kBf16, false>, cluster, dim3(plan.warps * cluster), dim3(kRingThreads), ring_smem_bytes(g, in.mode), st, a, plan, in, nx);
        if (err == cudaSuccess && !plan.direct && !plan.fix)
            err = launch_kernel(finalize_flat_kernel, dim3((a.M + 255u) / 256u), dim3(256), 0, st, a.y32, a.bias, a.scale, a.y, a.M, g.rows, plan);
        return err;
    }
    if (layout == 0) err = elem == kFp8 ? launch_modes<0, kFp8>(mode, grid, smem, st, a) : launch_modes<0, kBf16>(mode, grid, smem, st, a);
    else if (layout == 1) err = elem == kFp8 ? launch_modes<1, kFp8>(mode, grid, smem, st, a) : launch_modes<1, kBf16>(mode, grid, smem, st, a);
    else err = elem == kFp8 ? launch_modes<2, kFp8>(mode, grid, smem, st, a) : launch_modes<2, kBf16>(mode, grid, smem, st, a);
    if (err != cudaSuccess) return err;
    if (mode == kModeLinear && a.splits > 1) {
        finalize_kernel<<<(a.M + 255u) / 256u, 256, 0, st>>>(a.y32, a.bias, a.scale, a.y, a.M, a.splits);
        err = cudaGetLastError();
    }
    return err;
}

template <int LAYOUT, int ELEM>
static void opt_in_smem() {
    const int bytes = (int)(kTableSmemBytes + (kSegmentThreads / 32u) * 64u * sizeof(float));
    cudaFuncSetAttribute(segment_kernel<LAYOUT, ELEM, kModeLinear, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes);
    cudaFuncSetAttribute(segment_kernel<LAYOUT, ELEM, kModeLinear, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes);
    cudaFuncSetAttribute(segment_kernel<LAYOUT, ELEM, kModeDequant, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes);
    cudaFuncSetAttribute(segment_kernel<LAYOUT, ELEM, kModeAtomic, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes);
}
static ClusterRoom cluster_room(int sms) {
    static ClusterRoom cache[64];
    static bool known[64];
    static std::mutex guard;                                     /* launches may come from several host threads */
    std::lock_guard<std::mutex> hold(guard);
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev < 0 || dev >= 64) dev = 0;
    if (!known[dev]) {
        ClusterRoom r{{sms, 0, 0, 0}};
        cudaFuncSetAttribute(ring_kernel_layout2<kBf16, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kRingMaxSmem);
        for (int lg = 1; lg < 4; lg++) {
            cudaLaunchConfig_t cfg = {};
            cfg.gridDim = dim3((unsigned)sms / (1u << lg) * (1u << lg)); cfg.blockDim = dim3(kRingThreads); cfg.dynamicSmemBytes = kRingMaxSmem;
            cudaLaunchAttribute attr[1];
            attr[0].id = cudaLaunchAttributeClusterDimension; attr[0].val.clusterDim.x = 1u << lg; attr[0].val.clusterDim.y = 1; attr[0].val.clusterDim.z = 1;
            cfg.attrs = attr; cfg.numAttrs = 1;
            int n = 0;
            if (cudaOccupancyMaxActiveClusters(&n, ring_kernel_layout2<kBf16, false>, &cfg) == cudaSuccess) r.count[lg] = n; else cudaGetLastError();
        }
        cache[dev] = r; known[dev] = true;
    }
    return cache[dev];
}

cudaError_t launch_side_table(int code, cudaStream_t st, const uint8_t *data, const uint32_t *bases, const uint8_t *hdr, uint16_t *side, uint32_t nb) {
    const unsigned grid = (nb + 3u) / 4u;
    if (type_of(code) == kFp8) side_table_kernel<kFp8><<<grid, 128, 0, st>>>(data, bases, hdr, side, nb);
    else side_table_kernel<kBf16><<<grid, 128, 0, st>>>(data, bases, hdr, side, nb);
    return cudaGetLastError();
}

void configure_segment_kernels() {
    cudaFuncSetAttribute(small_split_kernel_layout0<kBf16>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kRingMaxSmem);
    cudaFuncSetAttribute(small_split_kernel_layout0<kFp8>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kRingMaxSmem);
    cudaFuncSetAttribute(small_kernel_layout0<kBf16>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kRingMaxSmem);
    cudaFuncSetAttribute(small_kernel_layout0<kFp8>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kRingMaxSmem);
    cudaFuncSetAttribute(ring_kernel_layout2<kBf16, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kRingMaxSmem);
    cudaFuncSetAttribute(ring_kernel_layout2<kFp8, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kRingMaxSmem);
    cudaFuncSetAttribute(ring_kernel_layout2<kBf16, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kRingMaxSmem);
    cudaFuncSetAttribute(ring_kernel_layout2<kFp8, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kRingMaxSmem);
    cudaFuncSetAttribute(pool_kernel_layout2<kBf16>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kRingMaxSmem);
    cudaFuncSetAttribute(pool_kernel_layout2<kFp8>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kRingMaxSmem);
    {                                                             /* no CTA has left a part of a row group for another one yet */
        void *parts = nullptr;
        if (cudaGetSymbolAddress(&parts, g_cut_part) == cudaSuccess) cudaMemset(parts, 0xFF, sizeof(g_cut_part)); else cudaGetLastError();
    }
    cudaFuncSetAttribute(prefix_ring_kernel_layout1<kBf16>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kRingMaxSmem);      /* rings (+ the activation vector) */
    cudaFuncSetAttribute(prefix_ring_kernel_layout1<kFp8>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kRingMaxSmem);
    cudaFuncSetAttribute(prefix_ring_kernel_layout0<kBf16, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kRingMaxSmem);
    cudaFuncSetAttribute(prefix_ring_kernel_layout0<kBf16, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kRingMaxSmem);
    cudaFuncSetAttribute(prefix_ring_kernel_layout0<kFp8, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kRingMaxSmem);
    cudaFuncSetAttribute(prefix_ring_kernel_layout0<kFp8, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kRingMaxSmem);
    opt_in_smem<0, kBf16>(); opt_in_smem<0, kFp8>(); opt_in_smem<1, kBf16>(); opt_in_smem<1, kFp8>();
}

}  // namespace nwc
