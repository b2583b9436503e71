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
#include "nwc_decode.cuh"
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

template <int ELEM, int MODE>
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

        XFrag8<true> xa, xb;                                    /* columns 0..7 and 8..15 of the lane */
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
                    const XFrag8<true> &xf = k < 2 ? xa : xb;
                    const int w = 2 * (k & 1);
                    mma_bf16(d, pa[2 * k], pb[2 * k], pa[2 * k + 1], pb[2 * k + 1], xf.head[w], xf.head[w + 1]);
                    mma_bf16(d, pa[2 * k], pb[2 * k], pa[2 * k + 1], pb[2 * k + 1], xf.tail[w], xf.tail[w + 1]);
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

template <int ELEM, int MODE>
__device__ __forceinline__ void segment_layout1(const SegmentArgs &a, const Geometry &g, uint32_t rb, uint32_t cb0, uint32_t cb1,
                                                uint32_t split, uint32_t lane, uint32_t table, const uint8_t *sym) {
    constexpr uint32_t MR = ELEM == kFp8 ? kMaxRankFp8 : kMaxRankBf16;
    constexpr uint32_t RB = ELEM == kFp8 ? 8u : 16u;             /* raw bytes per lane and super-chunk */
    constexpr bool XF32 = MODE == kModeAtomic;
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
template <int ELEM, int MODE, int SC_PARITY>
__device__ __forceinline__ void fixed_super_chunk(const SegmentArgs &a, const Geometry &g, const FixedTables &t, uint2 nib, uint4 raw,
                                                  uint32_t f0, uint32_t f1, uint32_t f2, uint32_t row0, uint32_t r, uint32_t kc, float (&d)[4]) {
    constexpr bool XF32 = MODE == kModeAtomic;
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

template <int ELEM, int MODE>
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
                fixed_super_chunk<ELEM, MODE, 0>(a, g, t, n0, make_uint4(0u, 0u, 0u, 0u), f0, f1, f2, row0, r, kbase + sc * 32u, d);
                if (sc + 1u < nsc) {
                    const uint2 n1 = ldg_stream64(np + kLanes * 8u);
                    fixed_super_chunk<ELEM, MODE, 1>(a, g, t, n1, make_uint4(0u, 0u, 0u, 0u), f0, f1, f2, row0, r, kbase + (sc + 1u) * 32u, d);
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
                fixed_super_chunk<ELEM, MODE, 0>(a, g, t, nib, raw, 0u, 0u, 0u, row0, r, kbase + sc * 32u, d);
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
                const float xv = MODE == kModeLinear ? bf16_to_float(__ldg(static_cast<const uint16_t *>(a.x) + col)) : __ldg(static_cast<const float *>(a.x) + col);
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

/* ---- the persistent segment kernel -------------------------------------------------------------------------------- */
template <int LAYOUT, int ELEM, int MODE>
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
        if (LAYOUT == 0) segment_layout0<ELEM, MODE>(a, g, rb, cb0, cb1, split, lane, table, sym, stash);
        else if (LAYOUT == 1) segment_layout1<ELEM, MODE>(a, g, rb, cb0, cb1, split, lane, table, sym);
        else segment_layout2<ELEM, MODE>(a, g, rb, cb0, cb1, split, lane);
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
    switch (mode) {
        case kModeLinear: segment_kernel<LAYOUT, ELEM, kModeLinear><<<grid, kSegmentThreads, smem, st>>>(a); break;
        case kModeDequant: segment_kernel<LAYOUT, ELEM, kModeDequant><<<grid, kSegmentThreads, smem, st>>>(a); break;
        default: segment_kernel<LAYOUT, ELEM, kModeAtomic><<<grid, kSegmentThreads, smem, st>>>(a); break;
    }
    return cudaGetLastError();
}

/* number of K splits: one segment per row group when there are enough row groups to give every resident warp work,
   otherwise the fewest splits (at most one per column block) that reach two segments per warp */
uint32_t choose_splits(const Geometry &g, int mode, int sms) {
    if (mode == kModeDequant) return g.CB;                       /* no sums: finest grain */
    const uint64_t warps = (uint64_t)sms * (kSegmentThreads / 32u);
    if (g.groups >= 2u * warps || g.CB == 1u) return 1u;
    const uint64_t want = (2u * warps + g.groups - 1u) / g.groups;
    return (uint32_t)(want < g.CB ? want : g.CB);
}

cudaError_t launch_segments(int mode, int code, int sms, cudaStream_t st, SegmentArgs a) {
    const int layout = layout_of(code), elem = type_of(code);
    const Geometry g(a.M, a.K, layout);
    if (a.splits == 0) a.splits = choose_splits(g, mode, sms);
    const uint32_t warps_per_cta = kSegmentThreads / 32u;
    const uint64_t items = (uint64_t)g.groups * a.splits;
    int grid = (int)((items + warps_per_cta - 1) / warps_per_cta);
    if (grid > sms) grid = sms;
    const size_t smem = layout == 2 ? 0 : kTableSmemBytes + (size_t)warps_per_cta * 64u * sizeof(float);
    cudaError_t err;
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

template <int LAYOUT, int ELEM, int MODE>
static void opt_in_smem() {
    cudaFuncSetAttribute(segment_kernel<LAYOUT, ELEM, MODE>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                         (int)(kTableSmemBytes + (kSegmentThreads / 32u) * 64u * sizeof(float)));
}
void configure_segment_kernels() {
    opt_in_smem<0, kBf16, 0>(); opt_in_smem<0, kBf16, 1>(); opt_in_smem<0, kBf16, 2>();
    opt_in_smem<0, kFp8, 0>(); opt_in_smem<0, kFp8, 1>(); opt_in_smem<0, kFp8, 2>();
    opt_in_smem<1, kBf16, 0>(); opt_in_smem<1, kBf16, 1>(); opt_in_smem<1, kBf16, 2>();
    opt_in_smem<1, kFp8, 0>(); opt_in_smem<1, kFp8, 1>(); opt_in_smem<1, kFp8, 2>();
}

}  // namespace nwc
