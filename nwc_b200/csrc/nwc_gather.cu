/* Row gather from the compressed matrix (embedding lookup) and the uncompressed fp8 weight-only matvec that serves as
 * the "native fp8" comparison.
 *
 * Gather: one warp per (requested row, column block), so a single token's row is decoded by CB warps in parallel
 * instead of one warp walking all column blocks.
 *   layout 0  every lane owns 16 columns of each of the block's 8 rows; the rows in front of the requested one are
 *             decoded and dropped (their symbols precede it in the lane stream).
 *   layout 1  only the four lanes of the quad that holds the row (r = row mod 8) carry useful streams; they decode and
 *             write, the others only take part in the header prefix sum.
 *   layout 2  fixed-width: the quad's nibble and raw cells are addressed directly, and all 32 lanes of the warp share
 *             the block's 16 super-chunks (lane -> super-chunk lane/4 and lane/4 + 8, source lane 4 r + lane%4).
 *
 * Interfaces replaced (reference: csrc/nwc_ops.cu): kern_gather 568-601, kern_gather1 707-745, kern_gather2 985-1042,
 * kern_ref_fp8 760-829.
 */
#include <cuda_fp16.h>
#include "nwc_decode.cuh"
#include "nwc_launch.h"

namespace nwc {

constexpr uint32_t kGatherThreads = 128;

/* side (may be null): per block and lane the bit positions at which rows 2, 4 and 6 begin in the lane's stream
   (launch_side_table); with it the walk starts at the row pair that holds the row instead of at the block's first row. */
template <int ELEM>
__device__ __forceinline__ void gather_block0(const SegmentArgs &a, const Geometry &g, uint32_t row, uint32_t cb, uint32_t lane,
                                              uint32_t table, const uint8_t *sym, uint16_t *dst, const uint16_t *side) {
    constexpr uint32_t MR = ELEM == kFp8 ? kMaxRankFp8 : kMaxRankBf16;
    const uint32_t rb = row >> 3, b = rb * g.CB + cb, col0 = cb * kBlockCols + lane * 16u;
    uint32_t skip = row & 7u, start_bit = 0u;
    if (side != nullptr && skip >= 2u) { start_bit = __ldg(side + ((uint64_t)b * 3u + ((skip >> 1) - 1u)) * kLanes + lane); skip &= 1u; }
    const bool col_ok = col0 < g.K16;
    uint32_t total;
    const uint32_t words = __ldg(a.hdr + (uint64_t)b * kLanes + lane), before = warp_exclusive_sum(words, lane, total);
    BitWindow<MR> W; W.open(reinterpret_cast<const uint32_t *>(a.data + __ldg(a.bases + b)) + before + (start_bit >> 5));
    if (start_bit & 31u) W.consume(start_bit & 31u);
    uint4 raw = make_uint4(0u, 0u, 0u, 0u);
    if (col_ok) raw = ELEM == kFp8 ? expand_nibbles(ldg_stream64(a.low + (uint64_t)row * (g.K16 >> 1) + (col0 >> 1)))
                                   : ldg_stream128(a.low + (uint64_t)row * g.K16 + col0);
    for (uint32_t z = 0; z < skip * 4u; z++) { uint32_t e0, e1; W.quad(table, sym, e0, e1); }
    const uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
    uint32_t p[8];
#pragma unroll
    for (int k = 0; k < 4; k++) { uint32_t e01, e23; W.quad(table, sym, e01, e23); p[2 * k] = weave<0>(w[k], e01); p[2 * k + 1] = weave<2>(w[k], e23); }
    if (col_ok) {
        uint4 *o = reinterpret_cast<uint4 *>(dst + col0);
        o[0] = make_uint4(p[0], p[1], p[2], p[3]); o[1] = make_uint4(p[4], p[5], p[6], p[7]);
    }
}

template <int ELEM>
__device__ __forceinline__ void gather_block1(const SegmentArgs &a, const Geometry &g, uint32_t row, uint32_t cb, uint32_t lane,
                                              uint32_t table, const uint8_t *sym, uint16_t *dst) {
    constexpr uint32_t MR = ELEM == kFp8 ? kMaxRankFp8 : kMaxRankBf16;
    constexpr uint32_t RB = ELEM == kFp8 ? 8u : 16u;
    const uint32_t rb = row >> 4, rr = row & 15u, b = rb * g.CB + cb, nsc = g.supers_in(cb), r = lane >> 2, q = lane & 3u;
    const bool upper = rr >= 8u;
    uint32_t total;
    const uint32_t words = __ldg(a.hdr + (uint64_t)b * kLanes + lane), before = warp_exclusive_sum(words, lane, total);
    if (r != (rr & 7u)) return;                                  /* this lane's stream holds other rows */
    BitWindow<MR> W; W.open(reinterpret_cast<const uint32_t *>(a.data + __ldg(a.bases + b)) + before);
    const uint8_t *rp = a.low + ((uint64_t)(rb * g.slots + cb * 16u) * kLanes + lane) * RB;
    for (uint32_t sc = 0; sc < nsc; sc++, rp += kLanes * RB) {
        const uint4 cw = ELEM == kFp8 ? expand_nibbles(ldg_stream64(rp)) : ldg_stream128(rp);
        const uint32_t c[4] = {cw.x, cw.y, cw.z, cw.w};
#pragma unroll
        for (int h = 0; h < 2; h++) {
            uint32_t e0, e1, e2, e3;
            W.quad(table, sym, e0, e1); W.quad(table, sym, e2, e3);
            const uint32_t col = cb * kBlockCols + sc * 32u + 8u * q + 4u * h;
            if (col < g.K16) {
                const uint32_t v0 = upper ? weave<2>(c[2 * h], e1) : weave<0>(c[2 * h], e0);
                const uint32_t v1 = upper ? weave<2>(c[2 * h + 1], e3) : weave<0>(c[2 * h + 1], e2);
                *reinterpret_cast<uint2 *>(dst + col) = make_uint2(v0, v1);
            }
        }
    }
}

template <int ELEM>
__device__ __forceinline__ void gather_block2(const SegmentArgs &a, const Geometry &g, const FixedTables &t, uint32_t row, uint32_t cb,
                                              uint32_t lane, uint16_t *dst) {
    constexpr uint32_t ES = ELEM == kFp8 ? 2u : 3u;
    const uint32_t rb = row >> 4, rr = row & 15u, b = rb * g.CB + cb, nsc = g.supers_in(cb), q = lane & 3u;
    const uint32_t src_lane = ((rr & 7u) << 2) | q;               /* lane whose cells hold the row */
    const bool upper = rr >= 8u;
    const uint32_t slot0 = rb * g.slots + cb * 16u;
    const uint8_t *raw_plane = a.low + g.nibble_plane_bytes();
    for (uint32_t sc = lane >> 2; sc < nsc; sc += 8u) {
        const uint64_t cell = (uint64_t)(slot0 + sc) * kLanes + src_lane;
        const uint2 nib = ldg_stream64(a.low + cell * 8u);
        uint4 raw = make_uint4(0u, 0u, 0u, 0u); uint32_t f0 = 0, f1 = 0, f2 = 0;
        if (ELEM == kFp8) {
            const uint8_t *fp = raw_plane + ((((uint64_t)rb * g.pair_slots + cb * 8u + (sc >> 1)) * 3u) * kLanes + src_lane) * 4u;
            f0 = ldg_stream32(reinterpret_cast<const uint32_t *>(fp)); f1 = ldg_stream32(reinterpret_cast<const uint32_t *>(fp + kLanes * 4u));
            f2 = ldg_stream32(reinterpret_cast<const uint32_t *>(fp + 2u * kLanes * 4u));
        } else raw = ldg_stream128(raw_plane + cell * 16u);
        uint32_t v[4], a0, a1, a2, a3;
        if (sc & 1u) fixed_half<ELEM, 4>(t, nib.x, raw.x, raw.y, f0, f1, f2, a0, a1, a2, a3); else fixed_half<ELEM, 0>(t, nib.x, raw.x, raw.y, f0, f1, f2, a0, a1, a2, a3);
        v[0] = upper ? a1 : a0; v[1] = upper ? a3 : a2;
        if (sc & 1u) fixed_half<ELEM, 6>(t, nib.y, raw.z, raw.w, f0, f1, f2, a0, a1, a2, a3); else fixed_half<ELEM, 2>(t, nib.y, raw.z, raw.w, f0, f1, f2, a0, a1, a2, a3);
        v[2] = upper ? a1 : a0; v[3] = upper ? a3 : a2;
        const uint32_t col = cb * kBlockCols + sc * 32u + 8u * q;
        if (col < g.K16) *reinterpret_cast<uint2 *>(dst + col) = make_uint2(v[0], v[1]);
        if (col + 4u < g.K16) *reinterpret_cast<uint2 *>(dst + col + 4u) = make_uint2(v[2], v[3]);
    }
    /* exceptions of the row's quad: the plane values written above were +-0 placeholders */
    uint32_t total;
    const uint32_t count = __ldg(a.hdr + (uint64_t)b * kLanes + lane), before = warp_exclusive_sum(count, lane, total);
    __syncwarp();
    if (total && (lane >> 2) == (rr & 7u)) {
        const uint8_t *ep = a.data + __ldg(a.bases + b) + (uint64_t)before * ES;
        for (uint32_t k = 0; k < count; k++, ep += ES) {
            const uint32_t i = ep[0], j = i & 15u;
            if ((((j >> 1) & 1u) != 0u) != upper) continue;
            const float w = ELEM == kFp8 ? fp8_to_float(ep[1]) : __uint_as_float(((uint32_t)ep[1] | ((uint32_t)ep[2] << 8)) << 16);
            dst[cb * kBlockCols + (i >> 4) * 32u + frag_col(lane, j)] = (uint16_t)(__float_as_uint(w) >> 16);
        }
    }
}

template <int LAYOUT, int ELEM>
__global__ void __launch_bounds__(kGatherThreads) gather_kernel(const SegmentArgs a, const int64_t *__restrict__ ids, uint32_t n_ids, const uint16_t *__restrict__ side) {
    __shared__ __align__(16) uint32_t smem[LAYOUT == 2 ? 4 : kTableWords + 4];
    uint32_t table = 0; const uint8_t *sym = nullptr;
    if constexpr (LAYOUT != 2) {
        stage_tables(smem, a.lut, threadIdx.x, kGatherThreads);
        table = (uint32_t)__cvta_generic_to_shared(smem);
        sym = reinterpret_cast<const uint8_t *>(smem + kTableWords);
    }
    const Geometry g(a.M, a.K, LAYOUT);
    const uint32_t lane = threadIdx.x & 31u;
    const uint64_t item = ((uint64_t)blockIdx.x * kGatherThreads + threadIdx.x) >> 5;
    if (item >= (uint64_t)n_ids * g.CB) return;
    const uint32_t which = (uint32_t)(item / g.CB), cb = (uint32_t)(item - (uint64_t)which * g.CB);
    const int64_t id = ids[which];
    if (id < 0 || id >= (int64_t)a.M) return;                    /* ids outside the matrix leave their output row untouched */
    uint16_t *dst = a.out + (uint64_t)which * g.K16;
    if (LAYOUT == 0) gather_block0<ELEM>(a, g, (uint32_t)id, cb, lane, table, sym, dst, side);
    else if (LAYOUT == 1) gather_block1<ELEM>(a, g, (uint32_t)id, cb, lane, table, sym, dst);
    else { FixedTables t; t.load(a.lut); gather_block2<ELEM>(a, g, t, (uint32_t)id, cb, lane, dst); }
}

cudaError_t launch_gather(int code, cudaStream_t st, const SegmentArgs &a, const int64_t *ids, uint32_t n_ids, const uint16_t *side) {
    const int layout = layout_of(code), elem = type_of(code);
    const Geometry g(a.M, a.K, layout);
    const uint64_t warps = (uint64_t)n_ids * g.CB;
    const unsigned grid = (unsigned)((warps * 32u + kGatherThreads - 1) / kGatherThreads);
    if (layout == 0) { if (elem == kFp8) gather_kernel<0, kFp8><<<grid, kGatherThreads, 0, st>>>(a, ids, n_ids, side); else gather_kernel<0, kBf16><<<grid, kGatherThreads, 0, st>>>(a, ids, n_ids, side); }
    else if (layout == 1) { if (elem == kFp8) gather_kernel<1, kFp8><<<grid, kGatherThreads, 0, st>>>(a, ids, n_ids, side); else gather_kernel<1, kBf16><<<grid, kGatherThreads, 0, st>>>(a, ids, n_ids, side); }
    else { if (elem == kFp8) gather_kernel<2, kFp8><<<grid, kGatherThreads, 0, st>>>(a, ids, n_ids, side); else gather_kernel<2, kBf16><<<grid, kGatherThreads, 0, st>>>(a, ids, n_ids, side); }
    return cudaGetLastError();
}

/* ---- uncompressed fp8 weight-only matvec: y[i] = bf16(scale[i] * sum_k fp8[i][k] x[k]) ----------------------------- */
/* One warp per two rows; 16 weights per lane and step (128-bit loads), e4m3 pairs converted to f16x2 in hardware and
   multiplied with f16x2 x; every 16 products are summed in f16x2 and then folded into fp32. */
__device__ __forceinline__ uint32_t e4m3x2_to_f16x2(uint32_t two_bytes) {
    uint32_t r; asm("cvt.rn.f16x2.e4m3x2 %0, %1;" : "=r"(r) : "h"((unsigned short)two_bytes)); return r;
}
__device__ __forceinline__ float dot16_fp8(uint4 w, const uint32_t (&xh)[8]) {
    const uint32_t c[4] = {w.x, w.y, w.z, w.w};
    __half2 s0 = __float2half2_rn(0.f), s1 = s0;
#pragma unroll
    for (int j = 0; j < 4; j++) {
        const uint32_t lo = e4m3x2_to_f16x2(c[j] & 0xFFFFu), hi = e4m3x2_to_f16x2(c[j] >> 16);
        s0 = __hfma2(*reinterpret_cast<const __half2 *>(&lo), *reinterpret_cast<const __half2 *>(&xh[2 * j]), s0);
        s1 = __hfma2(*reinterpret_cast<const __half2 *>(&hi), *reinterpret_cast<const __half2 *>(&xh[2 * j + 1]), s1);
    }
    const float2 f0 = __half22float2(s0), f1 = __half22float2(s1);
    return (f0.x + f0.y) + (f1.x + f1.y);
}

/* Uncompressed fp8 weight-only matvec (the bandwidth baseline NWC-fp8 is compared with).  A warp takes kNativeRows rows at
   a time so that the fp32 -> half conversion of its slice of x is paid once per kNativeRows rows and that many 16-byte
   loads per lane are in flight. */
constexpr uint32_t kNativeRows = 8;
__global__ void __launch_bounds__(256) native_fp8_kernel(const uint8_t *__restrict__ w, const float *__restrict__ scale, const float *__restrict__ x,
                                                         uint16_t *__restrict__ y, uint32_t M, uint32_t K) {
    const uint32_t lane = threadIdx.x & 31u, warps = gridDim.x * (blockDim.x >> 5);
    for (uint32_t row0 = kNativeRows * (blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5)); row0 < M; row0 += kNativeRows * warps) {
        const uint32_t rows = min(kNativeRows, M - row0);
        float acc[kNativeRows];
#pragma unroll
        for (uint32_t r = 0; r < kNativeRows; r++) acc[r] = 0.f;
        if ((K & 15u) == 0u) {
            for (uint32_t k = lane * 16u; k < K; k += 512u) {
                uint4 wv[kNativeRows];
#pragma unroll
                for (uint32_t r = 0; r < kNativeRows; r++) wv[r] = r < rows ? ldg_stream128(w + (uint64_t)(row0 + r) * K + k) : make_uint4(0u, 0u, 0u, 0u);
                uint32_t xh[8];
#pragma unroll
                for (int i = 0; i < 4; i++) {
                    const float4 v = __ldg(reinterpret_cast<const float4 *>(x + k) + i);
                    const __half2 p0 = __floats2half2_rn(v.x, v.y), p1 = __floats2half2_rn(v.z, v.w);
                    xh[2 * i] = *reinterpret_cast<const uint32_t *>(&p0); xh[2 * i + 1] = *reinterpret_cast<const uint32_t *>(&p1);
                }
#pragma unroll
                for (uint32_t r = 0; r < kNativeRows; r++) acc[r] += dot16_fp8(wv[r], xh);
            }
        } else {
            for (uint32_t k = lane; k < K; k += 32u) {
                const float xv = __ldg(x + k);
#pragma unroll
                for (uint32_t r = 0; r < kNativeRows; r++) if (r < rows) acc[r] = fmaf(fp8_to_float(w[(uint64_t)(row0 + r) * K + k]), xv, acc[r]);
            }
        }
#pragma unroll
        for (uint32_t r = 0; r < kNativeRows; r++) {
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) acc[r] += __shfl_xor_sync(0xffffffffu, acc[r], o);
        }
        if (lane == 0) {
#pragma unroll
            for (uint32_t r = 0; r < kNativeRows; r++) if (r < rows) y[row0 + r] = bf16_round(acc[r] * scale[row0 + r]);
        }
    }
}

cudaError_t launch_native_fp8(int sms, cudaStream_t st, const uint8_t *w, const float *scale, const float *x, uint16_t *y, uint32_t M, uint32_t K) {
    const uint32_t units = (M + kNativeRows - 1u) / kNativeRows;
    unsigned grid = (units + 7u) / 8u;
    if (grid > (unsigned)sms * 8u) grid = (unsigned)sms * 8u;
    native_fp8_kernel<<<grid, 256, 0, st>>>(w, scale, x, y, M, K);
    return cudaGetLastError();
}

}  // namespace nwc
