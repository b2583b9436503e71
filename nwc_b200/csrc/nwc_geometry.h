/* Block geometry of the NWC on-disk formats v9 / v10 / v11 (layouts 0, 1, 2), shared by host and device code.
 *
 * A matrix of M rows and K columns is tiled into blocks of `rows` x 512 weights (rows = 8 for layout 0, 16 for
 * layouts 1 and 2).  Blocks are numbered row-group-major: block = row_group * CB + column_block.  Every block holds
 * 32 lane streams.  The sizes below are the ones the reference library reports through nwc_layout
 * (reference: csrc/nwc_ops.cu:87-126).
 */
#pragma once
#include <cstdint>

#if defined(__CUDACC__)
#define NWC_HD __host__ __device__ __forceinline__
#else
#define NWC_HD inline
#endif

namespace nwc {

constexpr uint32_t kLanes = 32;            /* lane streams per block                                    */
constexpr uint32_t kBlockCols = 512;       /* columns per block                                         */
constexpr uint32_t kBlockWeights = 4096;   /* the `block` argument of the C-ABI (8 x 512)               */
constexpr uint32_t kPeekBits = 12;         /* index width of the on-disk decoder table                  */
constexpr uint32_t kTableWords = 1u << kPeekBits;
constexpr uint32_t kSymTableLen = 1024;    /* length of the freq / psym arrays of the encoder interface */
constexpr uint32_t kEscape = 1u << 30;     /* table entry: "not two complete codes"                     */
constexpr int kFormatVersion = 11;

enum ElemType : int { kBf16 = 0, kFp8 = 1 };

NWC_HD int type_of(int code) { return code & 15; }
NWC_HD int layout_of(int code) { return (code >> 4) & 15; }

struct Geometry {
    uint32_t M, K;
    uint32_t rows;             /* rows per block                                                       */
    uint32_t K16;              /* K rounded up to 16: row stride of dequantised output                 */
    uint32_t CB;               /* column blocks                                                        */
    uint32_t groups;           /* row groups                                                           */
    uint32_t nb;               /* blocks                                                               */
    uint32_t last_chunks;      /* coded 16-column chunks in the last column block                      */
    uint32_t last_super;       /* 32-column super-chunks in the last column block                      */
    uint32_t slots;            /* super-chunk slots per row group in the planes of layouts 1 / 2       */
    uint32_t pair_slots;       /* super-chunk pairs per row group (layout 2 fp8 raw plane)             */

    NWC_HD Geometry(uint32_t m, uint32_t k, int layout) : M(m), K(k) {
        rows = layout ? 16u : 8u;
        K16 = (K + 15u) & ~15u;
        CB = (K + kBlockCols - 1) / kBlockCols;
        groups = (M + rows - 1) / rows;
        nb = groups * CB;
        last_chunks = (K16 - (CB - 1) * kBlockCols) >> 4;
        last_super = (last_chunks + 1) >> 1;
        slots = 16u * (CB - 1) + last_super;
        pair_slots = 8u * (CB - 1) + ((last_super + 1) >> 1);
    }
    NWC_HD uint32_t padded_rows() const { return groups * rows; }
    /* super-chunks coded in column block cb */
    NWC_HD uint32_t supers_in(uint32_t cb) const { return cb == CB - 1 ? last_super : 16u; }
    NWC_HD uint64_t nibble_plane_bytes() const { return (uint64_t)groups * slots * kLanes * 8u; }
    NWC_HD uint64_t raw_plane_bytes(int code) const {
        const int t = type_of(code), lay = layout_of(code);
        if (lay == 2)
            return nibble_plane_bytes() + (t == kFp8 ? (uint64_t)groups * pair_slots * 3u * kLanes * 4u
                                                     : (uint64_t)groups * slots * kLanes * 16u);
        if (lay == 1) return (uint64_t)groups * slots * kLanes * (t == kFp8 ? 8u : 16u);
        return t == kFp8 ? (uint64_t)M * (K16 >> 1) : (uint64_t)M * K16;
    }
    NWC_HD uint64_t scratch_floats() const { return (uint64_t)padded_rows() * CB; }
};

/* (row, column) inside a 16 x 32 super-chunk of element i (0..15) of lane L: the element order of two m16n8k16
   A fragments (reference: csrc/nwc_ops.cu:154-160). */
NWC_HD uint32_t frag_row(uint32_t L, uint32_t i) { return (L >> 2) + (((i >> 1) & 1u) << 3); }
NWC_HD uint32_t frag_col(uint32_t L, uint32_t i) { return ((L & 3u) << 3) + (((i >> 3) & 1u) << 2) + (((i >> 2) & 1u) << 1) + (i & 1u); }

}  // namespace nwc
