/* Prefill (many tokens at once): Y[T][M] = X[T][K] * W^T with W decoded tile by tile straight into the operands of a
 * tcgen05 tensor-core GEMM - no decompressed copy of W is ever written to global memory.
 *
 * The reference dequantises the whole matrix into a temporary bf16 buffer and calls a dense matmul on it
 * (nwc/nwc_torch.py:320-323, csrc/nwc_ops.cu:1121-1126); at prefill the contraction is dense, so here it runs on the
 * 5th-generation tensor cores: tcgen05.mma (cta_group::1, kind::f16, bf16 in, fp32 accumulate in tensor memory),
 * issued by one thread, operands in shared memory in the K-major 128-byte-swizzled layout, completion signalled
 * through tcgen05.commit on an mbarrier, accumulator read back with tcgen05.ld for the epilogue.
 *
 * One CTA owns 128 rows of W (the MMA's M) and up to 256 tokens (N); tensor memory holds the 128 x N fp32 tile.
 * K advances in chunks of 64 columns (one swizzle atom) through four operand stages.  Sixteen warps decode the chunk of
 * W - layout 2: one super-chunk slot per warp, nibble + raw bytes -> bf16 fragments -> 8-byte swizzled stores - one lane
 * of a seventeenth warp fetches the chunk of X with one tensor-map copy (cp.async.bulk.tensor from this GPU's own memory to this
 * CTA only; the copy engine swizzles), one lane of an eighteenth issues the four K = 16 MMAs.  The roles hand stages
 * over through mbarriers only, so decoding runs ahead of the tensor core instead of in step with it.  Every wait is
 * bounded; on a timeout the role records the status word and stops, the CTA frees its tensor memory and leaves.
 * Layout 2 / bf16 only for now; other layouts take the dequantise-then-matmul route in the Python module.
 */
#include <atomic>
#include <cuda.h>
#include "nwc_decode.cuh"
#include "nwc_async.cuh"
#include "nwc_launch.h"

namespace nwc {

constexpr uint32_t kPfDecodeThreads = 512, kPfThreads = kPfDecodeThreads + 64u /* + the warp that copies X and the warp that issues the MMAs */, kPfRows = 128, kPfK = 64, kPfHalfTokens = 256 /* most tokens of one MMA */, kPfAhead = 3, kPfFar = 12;
constexpr uint32_t kPfABytes = kPfRows * 128u, kPfHalfBytes = kPfHalfTokens * 128u;
/* A CTA multiplies its 128 rows with one or two halves of 256 tokens (HALVES): two halves reuse every decoded W tile for
   twice the tokens and fill all 512 columns of tensor memory, but their B tiles leave room for two operand stages only. */
__host__ __device__ constexpr uint32_t pf_stages(uint32_t halves) { return halves == 1u ? 4u : 2u; }
__host__ __device__ constexpr uint32_t pf_smem(uint32_t halves) { return 1024u /* alignment slack */ + pf_stages(halves) * (kPfABytes + halves * kPfHalfBytes) + 3u * pf_stages(halves) * 8u + 32u; }

/* shared-memory matrix descriptor: K-major tile, 128-byte swizzle, 8-row groups 1024 bytes apart */
__device__ __forceinline__ uint64_t smem_desc_sw128(uint32_t addr) {
    return (uint64_t)((addr & 0x3FFFFu) >> 4) | ((uint64_t)1u << 16) | ((uint64_t)(1024u >> 4) << 32) | ((uint64_t)1u << 46) | ((uint64_t)2u << 61);
}
/* instruction descriptor, kind::f16: fp32 accumulate, bf16 x bf16, both operands K-major, M x N */
__host__ __device__ constexpr uint32_t instr_desc_bf16(uint32_t M, uint32_t N) {
    return (1u << 4) | (1u << 7) | (1u << 10) | ((N >> 3) << 17) | ((M >> 4) << 24);
}
/* byte offset of (row, 16-byte chunk c) inside a swizzled K-major tile of 128-byte rows */
__device__ __forceinline__ uint32_t sw128(uint32_t row, uint32_t c) { return (row >> 3) * 1024u + (row & 7u) * 128u + ((c ^ (row & 7u)) << 4); }

__device__ __forceinline__ void sts64(uint32_t addr, uint32_t a, uint32_t b) { asm volatile("st.shared.v2.u32 [%0], {%1, %2};" ::"r"(addr), "r"(a), "r"(b) : "memory"); }
__device__ __forceinline__ void sts128(uint32_t addr, uint4 v) { asm volatile("st.shared.v4.u32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w) : "memory"); }
__device__ __forceinline__ void sts16(uint32_t addr, uint16_t v) { asm volatile("st.shared.u16 [%0], %1;" ::"r"(addr), "h"(v) : "memory"); }

struct PrefillArgs {
    SegmentArgs w;               /* the compressed matrix (x, y unused)               */
    const uint16_t *X;           /* bf16 [T][ldx]                                     */
    uint16_t *Y;                 /* bf16 [T][ldy]                                     */
    uint32_t T, ldx, ldy;
};

/* one 64-column x 256-token box of X, swizzled by the copy engine, into shared memory; completion = `bytes` on the barrier.
   (tiled TMA load from this GPU's own memory into this CTA only; x is a multiple of 64 elements = 128 bytes) */
__device__ __forceinline__ void tma_load_x(uint32_t dst, const CUtensorMap *map, uint32_t x, uint32_t y, uint32_t bar) {
    asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
                 ::"r"(dst), "l"(map), "r"(x), "r"(y), "r"(bar) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) { asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory"); }

/* Roles.  Warps 0..15 decode: chunk k of W (64 columns) into the A tile of stage k % kPfStages, one super-chunk slot per
   warp, from registers loaded three chunks earlier; they announce the tile on the stage's `filled` barrier (16 arrivals).
   Warp 16 (one lane) copies: the X tile of chunk k by one tensor-map copy into the stage's B tile, completion on the
   stage's `landed` barrier.  Warp 17 (one lane) multiplies: waits for `filled` and `landed`, issues the four K = 16 MMAs of
   the chunk and commits them to the stage's `freed` barrier, which the decoders and the copier wait for before they
   overwrite the stage four chunks later.  No CTA barrier inside the loop: the three roles run up to kPfStages chunks
   apart.  Every wait is bounded; a role that gives up records the status word and stops, the others then run out too. */
template <uint32_t HALVES>
__global__ void __launch_bounds__(kPfThreads, 1) prefill_kernel_layout2(const PrefillArgs p, const __grid_constant__ CUtensorMap xmap) {
    constexpr uint32_t kPfStages = pf_stages(HALVES), kPfMaxTokens = HALVES * kPfHalfTokens, kPfBBytes = HALVES * kPfHalfBytes;
    extern __shared__ uint8_t pf_smem_raw[];
    const uint32_t base = (smem_addr(pf_smem_raw) + 1023u) & ~1023u;            /* swizzled tiles want 1024-byte alignment */
    const uint32_t a_buf = base, b_buf = base + kPfStages * kPfABytes, bars = b_buf + kPfStages * kPfBBytes;
    const uint32_t filled = bars, landed = bars + kPfStages * 8u, freed = bars + 2u * kPfStages * 8u, tmem_slot = bars + 3u * kPfStages * 8u;
    const uint32_t tid = threadIdx.x, lane = tid & 31u, warp = tid >> 5, r = lane >> 2, q = lane & 3u;
    const SegmentArgs &a = p.w;
    const Geometry g(a.M, a.K, 2);
    const uint32_t m0 = blockIdx.x * kPfRows, t0 = blockIdx.y * kPfMaxTokens;
    const uint32_t nt = min(kPfMaxTokens, p.T - t0), N = (nt + 15u) & ~15u;         /* MMA N: multiple of 16 */
    uint32_t ncols = 32; while (ncols < N) ncols <<= 1;                              /* tensor-memory columns: power of two >= 32 */
    constexpr uint32_t kDecodeWarps = kPfDecodeThreads / 32u;
    if (warp == 0) {
        if (lane == 0) {
            for (uint32_t s = 0; s < kPfStages; s++) { mbar_init(filled + s * 8u, kDecodeWarps); mbar_init(landed + s * 8u, 1u); mbar_init(freed + s * 8u, 1u); }
            mbar_init_fence();
        }
        __syncwarp();
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(tmem_slot), "r"(ncols) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    const uint8_t *raw_plane = a.low + g.nibble_plane_bytes();
    const uint32_t chunks = (a.K + kPfK - 1u) / kPfK;
    const uint32_t n_lo = min(N, kPfHalfTokens), n_hi = N - n_lo;                   /* tokens of the first and the second MMA of a step */
    const uint32_t idesc = instr_desc_bf16(kPfRows, n_lo), idesc_hi = instr_desc_bf16(kPfRows, n_hi ? n_hi : 16u);
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem = lds32(tmem_slot);
    bool alive = true;
    if (warp < kDecodeWarps) {
        /* ---- decoders ---- */
        const uint32_t rg = (m0 >> 4) + (warp >> 1);                                /* this warp's row group */
        const bool rows_live = rg < g.groups;
        /* the slot of chunk k into registers; the slot of chunk k + kPfFar is asked into L2 at the same time, so that the
           register loads (three chunks ahead of their use) find their lines there instead of in HBM */
        auto load_w = [&](uint32_t k, uint2 &nib, uint4 &raw) {
            const uint32_t slot = 2u * k + (warp & 1u);
            nib = make_uint2(0u, 0u); raw = make_uint4(0u, 0u, 0u, 0u);
            if (k < chunks && rows_live && slot < g.slots) {
                const uint64_t cell = ((uint64_t)rg * g.slots + slot) * kLanes + lane;
                nib = ldg_stream64(a.low + cell * 8u);
                raw = ldg_stream128(raw_plane + cell * 16u);
                if (slot + 2u * kPfFar < g.slots) {
                    const uint64_t far = cell + (uint64_t)2u * kPfFar * kLanes;
                    if ((lane & 15u) == 0u) asm volatile("prefetch.global.L2 [%0];" ::"l"(a.low + far * 8u));          /* 128 bytes per 16 lanes */
                    if ((lane & 7u) == 0u) asm volatile("prefetch.global.L2 [%0];" ::"l"(raw_plane + far * 16u));       /* 128 bytes per 8 lanes  */
                }
            }
        };
        /* exception count of this lane and data offset of the block (512 columns = 8 chunks) that holds chunk k; the next
           block's are loaded while this one is in use and its entries are pulled towards L1 */
        uint32_t cnt = 0, ebase = 0, cnt_next = 0, ebase_next = 0, before = 0, total = 0, before_next = 0, total_next = 0;
        uint32_t e0 = 0, e1 = 0, e0_next = 0, e1_next = 0;       /* this lane's first two exception entries of the block: index | value << 8 */
        auto load_block = [&](uint32_t cb, uint32_t &c, uint32_t &b) {
            c = 0u; b = 0u;
            if (rows_live && cb < g.CB) { const uint32_t blk = rg * g.CB + cb; c = __ldg(a.hdr + (uint64_t)blk * kLanes + lane); b = __ldg(a.bases + blk); }
        };
        /* where the lane's entries of the next block start, and its first two entries, into registers (the rest, rare, is
           read when needed) */
        auto load_entries = [&]() {
            before_next = warp_exclusive_sum(cnt_next, lane, total_next);
            const uint8_t *ep = a.data + ebase_next + (uint64_t)before_next * 3u;
            e0_next = cnt_next >= 1u ? (uint32_t)ep[0] | ((uint32_t)ep[1] << 8) | ((uint32_t)ep[2] << 16) : 0u;
            e1_next = cnt_next >= 2u ? (uint32_t)ep[3] | ((uint32_t)ep[4] << 8) | ((uint32_t)ep[5] << 16) : 0u;
        };
        FixedTables tab; tab.load(a.lut);
        uint2 n0, n1, n2; uint4 r0, r1, r2;
        static_assert(kPfAhead == 3u, "three register sets travel ahead of the decode");
        load_w(0u, n0, r0); load_w(1u, n1, r1); load_w(2u, n2, r2);
        load_block(0u, cnt_next, ebase_next);
        load_entries();
        const uint32_t mm = (warp >> 1) * 16u + r, cc = (warp & 1u) * 4u + q;
        const uint32_t off_lo = sw128(mm, cc), off_hi = sw128(mm + 8u, cc);       /* where this lane's two rows of the slot go */
        /* one chunk; (wn, wr) = the register set that holds its compressed slot and is reloaded with chunk k + kPfAhead
           (the loop rotates three sets by name: a register that still waits for its load must not be moved) */
        auto step = [&](const uint32_t k, uint2 &wn, uint4 &wr) -> bool {
            const uint32_t s = k % kPfStages, abase = a_buf + s * kPfABytes;
            if ((k & 7u) == 0u) {                                                    /* a new block of W begins */
                cnt = cnt_next; ebase = ebase_next; before = before_next; total = total_next; e0 = e0_next; e1 = e1_next;
                load_block((k >> 3) + 1u, cnt_next, ebase_next);
            } else if ((k & 7u) == 4u) load_entries();                               /* (the next block's counts have arrived by now) */
            const uint32_t slot = 2u * k + (warp & 1u);
            const bool live = rows_live && slot < g.slots;
            uint32_t f[8];
            fixed_half<kBf16, 0>(tab, wn.x, wr.x, wr.y, 0u, 0u, 0u, f[0], f[1], f[2], f[3]);
            fixed_half<kBf16, 2>(tab, wn.y, wr.z, wr.w, 0u, 0u, 0u, f[4], f[5], f[6], f[7]);
            if (!live) { for (uint32_t e = 0; e < 8u; e++) f[e] = 0u; }
            load_w(k + kPfAhead, wn, wr);
            /* the stage's last user was chunk k - kPfStages: its MMAs must be done before the tile is overwritten */
            if (k >= kPfStages && !mbar_wait(freed + s * 8u, ((k / kPfStages) - 1u) & 1u)) return false;
            /* f[0], f[2]: row r, columns 8q + 0..3;  f[1], f[3]: row r + 8;  f[4..7]: the same for columns 8q + 4..7 */
            sts64(abase + off_lo, f[0], f[2]);      sts64(abase + off_lo + 8u, f[4], f[6]);
            sts64(abase + off_hi, f[1], f[3]);      sts64(abase + off_hi + 8u, f[5], f[7]);
            if (total && live) {                                  /* exceptions of this slot overwrite their +-0 placeholders */
                auto patch = [&](uint32_t entry) {
                    const uint32_t i = entry & 0xFFu, j = i & 15u;
                    if ((i >> 4) != (slot & 15u)) return;
                    const uint32_t col = (warp & 1u) * 32u + frag_col(lane, j), row = (warp >> 1) * 16u + frag_row(lane, j);
                    sts16(abase + sw128(row, col >> 3) + (col & 7u) * 2u, (uint16_t)(entry >> 8));
                };
                if (cnt >= 1u) patch(e0);
                if (cnt >= 2u) patch(e1);
                if (cnt > 2u) {
                    const uint8_t *ep = a.data + ebase + (uint64_t)before * 3u + 6u;
                    for (uint32_t e = 2; e < cnt; e++, ep += 3) patch((uint32_t)ep[0] | ((uint32_t)ep[1] << 8) | ((uint32_t)ep[2] << 16));
                }
            }
            async_proxy_fence();                                                     /* generic-proxy stores -> visible to the tensor core */
            __syncwarp();
            if (lane == 0) mbar_arrive(filled + s * 8u);
            return true;
        };
        for (uint32_t k = 0; k < chunks && alive; k += 3u) {
            alive = step(k, n0, r0);
            if (alive && k + 1u < chunks) alive = step(k + 1u, n1, r1);
            if (alive && k + 2u < chunks) alive = step(k + 2u, n2, r2);
        }
    } else if (warp == kDecodeWarps) {
        /* ---- copier: the X tile of every chunk, kPfStages chunks ahead of the MMAs at most ---- */
        if (lane == 0) {
            for (uint32_t k = 0; k < chunks; k++) {
                const uint32_t s = k % kPfStages;
                if (k >= kPfStages && !mbar_wait_one(freed + s * 8u, ((k / kPfStages) - 1u) & 1u)) { alive = false; break; }
                mbar_expect(landed + s * 8u, kPfBBytes);
#pragma unroll
                for (uint32_t h = 0; h < HALVES; h++)                               /* (a box wholly beyond T arrives as zeros) */
                    tma_load_x(b_buf + s * kPfBBytes + h * kPfHalfBytes, &xmap, k * kPfK, t0 + h * kPfHalfTokens, landed + s * 8u);
            }
        }
        alive = __shfl_sync(0xffffffffu, alive ? 1 : 0, 0) != 0;
    } else {
        /* ---- multiplier ---- */
        if (lane == 0) {
            const uint64_t adesc0 = smem_desc_sw128(a_buf), bdesc0 = smem_desc_sw128(b_buf);
            for (uint32_t k = 0; k < chunks; k++) {
                const uint32_t s = k % kPfStages, phase = (k / kPfStages) & 1u;
                if (!mbar_wait_one(filled + s * 8u, phase) || !mbar_wait_one(landed + s * 8u, phase)) { alive = false; break; }
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                const uint64_t adesc = adesc0 + ((s * kPfABytes) >> 4), bdesc = bdesc0 + ((s * kPfBBytes) >> 4);
#pragma unroll
                for (uint32_t kk = 0; kk < kPfK / 16u; kk++) {                      /* 16 bf16 = 32 bytes further along K: +2 in the descriptor's address field */
                    const uint32_t accumulate = (k | kk) ? 1u : 0u;
                    asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\ttcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
                                 ::"r"(tmem), "l"(adesc + 2u * kk), "l"(bdesc + 2u * kk), "r"(idesc), "r"(accumulate) : "memory");
                    if (HALVES > 1u && n_hi)                                        /* the same W tile against the second half of the tokens */
                        asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\ttcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
                                     ::"r"(tmem + kPfHalfTokens), "l"(adesc + 2u * kk), "l"(bdesc + (kPfHalfBytes >> 4) + 2u * kk), "r"(idesc_hi), "r"(accumulate) : "memory");
                }
                asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(freed + s * 8u) : "memory");
            }
        }
        alive = __shfl_sync(0xffffffffu, alive ? 1 : 0, 0) != 0;
    }
    /* ---- epilogue: wait for the last MMAs, read the accumulator, scale, bias, round, store ---- */
    {
        bool done = alive;
        if (done && chunks) done = mbar_wait(freed + ((chunks - 1u) % kPfStages) * 8u, ((chunks - 1u) / kPfStages) & 1u);
        alive = __syncthreads_and(done);
    }
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    if (alive && warp < kDecodeWarps) {
        const uint32_t quarter = warp & 3u, row = m0 + quarter * 32u + lane;       /* a warp reads the 32 tensor-memory lanes of its quarter */
        const float sc = (a.scale && row < a.M) ? __ldg(a.scale + row) : 1.f, bi = (a.bias && row < a.M) ? bf16_to_float(__ldg(a.bias + row)) : 0.f;
        for (uint32_t c0 = (warp >> 2) * 16u; c0 < N; c0 += 64u) {                 /* the four warps of a quarter take every fourth 16-column group */
            uint32_t v[16];
            asm volatile("tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
                         : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]), "=r"(v[8]), "=r"(v[9]), "=r"(v[10]),
                           "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15])
                         : "r"(tmem + ((quarter * 32u) << 16) + c0));
            asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
            if (row < a.M) {
#pragma unroll
                for (uint32_t e = 0; e < 16u; e++)
                    if (c0 + e < nt) p.Y[(uint64_t)(t0 + c0 + e) * p.ldy + row] = bf16_round_nan(__uint_as_float(v[e]) * sc + bi);
            }
        }
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (warp == 0) asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(ncols) : "memory");
}

/* cuTensorMapEncodeTiled through the runtime's driver entry point (the library does not link against the driver) */
typedef CUresult (*EncodeTiledFn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *, const cuuint64_t *, const cuuint32_t *,
                                  const cuuint32_t *, CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
static EncodeTiledFn encode_tiled() {
    static std::atomic<void *> cached{nullptr};
    void *fn = cached.load(std::memory_order_acquire);
    if (!fn) {
        cudaDriverEntryPointQueryResult res;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &res) != cudaSuccess || res != cudaDriverEntryPointSuccess) { cudaGetLastError(); return nullptr; }
        cached.store(fn, std::memory_order_release);
    }
    return reinterpret_cast<EncodeTiledFn>(fn);
}

static uint32_t g_prefill_halves = 0;                            /* 0 = choose per launch; 1 or 2 = the tests' choice */
void set_prefill_halves(int halves) { g_prefill_halves = halves == 1 || halves == 2 ? (uint32_t)halves : 0u; }

cudaError_t launch_prefill_layout2(cudaStream_t st, const SegmentArgs &w, const uint16_t *X, uint16_t *Y, uint32_t T, uint32_t ldx, uint32_t ldy) {
    PrefillArgs p{w, X, Y, T, ldx, ldy};
    /* X as a 2-D tensor (K innermost, T rows of ldx elements), boxes of 64 columns x 256 tokens, 128-byte swizzle, zeros
       outside the tensor: the layout the B operand's shared-memory descriptor describes */
    const EncodeTiledFn encode = encode_tiled();
    if (!encode) return cudaErrorNotSupported;
    alignas(64) CUtensorMap xmap;
    const cuuint64_t dims[2] = {w.K, T}, strides[1] = {(cuuint64_t)ldx * 2u};
    const cuuint32_t box[2] = {kPfK, kPfHalfTokens}, elem_strides[2] = {1u, 1u};
    if (encode(&xmap, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2u, const_cast<uint16_t *>(X), dims, strides, box, elem_strides, CU_TENSOR_MAP_INTERLEAVE_NONE,
               CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS) return cudaErrorInvalidValue;
    /* Two halves per CTA halve the decode work per token but also the number of CTAs, and a two-halves CTA takes about
       1.15 x as long (measured: 6144 x 2560 x 512 runs 44 us on 96 one-half CTAs, 50 us on 48 two-halves CTAs; 19456 x 2560
       x 512 runs 106 us on 304 and 92 us on 152): take them when they save whole waves of CTAs. */
    int dev = 0, sms = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || sms <= 0) return cudaErrorNoDevice;
    const uint32_t row_tiles = (w.M + kPfRows - 1u) / kPfRows;
    const uint64_t ctas1 = (uint64_t)row_tiles * ((T + kPfHalfTokens - 1u) / kPfHalfTokens), ctas2 = (uint64_t)row_tiles * ((T + 2u * kPfHalfTokens - 1u) / (2u * kPfHalfTokens));
    const uint64_t waves1 = (ctas1 + (uint64_t)sms - 1u) / (uint64_t)sms, waves2 = (ctas2 + (uint64_t)sms - 1u) / (uint64_t)sms;
    const uint32_t halves = g_prefill_halves ? g_prefill_halves : (T > kPfHalfTokens && waves2 * 115u < waves1 * 100u ? 2u : 1u), tokens = halves * kPfHalfTokens;
    const dim3 grid(row_tiles, (T + tokens - 1u) / tokens);
    if (halves == 2u) prefill_kernel_layout2<2u><<<grid, kPfThreads, pf_smem(2u), st>>>(p, xmap);
    else prefill_kernel_layout2<1u><<<grid, kPfThreads, pf_smem(1u), st>>>(p, xmap);
    return cudaGetLastError();
}

/* shared-memory opt-in of the prefill kernel on the current device (attributes of a function are per device) */
void configure_prefill_kernels() {
    cudaFuncSetAttribute(prefill_kernel_layout2<1u>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)pf_smem(1u));
    cudaFuncSetAttribute(prefill_kernel_layout2<2u>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)pf_smem(2u));
}

int read_prefill_status(bool clear) {
    int v = 0;
    if (cudaMemcpyFromSymbol(&v, g_kernel_status, sizeof(int)) != cudaSuccess) return -1;
    if (clear && v) { const int z = 0; cudaMemcpyToSymbol(g_kernel_status, &z, sizeof(int)); }
    return v;
}

}  // namespace nwc
