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
 * K advances in chunks of 64 columns (one swizzle atom): the CTA's 16 warps decode the chunk of W - layout 2: one
 * super-chunk slot per warp, nibble + raw bytes -> bf16 fragments -> 8-byte swizzled stores - and copy the chunk of X,
 * then one thread issues four K = 16 MMAs.  Two operand buffers alternate, so decoding chunk k + 1 overlaps the MMAs of
 * chunk k.  Every wait is bounded; on a timeout the CTA records the status word, frees its tensor memory and leaves.
 * Layout 2 / bf16 only for now; other layouts take the dequantise-then-matmul route in the Python module.
 */
#include "nwc_decode.cuh"
#include "nwc_async.cuh"
#include "nwc_launch.h"

namespace nwc {

constexpr uint32_t kPfDecodeThreads = 512, kPfThreads = kPfDecodeThreads + 32u /* + the warp that issues the MMAs */, kPfRows = 128, kPfK = 64, kPfMaxTokens = 256, kPfStages = 4, kPfAhead = 3, kPfAheadX = 2;
constexpr uint32_t kPfABytes = kPfRows * 128u, kPfBBytes = kPfMaxTokens * 128u;
constexpr uint32_t kPfSmem = 1024u /* alignment slack */ + kPfStages * (kPfABytes + kPfBBytes) + 64u;

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

/* 16 bytes global -> shared without passing through registers; bytes beyond src_bytes are written as zeros */
__device__ __forceinline__ void cp_async16(uint32_t dst, const void *src, uint32_t src_bytes) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(src), "r"(src_bytes) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N> __device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

__global__ void __launch_bounds__(kPfThreads, 1) prefill_kernel_layout2(const PrefillArgs p) {
    extern __shared__ uint8_t pf_smem_raw[];
    const uint32_t base = (smem_addr(pf_smem_raw) + 1023u) & ~1023u;            /* swizzled tiles want 1024-byte alignment */
    const uint32_t a_buf = base, b_buf = base + kPfStages * kPfABytes, bars = b_buf + kPfStages * kPfBBytes, tmem_slot = bars + kPfStages * 8u;
    const uint32_t tid = threadIdx.x, lane = tid & 31u, warp = tid >> 5, r = lane >> 2, q = lane & 3u;
    const SegmentArgs &a = p.w;
    const Geometry g(a.M, a.K, 2);
    const uint32_t m0 = blockIdx.x * kPfRows, t0 = blockIdx.y * kPfMaxTokens;
    const uint32_t nt = min(kPfMaxTokens, p.T - t0), N = (nt + 15u) & ~15u;         /* MMA N: multiple of 16 */
    uint32_t ncols = 32; while (ncols < N) ncols <<= 1;                              /* tensor-memory columns: power of two >= 32 */
    if (warp == 0) {
        if (lane == 0) { for (uint32_t s = 0; s < kPfStages; s++) mbar_init(bars + s * 8u, 1u); mbar_init_fence(); }
        __syncwarp();
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(tmem_slot), "r"(ncols) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    const uint8_t *raw_plane = a.low + g.nibble_plane_bytes();
    const uint32_t chunks = (a.K + kPfK - 1u) / kPfK, idesc = instr_desc_bf16(kPfRows, N);
    const uint32_t rg = (m0 >> 4) + (warp >> 1);                                    /* this warp's row group */
    /* The pipeline.  Chunk k (64 columns of K) lives in stage k % kPfStages.  Its X tile is copied asynchronously (16 bytes
       per copy, straight to the swizzled position) and its compressed W slot is loaded into registers kPfAhead chunks
       before it is needed (X two chunks); in iteration k the warps decode W(k) into the stage's A tile while the tensor
       core still works on chunks k - 2 and k - 1, then one thread issues the MMAs of chunk k, then everybody waits for the
       MMAs of chunk k - 2 (bounded) and refills that chunk's stage with the copies of chunk k + 2. */
    auto load_w = [&](uint32_t k, uint2 &nib, uint4 &raw) {
        const uint32_t slot = 2u * k + (warp & 1u);
        nib = make_uint2(0u, 0u); raw = make_uint4(0u, 0u, 0u, 0u);
        if (k < chunks && rg < g.groups && slot < g.slots) {
            const uint64_t cell = ((uint64_t)rg * g.slots + slot) * kLanes + lane;
            nib = ldg_stream64(a.low + cell * 8u);
            raw = ldg_stream128(raw_plane + cell * 16u);
        }
    };
    /* X tile: N rows of 128 bytes, zero beyond T and beyond K.  Decode thread i copies the 16-byte column i & 7 of rows
       (i >> 3) + 64 j: the same column and, 64 rows = 8 swizzle groups further on, the same offset + 8192 j in the tile. */
    const uint32_t xt = tid >> 3, xc = tid & 7u, x_smem = sw128(xt, xc);
    const uint16_t *x_src = p.X + (uint64_t)(t0 + xt) * p.ldx + xc * 8u;
    const uint64_t x_rows64 = 64ull * p.ldx;
    auto load_x = [&](uint32_t k) {
        if (k < chunks) {
            const uint32_t bbase = b_buf + (k % kPfStages) * kPfBBytes + x_smem, col = k * kPfK + xc * 8u;
            const uint32_t bytes = col < a.K ? min(16u, (a.K - col) * 2u) : 0u;
#pragma unroll
            for (uint32_t j = 0; j < kPfMaxTokens / 64u; j++) {
                const uint32_t row = xt + 64u * j;
                if (row < N) cp_async16(bbase + j * 8192u, row < nt ? x_src + j * x_rows64 + k * kPfK : p.X, row < nt ? bytes : 0u);
            }
        }
        cp_async_commit();                                                           /* one group per chunk, empty or not */
    };
    /* exception count of this lane and data offset of the block (512 columns = 8 chunks) that holds chunk k; the next block's
       are loaded while this one is in use and its entries are pulled towards L1 */
    uint32_t cnt = 0, ebase = 0, cnt_next = 0, ebase_next = 0, before = 0, total = 0;
    auto load_block = [&](uint32_t cb, uint32_t &c, uint32_t &b) {
        c = 0u; b = 0u;
        if (rg < g.groups && cb < g.CB) { const uint32_t blk = rg * g.CB + cb; c = __ldg(a.hdr + (uint64_t)blk * kLanes + lane); b = __ldg(a.bases + blk); }
    };
    uint2 n0, n1, n2; uint4 r0, r1, r2;
    static_assert(kPfAhead == 3u, "three register sets travel ahead of the decode");
    const bool decoder = warp < kPfDecodeThreads / 32u;                              /* the last warp only issues MMAs */
    if (decoder) {
        load_w(0u, n0, r0); load_w(1u, n1, r1); load_w(2u, n2, r2);
        load_block(0u, cnt_next, ebase_next);
        for (uint32_t k = 0; k < kPfAheadX; k++) load_x(k);
    }
    const uint64_t adesc0 = smem_desc_sw128(a_buf), bdesc0 = smem_desc_sw128(b_buf);
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem = lds32(tmem_slot);
    FixedTables tab; tab.load(a.lut);
    bool alive = true;
    /* one chunk; (wn, wr) = the register set that holds its compressed slot and is reloaded with chunk k + kPfAhead (the
       loop below rotates three sets by name: a register that still waits for its load must not be moved) */
    auto step = [&](const uint32_t k, uint2 &wn, uint4 &wr) -> bool {
        const uint32_t s = k % kPfStages, abase = a_buf + s * kPfABytes, bbase = b_buf + s * kPfBBytes;
        if (decoder) {
        if ((k & 7u) == 0u) {                                                        /* a new block of W begins */
            cnt = cnt_next; ebase = ebase_next;
            before = warp_exclusive_sum(cnt, lane, total);
            load_block((k >> 3) + 1u, cnt_next, ebase_next);
            if (cnt) asm volatile("prefetch.global.L1 [%0];" ::"l"(a.data + ebase + (uint64_t)before * 3u));
        }
        /* ---- W chunk: one super-chunk slot (16 rows x 32 columns) per warp, from the registers loaded three chunks ago ---- */
        {
            const uint32_t slot = 2u * k + (warp & 1u), mm = (warp >> 1) * 16u + r, c = (warp & 1u) * 4u + q;
            uint32_t f[8];
            fixed_half<kBf16, 0>(tab, wn.x, wr.x, wr.y, 0u, 0u, 0u, f[0], f[1], f[2], f[3]);
            fixed_half<kBf16, 2>(tab, wn.y, wr.z, wr.w, 0u, 0u, 0u, f[4], f[5], f[6], f[7]);
            if (!(rg < g.groups && slot < g.slots)) { for (uint32_t e = 0; e < 8u; e++) f[e] = 0u; }
            /* f[0], f[2]: row r, columns 8q + 0..3;  f[1], f[3]: row r + 8;  f[4..7]: the same for columns 8q + 4..7 */
            sts64(abase + sw128(mm, c), f[0], f[2]);          sts64(abase + sw128(mm, c) + 8u, f[4], f[6]);
            sts64(abase + sw128(mm + 8u, c), f[1], f[3]);     sts64(abase + sw128(mm + 8u, c) + 8u, f[5], f[7]);
            if (total && rg < g.groups && slot < g.slots) {   /* exceptions of this slot overwrite their +-0 placeholders */
                __syncwarp();                                  /* (another lane's store above may cover the same 8 bytes) */
                const uint8_t *ep = a.data + ebase + (uint64_t)before * 3u;
                for (uint32_t e = 0; e < cnt; e++, ep += 3) {
                    const uint32_t i = ep[0], j = i & 15u;
                    if ((i >> 4) != (slot & 15u)) continue;
                    const uint32_t col = (warp & 1u) * 32u + frag_col(lane, j), row = (warp >> 1) * 16u + frag_row(lane, j);
                    sts16(abase + sw128(row, col >> 3) + (col & 7u) * 2u, (uint16_t)(ep[1] | (ep[2] << 8)));
                }
            }
        }
        load_w(k + kPfAhead, wn, wr);
        cp_async_wait<(int)kPfAheadX - 1>();                                          /* this thread's copies of the X tile of chunk k have landed */
        async_proxy_fence();                                                         /* generic-proxy writes (stores above, copies) -> visible to the tensor core */
        }
        asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
        if (!__syncthreads_and(alive)) { alive = false; return false; }              /* one decision for the whole CTA */
        if (!decoder) {                                                              /* the MMAs of chunk k go out while the other warps decode chunk k + 1 */
          if (lane == 0) {
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            const uint64_t adesc = adesc0 + ((s * kPfABytes) >> 4), bdesc = bdesc0 + ((s * kPfBBytes) >> 4);
#pragma unroll
            for (uint32_t kk = 0; kk < kPfK / 16u; kk++) {                          /* 16 bf16 = 32 bytes further along K: +2 in the descriptor's address field */
                const uint32_t accumulate = (k | kk) ? 1u : 0u;
                asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\ttcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
                             ::"r"(tmem), "l"(adesc + 2u * kk), "l"(bdesc + 2u * kk), "r"(idesc), "r"(accumulate) : "memory");
            }
            asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bars + s * 8u) : "memory");
          }
          __syncwarp();
          return true;
        }
        /* The stage that chunk k + kPfAheadX will use held chunk k - 2: free once those MMAs are done.  Waiting for chunk
           k - 2, not k - 1, keeps two chunks' MMAs in flight behind the decode (the wait costs the MMA's latency). */
        static_assert(kPfAheadX + 2u == kPfStages, "the refilled stage is the one of chunk k - 2");
        if (k >= 2u) alive = mbar_wait(bars + ((k - 2u) % kPfStages) * 8u, ((k - 2u) / kPfStages) & 1u);
        if (alive) load_x(k + kPfAheadX); else cp_async_commit();
        return true;
    };
    for (uint32_t k = 0; k < chunks; k += 3u) {
        if (!step(k, n0, r0)) break;
        if (k + 1u < chunks && !step(k + 1u, n1, r1)) break;
        if (k + 2u < chunks && !step(k + 2u, n2, r2)) break;
    }
    cp_async_wait<0>();
    /* ---- epilogue: wait for the last MMAs, read the accumulator, scale, bias, round, store ---- */
    {
        bool done = alive;
        if (done && chunks) done = mbar_wait(bars + ((chunks - 1u) % kPfStages) * 8u, ((chunks - 1u) / kPfStages) & 1u);
        alive = __syncthreads_and(done);
    }
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    if (alive && decoder) {
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

cudaError_t launch_prefill_layout2(cudaStream_t st, const SegmentArgs &w, const uint16_t *X, uint16_t *Y, uint32_t T, uint32_t ldx, uint32_t ldy) {
    PrefillArgs p{w, X, Y, T, ldx, ldy};
    const dim3 grid((w.M + kPfRows - 1u) / kPfRows, (T + kPfMaxTokens - 1u) / kPfMaxTokens);
    prefill_kernel_layout2<<<grid, kPfThreads, kPfSmem, st>>>(p);
    return cudaGetLastError();
}

/* shared-memory opt-in of the prefill kernel on the current device (attributes of a function are per device) */
void configure_prefill_kernels() { cudaFuncSetAttribute(prefill_kernel_layout2, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kPfSmem); }

int read_prefill_status(bool clear) {
    int v = 0;
    if (cudaMemcpyFromSymbol(&v, g_kernel_status, sizeof(int)) != cudaSuccess) return -1;
    if (clear && v) { const int z = 0; cudaMemcpyToSymbol(g_kernel_status, &z, sizeof(int)); }
    return v;
}

}  // namespace nwc
