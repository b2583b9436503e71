/* Tensor-parallel decode: the sum of the ranks' partial o / down outputs, fused with the residual add and the RMSNorm
 * that follow it, as one kernel over NVLink peer memory.
 *
 * Every rank owns one exchange buffer in its own HBM (cudaMalloc, exported to the other ranks of the node with CUDA IPC);
 * its layout is in nwc_comm.h.  This kernel is the "pull" protocol: the call counter and the arrival words of the
 * header, and the two pull slots (partial vectors of H bf16 values written by this rank's own matvec kernels).
 *
 * Call n of every rank (one cluster of 8 CTAs; CTA 0 does the signalling): announce n to all peers (store into their arrival words, after a system-scope fence so that the
 * partial written by the preceding matvec is visible), wait until every peer has announced n, read all W partials with
 * plain peer loads (no multicast, no multimem), add them in rank order in fp32 - so every rank gets the same bits - and
 * finish with h_out = bf16(h_in + bf16(sum)), x = RMSNorm(h_out) * w.  The o projection uses slot 0 and the down
 * projection slot 1 in turn; a rank can only reach its next write of a slot after all peers have announced the call in
 * between, i.e. after they finished reading that slot, so two slots need no further barrier.
 * The wait is bounded: after kCommPolls polls the kernel records status 3 and carries on with what it has, the context
 * stays usable and the host reads the status through nwc_kernel_status().
 */
#include <cstdint>
#include <cuda_runtime.h>
#include <cooperative_groups.h>
#include "../../include/nwc_ops.h"
#include "nwc_launch.h"

namespace nwc {
namespace {

constexpr uint32_t kCommPolls = 1u << 21;
__device__ int g_comm_status;

struct CommPeers { uint8_t *buf[kCommMaxRanks]; };

__device__ __forceinline__ float bf2f(uint32_t h) { return __uint_as_float(h << 16); }
__device__ __forceinline__ uint32_t f2bf(float v) {
    uint32_t u = __float_as_uint(v);
    if ((u & 0x7FFFFFFFu) > 0x7F800000u) return (u >> 16) | 0x40u;
    u += 0x7FFFu + ((u >> 16) & 1u);
    return u >> 16;
}
__device__ __forceinline__ float bfround(float v) { return bf2f(f2bf(v)); }
__device__ __forceinline__ uint4 load_peer(const uint8_t *p) {          /* never from L1: the same addresses carry new data every second call */
    uint4 v;
    asm volatile("ld.volatile.global.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
    return v;
}

/* One cluster of kCommCtas CTAs per rank: every CTA owns 1 / kCommCtas of the vector, so the peer loads run from
   several SMs at once; the sum of squares of the RMSNorm crosses the cluster through distributed shared memory. */
constexpr uint32_t kCommCtas = 8, kCommThreads = 256;

__global__ void __launch_bounds__(kCommThreads, 1) allreduce_add_rmsnorm_kernel(const CommPeers peers, int rank, int world, uint32_t slot_offset, const uint16_t *h_in,
                                                                              uint16_t *h_out, const uint16_t *__restrict__ norm_w, float eps, uint32_t H, uint16_t *xn) {
    namespace cg = cooperative_groups;
    cg::cluster_group cluster = cg::this_cluster();
    __shared__ float red[kCommThreads / 32u];
    __shared__ float cta_squares[kCommCtas];       /* CTA 0's copy collects every CTA's sum of squares */
    __shared__ uint32_t call_number;               /* CTA 0's copy is the one the cluster reads */
    const uint32_t tid = threadIdx.x, lane = tid & 31u, warp = tid >> 5, cta = cluster.block_rank(), ctas = cluster.num_blocks();
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    asm volatile("griddepcontrol.wait;" ::: "memory");                 /* this rank's partial is complete */
    uint8_t *mine = peers.buf[rank];
    if (cta == 0) {                                                     /* CTA 0 talks to the other ranks */
        if (tid == 0) {
            volatile uint32_t *counter = &reinterpret_cast<CommControl *>(mine)->pull_calls;
            const uint32_t n = *counter + 1u;
            *counter = n; call_number = n;
        }
        __syncthreads();
        const uint32_t n = call_number;
        bool arrived = true;
        if (tid < (uint32_t)world && tid != (uint32_t)rank) {
            __threadfence_system();
            *reinterpret_cast<volatile uint32_t *>(&reinterpret_cast<CommControl *>(peers.buf[tid])->pull_arrived[rank]) = n;
            const volatile uint32_t *word = &reinterpret_cast<const CommControl *>(mine)->pull_arrived[tid];
            uint32_t polls = 0;
            while ((int32_t)(*word - n) < 0) {
                if (++polls > kCommPolls) { arrived = false; break; }
                __nanosleep(64);
            }
            __threadfence_system();
        }
        if (!__syncthreads_and(arrived) && tid == 0) atomicExch(&g_comm_status, kStatusPeerTimeout);
    }
    cluster.sync();                                                     /* every peer's partial is complete (or the wait ran out) */
    /* this CTA's part of the vector: sum of the partials in rank order, residual add, sum of squares */
    const uint32_t chunks = H >> 3, c0 = (uint32_t)((uint64_t)chunks * cta / ctas), c1 = (uint32_t)((uint64_t)chunks * (cta + 1u) / ctas);
    float ss = 0.f;
    for (uint32_t c = c0 + tid; c < c1; c += kCommThreads) {
        float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
        uint4 part[kCommMaxRanks];
#pragma unroll
        for (int r = 0; r < (int)kCommMaxRanks; r++)                    /* all peer loads in flight before the first add */
            part[r] = r < world ? load_peer(peers.buf[r] + slot_offset + (uint64_t)c * 16u) : make_uint4(0u, 0u, 0u, 0u);
#pragma unroll
        for (int r = 0; r < (int)kCommMaxRanks; r++) {
            if (r < world) {
                const uint32_t w[4] = {part[r].x, part[r].y, part[r].z, part[r].w};
#pragma unroll
                for (int k = 0; k < 4; k++) { acc[2 * k] += bf2f(w[k] & 0xFFFFu); acc[2 * k + 1] += bf2f(w[k] >> 16); }
            }
        }
        const uint4 hv = *(reinterpret_cast<const uint4 *>(h_in) + c);
        const uint32_t hw[4] = {hv.x, hv.y, hv.z, hv.w};
        uint32_t ow[4];
#pragma unroll
        for (int k = 0; k < 4; k++) {
            const float v0 = bfround(bf2f(hw[k] & 0xFFFFu) + bfround(acc[2 * k])), v1 = bfround(bf2f(hw[k] >> 16) + bfround(acc[2 * k + 1]));
            ss += v0 * v0; ss += v1 * v1;
            ow[k] = f2bf(v0) | (f2bf(v1) << 16);
        }
        *(reinterpret_cast<uint4 *>(h_out) + c) = make_uint4(ow[0], ow[1], ow[2], ow[3]);
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
    if (lane == 0) red[warp] = ss;
    __syncthreads();
    if (tid == 0) {
        float t = 0.f;
        for (uint32_t i = 0; i < kCommThreads / 32u; i++) t += red[i];
        cluster.map_shared_rank(cta_squares, 0)[cta] = t;               /* into CTA 0's shared memory */
    }
    cluster.sync();
    float tot = 0.f;
    {
        const float *all = cluster.map_shared_rank(cta_squares, 0);
        for (uint32_t i = 0; i < ctas; i++) tot += all[i];              /* same order in every CTA */
    }
    const float inv = rsqrtf(tot / (float)H + eps);
    for (uint32_t c = c0 + tid; c < c1; c += kCommThreads) {            /* each thread re-reads the chunks it wrote itself */
        const uint4 hv = *(reinterpret_cast<const uint4 *>(h_out) + c), wv = __ldg(reinterpret_cast<const uint4 *>(norm_w) + c);
        const uint32_t hw[4] = {hv.x, hv.y, hv.z, hv.w}, ww[4] = {wv.x, wv.y, wv.z, wv.w};
        uint32_t ow[4];
#pragma unroll
        for (int k = 0; k < 4; k++)
            ow[k] = f2bf(bf2f(ww[k] & 0xFFFFu) * bfround(bf2f(hw[k] & 0xFFFFu) * inv)) | (f2bf(bf2f(ww[k] >> 16) * bfround(bf2f(hw[k] >> 16) * inv)) << 16);
        *(reinterpret_cast<uint4 *>(xn) + c) = make_uint4(ow[0], ow[1], ow[2], ow[3]);
    }
    cluster.sync();                                                     /* CTA 0's shared memory stays alive until everybody has read it */
}

}  // namespace

int read_comm_status(bool clear) {
    int v = 0;
    if (cudaMemcpyFromSymbol(&v, g_comm_status, sizeof(int)) != cudaSuccess) return -1;
    if (clear && v) { const int z = 0; cudaMemcpyToSymbol(g_comm_status, &z, sizeof(int)); }
    return v;
}

}  // namespace nwc

using namespace nwc;

#define NWC_EXPORT extern "C" __attribute__((visibility("default")))

NWC_EXPORT uint64_t nwc_comm_bytes(uint32_t H) { return comm_total_bytes(H); }

NWC_EXPORT int nwc_comm_alloc(void **buffer, uint32_t H) {
    if (!buffer || !H || (H & 7u)) return -1;
    const cudaError_t e = cudaMalloc(buffer, nwc_comm_bytes(H));
    if (e != cudaSuccess) return (int)e;
    return (int)cudaMemset(*buffer, 0, nwc_comm_bytes(H));
}

NWC_EXPORT int nwc_comm_free(void *buffer) { return (int)cudaFree(buffer); }

NWC_EXPORT int nwc_comm_export(void *buffer, uint8_t *handle64) {
    cudaIpcMemHandle_t h;
    const cudaError_t e = cudaIpcGetMemHandle(&h, buffer);
    if (e != cudaSuccess) return (int)e;
    static_assert(sizeof(h) == 64, "CUDA IPC handles are 64 bytes");
    for (int i = 0; i < 64; i++) handle64[i] = reinterpret_cast<const uint8_t *>(&h)[i];
    return 0;
}

NWC_EXPORT int nwc_comm_import(const uint8_t *handle64, void **peer_buffer) {
    cudaIpcMemHandle_t h;
    for (int i = 0; i < 64; i++) reinterpret_cast<uint8_t *>(&h)[i] = handle64[i];
    return (int)cudaIpcOpenMemHandle(peer_buffer, h, cudaIpcMemLazyEnablePeerAccess);
}

NWC_EXPORT int nwc_comm_release(void *peer_buffer) { return (int)cudaIpcCloseMemHandle(peer_buffer); }

NWC_EXPORT uint16_t *nwc_comm_slot(void *buffer, uint32_t H, int slot) {
    return reinterpret_cast<uint16_t *>(static_cast<uint8_t *>(buffer) + comm_pull_offset(H, (uint32_t)slot));
}

NWC_EXPORT int nwc_allreduce_add_rmsnorm(void *stream, void *const *buffers, int rank, int world, int slot, const uint16_t *h_in, uint16_t *h_out,
                                         const uint16_t *norm_w, float eps, uint32_t H, uint16_t *xn) {
    if (!buffers || world < 1 || world > (int)kCommMaxRanks || rank < 0 || rank >= world || !H || (H & 7u) || !h_in || !h_out || !norm_w || !xn || h_in == h_out) return -1;
    if ((reinterpret_cast<uintptr_t>(h_in) | reinterpret_cast<uintptr_t>(h_out) | reinterpret_cast<uintptr_t>(norm_w) | reinterpret_cast<uintptr_t>(xn)) & 15u) return -1;
    CommPeers peers{};
    for (int r = 0; r < world; r++) { if (!buffers[r]) return -1; peers.buf[r] = static_cast<uint8_t *>(buffers[r]); }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(kCommCtas); cfg.blockDim = dim3(kCommThreads); cfg.dynamicSmemBytes = 0; cfg.stream = (cudaStream_t)stream;
    cudaLaunchAttribute attr[2];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = kCommCtas; attr[0].val.clusterDim.y = 1; attr[0].val.clusterDim.z = 1;
    attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[1].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr; cfg.numAttrs = dependent_launch() ? 2 : 1;
    return (int)cudaLaunchKernelEx(&cfg, allreduce_add_rmsnorm_kernel, peers, rank, world, (uint32_t)comm_pull_offset(H, (uint32_t)slot), h_in, h_out, norm_w, eps, H, xn);
}
