/* Layout of a tensor-parallel exchange buffer, shared by the kernels that write into peers' buffers (the row-parallel
 * token matvec, the greedy argmax) and the ones that read their own (the fused activation prologue, the pull-style
 * reduction kernel).
 *
 * Every rank owns one buffer in its own HBM and maps the buffers of the other ranks of the node (CUDA IPC).  Two
 * protocols share it:
 *
 *   pull  (nwc_allreduce_add_rmsnorm)   a rank's matvec writes its partial into its OWN pull slot, a reduction kernel
 *                                       announces the call to the peers, waits for theirs and loads their partials
 *                                       over NVLink;
 *   push  (nwc_linear_fused_opt)        a rank's matvec stores its partial into EVERY rank's push slot [slot][rank]
 *                                       as 8-byte words {two bf16 rows, call number}: a word is valid when it carries the
 *                                       call number the consumer expects, so there is no flag and no fence - the
 *                                       consumer (the next matvec's prologue) polls the words themselves in its own HBM
 *                                       and the exchange costs one NVLink store latency.
 *
 * Counters only ever grow (wrap-around compared as signed differences), so a captured CUDA graph replays unchanged.
 */
#pragma once
#include <cstdint>

namespace nwc {

constexpr uint32_t kCommMaxRanks = 8;
constexpr int kStatusPeerTimeout = 3;

struct CommControl {
    uint32_t pull_calls;                        /* [0]   calls of the pull kernel made by this rank                     */
    uint32_t pad0[15];
    uint32_t pull_arrived[kCommMaxRanks];       /* [64]  last pull call each rank has announced to this rank            */
    uint32_t pad1[8];
    uint32_t push_epoch[2];                     /* [128] pushes this rank has completed, per slot                       */
    uint32_t push_done;                         /* [136] CTAs of the running push kernel that have finished             */
    uint32_t argmax_epoch;                      /* [140] argmax exchanges this rank has made                            */
    uint32_t pad2[12];
    uint32_t reserved[2][kCommMaxRanks];        /* [192]                                                                */
    unsigned long long argmax_key[kCommMaxRanks]; /* [256] per source rank: epoch << 48 | value key << 32 | ~index      */
    uint32_t pad3[48];
};
static_assert(sizeof(CommControl) == 512, "exchange buffer header");

constexpr uint32_t kCommHeader = sizeof(CommControl);
#if defined(__CUDACC__)
#define NWC_COMM_HD __host__ __device__ __forceinline__
#else
#define NWC_COMM_HD inline
#endif
NWC_COMM_HD uint64_t comm_slot_bytes(uint32_t H) { return ((uint64_t)H * 2u + 255u) & ~255ull; }
/* this rank's own partial of pull slot `slot` */
NWC_COMM_HD uint64_t comm_pull_offset(uint32_t H, uint32_t slot) { return kCommHeader + (slot & 1u) * comm_slot_bytes(H); }
/* where rank `src`'s partial of push slot `slot` lands in every buffer */
/* a push slot holds H / 2 words of 8 bytes: {bf16 row 2i | bf16 row 2i + 1 << 16, call number} */
NWC_COMM_HD uint64_t comm_push_slot_bytes(uint32_t H) { return ((uint64_t)H * 4u + 255u) & ~255ull; }
NWC_COMM_HD uint64_t comm_push_offset(uint32_t H, uint32_t slot, uint32_t src) {
    return kCommHeader + 2u * comm_slot_bytes(H) + ((slot & 1u) * kCommMaxRanks + src) * comm_push_slot_bytes(H);
}
NWC_COMM_HD uint64_t comm_total_bytes(uint32_t H) { return kCommHeader + 2u * comm_slot_bytes(H) + 2u * kCommMaxRanks * comm_push_slot_bytes(H); }

/* Where a row-parallel matvec sends its bf16 output on a tensor-parallel group (world == 0: the local y instead). */
struct PeerOutput {
    uint8_t *buf[kCommMaxRanks];
    uint32_t world, rank, slot, H;
};

}  // namespace nwc
