/* Host-side launch interface between the C-ABI layer and the kernel translation units. */
#pragma once
#include <cstdint>
#include <cuda_runtime.h>
#include "nwc_geometry.h"
#include "nwc_comm.h"

namespace nwc {

constexpr uint32_t kSegmentThreads = 512;   /* 16 warps per CTA, one CTA per SM */

/* Arguments of the segment kernels; every pointer is device memory owned by the caller. */
struct SegmentArgs {
    const uint8_t *data;        /* lane streams (layouts 0, 1) or exception entries (layout 2)              */
    const uint32_t *bases;      /* byte offset of every block inside data                                   */
    const uint8_t *hdr;         /* per block and lane: stream words (layouts 0, 1) or exception count        */
    const uint32_t *lut;        /* 4096-word decoder table                                                   */
    const uint8_t *low;         /* raw plane(s)                                                              */
    const void *x;              /* activation vector: fp32 or bf16, see nwc_linear_bf16                      */
    float *y32;                 /* fp32 partial sums [padded rows][splits], or the fp32 result of nwc_matvec */
    uint16_t *out;              /* dequantised matrix, row stride K16                                        */
    const uint16_t *bias;       /* bf16 or null                                                              */
    const float *scale;         /* fp32 per row or null                                                      */
    uint16_t *y;                /* bf16 result                                                               */
    uint32_t M, K;
    uint32_t splits;            /* K splits per row group; 0 = let the launcher choose                       */
    int x_bf16;                 /* token path of layout 0: x is bf16[K16] instead of fp32[K16]                */
    uint32_t splits_forced;     /* the caller's own splits request (0 = none): forced splits take the plain kernels */
    uint32_t fixup;             /* 1: equal runs per CTA are allowed, row groups cut by a run boundary are completed inside
                                   the kernel by the CTA where the group begins (per-device exchange area: calls that set
                                   this must be in stream order on their device)                                    */
    PeerOutput push;            /* world > 0: y goes to every rank's exchange buffer instead of a.y                   */
};

/* How the fused small-matrix kernel builds its activation vector. */
enum FusedInputMode : int { kInputPlain = 0, kInputNorm = 1, kInputSwiglu = 2, kInputPeerNorm = 3 };
struct FusedInput {
    int mode;
    const uint16_t *h_in;       /* kInputNorm: residual stream in (bf16[K])                         */
    const uint16_t *delta;      /* kInputNorm: added to h_in first, or null                         */
    uint16_t *h_out;            /* kInputNorm: receives h_in + delta (must not alias h_in), or null */
    const uint16_t *norm_w;     /* kInputNorm: RMSNorm weight                                       */
    float eps;
    const uint16_t *gate_up;    /* kInputSwiglu: [gate | up], 2 K values                            */
    /* kInputPeerNorm: as kInputNorm with delta = the sum, in rank order, of the `world` partial vectors that the ranks of
       a tensor-parallel group pushed into push slot `slot` of this rank's exchange buffer `comm` */
    const uint8_t *comm;
    uint32_t world, slot;
    unsigned long long timeout_ns;   /* longest wait for the peers' flags */
    /* set by the launcher, kInputPeerNorm on the layout-2 ring kernel: bit 0 = the CTAs of a cluster each add up a share of
       the pushed partials and hand the sums to one another through distributed shared memory; bit 1 = the cluster exists
       for that alone (the plan's runs belong to single CTAs) */
    uint32_t share;
};
/* The matrix that the launch following this one on the stream will read (a hint; null low = none).  When both launches
   take the layout-2 ring kernel, this launch asks L2 for the next launch's first bytes while its own tail runs. */
struct NextMatrix {
    const uint8_t *low;
    uint32_t M, K;
    int code;                   /* layout / element code of the next matrix */
    int input_mode;             /* FusedInputMode of the next launch        */
    uint32_t fixup;             /* SegmentArgs::fixup of the next launch    */
};
/* side: per block and lane the bit positions where rows 2, 4, 6 begin (launch_side_table), or null */
cudaError_t launch_small_layout0(int code, int sms, cudaStream_t st, const SegmentArgs &a, const FusedInput &in, const uint16_t *side = nullptr);
cudaError_t launch_side_table(int code, cudaStream_t st, const uint8_t *data, const uint32_t *bases, const uint8_t *hdr, uint16_t *side, uint32_t nb);
void set_dependent_launch(bool on);           /* programmatic dependent launch for the decode-step launches */
bool dependent_launch();

uint32_t choose_splits(const Geometry &g, int mode, int code, int sms);
void set_ring_kernels(bool on);               /* tests: switch the bulk-copy ring kernels off to compare with the plain ones */
void set_peer_sharing(int min_world);         /* clusters share the sum of the pushed partials from this many ranks on (0 = never) */
void set_pool_kernels(bool on);               /* tests: layout-2 kernel whose warps draw stages from a per-CTA pool on / off */
void set_fixup_plans(bool on);                /* tests: equal runs with in-kernel fix-up of cut row groups on / off */
int read_kernel_status(bool clear);           /* 0, or 2 when a bounded wait gave up; synchronises */
/* input: how the token path builds its activation vector; only where token_path_fuses_input() says so, else null */
cudaError_t launch_segments(int mode, int code, int sms, cudaStream_t st, SegmentArgs a, const FusedInput *input = nullptr, const NextMatrix *next = nullptr);
void set_next_fill_stages(uint32_t stages);   /* tests and tuning: ring stages per warp fetched ahead for the next launch (0 = off) */
bool token_path_fuses_input(int code, uint32_t M, uint32_t K, int input_mode);
bool small_layout0_preferred(uint32_t M, uint32_t K, int sms, int input_mode);   /* layout 0: single-launch small-matrix kernel rather than prologue + ring kernel + finalize */
void configure_segment_kernels();
int count_token_launches(int code, int sms, uint32_t M, uint32_t K, bool allow_fix = false);

cudaError_t launch_prefill_layout2(cudaStream_t st, const SegmentArgs &w, const uint16_t *X, uint16_t *Y, uint32_t T, uint32_t ldx, uint32_t ldy);
void set_prefill_halves(int halves);         /* tests: 1 or 2 token halves of 256 per CTA of the prefill GEMM, 0 = chosen per launch */
int read_prefill_status(bool clear);
void configure_prefill_kernels();
void prepare_static_scratch();               /* nwc_linear_bf16_static: look up the built-in scratch area of the current device */
int read_model_status(bool clear);           /* 0, or 3 when the sharded argmax gave up waiting for a rank */
unsigned long long peer_timeout_ns();        /* longest wait for other ranks inside a kernel (nwc_comm_set_timeout_ms) */
void configure_model_kernels();              /* per-device opt-ins of the decode-step kernels */
int read_comm_status(bool clear);            /* 0, or 3 when a rank gave up waiting for its peers */
/* side: layout 0 only, the matrix's side table (launch_side_table) or null */
cudaError_t launch_gather(int code, cudaStream_t st, const SegmentArgs &a, const int64_t *ids, uint32_t n_ids, const uint16_t *side = nullptr);
cudaError_t launch_native_fp8(int sms, cudaStream_t st, const uint8_t *w, const float *scale, const float *x, uint16_t *y, uint32_t M, uint32_t K);

}  // namespace nwc
