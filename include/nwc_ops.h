/* C-ABI of the B200-native NWC kernel library (nwc_b200/lib/nwc_ops.so).
 *
 * The ten entry points below are exactly the ones the reference's ctypes bridge binds (reference:
 * nwc/nwc_torch.py:58-77) and have the reference's signatures, argument meaning and return codes, so the reference's
 * own Python package runs on this library unchanged (NWC_DLL=/path/to/nwc_ops.so).  Every pointer named "device" is
 * CUDA device memory owned by the caller; the library allocates no device memory on the decode path, launches only on
 * the stream it is given and never synchronises there, so every decode call can be captured in a CUDA graph.
 *
 * `elem` carries the element type in bits 0..3 (0 = bf16, 1 = fp8 e4m3 with per-row fp32 scale) and the block layout
 * in bits 4..7 (0 = 8 x 512 blocks, prefix code; 1 = 16 x 512 blocks in mma fragment order, prefix code; 2 = 16 x 512
 * blocks, fixed-width ranks plus exception lists).  `n` = M * K weights, `block` must be 4096.
 * Alignment: data, low, x, out and y must be 16-byte aligned (tensors from any CUDA allocator are).
 */
#ifndef NWC_OPS_H
#define NWC_OPS_H
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* Capabilities.  0: format version (11), 1: states per lane (1), 2: decoder table words (4096), 3: header bytes per
   block (32), 4: block size (4096), 5: elem parameter present (1), 6: layout 1 (1), 7: layout 2 (1); else -1.
   Replaces csrc/nwc_ops.cu:100-106. */
int nwc_info(int what);

/* out = [blocks, raw-plane bytes, scratch floats, K16].  0 ok, -1 bad shape.  Replaces csrc/nwc_ops.cu:121-126. */
int nwc_layout(uint64_t M, uint32_t K, int elem, uint64_t *out);

/* Encoder, HOST pointers in and out (w: n bf16 or fp8 values; freq, psym: uint16[1024]; bases: uint32[blocks];
   hdr: uint8[32 * blocks]; data: cap bytes; low: raw-plane bytes).  The work runs on the current CUDA device.
   Returns the data length including 64 bytes of slack; -1 bad shape or capacity (the caller retries with a larger
   cap); -2 fp8 NaN; -3 more than 255 exceptions in one lane (layout 2); <= -100: -(100 + cudaError).
   Replaces csrc/nwc_ops.cu:245-320 and 175-243. */
int64_t nwc_encode(const void *w, uint64_t n, uint32_t K, int elem, uint16_t *freq, uint16_t *psym, uint32_t *bases,
                   uint8_t *hdr, uint8_t *data, uint64_t cap, uint8_t *low);

/* 4096-word decoder table from the symbol table (host).  Replaces csrc/nwc_ops.cu:324-348. */
void nwc_build_tab(const uint16_t *freq, const uint16_t *psym, int elem, uint32_t *lut);

/* Token path: y = bf16(scale * (W x) + bias).  x is fp32[K16] for layout 0 and bf16[K rounded up to 32] for layouts
   1 and 2, zero beyond K; bias bf16[M] or NULL; scale fp32[M] or NULL; scratch fp32[padded rows * column blocks];
   y bf16[M].  Returns 0, -1 bad shape / alignment, or the CUDA error of the launch.  Replaces csrc/nwc_ops.cu:1130-1141. */
int nwc_linear_bf16(void *stream, const uint8_t *data, const uint32_t *bases, const uint8_t *hdr, const uint32_t *lut,
                    const uint8_t *low, const float *x, const uint16_t *bias, const float *scale, float *scratch,
                    uint16_t *y, uint64_t n, uint32_t block, uint32_t K, int elem);

/* fp32 test path: y = W x with fp32 x (K16, or K rounded up to 32 for layouts 1 and 2) and fp32 y[M]; accumulates
   with atomics after clearing y.  Replaces csrc/nwc_ops.cu:1110-1118. */
int nwc_matvec(void *stream, const uint8_t *data, const uint32_t *bases, const uint8_t *hdr, const uint32_t *lut,
               const uint8_t *low, const float *x, float *y, uint64_t n, uint32_t block, uint32_t K, int elem);

/* Whole matrix -> bf16[M][K16] (fp8: the unscaled fp8 values).  Replaces csrc/nwc_ops.cu:1121-1126. */
int nwc_dequant(void *stream, const uint8_t *data, const uint32_t *bases, const uint8_t *hdr, const uint32_t *lut,
                const uint8_t *low, uint16_t *out, uint64_t n, uint32_t block, uint32_t K, int elem);

/* Rows ids[0..n_ids) -> bf16[n_ids][K16]; ids outside [0, M) leave their output row untouched.
   Replaces csrc/nwc_ops.cu:1143-1160. */
int nwc_gather(void *stream, const uint8_t *data, const uint32_t *bases, const uint8_t *hdr, const uint32_t *lut,
               const uint8_t *low, const int64_t *ids, uint32_t n_ids, uint16_t *out, uint64_t n, uint32_t block,
               uint32_t K, int elem);

/* Uncompressed fp8 weight-only matvec (bandwidth baseline): y = bf16(scale * (W8 x)), x fp32[K16].
   Replaces csrc/nwc_ops.cu:1163-1168. */
int nwc_ref_fp8(void *stream, const uint8_t *w, const float *scale, const float *x, uint16_t *y, uint64_t M, uint32_t K);

/* SM count of the current device; prepares the kernels for it.  Replaces csrc/nwc_ops.cu:1170-1192. */
int nwc_setup(void);

/* ---- additions of this library (no counterpart in the reference) ------------------------------------------------ */

/* nwc_encode with DEVICE pointers for w, bases, hdr, data and low (psym stays host memory): lets a model that is
   already on the GPU be converted without a host round trip.  Synchronises `stream`.  Same return codes. */
int64_t nwc_encode_device(void *stream, const void *w, uint64_t n, uint32_t K, int elem, uint16_t *psym, uint32_t *bases,
                          uint8_t *hdr, uint8_t *data, uint64_t cap, uint8_t *low);

/* nwc_linear_bf16 with the number of K splits forced (1 .. column blocks; 0 = automatic): used by tests to cover both
   the direct-write and the partial-sum path on any shape. */
int nwc_linear_bf16_splits(void *stream, const uint8_t *data, const uint32_t *bases, const uint8_t *hdr,
                           const uint32_t *lut, const uint8_t *low, const float *x, const uint16_t *bias,
                           const float *scale, float *scratch, uint16_t *y, uint64_t n, uint32_t block, uint32_t K,
                           int elem, uint32_t splits);

/* Status word of the kernels' bounded waits: 0, 2 when a warp gave up waiting for a bulk copy (its rows are then
   missing from y), 3 when a kernel gave up waiting for a peer rank (nwc_allreduce_add_rmsnorm, nwc_linear_fused_opt,
   nwc_argmax_tp).  Synchronises the device;
   clear != 0 resets the word. */
int nwc_kernel_status(int clear);

/* ---- tensor-parallel decode on one node (no counterpart in the reference, which is single-GPU) ------------------------
   Each rank allocates one exchange buffer (nwc_comm_alloc; device memory of nwc_comm_bytes(H) bytes, zeroed), exports it
   as a 64-byte CUDA IPC handle, and opens the handles of the other ranks (nwc_comm_import; peer access is enabled on
   first use).  Row-parallel matvecs (o, down) write their bf16 partial output into nwc_comm_slot(buffer, H, slot), slot 0
   and 1 in turn.  nwc_allreduce_add_rmsnorm then is one kernel per rank: it announces the call to the peers, waits
   (bounded) for theirs, adds the `world` partials of `slot` in rank order in fp32 with plain peer loads over NVLink,
   and writes h_out = bf16(h_in + bf16(sum)) and xn = RMSNorm(h_out) * norm_w (H % 8 == 0, 16-byte aligned pointers,
   h_out != h_in).  `buffers` is a host array of `world` device pointers: this rank's own buffer at [rank], the imported
   ones elsewhere.  All ranks must make the same sequence of calls. */
uint64_t nwc_comm_bytes(uint32_t H);
int nwc_comm_alloc(void **buffer, uint32_t H);
int nwc_comm_free(void *buffer);
int nwc_comm_export(void *buffer, uint8_t *handle64);
int nwc_comm_import(const uint8_t *handle64, void **peer_buffer);
int nwc_comm_release(void *peer_buffer);
uint16_t *nwc_comm_slot(void *buffer, uint32_t H, int slot);
int nwc_allreduce_add_rmsnorm(void *stream, void *const *buffers, int rank, int world, int slot, const uint16_t *h_in,
                              uint16_t *h_out, const uint16_t *norm_w, float eps, uint32_t H, uint16_t *xn);

/* on = 0 routes every call through the kernels that load with plain vector loads instead of bulk-copy rings (A/B
   tests); on = 1 (default) restores the rings. */
void nwc_set_ring_kernels(int on);

/* on = 0 keeps nwc_linear_fused on work splits of whole row groups (or a finalize launch) instead of equal runs per CTA
   whose cut row groups are completed inside the kernel (A/B tests); on = 1 (default) restores them. */
void nwc_set_fixup_plans(int on);

/* on = 1 moves the layout-2 token matvec from the kernel in which every warp owns one contiguous run of its CTA's work
   to the one whose warps draw their stages from a per-CTA pool (all warps end together, more bookkeeping per stage; A/B
   tests); on = 0 (default) goes back. */
void nwc_set_pool_kernels(int on);

/* Tensor-parallel token matvecs whose input is the sum of the ranks' pushed partials (nwc_linear_fused_opt, tp_in): from
   min_world ranks on (0 = never, the default) the layout-2 kernel is launched as clusters of 2 or 4 CTAs that each add up
   a share of the partials and exchange the sums through distributed shared memory, instead of every CTA adding up all of
   them.  Same residual stream; the RMSNorm's sum of squares is added in another order.  Off by default: the sum itself
   gets cheaper (8.4 -> 4.4 us at 8 ranks) but a cluster launch gives up more than that at the kernel boundary before it
   (measured: 155 against 169 tokens/s on 8 GPUs); kept for A/B tests. */
void nwc_set_peer_sharing(int min_world);

/* nwc_linear_bf16 with a bf16 activation vector for every layout (layout 0: bf16[K16]; layouts 1, 2: bf16[K rounded up
   to 32]): the decode loop keeps activations in bf16, which spares layout 0 the fp32 copy and the second mma pass. */
int nwc_linear_x16(void *stream, const uint8_t *data, const uint32_t *bases, const uint8_t *hdr, const uint32_t *lut,
                   const uint8_t *low, const uint16_t *x, const uint16_t *bias, const float *scale, float *scratch,
                   uint16_t *y, uint64_t n, uint32_t block, uint32_t K, int elem);

/* nwc_linear_bf16 without the scratch argument, for hosts that cannot allocate device memory for us (a server whose
   runtime owns all of HBM from start-up, a sandbox without access to the allocator).  It has no counterpart in the
   reference.  The partial sums live in an area of NWC_STATIC_SCRATCH_FLOATS floats (4 MiB) built into the library; every
   GPU that loads the library carries it until the process exits.  The call allocates and frees nothing.
   Limit: padded rows x column blocks (the scratch size nwc_layout reports) must not exceed NWC_STATIC_SCRATCH_FLOATS,
   otherwise nothing is launched and NWC_ERR_STATIC_SCRATCH is returned.  Other return codes as nwc_linear_bf16.
   The area's device address is looked up once per device, when the device is prepared (nwc_setup, or the first call of
   any entry point with that device current) - or, failing that, by the first call of this entry point on the device; so
   call nwc_setup (or this entry point once) with the device current before any stream capture begins.  All calls on a device share the one area and it keeps whatever the last call
   left there: two calls whose kernels overlap on the GPU (different streams) race with each other, so keep calls on
   one device in stream order.  Nothing in the area needs clearing between calls. */
#define NWC_STATIC_SCRATCH_FLOATS 1048576
#define NWC_ERR_STATIC_SCRATCH (-4)
int nwc_linear_bf16_static(void *stream, const uint8_t *data, const uint32_t *bases, const uint8_t *hdr,
                           const uint32_t *lut, const uint8_t *low, const float *x, const uint16_t *bias,
                           const float *scale, uint16_t *y, uint64_t n, uint32_t block, uint32_t K, int elem);

/* ---- decode-step kernels (the reference leaves these operations to Transformers eager code inside its CUDA graph,
   scripts/graph_decode.py:46-60; there is no reference library entry point for them) ------------------------------- */

/* h_out <- bf16(h_in + delta) (delta may be NULL; h_out may be h_in); xn16 <- bf16(weight * bf16(h_out * rsqrt(mean(h_out^2)
   + eps))); xn32 (may be NULL) receives the same values as fp32.  All vectors have H elements. */
int nwc_add_rmsnorm(void *stream, const uint16_t *h_in, const uint16_t *delta, uint16_t *h_out, const uint16_t *weight,
                    float eps, uint32_t H, uint16_t *xn16, float *xn32);

/* Token matvec with its activation prologue fused: y = bf16(scale * (W x) + bias) where x is
     mode 0  the bf16 vector x (as nwc_linear_x16),
     mode 1  RMSNorm of the residual stream: h_out <- bf16(h_in + delta) (delta may be NULL, h_out may be NULL but must
             not be h_in), x = bf16(norm_w * bf16(h_out * rsqrt(mean(h_out^2) + eps))),
     mode 2  SwiGLU of a fused projection: x = bf16(bf16(silu(gate_up[i])) * gate_up[K + i]).
   Layout-0 matrices small enough that launch latency dominates run as ONE launch (prologue, decode, reduction and bf16
   output in a single kernel); every other matrix runs the prologue kernel into xtmp (bf16, K rounded up to 32; needed
   for modes 1 and 2) followed by the regular token path with `scratch`. */
int nwc_linear_fused(void *stream, const uint8_t *data, const uint32_t *bases, const uint8_t *hdr, const uint32_t *lut,
                     const uint8_t *low, int mode, const uint16_t *x, const uint16_t *h_in, const uint16_t *delta,
                     uint16_t *h_out, const uint16_t *norm_w, float eps, const uint16_t *gate_up, uint16_t *xtmp,
                     const uint16_t *bias, const float *scale, float *scratch, uint16_t *y, uint64_t n, uint32_t block,
                     uint32_t K, int elem);

/* nwc_linear_fused with options (opt == NULL is nwc_linear_fused).

   Tensor-parallel group of one node ("push" protocol; `buffers` as for nwc_allreduce_add_rmsnorm: a host array of `world`
   exchange buffers, this rank's own at [rank]; buffers == NULL: no group):
     out_slot >= 0  (row-parallel matrices: o, down) y is not written; the kernel stores its bf16 result into push slot
                    out_slot (0 or 1, used in turn) of EVERY rank's buffer over NVLink as 8-byte words {two rows, number of
                    this push}: a word is valid once it carries the number the reader expects, so there is no flag and
                    no fence.  M == H, no bias / scale.
     in_slot >= 0   (the matrix after a row-parallel one; mode must be 1, delta NULL, K == H) the prologue reads the
                    `world` partials of that slot in its own buffer - polling, bounded by nwc_comm_set_timeout_ms, any word
                    that does not carry the expected push number yet - adds them in rank order in fp32 (every rank gets
                    the same bits), and continues as mode 1 with that sum as delta.  After a timeout nwc_kernel_status()
                    reports 3 and y is NaN.
   So the sum over the ranks costs no kernel of its own and one NVLink store latency.  Only matrices that run on the layout-2 bf16
   ring kernel are covered (-2 otherwise: use nwc_allreduce_add_rmsnorm).  All ranks must make the same sequence of calls.

   side != NULL  (layout 0, matrices that take the single-launch small-matrix kernel) the table nwc_build_side_table made
                 for this matrix: four warps then decode each block in parallel, one row pair each.

   Calls on one device must be in stream order (the kernels share a per-device exchange area for row groups cut by CTA boundaries). */
typedef struct {
    void *const *buffers;
    int rank, world;
    int in_slot, out_slot;      /* -1: unused */
    uint32_t H;                 /* hidden size the buffers were allocated for */
    const uint16_t *side;
    /* A hint, all zero = none: the matrix that the NEXT nwc_linear_fused[_opt] call on this stream will read (its `low`
       pointer, n, K, elem and fused mode).  When both calls take the layout-2 ring kernel, this call's warps ask L2 for the
       first bytes the next call will request as soon as their own last copy is under way, so HBM keeps streaming across
       the kernel boundary.  A wrong hint costs bandwidth, never correctness; next_low must be readable device memory of
       that matrix's size. */
    const void *next_low;
    uint64_t next_n;
    uint32_t next_K;
    int next_elem, next_mode;
} nwc_fused_options;
int nwc_linear_fused_opt(void *stream, const uint8_t *data, const uint32_t *bases, const uint8_t *hdr, const uint32_t *lut,
                         const uint8_t *low, int mode, const uint16_t *x, const uint16_t *h_in, const uint16_t *delta,
                         uint16_t *h_out, const uint16_t *norm_w, float eps, const uint16_t *gate_up, uint16_t *xtmp,
                         const uint16_t *bias, const float *scale, float *scratch, uint16_t *y, uint64_t n, uint32_t block,
                         uint32_t K, int elem, const nwc_fused_options *opt);

/* Layout 0 side table (no counterpart in the reference; built when a matrix is loaded, never stored in checkpoints): for
   every block and lane the bit positions inside the lane's stream at which rows 2, 4 and 6 of the block begin - uint16
   side[blocks][3][32], nwc_side_table_bytes(M, K) bytes of device memory.  It lets several warps decode one block in
   parallel instead of one warp walking each 128-symbol stream from its first bit.  Returns 0, -1 for a bad shape or a
   layout other than 0, or a CUDA error. */
uint64_t nwc_side_table_bytes(uint64_t M, uint32_t K);
/* nwc_gather for a layout-0 matrix with its side table: the walk of a lane's stream starts at the row pair that holds
   the requested row (at most one row is decoded and dropped instead of up to seven).  side == NULL is nwc_gather;
   a side table with another layout returns -1.  Bit-identical output. */
int nwc_gather_side(void *stream, const uint8_t *data, const uint32_t *bases, const uint8_t *hdr, const uint32_t *lut,
                    const uint8_t *low, const int64_t *ids, uint32_t n_ids, uint16_t *out, uint64_t n, uint32_t block,
                    uint32_t K, int elem, const uint16_t *side);
int nwc_build_side_table(void *stream, const uint8_t *data, const uint32_t *bases, const uint8_t *hdr, uint16_t *side,
                         uint64_t n, uint32_t block, uint32_t K, int elem);

/* Longest time a kernel waits for the other ranks of a tensor-parallel group (fused prologue, sharded argmax) before it
   gives up with status 3; default 2000 ms. */
void nwc_comm_set_timeout_ms(uint32_t ms);

/* Prefill (T tokens at once): Y[t][m] = bf16(scale[m] * sum_k X[t][k] W[m][k] + bias[m]); X bf16 [T][ldx] (ldx a multiple
   of 8, 16-byte aligned), Y bf16 [T][ldy].  W is decoded tile by tile into the shared-memory operands of a tcgen05 /
   tensor-memory GEMM; no decompressed copy is written.  The reference dequantises into a temporary and calls a dense
   matmul instead (nwc/nwc_torch.py:320-323).  Returns 0, -1 bad arguments, -2 when the element type / layout is not
   covered by this path yet (layout 2 bf16 is), or a CUDA error. */
/* tests: 1 or 2 = every nwc_linear_prefill CTA multiplies its rows with that many halves of 256 tokens; 0 (default) = the
   launcher chooses (two halves when that saves whole waves of CTAs). */
void nwc_set_prefill_halves(int halves);
int nwc_linear_prefill(void *stream, const uint8_t *data, const uint32_t *bases, const uint8_t *hdr, const uint32_t *lut,
                       const uint8_t *low, const uint16_t *X, uint32_t T, uint32_t ldx, const uint16_t *bias,
                       const float *scale, uint16_t *Y, uint32_t ldy, uint64_t n, uint32_t block, uint32_t K, int elem);

/* Kernels one token-path call launches on the current device (for launch accounting): fused_mode -1 = nwc_linear_bf16 /
   nwc_linear_x16, 0..2 = nwc_linear_fused with that mode.  -1 on a bad shape or without a device. */
int nwc_linear_launches(uint64_t n, uint32_t K, int elem, int fused_mode);

/* on != 0: the decode-step launches (nwc_linear_fused's single-launch kernel, nwc_add_rmsnorm, nwc_attention_decode,
   nwc_swiglu, nwc_argmax) allow programmatic dependent launch, so each overlaps its set-up with the tail of the kernel
   before it; the kernels order themselves with griddepcontrol.wait.  Off by default. */
void nwc_set_dependent_launch(int on);

/* One token of grouped-query attention.  qkv = [n_q | n_kv | n_kv] heads x head_dim (bf16) of the token at position
   *pos; q_norm / k_norm: per-head RMSNorm weights (bf16[head_dim]) or NULL; cos_t / sin_t: bf16[max positions][head_dim];
   k_cache / v_cache: bf16[n_kv][max_len][head_dim], appended at *pos; out: bf16[n_q * head_dim].
   *status is set to 1 (and nothing is written) when *pos is outside [0, max_len).
   With dependent launch on, *pos and the cache rows below it are read while the kernel before this one may still run:
   they must come from work that completed earlier (in the decode loop: from the previous token, whose last kernel is
   followed by an ordinary launch, the embedding gather). */
int nwc_attention_decode(void *stream, const uint16_t *qkv, const uint16_t *q_norm, const uint16_t *k_norm,
                         const uint16_t *cos_t, const uint16_t *sin_t, uint16_t *k_cache, uint16_t *v_cache,
                         const int32_t *pos, uint32_t n_q, uint32_t n_kv, uint32_t head_dim, uint32_t max_len, float eps,
                         uint16_t *out, int *status);

/* on != 0 sends every head size through the general attention kernel (one thread per cached position) instead of the
   lane-per-dimension kernel that head sizes 64, 128 and 256 normally take (A/B tests). */
void nwc_set_plain_attention(int on);

/* a16 <- bf16(bf16(silu(gate)) * up) with gate = gate_up[0..I), up = gate_up[I..2I); a32 (may be NULL) as fp32 */
int nwc_swiglu(void *stream, const uint16_t *gate_up, uint32_t I, uint16_t *a16, float *a32);

/* Greedy choice over bf16 logits[V] (lowest index wins ties): cur[0] <- token; then, only while *step < log_len and
   *pos < max_pos (so a loop that runs past its buffers writes nothing out of bounds): log[*step] <- token (log may be
   NULL), *pos += 1 and *step += 1. */
int nwc_argmax(void *stream, const uint16_t *logits, uint32_t V, int64_t *cur, int64_t *log, int32_t *pos, int32_t *step,
               uint32_t log_len, uint32_t max_pos);

/* The same over vocabulary-sharded logits: every rank passes its V rows (global index = rank * V + local index), the
   ranks exchange one 8-byte (value, index) word each through their exchange buffers and all end with the same token.
   The wait for the other ranks is bounded (status 3, the local best is used). */
int nwc_argmax_tp(void *stream, const uint16_t *logits, uint32_t V, int64_t *cur, int64_t *log, int32_t *pos,
                  int32_t *step, uint32_t log_len, uint32_t max_pos, void *const *buffers, int rank, int world);

#ifdef __cplusplus
}
#endif
#endif
