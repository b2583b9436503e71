/* extern "C" surface of nwc_ops.so: argument checks, per-device set-up and dispatch.  See include/nwc_ops.h for the
 * contract of every entry point and the reference interface it replaces. */
#include <mutex>
#include "../../include/nwc_ops.h"
#include "nwc_encode.h"
#include "nwc_launch.h"

#define NWC_EXPORT extern "C" __attribute__((visibility("default")))

using namespace nwc;

namespace {

constexpr int kMaxDevices = 64;
int g_sm_count[kMaxDevices];         /* 0 = device not prepared yet */
std::mutex g_setup_lock;

/* SM count of the current device, preparing the kernels' shared-memory opt-in on first use of that device */
int device_sms() {
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return 0;
    if (g_sm_count[dev]) return g_sm_count[dev];
    std::lock_guard<std::mutex> hold(g_setup_lock);
    int sms = 0;
    if (cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || sms <= 0) return 0;
    configure_segment_kernels();
    configure_model_kernels();
    configure_prefill_kernels();
    prepare_static_scratch();
    g_sm_count[dev] = sms;
    return sms;
}

bool shape_ok(uint64_t n, uint32_t block, uint32_t K) { return block == kBlockWeights && K != 0 && n != 0 && n % K == 0 && n / K <= 0xFFFFFFFFull; }
bool aligned16(const void *p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

int run_segments(int mode, void *stream, const uint8_t *data, const uint32_t *bases, const uint8_t *hdr, const uint32_t *lut,
                 const uint8_t *low, const void *x, float *y32, uint16_t *out, const uint16_t *bias, const float *scale, uint16_t *y,
                 uint64_t n, uint32_t block, uint32_t K, int elem, uint32_t splits, int x_bf16 = 0) {
    if (!shape_ok(n, block, K) || layout_of(elem) > 2 || type_of(elem) > 1) return -1;
    if (!aligned16(data) || !aligned16(low) || !aligned16(lut) || (x && !aligned16(x)) || (out && !aligned16(out))) return -1;
    const int sms = device_sms();
    if (!sms) return (int)cudaErrorNoDevice;
    SegmentArgs a{data, bases, hdr, lut, low, x, y32, out, bias, scale, y, (uint32_t)(n / K), K, splits, x_bf16, 0};
    const Geometry g(a.M, K, layout_of(elem));
    if (a.splits > g.CB) a.splits = g.CB;
    return (int)launch_segments(mode, elem, sms, (cudaStream_t)stream, a);
}

}  // namespace

NWC_EXPORT int nwc_info(int what) {
    switch (what) {
        case 0: return kFormatVersion;
        case 1: return 1;
        case 2: return (int)kTableWords;
        case 3: return (int)kLanes;
        case 4: return (int)kBlockWeights;
        case 5: case 6: case 7: return 1;
        default: return -1;
    }
}

NWC_EXPORT int nwc_layout(uint64_t M, uint32_t K, int elem, uint64_t *out) {
    if (!M || !K || M > 0xFFFFFFFFull) return -1;
    const Geometry g((uint32_t)M, K, layout_of(elem));
    out[0] = g.nb; out[1] = g.raw_plane_bytes(elem); out[2] = g.scratch_floats(); out[3] = g.K16;
    return 0;
}

NWC_EXPORT int64_t nwc_encode(const void *w, uint64_t n, uint32_t K, int elem, uint16_t *freq, uint16_t *psym, uint32_t *bases,
                              uint8_t *hdr, uint8_t *data, uint64_t cap, uint8_t *low) {
    return encode_host(w, n, K, elem, freq, psym, bases, hdr, data, cap, low);
}

NWC_EXPORT int64_t nwc_encode_device(void *stream, const void *w, uint64_t n, uint32_t K, int elem, uint16_t *psym, uint32_t *bases,
                                     uint8_t *hdr, uint8_t *data, uint64_t cap, uint8_t *low) {
    if (!K || !n || n % K || n / K > 0xFFFFFFFFull) return -1;
    return encode_device((cudaStream_t)stream, w, n, K, elem, psym, bases, hdr, data, cap, low);
}

NWC_EXPORT void nwc_build_tab(const uint16_t *freq, const uint16_t *psym, int elem, uint32_t *lut) { (void)freq; build_table(psym, elem, lut); }

NWC_EXPORT int nwc_linear_bf16(void *stream, const uint8_t *data, const uint32_t *bases, const uint8_t *hdr, const uint32_t *lut,
                               const uint8_t *low, const float *x, const uint16_t *bias, const float *scale, float *scratch, uint16_t *y,
                               uint64_t n, uint32_t block, uint32_t K, int elem) {
    return run_segments(0, stream, data, bases, hdr, lut, low, x, scratch, nullptr, bias, scale, y, n, block, K, elem, 0);
}

NWC_EXPORT int nwc_linear_bf16_splits(void *stream, const uint8_t *data, const uint32_t *bases, const uint8_t *hdr, const uint32_t *lut,
                                      const uint8_t *low, const float *x, const uint16_t *bias, const float *scale, float *scratch,
                                      uint16_t *y, uint64_t n, uint32_t block, uint32_t K, int elem, uint32_t splits) {
    return run_segments(0, stream, data, bases, hdr, lut, low, x, scratch, nullptr, bias, scale, y, n, block, K, elem, splits);
}

NWC_EXPORT int nwc_linear_x16(void *stream, const uint8_t *data, const uint32_t *bases, const uint8_t *hdr, const uint32_t *lut,
                              const uint8_t *low, const uint16_t *x, const uint16_t *bias, const float *scale, float *scratch, uint16_t *y,
                              uint64_t n, uint32_t block, uint32_t K, int elem) {
    return run_segments(0, stream, data, bases, hdr, lut, low, x, scratch, nullptr, bias, scale, y, n, block, K, elem, 0, 1);
}

/* longest wait of a fused prologue for the other ranks' partials (nwc_comm_set_timeout_ms) */
unsigned long long g_peer_timeout_ns = 2000000000ull;

/* Token matvec with the activation prologue fused where that pays (layout 0 matrices of at most two blocks per resident
   warp: one launch in all; layout 2 bf16 on the ring kernel); other matrices run the prologue kernel into xtmp and then the
   regular token path.  `tp` (may be null) names the exchange buffers of a tensor-parallel group: in_slot >= 0 takes the
   summed partials of that push slot as the residual delta, out_slot >= 0 pushes y to every rank instead of writing it. */
static int linear_fused(void *stream, const uint8_t *data, const uint32_t *bases, const uint8_t *hdr, const uint32_t *lut,
                        const uint8_t *low, int mode, const uint16_t *x, const uint16_t *h_in, const uint16_t *delta, uint16_t *h_out,
                        const uint16_t *norm_w, float eps, const uint16_t *gate_up, uint16_t *xtmp, const uint16_t *bias, const float *scale,
                        float *scratch, uint16_t *y, uint64_t n, uint32_t block, uint32_t K, int elem, const nwc_fused_options *tp) {
    if (!shape_ok(n, block, K) || layout_of(elem) > 2 || type_of(elem) > 1 || mode < 0 || mode > 2) return -1;
    if (!aligned16(data) || !aligned16(low) || !aligned16(lut)) return -1;
    if (mode == kInputNorm && (!h_in || !norm_w || h_out == h_in)) return -1;
    if (mode == kInputNorm && (!aligned16(h_in) || !aligned16(delta) || !aligned16(h_out) || !aligned16(norm_w))) return -1;   /* read as 16-byte vectors */
    if (mode == kInputSwiglu && (!gate_up || !aligned16(gate_up))) return -1;
    if (mode == kInputPlain && (!x || !aligned16(x))) return -1;
    const int sms = device_sms();
    if (!sms) return (int)cudaErrorNoDevice;
    const uint32_t M = (uint32_t)(n / K);
    const Geometry g(M, K, layout_of(elem));
    const bool peer_in = tp && tp->buffers && tp->in_slot >= 0, peer_out = tp && tp->buffers && tp->out_slot >= 0;
    const uint16_t *side = tp && layout_of(elem) == 0 ? tp->side : nullptr;
    PeerOutput push{};
    int in_mode = mode;
    if (peer_in || peer_out) {
        if (tp->world < 1 || tp->world > (int)kCommMaxRanks || tp->rank < 0 || tp->rank >= tp->world || !tp->H || (tp->H & 7u)) return -1;
        for (int r = 0; r < tp->world; r++) if (!tp->buffers[r]) return -1;
        if (peer_in && (mode != kInputNorm || K != tp->H || tp->in_slot > 1 || delta)) return -1;
        if (peer_out && (M != tp->H || tp->out_slot > 1 || bias || scale)) return -1;     /* the consumer polls every word of the H-vector */
        if (peer_in) in_mode = kInputPeerNorm;
        /* both directions are part of the layout-2 ring kernel only */
        if (!token_path_fuses_input(elem, M, K, in_mode)) return -2;
        if (peer_out) {
            for (int r = 0; r < tp->world; r++) push.buf[r] = static_cast<uint8_t *>(tp->buffers[r]);
            push.world = (uint32_t)tp->world; push.rank = (uint32_t)tp->rank; push.slot = (uint32_t)tp->out_slot; push.H = tp->H;
        }
    }
    FusedInput in{in_mode, h_in, delta, h_out, norm_w, eps, gate_up, nullptr, 0u, 0u, g_peer_timeout_ns};
    if (peer_in) { in.comm = static_cast<const uint8_t *>(tp->buffers[tp->rank]); in.world = (uint32_t)tp->world; in.slot = (uint32_t)tp->in_slot; }
    if (!peer_in && !peer_out && layout_of(elem) == 0 && g.nb <= 2u * (uint32_t)sms * 32u && g.K16 <= 40960u && (side || small_layout0_preferred(M, K, sms, mode))) {
        SegmentArgs a{data, bases, hdr, lut, low, x, scratch, nullptr, bias, scale, y, M, K, 0, 1, 0};
        return (int)launch_small_layout0(elem, sms, (cudaStream_t)stream, a, in, side);
    }
    if (token_path_fuses_input(elem, M, K, in_mode)) {              /* the ring kernel builds x itself (a plain x too) */
        SegmentArgs a{data, bases, hdr, lut, low, x, scratch, nullptr, bias, scale, y, M, K, 0, 1, 0};
        a.fixup = 1u; a.push = push;
        NextMatrix next{};
        if (tp && tp->next_low && tp->next_K && tp->next_n && tp->next_n / tp->next_K <= 0xFFFFFFFFull && aligned16(tp->next_low) &&
            layout_of(tp->next_elem) == 2 && type_of(tp->next_elem) <= 1 && tp->next_mode >= 0 && tp->next_mode <= 2)
            next = NextMatrix{static_cast<const uint8_t *>(tp->next_low), (uint32_t)(tp->next_n / tp->next_K), tp->next_K, tp->next_elem, tp->next_mode, 1u};
        return (int)launch_segments(0, elem, sms, (cudaStream_t)stream, a, &in, &next);
    }
    const uint16_t *xin = x;
    if (mode != kInputPlain) {
        if (!xtmp || !aligned16(xtmp)) return -1;
        const int e = mode == kInputNorm ? nwc_add_rmsnorm(stream, h_in, delta, h_out ? h_out : xtmp, norm_w, eps, K, xtmp, nullptr)
                                         : nwc_swiglu(stream, gate_up, K, xtmp, nullptr);
        if (e) return e;
        xin = xtmp;
    }
    return run_segments(0, stream, data, bases, hdr, lut, low, xin, scratch, nullptr, bias, scale, y, n, block, K, elem, 0, 1);
}

NWC_EXPORT int nwc_linear_fused(void *stream, const uint8_t *data, const uint32_t *bases, const uint8_t *hdr, const uint32_t *lut,
                                const uint8_t *low, int mode, const uint16_t *x, const uint16_t *h_in, const uint16_t *delta, uint16_t *h_out,
                                const uint16_t *norm_w, float eps, const uint16_t *gate_up, uint16_t *xtmp, const uint16_t *bias, const float *scale,
                                float *scratch, uint16_t *y, uint64_t n, uint32_t block, uint32_t K, int elem) {
    return linear_fused(stream, data, bases, hdr, lut, low, mode, x, h_in, delta, h_out, norm_w, eps, gate_up, xtmp, bias, scale, scratch, y, n, block, K, elem, nullptr);
}

NWC_EXPORT int nwc_linear_fused_opt(void *stream, const uint8_t *data, const uint32_t *bases, const uint8_t *hdr, const uint32_t *lut,
                                   const uint8_t *low, int mode, const uint16_t *x, const uint16_t *h_in, const uint16_t *delta, uint16_t *h_out,
                                   const uint16_t *norm_w, float eps, const uint16_t *gate_up, uint16_t *xtmp, const uint16_t *bias, const float *scale,
                                   float *scratch, uint16_t *y, uint64_t n, uint32_t block, uint32_t K, int elem, const nwc_fused_options *tp) {
    return linear_fused(stream, data, bases, hdr, lut, low, mode, x, h_in, delta, h_out, norm_w, eps, gate_up, xtmp, bias, scale, scratch, y, n, block, K, elem, tp);
}

NWC_EXPORT uint64_t nwc_side_table_bytes(uint64_t M, uint32_t K) {
    if (!M || !K || M > 0xFFFFFFFFull) return 0;
    return (uint64_t)Geometry((uint32_t)M, K, 0).nb * 192u;
}

NWC_EXPORT int nwc_build_side_table(void *stream, const uint8_t *data, const uint32_t *bases, const uint8_t *hdr, uint16_t *side, uint64_t n, uint32_t block,
                                    uint32_t K, int elem) {
    if (!shape_ok(n, block, K) || layout_of(elem) != 0 || type_of(elem) > 1 || !side) return -1;
    if (!device_sms()) return (int)cudaErrorNoDevice;
    return (int)launch_side_table(elem, (cudaStream_t)stream, data, bases, hdr, side, Geometry((uint32_t)(n / K), K, 0).nb);
}

NWC_EXPORT void nwc_comm_set_timeout_ms(uint32_t ms) { g_peer_timeout_ns = (unsigned long long)(ms ? ms : 1u) * 1000000ull; }
namespace nwc { unsigned long long peer_timeout_ns() { return g_peer_timeout_ns; } }

/* number of kernels one token-path call launches on the current device: fused_mode -1 = nwc_linear_bf16 / nwc_linear_x16,
   0..2 = nwc_linear_fused with that mode */
NWC_EXPORT int nwc_linear_launches(uint64_t n, uint32_t K, int elem, int fused_mode) {
    if (!shape_ok(n, kBlockWeights, K)) return -1;
    const int sms = device_sms();
    if (!sms) return -1;
    const uint32_t M = (uint32_t)(n / K);
    const Geometry g(M, K, layout_of(elem));
    if (fused_mode >= 0 && layout_of(elem) == 0 && g.nb <= 2u * (uint32_t)sms * 32u && g.K16 <= 40960u && small_layout0_preferred(M, K, sms, fused_mode)) return 1;
    const bool ring = fused_mode >= 0 && token_path_fuses_input(elem, M, K, fused_mode);
    return count_token_launches(elem, sms, M, K, ring) + (fused_mode > 0 && !ring ? 1 : 0);
}

NWC_EXPORT void nwc_set_dependent_launch(int on) { set_dependent_launch(on != 0); }

NWC_EXPORT int nwc_matvec(void *stream, const uint8_t *data, const uint32_t *bases, const uint8_t *hdr, const uint32_t *lut,
                          const uint8_t *low, const float *x, float *y, uint64_t n, uint32_t block, uint32_t K, int elem) {
    if (!shape_ok(n, block, K)) return -1;
    const cudaError_t e = cudaMemsetAsync(y, 0, 4ull * (n / K), (cudaStream_t)stream);
    if (e != cudaSuccess) return (int)e;
    return run_segments(2, stream, data, bases, hdr, lut, low, x, y, nullptr, nullptr, nullptr, nullptr, n, block, K, elem, 0);
}

NWC_EXPORT int nwc_dequant(void *stream, const uint8_t *data, const uint32_t *bases, const uint8_t *hdr, const uint32_t *lut,
                           const uint8_t *low, uint16_t *out, uint64_t n, uint32_t block, uint32_t K, int elem) {
    return run_segments(1, stream, data, bases, hdr, lut, low, nullptr, nullptr, out, nullptr, nullptr, nullptr, n, block, K, elem, 0);
}

static int gather_rows(void *stream, const uint8_t *data, const uint32_t *bases, const uint8_t *hdr, const uint32_t *lut, const uint8_t *low,
                       const int64_t *ids, uint32_t n_ids, uint16_t *out, uint64_t n, uint32_t block, uint32_t K, int elem, const uint16_t *side) {
    if (!shape_ok(n, block, K) || layout_of(elem) > 2 || type_of(elem) > 1) return -1;
    if (side && layout_of(elem) != 0) return -1;
    if (n_ids == 0) return 0;
    if (!aligned16(data) || !aligned16(low) || !aligned16(lut) || !aligned16(out)) return -1;
    if (!device_sms()) return (int)cudaErrorNoDevice;
    SegmentArgs a{data, bases, hdr, lut, low, nullptr, nullptr, out, nullptr, nullptr, nullptr, (uint32_t)(n / K), K, 1, 0, 0};
    return (int)launch_gather(elem, (cudaStream_t)stream, a, ids, n_ids, side);
}

NWC_EXPORT int nwc_gather(void *stream, const uint8_t *data, const uint32_t *bases, const uint8_t *hdr, const uint32_t *lut,
                          const uint8_t *low, const int64_t *ids, uint32_t n_ids, uint16_t *out, uint64_t n, uint32_t block, uint32_t K, int elem) {
    return gather_rows(stream, data, bases, hdr, lut, low, ids, n_ids, out, n, block, K, elem, nullptr);
}

NWC_EXPORT int nwc_gather_side(void *stream, const uint8_t *data, const uint32_t *bases, const uint8_t *hdr, const uint32_t *lut,
                               const uint8_t *low, const int64_t *ids, uint32_t n_ids, uint16_t *out, uint64_t n, uint32_t block, uint32_t K, int elem,
                               const uint16_t *side) {
    return gather_rows(stream, data, bases, hdr, lut, low, ids, n_ids, out, n, block, K, elem, side);
}

NWC_EXPORT int nwc_ref_fp8(void *stream, const uint8_t *w, const float *scale, const float *x, uint16_t *y, uint64_t M, uint32_t K) {
    if (!M || !K || M > 0xFFFFFFFFull) return -1;
    if (((K & 15u) == 0u) && (!aligned16(w) || !aligned16(x))) return -1;
    const int sms = device_sms();
    if (!sms) return (int)cudaErrorNoDevice;
    return (int)launch_native_fp8(sms, (cudaStream_t)stream, w, scale, x, y, (uint32_t)M, K);
}

NWC_EXPORT int nwc_setup(void) { return device_sms(); }

NWC_EXPORT int nwc_kernel_status(int clear) {
    const int v[4] = {read_kernel_status(clear != 0), read_prefill_status(clear != 0), read_comm_status(clear != 0), read_model_status(clear != 0)};
    int worst = v[0];
    for (int i = 1; i < 4; i++) if (v[i] > worst) worst = v[i];
    return worst;
}

/* Prefill: Y[T][ldy] = bf16(scale * (X[T][ldx] W^T) + bias) on the tcgen05 tensor cores, W decoded tile by tile.
   Returns -2 for element types / layouts this path does not cover yet (the caller then dequantises and calls a matmul). */
NWC_EXPORT int nwc_linear_prefill(void *stream, const uint8_t *data, const uint32_t *bases, const uint8_t *hdr, const uint32_t *lut,
                                  const uint8_t *low, const uint16_t *X, uint32_t T, uint32_t ldx, const uint16_t *bias, const float *scale,
                                  uint16_t *Y, uint32_t ldy, uint64_t n, uint32_t block, uint32_t K, int elem) {
    if (!shape_ok(n, block, K) || !T || ldx < K || ldy < n / K) return -1;
    if (layout_of(elem) != 2 || type_of(elem) != kBf16) return -2;
    if (!aligned16(data) || !aligned16(low) || !aligned16(lut) || !aligned16(X) || (ldx & 7u)) return -1;
    if (!device_sms()) return (int)cudaErrorNoDevice;
    SegmentArgs a{data, bases, hdr, lut, low, nullptr, nullptr, nullptr, bias, scale, nullptr, (uint32_t)(n / K), K, 1, 1, 0};
    return (int)launch_prefill_layout2((cudaStream_t)stream, a, X, Y, T, ldx, ldy);
}

NWC_EXPORT void nwc_set_prefill_halves(int halves) { set_prefill_halves(halves); }
NWC_EXPORT void nwc_set_ring_kernels(int on) { set_ring_kernels(on != 0); }
NWC_EXPORT void nwc_set_fixup_plans(int on) { set_fixup_plans(on != 0); }
NWC_EXPORT void nwc_set_pool_kernels(int on) { set_pool_kernels(on != 0); }
NWC_EXPORT void nwc_set_peer_sharing(int min_world) { set_peer_sharing(min_world); }
