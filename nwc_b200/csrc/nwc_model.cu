/* The kernels between the compressed matvecs of one decode step (batch 1): residual add + RMSNorm, per-head
 * q/k-norm + rotary embedding + KV-cache append + grouped-query attention over the cache, SwiGLU, greedy argmax.
 *
 * The reference leaves these operations to Hugging Face eager code captured into its CUDA graph (reference:
 * scripts/graph_decode.py:46-60); here each is one small kernel so a whole token is a short fixed chain of launches
 * that reads its position and token from device memory and can be replayed as one graph.
 * Rounding follows the bf16 module semantics of the Transformers Qwen3 / Llama decoder layers: the residual stream is
 * bf16, RMSNorm normalises in fp32, rounds to bf16 and then multiplies by the bf16 weight, rotary products and sums
 * are rounded to bf16 one by one, SiLU is rounded before the multiply; attention accumulates in fp32.
 */
#include <cstdint>
#include <cuda_runtime.h>
#include "../../include/nwc_ops.h"
#include "nwc_launch.h"

#define NWC_EXPORT extern "C" __attribute__((visibility("default")))

namespace {

__device__ __forceinline__ float bf2f(uint16_t h) { return __uint_as_float((uint32_t)h << 16); }
/* round to nearest even with NaN kept (activations, unlike weights, may legitimately overflow) */
__device__ __forceinline__ uint16_t f2bf(float v) {
    uint32_t u = __float_as_uint(v);
    if ((u & 0x7FFFFFFFu) > 0x7F800000u) return (uint16_t)((u >> 16) | 0x40u);
    u += 0x7FFFu + ((u >> 16) & 1u);
    return (uint16_t)(u >> 16);
}
__device__ __forceinline__ float bfround(float v) { return bf2f(f2bf(v)); }
/* let the next kernel of the stream start its own prologue, then wait until everything before this kernel is complete
   (both are no-ops unless the launch allowed programmatic dependent launch) */
__device__ __forceinline__ void dependency_sync() {
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    asm volatile("griddepcontrol.wait;" ::: "memory");
}

__device__ __forceinline__ float block_sum(float v, float *red) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nw = (blockDim.x + 31) >> 5;
    __syncthreads();
    if (lane == 0) red[warp] = v;
    __syncthreads();
    float t = 0.f;
    for (int i = 0; i < nw; i++) t += red[i];
    return t;
}
__device__ __forceinline__ float block_max(float v, float *red) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nw = (blockDim.x + 31) >> 5;
    __syncthreads();
    if (lane == 0) red[warp] = v;
    __syncthreads();
    float t = -INFINITY;
    for (int i = 0; i < nw; i++) t = fmaxf(t, red[i]);
    return t;
}

/* h <- bf16(h_in + delta) (delta may be null, h may alias h_in); xn <- bf16(weight * bf16(h * rsqrt(mean(h^2) + eps))); optional fp32 copy */
__global__ void __launch_bounds__(1024) add_rmsnorm_kernel(const uint16_t *h_in, const uint16_t *__restrict__ delta, uint16_t *h, const uint16_t *__restrict__ weight,
                                                            float eps, uint32_t H, uint16_t *__restrict__ xn16, float *__restrict__ xn32) {
    __shared__ float red[32];
    dependency_sync();
    float ss = 0.f;
    for (uint32_t i = threadIdx.x; i < H; i += blockDim.x) {
        float v = bf2f(h_in[i]);
        if (delta) v = bfround(v + bf2f(delta[i]));
        if (delta || h != h_in) h[i] = f2bf(v);
        ss += v * v;
    }
    const float inv = rsqrtf(block_sum(ss, red) / (float)H + eps);
    for (uint32_t i = threadIdx.x; i < H; i += blockDim.x) {
        const float y = bfround(bf2f(weight[i]) * bfround(bf2f(h[i]) * inv));
        xn16[i] = f2bf(y);
        if (xn32) xn32[i] = y;
    }
}

/* One CTA per query head.  qkv = [q heads | k heads | v heads] x head_dim of the current token.
   cos / sin: bf16 [max_pos][head_dim] tables.  Caches: bf16 [n_kv][max_len][head_dim].  pos_ptr: position of the token. */
__global__ void __launch_bounds__(256) attention_decode_kernel(const uint16_t *__restrict__ qkv, const uint16_t *__restrict__ q_norm, const uint16_t *__restrict__ k_norm,
                                                                const uint16_t *__restrict__ cos_t, const uint16_t *__restrict__ sin_t, uint16_t *__restrict__ k_cache,
                                                                uint16_t *__restrict__ v_cache, const int32_t *__restrict__ pos_ptr, uint32_t n_q, uint32_t n_kv, uint32_t hd,
                                                                uint32_t max_len, float eps, float scale, uint16_t *__restrict__ out, int *__restrict__ status) {
    extern __shared__ float sm[];
    float *qs = sm, *ks = sm + hd, *scores = sm + 2 * hd;          /* q, current k (fp32), scores [max_len] */
    __shared__ float red[32];
    const uint32_t head = blockIdx.x, kvh = head / (n_q / n_kv), tid = threadIdx.x;
    /* Before the dependency wait: everything that the kernels of this token do not write.  The norm weights and the
       rotary tables are constants.  The position and the cache rows below it were written while earlier tokens were
       decoded, and the step's first kernel (the embedding gather) is an ordinary launch, so all of that is complete
       before any kernel of this token starts.  The cached rows are pulled towards L1 for the score and value loops. */
    float qw = 0.f, kw = 0.f;
    if (q_norm && tid < hd) { qw = bf2f(q_norm[tid]); kw = bf2f(k_norm[tid]); }
    const int32_t pos = *pos_ptr;
    const bool pos_ok = pos >= 0 && (uint32_t)pos < max_len;
    float rc = 0.f, rs = 0.f;
    if (pos_ok) {
        if (tid < hd) { rc = bf2f(cos_t[(uint64_t)pos * hd + tid]); rs = bf2f(sin_t[(uint64_t)pos * hd + tid]); }
        const uint32_t lines_per_row = (hd * 2u + 127u) >> 7, lines = (uint32_t)pos * lines_per_row;
        const uint8_t *kbase = reinterpret_cast<const uint8_t *>(k_cache + (uint64_t)kvh * max_len * hd), *vbase = reinterpret_cast<const uint8_t *>(v_cache + (uint64_t)kvh * max_len * hd);
        for (uint32_t i = tid; i < lines && i < 1024u; i += blockDim.x) {      /* up to 128 KB of each: what L1 can hold */
            asm volatile("prefetch.global.L1 [%0];" ::"l"(kbase + (uint64_t)i * 128u));
            asm volatile("prefetch.global.L1 [%0];" ::"l"(vbase + (uint64_t)i * 128u));
        }
    }
    dependency_sync();
    if (!pos_ok) { if (tid == 0) atomicExch(status, 1); return; }
    const uint16_t *qp = qkv + (uint64_t)head * hd, *kp = qkv + (uint64_t)(n_q + kvh) * hd, *vp = qkv + (uint64_t)(n_q + n_kv + kvh) * hd;
    float qv = 0.f, kv = 0.f;
    if (tid < hd) { qv = bf2f(qp[tid]); kv = bf2f(kp[tid]); }
    /* per-head RMSNorm of q and k (Qwen3), then rotary embedding with bf16 rounding per operation */
    if (q_norm) {
        const float qi = rsqrtf(block_sum(qv * qv, red) / (float)hd + eps), ki = rsqrtf(block_sum(kv * kv, red) / (float)hd + eps);
        if (tid < hd) { qv = bfround(qw * bfround(qv * qi)); kv = bfround(kw * bfround(kv * ki)); }
    }
    if (tid < hd) { qs[tid] = qv; ks[tid] = kv; }
    __syncthreads();
    if (tid < hd) {
        const uint32_t half = hd >> 1, other = tid < half ? tid + half : tid - half;
        const float sgn = tid < half ? -1.f : 1.f, c = rc, s = rs;
        qv = bfround(bfround(qs[tid] * c) + bfround(sgn * qs[other] * s));
        kv = bfround(bfround(ks[tid] * c) + bfround(sgn * ks[other] * s));
    }
    __syncthreads();
    if (tid < hd) {
        qs[tid] = qv * scale; ks[tid] = kv;
        if (head == kvh * (n_q / n_kv)) {                            /* first query head of the group appends to the cache */
            k_cache[((uint64_t)kvh * max_len + pos) * hd + tid] = f2bf(kv);
            v_cache[((uint64_t)kvh * max_len + pos) * hd + tid] = vp[tid];
        }
    }
    __syncthreads();
    /* scores: one thread per cached position; the current position comes from shared memory */
    const uint16_t *kc = k_cache + (uint64_t)kvh * max_len * hd;
    float best = -INFINITY;
    for (int32_t t = tid; t <= pos; t += blockDim.x) {
        float s = 0.f;
        if (t == pos) { for (uint32_t d = 0; d < hd; d++) s = fmaf(qs[d], ks[d], s); }
        else {
            const uint4 *row = reinterpret_cast<const uint4 *>(kc + (uint64_t)t * hd);
            for (uint32_t d8 = 0; d8 < hd / 8; d8++) {
                const uint4 w = row[d8];
                const uint32_t p[4] = {w.x, w.y, w.z, w.w};
#pragma unroll
                for (int j = 0; j < 4; j++) { s = fmaf(qs[d8 * 8 + 2 * j], __uint_as_float(p[j] << 16), s); s = fmaf(qs[d8 * 8 + 2 * j + 1], __uint_as_float(p[j] & 0xFFFF0000u), s); }
            }
        }
        scores[t] = s; best = fmaxf(best, s);
    }
    best = block_max(best, red);
    float denom = 0.f;
    for (int32_t t = tid; t <= pos; t += blockDim.x) { const float e = __expf(scores[t] - best); scores[t] = e; denom += e; }
    denom = block_sum(denom, red);                                 /* also orders the score writes before the reads below */
    /* out[d] = sum_t p[t] v[t][d]: hd / 8 threads cover one cached row with 128-bit loads, the thread groups take
       positions t = g mod groups and are added through shared memory in group order */
    const uint32_t per_row = hd >> 3, groups = blockDim.x / per_row, g = tid / per_row, c = tid - g * per_row;
    const uint16_t *vc = v_cache + (uint64_t)kvh * max_len * hd;
    float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
    if (g < groups) {
        for (int32_t t = g; t <= pos; t += groups) {
            const uint4 w = *reinterpret_cast<const uint4 *>((t == pos ? vp : vc + (uint64_t)t * hd) + 8u * c);
            const float p = scores[t];
            const uint32_t u[4] = {w.x, w.y, w.z, w.w};
#pragma unroll
            for (int j = 0; j < 4; j++) { acc[2 * j] = fmaf(p, __uint_as_float(u[j] << 16), acc[2 * j]); acc[2 * j + 1] = fmaf(p, __uint_as_float(u[j] & 0xFFFF0000u), acc[2 * j + 1]); }
        }
    }
    float *part = sm;                                              /* [groups][hd] over q, k and the scores: all dead now */
    __syncthreads();
    if (g < groups) {
#pragma unroll
        for (int j = 0; j < 8; j++) part[g * hd + 8u * c + j] = acc[j];
    }
    __syncthreads();
    if (tid < hd) {
        float o = 0.f;
        for (uint32_t i = 0; i < groups; i++) o += part[i * hd + tid];
        out[(uint64_t)head * hd + tid] = f2bf(o / denom);
    }
}

/* The same token of attention for head sizes of 64, 128 or 256 (VPL = head_dim / 32 values per lane), organised for
   latency: one CTA of eight warps per query head, and inside a warp every lane owns VPL consecutive dimensions, so a cached
   row is one coalesced load per warp, a score is VPL multiply-adds and five shuffles, and nothing between the prologue and
   the final combine needs a CTA barrier.  Warp w takes the cached positions w, w + 8, ... with an online softmax (running
   maximum, denominator and weighted value sum in fp32); the eight partial results meet once in shared memory.  The query
   (per-head RMSNorm, rotary embedding, bf16 rounding per step as in the kernel above) is computed by every warp for its own
   lanes - the rotary partner of a dimension lives in lane ^ 16 - and warp 0 also prepares the new key, appends key and value
   to the cache (first query head of the group) and scores the current position from registers. */
template <int VPL> struct LaneRow;
template <> struct LaneRow<2> { using T = uint32_t; };
template <> struct LaneRow<4> { using T = uint2; };
template <> struct LaneRow<8> { using T = uint4; };
template <int VPL> __device__ __forceinline__ void unpack_row(const typename LaneRow<VPL>::T &w, float (&v)[VPL]);
template <> __device__ __forceinline__ void unpack_row<2>(const uint32_t &w, float (&v)[2]) { v[0] = __uint_as_float(w << 16); v[1] = __uint_as_float(w & 0xFFFF0000u); }
template <> __device__ __forceinline__ void unpack_row<4>(const uint2 &w, float (&v)[4]) {
    v[0] = __uint_as_float(w.x << 16); v[1] = __uint_as_float(w.x & 0xFFFF0000u); v[2] = __uint_as_float(w.y << 16); v[3] = __uint_as_float(w.y & 0xFFFF0000u);
}
template <> __device__ __forceinline__ void unpack_row<8>(const uint4 &w, float (&v)[8]) {
    const uint32_t u[4] = {w.x, w.y, w.z, w.w};
#pragma unroll
    for (int j = 0; j < 4; j++) { v[2 * j] = __uint_as_float(u[j] << 16); v[2 * j + 1] = __uint_as_float(u[j] & 0xFFFF0000u); }
}
__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}

/* Long caches: gridDim.y CTAs per query head, CTA y takes an equal share of the cached positions (the first one also the
   current position).  Each CTA leaves its (maximum, denominator, value sum) in a per-device work area; the CTA of a head that
   arrives last at the head's counter combines the shares in split order and writes the output (so the result does not depend
   on timing).  One work area per device: calls on one device must not overlap. */
constexpr uint32_t kAttnMaxSplits = 8, kAttnMaxHeads = 256, kAttnMaxDim = 256;
static __device__ float g_attn_share[kAttnMaxHeads * kAttnMaxSplits * (kAttnMaxDim + 2u)];
static __device__ unsigned int g_attn_arrived[kAttnMaxHeads];

template <int VPL>
__global__ void __launch_bounds__(256) attention_decode_lanes_kernel(const uint16_t *__restrict__ qkv, const uint16_t *__restrict__ q_norm, const uint16_t *__restrict__ k_norm,
                                                                      const uint16_t *__restrict__ cos_t, const uint16_t *__restrict__ sin_t, uint16_t *__restrict__ k_cache,
                                                                      uint16_t *__restrict__ v_cache, const int32_t *__restrict__ pos_ptr, uint32_t n_q, uint32_t n_kv,
                                                                      uint32_t max_len, float eps, float scale, uint16_t *__restrict__ out, int *__restrict__ status) {
    constexpr uint32_t hd = 32u * VPL, kWarps = 8;
    using Row = typename LaneRow<VPL>::T;
    __shared__ float part_max[kWarps], part_den[kWarps], part_acc[kWarps][hd];
    __shared__ unsigned int last_of_head;
    const uint32_t head = blockIdx.x, kvh = head / (n_q / n_kv), tid = threadIdx.x, lane = tid & 31u, warp = tid >> 5, d0 = lane * VPL;
    const uint32_t split = blockIdx.y, splits = gridDim.y;
    /* before the dependency wait: constants and what earlier tokens left (position, rotary row, norm weights, cached rows) */
    const int32_t pos = *pos_ptr;
    const bool pos_ok = pos >= 0 && (uint32_t)pos < max_len;
    float cs[VPL], sn[VPL], qw[VPL], kw[VPL];
#pragma unroll
    for (int j = 0; j < VPL; j++) { cs[j] = sn[j] = 0.f; qw[j] = kw[j] = 1.f; }
    const uint16_t *kc = k_cache + (uint64_t)kvh * max_len * hd, *vc = v_cache + (uint64_t)kvh * max_len * hd;
    if (pos_ok) {
#pragma unroll
        for (int j = 0; j < VPL; j++) {
            cs[j] = bf2f(cos_t[(uint64_t)pos * hd + d0 + j]); sn[j] = bf2f(sin_t[(uint64_t)pos * hd + d0 + j]);
            if (q_norm) { qw[j] = bf2f(q_norm[d0 + j]); kw[j] = bf2f(k_norm[d0 + j]); }
        }
        const uint32_t lines_per_row = (hd * 2u + 127u) >> 7, lines = (uint32_t)pos * lines_per_row;
        for (uint32_t i = tid; i < lines && i < 1024u; i += 256u) {          /* up to 128 KB of each: what L1 can hold */
            asm volatile("prefetch.global.L1 [%0];" ::"l"(reinterpret_cast<const uint8_t *>(kc) + (uint64_t)i * 128u));
            asm volatile("prefetch.global.L1 [%0];" ::"l"(reinterpret_cast<const uint8_t *>(vc) + (uint64_t)i * 128u));
        }
    }
    dependency_sync();
    if (!pos_ok) { if (tid == 0) atomicExch(status, 1); return; }
    /* per-head RMSNorm (Qwen3), then rotary embedding with bf16 rounding per operation; partner dimension = lane ^ 16 */
    auto prepare = [&](const uint16_t *src, const float (&w)[VPL], bool norm, float (&v)[VPL]) {
        Row raw = *reinterpret_cast<const Row *>(src + d0);
        unpack_row<VPL>(raw, v);
        if (norm) {
            float ss = 0.f;
#pragma unroll
            for (int j = 0; j < VPL; j++) ss += v[j] * v[j];
            const float inv = rsqrtf(warp_sum(ss) / (float)hd + eps);
#pragma unroll
            for (int j = 0; j < VPL; j++) v[j] = bfround(w[j] * bfround(v[j] * inv));
        }
        const float sgn = lane < 16u ? -1.f : 1.f;
#pragma unroll
        for (int j = 0; j < VPL; j++) {
            const float other = __shfl_xor_sync(0xffffffffu, v[j], 16);
            v[j] = bfround(bfround(v[j] * cs[j]) + bfround(sgn * other * sn[j]));
        }
    };
    float q[VPL];
    prepare(qkv + (uint64_t)head * hd, qw, q_norm != nullptr, q);
#pragma unroll
    for (int j = 0; j < VPL; j++) q[j] *= scale;
    float m = -INFINITY, den = 0.f, acc[VPL];
#pragma unroll
    for (int j = 0; j < VPL; j++) acc[j] = 0.f;
    auto absorb = [&](const float (&kr)[VPL], const float (&vr)[VPL]) {
        float s = 0.f;
#pragma unroll
        for (int j = 0; j < VPL; j++) s = fmaf(q[j], kr[j], s);
        s = warp_sum(s);
        const float m_new = fmaxf(m, s), corr = __expf(m - m_new), p = __expf(s - m_new);
        den = den * corr + p;
#pragma unroll
        for (int j = 0; j < VPL; j++) acc[j] = fmaf(p, vr[j], acc[j] * corr);
        m = m_new;
    };
    /* this CTA's share of the cached positions [t_begin, t_end) */
    const int32_t share_len = (pos + (int32_t)splits - 1) / (int32_t)splits, t_begin = (int32_t)split * share_len, t_end = min(pos, t_begin + share_len);
    if (warp == 0 && split == 0) {                                   /* the current position: key and value of this token, from registers */
        float k[VPL], v[VPL];
        prepare(qkv + (uint64_t)(n_q + kvh) * hd, kw, k_norm != nullptr, k);
        const Row vraw = *reinterpret_cast<const Row *>(qkv + (uint64_t)(n_q + n_kv + kvh) * hd + d0);
        unpack_row<VPL>(vraw, v);
        if (head == kvh * (n_q / n_kv)) {                            /* first query head of the group appends to the cache */
#pragma unroll
            for (int j = 0; j < VPL; j++) k_cache[((uint64_t)kvh * max_len + pos) * hd + d0 + j] = f2bf(k[j]);
            *reinterpret_cast<Row *>(v_cache + ((uint64_t)kvh * max_len + pos) * hd + d0) = vraw;
        }
        absorb(k, v);
    }
    /* cached positions: two rows of each cache in flight per step */
    int32_t t = t_begin + (int32_t)warp;
    for (; t + (int32_t)kWarps < t_end; t += 2 * (int32_t)kWarps) {
        const Row ka = *reinterpret_cast<const Row *>(kc + (uint64_t)t * hd + d0), kb = *reinterpret_cast<const Row *>(kc + (uint64_t)(t + kWarps) * hd + d0);
        const Row va = *reinterpret_cast<const Row *>(vc + (uint64_t)t * hd + d0), vb = *reinterpret_cast<const Row *>(vc + (uint64_t)(t + kWarps) * hd + d0);
        float kr[VPL], vr[VPL];
        unpack_row<VPL>(ka, kr); unpack_row<VPL>(va, vr); absorb(kr, vr);
        unpack_row<VPL>(kb, kr); unpack_row<VPL>(vb, vr); absorb(kr, vr);
    }
    if (t < t_end) {
        float kr[VPL], vr[VPL];
        unpack_row<VPL>(*reinterpret_cast<const Row *>(kc + (uint64_t)t * hd + d0), kr); unpack_row<VPL>(*reinterpret_cast<const Row *>(vc + (uint64_t)t * hd + d0), vr);
        absorb(kr, vr);
    }
    /* combine the eight warps: common maximum, then denominators and value sums rescaled to it, in warp order */
    if (lane == 0) { part_max[warp] = m; part_den[warp] = den; }
#pragma unroll
    for (int j = 0; j < VPL; j++) part_acc[warp][d0 + j] = acc[j];
    __syncthreads();
    float top = part_max[0], total = 0.f, o = 0.f;
    for (uint32_t w = 1; w < kWarps; w++) top = fmaxf(top, part_max[w]);
    if (tid < hd) {
        for (uint32_t w = 0; w < kWarps; w++) {
            const float f = top == -INFINITY ? 0.f : __expf(part_max[w] - top);      /* a warp without positions: exp(-inf) = 0 */
            total = fmaf(part_den[w], f, total); o = fmaf(part_acc[w][tid], f, o);
        }
    }
    if (splits == 1u) {
        if (tid < hd) out[(uint64_t)head * hd + tid] = f2bf(o / total);
        return;
    }
    /* several CTAs per head: leave this share, the last CTA to arrive combines all of them in split order */
    float *mine = g_attn_share + ((uint64_t)head * kAttnMaxSplits + split) * (kAttnMaxDim + 2u);
    if (tid < hd) mine[2u + tid] = o;
    if (tid == 0) { mine[0] = top; mine[1] = total; }
    __syncthreads();
    if (tid == 0) { __threadfence(); last_of_head = atomicAdd(&g_attn_arrived[head], 1u) == splits - 1u ? 1u : 0u; }
    __syncthreads();
    if (!last_of_head) return;
    __threadfence();
    const float *shares = g_attn_share + (uint64_t)head * kAttnMaxSplits * (kAttnMaxDim + 2u);
    float best = -INFINITY;
    for (uint32_t y = 0; y < splits; y++) best = fmaxf(best, __ldcg(shares + y * (kAttnMaxDim + 2u)));
    if (tid < hd) {
        float den_all = 0.f, sum = 0.f;
        for (uint32_t y = 0; y < splits; y++) {
            const float *sh = shares + y * (kAttnMaxDim + 2u);
            const float my = __ldcg(sh), f = my == -INFINITY ? 0.f : __expf(my - best);
            den_all = fmaf(__ldcg(sh + 1), f, den_all); sum = fmaf(__ldcg(sh + 2u + tid), f, sum);
        }
        out[(uint64_t)head * hd + tid] = f2bf(sum / den_all);
    }
    if (tid == 0) g_attn_arrived[head] = 0u;
}

/* a <- bf16(bf16(silu(gate)) * up), gate = gu[0..I), up = gu[I..2I); optional fp32 copy */
__global__ void swiglu_kernel(const uint16_t *__restrict__ gu, uint32_t I, uint16_t *__restrict__ a16, float *__restrict__ a32) {
    const uint32_t i = blockIdx.x * blockDim.x + threadIdx.x;
    dependency_sync();
    if (i >= I) return;
    const float g = bf2f(gu[i]), u = bf2f(gu[I + i]);
    const float y = bfround(bfround(g / (1.f + __expf(-g))) * u);
    a16[i] = f2bf(y);
    if (a32) a32[i] = y;
}

/* Greedy choice: smallest index of the largest logit.  Every CTA folds its slice into one 64-bit key (order-preserving
   image of the value in the high word, inverted index in the low word) and takes the maximum into a device word; the
   CTA that arrives last writes the token for the next step, logs it, advances pos and step (only while the log and the
   position range have room), and clears the two words for the next call.  Calls on one device must not overlap (they
   share the two words).
   Vocabulary-sharded logits (peers.world > 0): the last CTA first exchanges its rank's best with the other ranks - one
   8-byte word per rank, stored into every rank's exchange buffer: call number (16 bits) | order-preserving bf16 value
   (16 bits) | inverted GLOBAL index (32 bits) - then waits (bounded) until the word of every rank carries this call's
   number and takes the largest.  Every rank ends with the same token without an all-gather of the logits. */
static __device__ unsigned long long g_argmax_key;
static __device__ unsigned int g_argmax_arrived;
static __device__ int g_model_status;

__device__ __forceinline__ unsigned long long argmax_key(float v, uint32_t i) {
    uint32_t u = __float_as_uint(v);
    u = (u & 0x80000000u) ? ~u : (u | 0x80000000u);
    return ((unsigned long long)u << 32) | (0xFFFFFFFFu - i);
}
__device__ __forceinline__ unsigned long long timer_ns() { unsigned long long t; asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t)); return t; }

__global__ void __launch_bounds__(256) argmax_kernel(const uint16_t *__restrict__ logits, uint32_t V, int64_t *__restrict__ cur, int64_t *__restrict__ log,
                                                      int32_t *__restrict__ pos, int32_t *__restrict__ step, uint32_t log_len, uint32_t max_pos,
                                                      const nwc::PeerOutput peers, unsigned long long timeout_ns) {
    __shared__ unsigned long long best_of_warp[8];
    dependency_sync();
    unsigned long long best = 0ull;
    const uint32_t chunks = V >> 3, stride = gridDim.x * blockDim.x;
    for (uint32_t k = blockIdx.x * blockDim.x + threadIdx.x; k < chunks; k += stride) {
        const uint4 w = *reinterpret_cast<const uint4 *>(logits + 8ull * k);
        const uint32_t u[4] = {w.x, w.y, w.z, w.w};
#pragma unroll
        for (int j = 0; j < 4; j++) {
            const unsigned long long a = argmax_key(__uint_as_float(u[j] << 16), 8u * k + 2u * j), b = argmax_key(__uint_as_float(u[j] & 0xFFFF0000u), 8u * k + 2u * j + 1u);
            best = a > best ? a : best; best = b > best ? b : best;
        }
    }
    if (blockIdx.x == 0 && threadIdx.x < (V & 7u)) { const uint32_t i = (V & ~7u) + threadIdx.x; const unsigned long long a = argmax_key(bf2f(logits[i]), i); best = a > best ? a : best; }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) { const unsigned long long other = __shfl_xor_sync(0xffffffffu, best, o); best = other > best ? other : best; }
    if ((threadIdx.x & 31) == 0) best_of_warp[threadIdx.x >> 5] = best;
    __syncthreads();
    if (threadIdx.x == 0) {
        for (uint32_t w = 1; w < (blockDim.x >> 5); w++) best = best_of_warp[w] > best ? best_of_warp[w] : best;
        atomicMax(&g_argmax_key, best);
        __threadfence();
        if (atomicAdd(&g_argmax_arrived, 1u) == gridDim.x - 1u) {
            __threadfence();
            const unsigned long long key = atomicExch(&g_argmax_key, 0ull);
            g_argmax_arrived = 0u;
            uint32_t idx = key ? 0xFFFFFFFFu - (uint32_t)key : 0u;
            if (peers.world) {
                nwc::CommControl *own = reinterpret_cast<nwc::CommControl *>(peers.buf[peers.rank]);
                volatile uint32_t *calls = &own->argmax_epoch;
                const uint32_t call = *calls + 1u;
                *calls = call;
                const unsigned long long tag = (unsigned long long)(call & 0xFFFFu) << 48;
                const unsigned long long mine = tag | ((key >> 48) << 32) | (unsigned long long)(0xFFFFFFFFu - (idx + peers.rank * V));
                for (uint32_t p = 0; p < peers.world; p++)
                    *reinterpret_cast<volatile unsigned long long *>(&reinterpret_cast<nwc::CommControl *>(peers.buf[p])->argmax_key[peers.rank]) = mine;
                unsigned long long top = 0ull;
                const unsigned long long t0 = timer_ns();
                for (uint32_t r = 0; r < peers.world; r++) {
                    const volatile unsigned long long *slot = &own->argmax_key[r];
                    unsigned long long w = *slot;
                    while ((w >> 48) != (tag >> 48)) {
                        if (timer_ns() - t0 > timeout_ns) { atomicExch(&g_model_status, nwc::kStatusPeerTimeout); w = mine; break; }
                        __nanosleep(20);
                        w = *slot;
                    }
                    w &= 0xFFFFFFFFFFFFull;
                    top = w > top ? w : top;
                }
                idx = 0xFFFFFFFFu - (uint32_t)top;
            }
            cur[0] = (int64_t)idx;
            const int32_t s = *step, p = *pos;
            if (s >= 0 && (uint32_t)s < log_len && p >= 0 && (uint32_t)p < max_pos) {
                if (log) log[s] = (int64_t)idx;
                *pos = p + 1; *step = s + 1;
            }
        }
    }
}

bool g_plain_attention = false;          /* tests: route every head size through the general kernel */

template <class... Params, class... Args>
cudaError_t launch(void (*kernel)(Params...), dim3 grid, dim3 block, size_t smem, void *stream, Args... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid; cfg.blockDim = block; cfg.dynamicSmemBytes = smem; cfg.stream = (cudaStream_t)stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr; cfg.numAttrs = nwc::dependent_launch() ? 1 : 0;
    return cudaLaunchKernelEx(&cfg, kernel, static_cast<Params>(args)...);
}

}  // namespace

/* ---- decode-step entry points (no counterpart in the reference's library; its decode step is Transformers code) --- */

NWC_EXPORT int nwc_add_rmsnorm(void *stream, const uint16_t *h_in, const uint16_t *delta, uint16_t *h_out, const uint16_t *weight, float eps, uint32_t H,
                               uint16_t *xn16, float *xn32) {
    if (!H) return -1;
    return (int)launch(add_rmsnorm_kernel, dim3(1), dim3(H >= 4096 ? 1024 : (H >= 1024 ? 512 : 256)), 0, stream, h_in, delta, h_out, weight, eps, H, xn16, xn32);
}

NWC_EXPORT int nwc_attention_decode(void *stream, const uint16_t *qkv, const uint16_t *q_norm, const uint16_t *k_norm, const uint16_t *cos_t, const uint16_t *sin_t,
                                    uint16_t *k_cache, uint16_t *v_cache, const int32_t *pos, uint32_t n_q, uint32_t n_kv, uint32_t head_dim, uint32_t max_len,
                                    float eps, uint16_t *out, int *status) {
    if (!n_q || !n_kv || n_q % n_kv || head_dim % 8 || head_dim > 256 || head_dim < 32 || max_len == 0 || max_len > 8192) return -1;
    const size_t floats = 2 * (size_t)head_dim + max_len, need = (256u / (head_dim / 8u)) * (size_t)head_dim;   /* scores, or the group partials */
    const size_t smem = (floats > need ? floats : need) * sizeof(float);
    if (!nwc_setup()) return (int)cudaErrorNoDevice;             /* prepares this device's kernels on first use */
    const float scale = 1.0f / sqrtf((float)head_dim);
    if (!g_plain_attention && (head_dim == 64 || head_dim == 128 || head_dim == 256) && !((reinterpret_cast<uintptr_t>(qkv) | reinterpret_cast<uintptr_t>(k_cache) | reinterpret_cast<uintptr_t>(v_cache)) & 15u)) {
        /* the grid is fixed when a decode graph is captured, the position is not: the split count follows the cache length */
        const uint32_t splits = n_q > kAttnMaxHeads ? 1u : (max_len <= 384u ? 1u : (max_len <= 1024u ? 2u : (max_len <= 2048u ? 4u : kAttnMaxSplits)));
        const dim3 grid(n_q, splits), block(256);
        if (head_dim == 64) return (int)launch(attention_decode_lanes_kernel<2>, grid, block, 0, stream, qkv, q_norm, k_norm, cos_t, sin_t, k_cache, v_cache, pos, n_q, n_kv, max_len, eps, scale, out, status);
        if (head_dim == 128) return (int)launch(attention_decode_lanes_kernel<4>, grid, block, 0, stream, qkv, q_norm, k_norm, cos_t, sin_t, k_cache, v_cache, pos, n_q, n_kv, max_len, eps, scale, out, status);
        return (int)launch(attention_decode_lanes_kernel<8>, grid, block, 0, stream, qkv, q_norm, k_norm, cos_t, sin_t, k_cache, v_cache, pos, n_q, n_kv, max_len, eps, scale, out, status);
    }
    return (int)launch(attention_decode_kernel, dim3(n_q), dim3(256), smem, stream, qkv, q_norm, k_norm, cos_t, sin_t, k_cache, v_cache, pos, n_q, n_kv, head_dim,
                       max_len, eps, 1.0f / sqrtf((float)head_dim), out, status);
}

NWC_EXPORT void nwc_set_plain_attention(int on) { g_plain_attention = on != 0; }

NWC_EXPORT int nwc_swiglu(void *stream, const uint16_t *gate_up, uint32_t I, uint16_t *a16, float *a32) {
    if (!I) return -1;
    return (int)launch(swiglu_kernel, dim3((I + 255) / 256), dim3(256), 0, stream, gate_up, I, a16, a32);
}

static int run_argmax(void *stream, const uint16_t *logits, uint32_t V, int64_t *cur, int64_t *log, int32_t *pos, int32_t *step, uint32_t log_len,
                      uint32_t max_pos, const nwc::PeerOutput &peers) {
    if (!V || !cur || !pos || !step) return -1;
    if (reinterpret_cast<uintptr_t>(logits) & 15u) return -1;
    const uint32_t chunks = V >> 3, grid = chunks >= 256u * 64u ? 64u : (chunks + 255u) / 256u + (chunks ? 0u : 1u);
    return (int)launch(argmax_kernel, dim3(grid ? grid : 1u), dim3(256), 0, stream, logits, V, cur, log, pos, step, log_len, max_pos, peers, nwc::peer_timeout_ns());
}

NWC_EXPORT int nwc_argmax(void *stream, const uint16_t *logits, uint32_t V, int64_t *cur, int64_t *log, int32_t *pos, int32_t *step, uint32_t log_len,
                          uint32_t max_pos) {
    return run_argmax(stream, logits, V, cur, log, pos, step, log_len, max_pos, nwc::PeerOutput{});
}

NWC_EXPORT int nwc_argmax_tp(void *stream, const uint16_t *logits, uint32_t V, int64_t *cur, int64_t *log, int32_t *pos, int32_t *step, uint32_t log_len,
                             uint32_t max_pos, void *const *buffers, int rank, int world) {
    if (!buffers || world < 1 || world > (int)nwc::kCommMaxRanks || rank < 0 || rank >= world || (uint64_t)V * (uint64_t)world > 0xFFFFFFFFull) return -1;
    nwc::PeerOutput peers{};
    for (int r = 0; r < world; r++) { if (!buffers[r]) return -1; peers.buf[r] = static_cast<uint8_t *>(buffers[r]); }
    peers.world = (uint32_t)world; peers.rank = (uint32_t)rank;
    return run_argmax(stream, logits, V, cur, log, pos, step, log_len, max_pos, peers);
}

namespace nwc {
/* dynamic shared memory beyond 48 KB for long caches; attributes of a function are per device */
void configure_model_kernels() { cudaFuncSetAttribute(attention_decode_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 64 * 1024); }

int read_model_status(bool clear) {
    int v = 0;
    if (cudaMemcpyFromSymbol(&v, g_model_status, sizeof(int)) != cudaSuccess) return -1;
    if (clear && v) { const int z = 0; cudaMemcpyToSymbol(g_model_status, &z, sizeof(int)); }
    return v;
}
}  // namespace nwc
