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

/* h <- bf16(h + delta) (delta may be null); xn <- bf16(weight * bf16(h * rsqrt(mean(h^2) + eps))); optional fp32 copy */
__global__ void __launch_bounds__(1024) add_rmsnorm_kernel(uint16_t *__restrict__ h, const uint16_t *__restrict__ delta, const uint16_t *__restrict__ weight,
                                                            float eps, uint32_t H, uint16_t *__restrict__ xn16, float *__restrict__ xn32) {
    __shared__ float red[32];
    float ss = 0.f;
    for (uint32_t i = threadIdx.x; i < H; i += blockDim.x) {
        float v = bf2f(h[i]);
        if (delta) { v = bfround(v + bf2f(delta[i])); h[i] = f2bf(v); }
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
    const int32_t pos = *pos_ptr;
    if (pos < 0 || (uint32_t)pos >= max_len) { if (tid == 0) atomicExch(status, 1); return; }
    const uint16_t *qp = qkv + (uint64_t)head * hd, *kp = qkv + (uint64_t)(n_q + kvh) * hd, *vp = qkv + (uint64_t)(n_q + n_kv + kvh) * hd;
    const uint16_t *cs = cos_t + (uint64_t)pos * hd, *sn = sin_t + (uint64_t)pos * hd;
    /* per-head RMSNorm of q and k (Qwen3), then rotary embedding with bf16 rounding per operation */
    float qv = 0.f, kv = 0.f;
    if (tid < hd) { qv = bf2f(qp[tid]); kv = bf2f(kp[tid]); }
    if (q_norm) {
        const float qi = rsqrtf(block_sum(qv * qv, red) / (float)hd + eps), ki = rsqrtf(block_sum(kv * kv, red) / (float)hd + eps);
        if (tid < hd) { qv = bfround(bf2f(q_norm[tid]) * bfround(qv * qi)); kv = bfround(bf2f(k_norm[tid]) * bfround(kv * ki)); }
    }
    if (tid < hd) { qs[tid] = qv; ks[tid] = kv; }
    __syncthreads();
    if (tid < hd) {
        const uint32_t half = hd >> 1, other = tid < half ? tid + half : tid - half;
        const float sgn = tid < half ? -1.f : 1.f, c = bf2f(cs[tid]), s = bf2f(sn[tid]);
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
    /* out[d] = sum_t p[t] v[t][d]: thread (g, d) takes positions t = g mod groups; groups are added through shared memory */
    const uint32_t groups = blockDim.x / hd, g = tid / hd, d = tid - g * hd;
    const uint16_t *vc = v_cache + (uint64_t)kvh * max_len * hd;
    float acc = 0.f;
    if (g < groups) {
        for (int32_t t = g; t < pos; t += groups) acc = fmaf(scores[t], bf2f(vc[(uint64_t)t * hd + d]), acc);
        if (g == (uint32_t)pos % groups) acc = fmaf(scores[pos], bf2f(vp[d]), acc);
    }
    float *part = sm;                                              /* [groups][hd] over q, k and the head of scores: all dead now */
    __syncthreads();
    if (g < groups) part[g * hd + d] = acc;
    __syncthreads();
    if (tid < hd) {
        float o = 0.f;
        for (uint32_t i = 0; i < groups; i++) o += part[i * hd + tid];
        out[(uint64_t)head * hd + tid] = f2bf(o / denom);
    }
}

/* a <- bf16(bf16(silu(gate)) * up), gate = gu[0..I), up = gu[I..2I); optional fp32 copy */
__global__ void swiglu_kernel(const uint16_t *__restrict__ gu, uint32_t I, uint16_t *__restrict__ a16, float *__restrict__ a32) {
    const uint32_t i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= I) return;
    const float g = bf2f(gu[i]), u = bf2f(gu[I + i]);
    const float y = bfround(bfround(g / (1.f + __expf(-g))) * u);
    a16[i] = f2bf(y);
    if (a32) a32[i] = y;
}

/* Greedy choice: smallest index of the largest logit.  Writes the token for the next step, logs it, advances pos. */
__global__ void __launch_bounds__(1024) argmax_kernel(const uint16_t *__restrict__ logits, uint32_t V, int64_t *__restrict__ cur, int64_t *__restrict__ log,
                                                       int32_t *__restrict__ pos, int32_t *__restrict__ step) {
    __shared__ float bv[32]; __shared__ uint32_t bi[32];
    float best = -INFINITY; uint32_t idx = 0xFFFFFFFFu;
    for (uint32_t i = threadIdx.x; i < V; i += blockDim.x) { const float v = bf2f(logits[i]); if (v > best) { best = v; idx = i; } }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, best, o); const uint32_t oi = __shfl_xor_sync(0xffffffffu, idx, o);
        if (ov > best || (ov == best && oi < idx)) { best = ov; idx = oi; }
    }
    if ((threadIdx.x & 31) == 0) { bv[threadIdx.x >> 5] = best; bi[threadIdx.x >> 5] = idx; }
    __syncthreads();
    if (threadIdx.x == 0) {
        for (uint32_t w = 1; w < (blockDim.x + 31) / 32; w++) if (bv[w] > best || (bv[w] == best && bi[w] < idx)) { best = bv[w]; idx = bi[w]; }
        if (idx == 0xFFFFFFFFu) idx = 0;
        cur[0] = (int64_t)idx;
        if (log) log[*step] = (int64_t)idx;
        *pos += 1; *step += 1;
    }
}

}  // namespace

/* ---- decode-step entry points (no counterpart in the reference's library; its decode step is Transformers code) --- */

NWC_EXPORT int nwc_add_rmsnorm(void *stream, uint16_t *h, const uint16_t *delta, const uint16_t *weight, float eps, uint32_t H, uint16_t *xn16, float *xn32) {
    if (!H) return -1;
    add_rmsnorm_kernel<<<1, H >= 4096 ? 1024 : (H >= 1024 ? 512 : 256), 0, (cudaStream_t)stream>>>(h, delta, weight, eps, H, xn16, xn32);
    return (int)cudaGetLastError();
}

NWC_EXPORT int nwc_attention_decode(void *stream, const uint16_t *qkv, const uint16_t *q_norm, const uint16_t *k_norm, const uint16_t *cos_t, const uint16_t *sin_t,
                                    uint16_t *k_cache, uint16_t *v_cache, const int32_t *pos, uint32_t n_q, uint32_t n_kv, uint32_t head_dim, uint32_t max_len,
                                    float eps, uint16_t *out, int *status) {
    if (!n_q || !n_kv || n_q % n_kv || head_dim % 8 || head_dim > 256 || head_dim < 32 || max_len == 0 || max_len > 8192) return -1;
    const size_t smem = (2 * (size_t)head_dim + (max_len > 256u ? max_len : 256u)) * sizeof(float);
    static bool opted = false;
    if (smem > 48 * 1024 && !opted) { cudaFuncSetAttribute(attention_decode_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 64 * 1024); opted = true; }
    attention_decode_kernel<<<n_q, 256, smem, (cudaStream_t)stream>>>(qkv, q_norm, k_norm, cos_t, sin_t, k_cache, v_cache, pos, n_q, n_kv, head_dim, max_len, eps,
                                                                     rsqrtf((float)head_dim), out, status);
    return (int)cudaGetLastError();
}

NWC_EXPORT int nwc_swiglu(void *stream, const uint16_t *gate_up, uint32_t I, uint16_t *a16, float *a32) {
    if (!I) return -1;
    swiglu_kernel<<<(I + 255) / 256, 256, 0, (cudaStream_t)stream>>>(gate_up, I, a16, a32);
    return (int)cudaGetLastError();
}

NWC_EXPORT int nwc_argmax(void *stream, const uint16_t *logits, uint32_t V, int64_t *cur, int64_t *log, int32_t *pos, int32_t *step) {
    if (!V) return -1;
    argmax_kernel<<<1, 1024, 0, (cudaStream_t)stream>>>(logits, V, cur, log, pos, step);
    return (int)cudaGetLastError();
}
