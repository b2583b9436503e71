/* GPU encoder: weights -> NWC streams, planes and tables, byte-identical to the reference's host encoder.
 *
 * Passes (all on one stream, two small host round trips):
 *   1. histogram of the 7-bit symbols (shared-memory bins per CTA, 64-bit global bins); fp8 NaN raises the status word
 *   2. host: frequency order with the reference's exchange rule, rank table back to the device, symbol table out
 *   3. one thread per (block, lane) measures its stream -> header byte; over-long streams raise the status word
 *   4. one CTA turns block sizes into 8-byte aligned block offsets (exclusive scan) and the total length
 *   5. one thread per (block, lane) re-walks its stream and writes words / exception entries and the planes of
 *      layouts 1 and 2; layout 0's row-major raw plane has its own element-wise kernel
 *
 * Interfaces replaced (reference: csrc/nwc_ops.cu): nwc_encode 245-320, encode2 175-243, nwc_build_tab 324-348.
 */
#include <cstdlib>
#include <cstring>
#include "nwc_encode_core.h"
#include "nwc_encode.h"

namespace nwc {

namespace {

constexpr int kEncThreads = 256;

__global__ void histogram_kernel(const void *w, uint64_t n, int type, int layout, unsigned long long *hist, int *status) {
    __shared__ unsigned int bins[128];
    for (int i = threadIdx.x; i < 128; i += blockDim.x) bins[i] = 0;
    __syncthreads();
    const uint64_t stride = (uint64_t)gridDim.x * blockDim.x;
    for (uint64_t i = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride) {
        uint32_t sym;
        if (type == kFp8) {
            const uint32_t b = static_cast<const uint8_t *>(w)[i];
            uint32_t raw;
            const bool ok = layout == 2 ? fp8_split_fixed(b, sym, raw) : fp8_split_prefix(b, sym, raw);
            if (!ok) { atomicExch(status, -2); continue; }
        } else sym = (static_cast<const uint16_t *>(w)[i] >> 8) & 0x7Fu;
        atomicAdd(&bins[sym], 1u);
    }
    __syncthreads();
    for (int i = threadIdx.x; i < 128; i += blockDim.x) if (bins[i]) atomicAdd(&hist[i], (unsigned long long)bins[i]);
}

/* pass 3: header byte of every lane stream */
__global__ void measure_kernel(EncodeJob j, uint8_t *hdr, int *status) {
    const Geometry g(j.M, j.K, j.layout);
    const uint64_t t = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (t >= (uint64_t)g.nb * kLanes) return;
    const uint32_t b = (uint32_t)(t >> 5), L = (uint32_t)(t & 31u);
    CountSink s;
    if (j.layout == 2) {
        if (!encode_fixed_stream(j, g, b, L, s)) { atomicCAS(status, 0, -3); hdr[t] = 255; return; }
        hdr[t] = (uint8_t)s.exceptions;
    } else {
        encode_prefix_stream(j, g, b, L, s);
        const uint32_t words = (s.nbits + 31u) >> 5;
        if (words > 255u) atomicCAS(status, 0, -1);
        hdr[t] = (uint8_t)(words > 255u ? 255u : words);
    }
}

/* pass 4: bases[b] = sum over earlier blocks of their size rounded up to 8; total[0] = end of the last block (not
   rounded), total[1] = sum of all rounded sizes */
__global__ void offsets_kernel(const uint8_t *hdr, uint32_t nb, uint32_t unit, uint32_t *bases, unsigned long long *total) {
    __shared__ unsigned long long part[1024];
    const uint32_t per = (nb + blockDim.x - 1) / blockDim.x, first = threadIdx.x * per, last = min(nb, first + per);
    unsigned long long sum = 0;
    for (uint32_t b = first; b < last; b++) {
        uint32_t size = 0;
        const uint4 *h = reinterpret_cast<const uint4 *>(hdr + (uint64_t)b * kLanes);
        for (int k = 0; k < 2; k++) { const uint4 v = h[k]; size += __dp4a(v.x, 0x01010101u, 0u) + __dp4a(v.y, 0x01010101u, 0u) + __dp4a(v.z, 0x01010101u, 0u) + __dp4a(v.w, 0x01010101u, 0u); }
        sum += ((unsigned long long)size * unit + 7ull) & ~7ull;
    }
    part[threadIdx.x] = sum;
    __syncthreads();
    if (threadIdx.x == 0) {
        unsigned long long run = 0;
        for (uint32_t i = 0; i < blockDim.x; i++) { const unsigned long long v = part[i]; part[i] = run; run += v; }
        total[1] = run;
    }
    __syncthreads();
    unsigned long long pos = part[threadIdx.x];
    for (uint32_t b = first; b < last; b++) {
        uint32_t size = 0;
        const uint8_t *h = hdr + (uint64_t)b * kLanes;
        for (int k = 0; k < 32; k++) size += h[k];
        bases[b] = (uint32_t)pos;
        if (b == nb - 1) total[0] = pos + (unsigned long long)size * unit;
        pos += ((unsigned long long)size * unit + 7ull) & ~7ull;
    }
}

/* pass 5: write streams / exception entries and the planes of layouts 1 and 2; one warp = one block */
__global__ void pack_kernel(EncodeJob j, const uint8_t *hdr, const uint32_t *bases, uint8_t *data, uint8_t *low) {
    const Geometry g(j.M, j.K, j.layout);
    const uint64_t t = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x;
    const bool live = t < (uint64_t)g.nb * kLanes;
    const uint32_t b = live ? (uint32_t)(t >> 5) : 0u, L = (uint32_t)(t & 31u);
    uint32_t mine = live ? hdr[(uint64_t)b * kLanes + L] : 0u, run = mine;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) { const uint32_t v = __shfl_up_sync(0xffffffffu, run, o); if (L >= (uint32_t)o) run += v; }
    if (!live) return;
    const uint32_t before = run - mine;
    uint8_t *block = data + bases[b];
    if (j.layout == 2) {
        WriteSink s(g, j.type, nullptr, block + (uint64_t)before * (j.type == kFp8 ? 2u : 3u), low);
        encode_fixed_stream(j, g, b, L, s);
    } else {
        WriteSink s(g, j.type, reinterpret_cast<uint32_t *>(block) + before, nullptr, low);
        encode_prefix_stream(j, g, b, L, s);
        s.flush();
    }
}

/* layout 0 raw plane: row-major, stride K16 (bf16 low bytes) or K16 / 2 (fp8 nibbles, interleaved per 16 columns) */
__global__ void plane0_kernel(EncodeJob j, uint8_t *low) {
    const Geometry g(j.M, j.K, 0);
    const uint32_t chunks = g.K16 >> 4;
    const uint64_t t = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (t >= (uint64_t)j.M * chunks) return;
    const uint32_t m = (uint32_t)(t / chunks), c = (uint32_t)(t - (uint64_t)m * chunks);
    plane0_cell(j, g, m, c, low);
}

}  // namespace

void build_table(const uint16_t *psym, int code, uint32_t *lut) { build_table_words(psym, code, lut); }

#define ENC_CHECK(call) do { cudaError_t e_ = (call); if (e_ != cudaSuccess) { rc = -100 - (int64_t)e_; goto done; } } while (0)

/* Encodes device-resident weights into device buffers.  psym is host memory.  Synchronises `st`. */
int64_t encode_device(cudaStream_t st, const void *w, uint64_t n, uint32_t K, int code, uint16_t *psym, uint32_t *bases, uint8_t *hdr,
                      uint8_t *data, uint64_t cap, uint8_t *low) {
    const int type = type_of(code), layout = layout_of(code);
    const uint32_t M = (uint32_t)(n / K);
    const Geometry g(M, K, layout);
    int64_t rc = -1;
    struct Work { unsigned long long hist[128]; unsigned long long total[2]; uint8_t rank_of[128]; int status; };
    Work *dev = nullptr; Work host;
    ENC_CHECK(cudaMalloc(&dev, sizeof(Work)));
    ENC_CHECK(cudaMemsetAsync(dev, 0, sizeof(Work), st));
    ENC_CHECK(cudaMemsetAsync(low, 0, g.raw_plane_bytes(code), st));
    {
        const int grid = (int)std::min<uint64_t>((n + kEncThreads * 16ull - 1) / (kEncThreads * 16ull), 4096ull);
        histogram_kernel<<<grid, kEncThreads, 0, st>>>(w, n, type, layout, dev->hist, &dev->status);
        ENC_CHECK(cudaGetLastError());
        ENC_CHECK(cudaMemcpyAsync(&host, dev, sizeof(Work), cudaMemcpyDeviceToHost, st));
        ENC_CHECK(cudaStreamSynchronize(st));
        if (host.status) { rc = host.status; goto done; }
        build_symbol_tables(host.hist, type, layout, psym, host.rank_of);
        ENC_CHECK(cudaMemcpyAsync(dev->rank_of, host.rank_of, 128, cudaMemcpyHostToDevice, st));
        EncodeJob j{w, dev->rank_of, type, layout, M, K};
        const uint64_t streams = (uint64_t)g.nb * kLanes;
        const unsigned sgrid = (unsigned)((streams + kEncThreads - 1) / kEncThreads);
        measure_kernel<<<sgrid, kEncThreads, 0, st>>>(j, hdr, &dev->status);
        ENC_CHECK(cudaGetLastError());
        offsets_kernel<<<1, 1024, 0, st>>>(hdr, g.nb, layout == 2 ? (type == kFp8 ? 2u : 3u) : 4u, bases, dev->total);
        ENC_CHECK(cudaGetLastError());
        ENC_CHECK(cudaMemcpyAsync(&host, dev, sizeof(Work), cudaMemcpyDeviceToHost, st));
        ENC_CHECK(cudaStreamSynchronize(st));
        if (host.status) { rc = host.status; goto done; }
        if (host.total[0] + 64ull > cap || host.total[1] > 0xFFFFFFFFull) { rc = -1; goto done; }
        pack_kernel<<<sgrid, kEncThreads, 0, st>>>(j, hdr, bases, data, low);
        ENC_CHECK(cudaGetLastError());
        if (layout == 0) {
            const uint64_t cells = (uint64_t)M * (g.K16 >> 4);
            plane0_kernel<<<(unsigned)((cells + kEncThreads - 1) / kEncThreads), kEncThreads, 0, st>>>(j, low);
            ENC_CHECK(cudaGetLastError());
        }
        ENC_CHECK(cudaStreamSynchronize(st));
        rc = (int64_t)(host.total[1] + 64ull);
    }
done:
    if (dev) cudaFree(dev);
    return rc;
}

/* Host-pointer front end with the reference's nwc_encode contract: stages through the device encoder. */
int64_t encode_host(const void *w, uint64_t n, uint32_t K, int code, uint16_t *freq, uint16_t *psym, uint32_t *bases, uint8_t *hdr,
                    uint8_t *data, uint64_t cap, uint8_t *low) {
    if (!K || n % K || n / K > 0xFFFFFFFFull || n == 0) return -1;
    for (uint32_t i = 0; i < kSymTableLen; i++) freq[i] = 0;
    const int type = type_of(code), layout = layout_of(code);
    const Geometry g((uint32_t)(n / K), K, layout);
    const uint64_t wbytes = n * (type == kFp8 ? 1u : 2u), lowbytes = g.raw_plane_bytes(code);
    void *dw = nullptr; uint32_t *dbases = nullptr; uint8_t *dhdr = nullptr, *ddata = nullptr, *dlow = nullptr;
    int64_t rc = -1;
    ENC_CHECK(cudaMalloc(&dw, wbytes));
    ENC_CHECK(cudaMalloc(&dbases, (uint64_t)g.nb * 4u));
    ENC_CHECK(cudaMalloc(&dhdr, (uint64_t)g.nb * kLanes));
    ENC_CHECK(cudaMalloc(&ddata, cap));
    ENC_CHECK(cudaMalloc(&dlow, lowbytes ? lowbytes : 16));
    ENC_CHECK(cudaMemcpy(dw, w, wbytes, cudaMemcpyHostToDevice));
    rc = encode_device(nullptr, dw, n, K, code, psym, dbases, dhdr, ddata, cap, dlow);
    if (rc >= 0) {
        const int64_t len = rc;
        ENC_CHECK(cudaMemcpy(bases, dbases, (uint64_t)g.nb * 4u, cudaMemcpyDeviceToHost));
        ENC_CHECK(cudaMemcpy(hdr, dhdr, (uint64_t)g.nb * kLanes, cudaMemcpyDeviceToHost));
        ENC_CHECK(cudaMemcpy(data, ddata, (uint64_t)std::min<uint64_t>((uint64_t)len - 64ull, cap), cudaMemcpyDeviceToHost));
        ENC_CHECK(cudaMemcpy(low, dlow, lowbytes, cudaMemcpyDeviceToHost));
        rc = len;
    }
done:
    cudaFree(dw); cudaFree(dbases); cudaFree(dhdr); cudaFree(ddata); cudaFree(dlow);
    return rc;
}

}  // namespace nwc
