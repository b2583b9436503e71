/* Encoder entry points shared between nwc_encode.cu and the C-ABI layer. */
#pragma once
#include <cstdint>
#include <cuda_runtime.h>

namespace nwc {

/* 4096-word decoder table from the symbol table (host). */
void build_table(const uint16_t *psym, int code, uint32_t *lut);

/* Device-resident weights -> device buffers; psym is host memory; synchronises the stream.
   Returns the data length (payload rounded up to 8, plus 64 bytes of slack), -1 shape / capacity / over-long stream,
   -2 fp8 NaN, -3 more than 255 exceptions in a lane of layout 2, <= -100: -(100 + cudaError). */
int64_t encode_device(cudaStream_t st, const void *w, uint64_t n, uint32_t K, int code, uint16_t *psym, uint32_t *bases,
                      uint8_t *hdr, uint8_t *data, uint64_t cap, uint8_t *low);

/* Host buffers in and out (the reference's nwc_encode contract), staged through encode_device. */
int64_t encode_host(const void *w, uint64_t n, uint32_t K, int code, uint16_t *freq, uint16_t *psym, uint32_t *bases,
                    uint8_t *hdr, uint8_t *data, uint64_t cap, uint8_t *low);

}  // namespace nwc
