// Weight-only quantisation kernels for frozen base weights (QLoRA).
//
//  * nf4_dequant: 4-bit NormalFloat codes (two per byte, first element in the high nibble) x fp32
//    absmax per 64-element block -> bf16. The absmax vector is already "double-dequantised" by the
//    caller (8-bit codes x per-256 scale + offset), as it is 1/64 of the data.
//    Storage contract of the bitsandbytes 4-bit format the reference dequantises through ctypes
//    (src/axolotl/kernels/quantize.py:27-106).
//  * fp8_block_dequant: E4M3 weights x fp32 inverse scale per 128x128 block -> bf16
//    (src/axolotl/kernels/quantize.py:109-135).
#include <cuda_fp8.h>

#include "axb_common.cuh"

namespace {

__constant__ float kNF4[16] = {-1.0f,
                               -0.6961928009986877f,
                               -0.5250730514526367f,
                               -0.39491748809814453f,
                               -0.28444138169288635f,
                               -0.18477343022823334f,
                               -0.09105003625154495f,
                               0.0f,
                               0.07958029955625534f,
                               0.16093020141124725f,
                               0.24611230194568634f,
                               0.33791524171829224f,
                               0.44070982933044434f,
                               0.5626170039176941f,
                               0.7229568362236023f,
                               1.0f};

// one thread per 16 values (8 packed bytes); blocksize must be a multiple of 16
__global__ void nf4_dequant_kernel(const uint8_t* __restrict__ q, const float* __restrict__ absmax,
                                   __nv_bfloat16* __restrict__ out, long long n_chunks,
                                   int chunks_per_block) {
  for (long long c = (long long)blockIdx.x * blockDim.x + threadIdx.x; c < n_chunks;
       c += (long long)gridDim.x * blockDim.x) {
    const float s = absmax[c / chunks_per_block];
    const uint2 packed = *reinterpret_cast<const uint2*>(q + c * 8);
    const uint32_t w[2] = {packed.x, packed.y};
    uint32_t o[8];
#pragma unroll
    for (int i = 0; i < 2; ++i)
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const uint32_t byte = (w[i] >> (8 * j)) & 0xFF;
        o[i * 4 + j] = pack_bf16x2(kNF4[byte >> 4] * s, kNF4[byte & 0xF] * s);
      }
    uint4* dst = reinterpret_cast<uint4*>(out + c * 16);
    dst[0] = make_uint4(o[0], o[1], o[2], o[3]);
    dst[1] = make_uint4(o[4], o[5], o[6], o[7]);
  }
}

// one thread per 8 consecutive values of a row
__global__ void fp8_block_dequant_kernel(const __nv_fp8_e4m3* __restrict__ w,
                                         const float* __restrict__ scale_inv,
                                         __nv_bfloat16* __restrict__ out, long long rows, long long cols,
                                         int block, long long scale_cols) {
  const long long per_row = cols / 8;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < rows * per_row;
       i += (long long)gridDim.x * blockDim.x) {
    const long long r = i / per_row, c = (i - r * per_row) * 8;
    const float s = scale_inv[(r / block) * scale_cols + c / block];
    const uint2 raw = *reinterpret_cast<const uint2*>(w + r * cols + c);
    const __nv_fp8_e4m3* v = reinterpret_cast<const __nv_fp8_e4m3*>(&raw);
    uint32_t o[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) o[j] = pack_bf16x2(float(v[2 * j]) * s, float(v[2 * j + 1]) * s);
    *reinterpret_cast<uint4*>(out + r * cols + c) = make_uint4(o[0], o[1], o[2], o[3]);
  }
}

}  // namespace

// q: n_values / 2 bytes; absmax: fp32 [n_values / blocksize]; out: bf16 [n_values]
extern "C" int axb_nf4_dequant(const void* q, const float* absmax, void* out, long long n_values,
                               int blocksize, void* stream) {
  if (n_values % 16 || blocksize % 16) return -2;
  const long long n_chunks = n_values / 16;
  if (n_chunks <= 0) return 0;
  const long long want = (n_chunks + 255) / 256;
  const int grid = (int)(want > 148 * 16 ? 148 * 16 : want);
  nf4_dequant_kernel<<<grid, 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
      (const uint8_t*)q, absmax, (__nv_bfloat16*)out, n_chunks, blocksize / 16);
  return (int)cudaGetLastError();
}

// w: e4m3 [rows, cols] (cols % 8 == 0); scale_inv: fp32 [ceil(rows/block), ceil(cols/block)]
extern "C" int axb_fp8_block_dequant(const void* w, const float* scale_inv, void* out, long long rows,
                                     long long cols, int block, void* stream) {
  if (cols % 8 || block % 8) return -2;
  const long long n = rows * (cols / 8);
  if (n <= 0) return 0;
  const long long want = (n + 255) / 256;
  const int grid = (int)(want > 148 * 16 ? 148 * 16 : want);
  fp8_block_dequant_kernel<<<grid, 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
      (const __nv_fp8_e4m3*)w, scale_inv, (__nv_bfloat16*)out, rows, cols, block, (cols + block - 1) / block);
  return (int)cudaGetLastError();
}
