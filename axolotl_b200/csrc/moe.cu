// Mixture-of-experts support kernels for sm_100a.
//
//  * nvfp4_dequant     : packed E2M1 nibbles x E4M3 block scales (16 elements) x fp32 per-tensor
//                        scale -> bf16 rows, for the frozen NVFP4 expert weights (storage contract
//                        of src/axolotl/integrations/kernels/libs/scattermoe_lora/dequant_grouped.py:63-111).
//  * ep_gather_rows    : expert-parallel DISPATCH. Every destination rank pulls the token rows
//                        routed to its experts straight out of the source ranks' symmetric
//                        activation buffers with peer loads over NVLink (row list: source rank +
//                        source row), writing them expert-sorted into a local buffer.
//  * ep_scatter_add    : expert-parallel COMBINE. Expert outputs are multiplied by their routing
//                        weight and reduce-added (bf16x2 atomics over NVLink) into the source
//                        rank's output buffer at the token's row.
//  * peer_put_i32      : routing metadata exchange (plain peer stores).
// Together they replace DeepEP's dispatch / combine + host barrier of the reference
// (src/axolotl/integrations/expert_parallel/experts_fn.py:185-342).
#include "axb_common.cuh"

namespace {

__constant__ float kE2M1[16] = {0.f, 0.5f, 1.f, 1.5f, 2.f, 3.f, 4.f, 6.f,
                                -0.f, -0.5f, -1.f, -1.5f, -2.f, -3.f, -4.f, -6.f};

AXB_DEVICE float e4m3_to_float(uint8_t v) {
  const uint32_t sign = (v >> 7) & 1, exp = (v >> 3) & 0xF, man = v & 7;
  float f;
  if (exp == 0) f = ldexpf((float)man, -9);                 // subnormal: man * 2^-3 * 2^-6
  else if (exp == 15 && man == 7) f = __int_as_float(0x7fc00000);
  else f = ldexpf(1.f + man * 0.125f, (int)exp - 7);
  return sign ? -f : f;
}

// one thread per 16-element block: 8 packed bytes in, 16 bf16 out
__global__ void nvfp4_dequant_kernel(const uint8_t* __restrict__ q, const uint8_t* __restrict__ scale,
                                     const float* __restrict__ pts, __nv_bfloat16* __restrict__ out,
                                     long long n_blocks, long long blocks_per_pts) {
  for (long long b = (long long)blockIdx.x * blockDim.x + threadIdx.x; b < n_blocks;
       b += (long long)gridDim.x * blockDim.x) {
    const float s = e4m3_to_float(scale[b]) * pts[b / blocks_per_pts];
    const uint2 packed = *reinterpret_cast<const uint2*>(q + b * 8);
    const uint32_t w[2] = {packed.x, packed.y};
    uint32_t o[8];
#pragma unroll
    for (int i = 0; i < 2; ++i)
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const uint32_t byte = (w[i] >> (8 * j)) & 0xFF;
        o[i * 4 + j] = pack_bf16x2(kE2M1[byte & 0xF] * s, kE2M1[byte >> 4] * s);
      }
    uint4* dst = reinterpret_cast<uint4*>(out + b * 16);
    dst[0] = make_uint4(o[0], o[1], o[2], o[3]);
    dst[1] = make_uint4(o[4], o[5], o[6], o[7]);
  }
}

struct PeerPtrs8 {
  unsigned long long p[8];
};

// out[i, :] = src_rank(i).buffer[src_row(i), :]   (one warp per row, 16-byte vectors)
__global__ void ep_gather_rows_kernel(PeerPtrs8 src, const int* __restrict__ src_rank,
                                      const int* __restrict__ src_row, __nv_bfloat16* __restrict__ out,
                                      long long n_rows, int width, long long src_ld) {
  const long long w = ((long long)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  const long long n_warps = ((long long)gridDim.x * blockDim.x) >> 5;
  for (long long i = w; i < n_rows; i += n_warps) {
    const __nv_bfloat16* s = reinterpret_cast<const __nv_bfloat16*>(src.p[src_rank[i]]) + (long long)src_row[i] * src_ld;
    for (int c = lane * 8; c < width; c += 256)
      *reinterpret_cast<uint4*>(out + i * width + c) = *reinterpret_cast<const uint4*>(s + c);
  }
}

// dst_rank(i).buffer[dst_row(i), :] += weight(i) * rows[i, :]
__global__ void ep_scatter_add_kernel(PeerPtrs8 dst, const int* __restrict__ dst_rank,
                                      const int* __restrict__ dst_row, const float* __restrict__ weight,
                                      const __nv_bfloat16* __restrict__ rows, long long n_rows, int width,
                                      long long dst_ld) {
  const long long w = ((long long)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  const long long n_warps = ((long long)gridDim.x * blockDim.x) >> 5;
  for (long long i = w; i < n_rows; i += n_warps) {
    const float g = weight ? weight[i] : 1.f;
    __nv_bfloat16* d = reinterpret_cast<__nv_bfloat16*>(dst.p[dst_rank[i]]) + (long long)dst_row[i] * dst_ld;
    for (int c = lane * 8; c < width; c += 256) {
      const uint4 v = *reinterpret_cast<const uint4*>(rows + i * width + c);
      const uint32_t in[4] = {v.x, v.y, v.z, v.w};
      uint32_t o[4];
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const float2 f = unpack_bf16x2(in[e]);
        o[e] = pack_bf16x2(f.x * g, f.y * g);
      }
      asm volatile("red.relaxed.sys.global.add.noftz.v4.bf16x2 [%0], {%1, %2, %3, %4};" ::"l"(d + c), "r"(o[0]),
                   "r"(o[1]), "r"(o[2]), "r"(o[3])
                   : "memory");
    }
  }
}

__global__ void peer_put_i32_kernel(int* __restrict__ dst, const int* __restrict__ src, long long n) {
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x)
    dst[i] = src[i];
}

int fill8(PeerPtrs8& d, const unsigned long long* s, int world) {
  if (world < 1 || world > 8) return -2;
  for (int i = 0; i < 8; ++i) d.p[i] = i < world ? s[i] : 0ull;
  return 0;
}
}  // namespace

#define ST(s) reinterpret_cast<cudaStream_t>(s)

// q: [rows, cols/2] uint8, scale: [rows, cols/16] e4m3 bytes, pts: device fp32 scalar -> out [rows, cols] bf16
extern "C" int axb_nvfp4_dequant(const void* q, const void* scale, const float* pts, void* out, long long rows,
                                 long long cols, void* stream) {
  if (cols % 16) return -2;
  const long long nb = rows * (cols / 16);
  if (nb <= 0) return 0;
  int grid = (int)((nb + 255) / 256 > 148 * 16 ? 148 * 16 : (nb + 255) / 256);
  nvfp4_dequant_kernel<<<grid, 256, 0, ST(stream)>>>((const uint8_t*)q, (const uint8_t*)scale, pts,
                                                     (__nv_bfloat16*)out, nb, nb);
  return (int)cudaGetLastError();
}

// batch of matrices (expert stacks): q [batch, rows, cols/2], scale [batch, rows, cols/16],
// pts [batch] fp32 -> out [batch, rows, cols] bf16, one launch
extern "C" int axb_nvfp4_dequant_batched(const void* q, const void* scale, const float* pts, void* out,
                                         long long batch, long long rows, long long cols, void* stream) {
  if (cols % 16) return -2;
  const long long per = rows * (cols / 16);
  const long long nb = batch * per;
  if (nb <= 0) return 0;
  int grid = (int)((nb + 255) / 256 > 148 * 16 ? 148 * 16 : (nb + 255) / 256);
  nvfp4_dequant_kernel<<<grid, 256, 0, ST(stream)>>>((const uint8_t*)q, (const uint8_t*)scale, pts,
                                                     (__nv_bfloat16*)out, nb, per);
  return (int)cudaGetLastError();
}

extern "C" int axb_ep_gather_rows(const unsigned long long* src_ptrs, int world, const int* src_rank,
                                  const int* src_row, void* out, long long n_rows, int width, long long src_ld,
                                  void* stream) {
  if (n_rows <= 0) return 0;
  if (width % 8 || src_ld % 8) return -2;
  PeerPtrs8 p;
  if (fill8(p, src_ptrs, world)) return -2;
  int grid = (int)((n_rows + 7) / 8 > 148 * 8 ? 148 * 8 : (n_rows + 7) / 8);
  ep_gather_rows_kernel<<<grid, 256, 0, ST(stream)>>>(p, src_rank, src_row, (__nv_bfloat16*)out, n_rows, width, src_ld);
  return (int)cudaGetLastError();
}

extern "C" int axb_ep_scatter_add(const unsigned long long* dst_ptrs, int world, const int* dst_rank,
                                  const int* dst_row, const float* weight, const void* rows, long long n_rows,
                                  int width, long long dst_ld, void* stream) {
  if (n_rows <= 0) return 0;
  if (width % 8 || dst_ld % 8) return -2;
  PeerPtrs8 p;
  if (fill8(p, dst_ptrs, world)) return -2;
  int grid = (int)((n_rows + 7) / 8 > 148 * 8 ? 148 * 8 : (n_rows + 7) / 8);
  ep_scatter_add_kernel<<<grid, 256, 0, ST(stream)>>>(p, dst_rank, dst_row, weight, (const __nv_bfloat16*)rows, n_rows,
                                                      width, dst_ld);
  return (int)cudaGetLastError();
}

extern "C" int axb_peer_put_i32(void* dst, const void* src, long long n, void* stream) {
  if (n <= 0) return 0;
  int grid = (int)((n + 255) / 256 > 148 * 4 ? 148 * 4 : (n + 255) / 256);
  peer_put_i32_kernel<<<grid, 256, 0, ST(stream)>>>((int*)dst, (const int*)src, n);
  return (int)cudaGetLastError();
}
