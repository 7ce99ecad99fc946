// Decode-time expert projection: a handful of routed slots (one new token per sequence, top-k experts each), so
// every slot is a matrix-vector product against its expert's weight and the work is reading that weight once.
//   out[s, n] = sum_k W[expert[s], n, k] * x[token[s], k]
// W is bf16 [E, N, K] or NVFP4 (packed E2M1 [E, N, K/2], E4M3 block scales [E, N, K/16], fp32 scale per expert),
// decoded in registers. One warp per output row, 8 rows per block, the activation row staged in shared memory; a
// grouped tensor-core launch would pad each of these slots to a 128-row tile.
// The reference's kernel for this case: src/axolotl/integrations/kernels/libs/scattermoe_lora/kernels/single.py:13-98.
#include "axb_common.cuh"

namespace {

constexpr int GV_WARPS = 8;

__device__ __forceinline__ float gv_warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ float gv_e2m1(uint32_t code) {
  constexpr unsigned long long lo = 0x3fc03f803f000000ull, hi = 0x40c0408040404000ull;
  const unsigned long long tbl = (code & 4) ? hi : lo;
  const uint32_t bits = (uint32_t)(tbl >> ((code & 3) * 16)) & 0xFFFFu;
  return __uint_as_float((bits | ((code & 8) << 12)) << 16);
}
__device__ __forceinline__ float gv_e4m3(uint32_t v) {
  const uint32_t mag = v & 0x7Fu;
  float f = __uint_as_float(mag << 20) * 1.329227995784916e36f;   // 2^120
  f = mag == 0x7Fu ? __int_as_float(0x7fc00000) : f;
  return (v & 0x80u) ? -f : f;
}

template <bool FP4>
__global__ void __launch_bounds__(GV_WARPS * 32)
    moe_gemv_kernel(const __nv_bfloat16* __restrict__ x, const int* __restrict__ slot_token,
                    const int* __restrict__ slot_expert, const void* __restrict__ W, const uint8_t* __restrict__ scale,
                    const float* __restrict__ pts, __nv_bfloat16* __restrict__ out, int E, int N, int K) {
  extern __shared__ __nv_bfloat16 xs[];
  const int s = blockIdx.y;
  const int e = slot_expert[s];
  if (!AXB_INDEX_OK(AXB_SITE_GROUPED_EXPERT, e, E)) return;
  const __nv_bfloat16* xr = x + (long long)slot_token[s] * K;
  for (int i = threadIdx.x * 8; i < K; i += blockDim.x * 8) *reinterpret_cast<uint4*>(xs + i) = *reinterpret_cast<const uint4*>(xr + i);
  __syncthreads();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int n = blockIdx.x * GV_WARPS + warp;
  if (n >= N) return;
  float acc = 0.f;
  if (!FP4) {
    const __nv_bfloat16* w = reinterpret_cast<const __nv_bfloat16*>(W) + ((long long)e * N + n) * K;
    for (int k = lane * 8; k < K; k += 256) {
      const uint4 wv = *reinterpret_cast<const uint4*>(w + k), xv = *reinterpret_cast<const uint4*>(xs + k);
      const uint32_t wa[4] = {wv.x, wv.y, wv.z, wv.w}, xa[4] = {xv.x, xv.y, xv.z, xv.w};
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float2 a = unpack_bf16x2(wa[j]), b = unpack_bf16x2(xa[j]);
        acc += a.x * b.x + a.y * b.y;
      }
    }
  } else {
    const uint8_t* q = reinterpret_cast<const uint8_t*>(W) + ((long long)e * N + n) * (K / 2);
    const uint8_t* sc = scale + ((long long)e * N + n) * (K / 16);
    for (int k = lane * 16; k < K; k += 512) {            // one 16-value scale group per lane and step
      const uint2 pk = *reinterpret_cast<const uint2*>(q + k / 2);
      const float sv = gv_e4m3(sc[k / 16]);
      const uint32_t words[2] = {pk.x, pk.y};
      float part = 0.f;
#pragma unroll
      for (int wi = 0; wi < 2; ++wi)
#pragma unroll
        for (int j = 0; j < 8; ++j)
          part += gv_e2m1((words[wi] >> (4 * j)) & 0xF) * __bfloat162float(xs[k + wi * 8 + j]);
      acc += part * sv;
    }
    acc *= pts[e];
  }
  acc = gv_warp_sum(acc);
  if (lane == 0) out[(long long)s * N + n] = __float2bfloat16(acc);
}

}  // namespace

// x [T, K] bf16; slot_token / slot_expert [S] int32; out [S, N] bf16. fp4 = 0: W bf16 [E, N, K]; fp4 = 1: W packed
// [E, N, K/2] with scale [E, N, K/16] and pts [E]. K % 8 == 0 (bf16) or K % 16 == 0 (fp4).
extern "C" int axb_moe_gemv(const void* x, const int* slot_token, const int* slot_expert, const void* W,
                            const void* scale, const float* pts, void* out, int S, int E, int N, int K, int fp4,
                            void* stream) {
  if (S <= 0 || N <= 0) return 0;
  if ((K & 7) || (fp4 && (K & 15)) || (size_t)K * 2 > 160 * 1024) return -2;
  dim3 grid((N + GV_WARPS - 1) / GV_WARPS, S);
  const size_t smem = (size_t)K * 2;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  if (fp4) {
    static bool attr = false;
    if (!attr) {
      cudaFuncSetAttribute(moe_gemv_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, 160 * 1024);
      attr = true;
    }
    moe_gemv_kernel<true><<<grid, GV_WARPS * 32, smem, st>>>((const __nv_bfloat16*)x, slot_token, slot_expert, W,
                                                             (const uint8_t*)scale, pts, (__nv_bfloat16*)out, E, N, K);
  } else {
    static bool attr = false;
    if (!attr) {
      cudaFuncSetAttribute(moe_gemv_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, 160 * 1024);
      attr = true;
    }
    moe_gemv_kernel<false><<<grid, GV_WARPS * 32, smem, st>>>((const __nv_bfloat16*)x, slot_token, slot_expert, W,
                                                              (const uint8_t*)scale, pts, (__nv_bfloat16*)out, E, N, K);
  }
  return (int)cudaGetLastError();
}
