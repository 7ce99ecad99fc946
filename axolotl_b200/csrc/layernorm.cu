// Residual-add + LayerNorm (mean-subtracting) for the architectures that use it instead of RMSNorm (Cohere, StarCoder 2,
// Nemotron, Phi, OLMo): one pass over HBM per direction.
//
//   s = x + residual (optional, written back as the new residual stream)
//   y = (s - mean(s)) * rstd(s) * (w + w_offset) + b         w, b optional (OLMo has neither; Cohere has no b)
//
// forward: one CTA per row (grid-stride); the row is read from HBM once, the second and third sweep hit L1 / L2; mean
// and rstd are kept per row for the backward pass. backward: dx = rstd * (g - mean(g) - xhat * mean(g * xhat)) with
// g = dy * (w + w_offset); the weight / bias gradients are accumulated per CTA in shared memory over the CTA's rows
// (every thread owns its columns, so no conflicts) and leave with one atomic per column per CTA.
// The reference reaches these norms through HF's modelling code (torch.nn.functional.layer_norm and hand-written
// variants such as CohereLayerNorm / NemotronLayerNorm1P).
#include "axb_common.cuh"

namespace {

constexpr int kThreads = 256;

AXB_DEVICE float block_sum(float v, float* red) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  __syncthreads();                 // red may still be read from the previous reduction
  if (lane == 0) red[warp] = v;
  __syncthreads();
  float t = lane < (kThreads >> 5) ? red[lane] : 0.f;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) t += __shfl_xor_sync(0xffffffffu, t, o);
  return t;
}

__global__ void __launch_bounds__(kThreads)
    layernorm_fwd_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ res,
                         const __nv_bfloat16* __restrict__ w, const __nv_bfloat16* __restrict__ b,
                         __nv_bfloat16* __restrict__ y, __nv_bfloat16* __restrict__ res_out, float* __restrict__ mean,
                         float* __restrict__ rstd, long long T, int D, float eps, float w_offset) {
  __shared__ float red[32];
  for (long long row = blockIdx.x; row < T; row += gridDim.x) {
    const __nv_bfloat16* xr = x + row * D;
    const __nv_bfloat16* rr = res ? res + row * D : nullptr;
    __nv_bfloat16* so = res_out ? res_out + row * D : nullptr;
    float s = 0.f;
    for (int i = threadIdx.x; i < D; i += kThreads) {
      float v = __bfloat162float(xr[i]);
      if (rr) {
        v += __bfloat162float(rr[i]);
        v = __bfloat162float(__float2bfloat16(v));       // the stream is stored in bf16: normalise what is stored
      }
      if (so) so[i] = __float2bfloat16(v);
      s += v;
    }
    const float mu = block_sum(s, red) / D;
    const __nv_bfloat16* src = so ? so : xr;              // (x + residual) as written, or x itself
    float q = 0.f;
    for (int i = threadIdx.x; i < D; i += kThreads) {
      const float d = __bfloat162float(src[i]) - mu;
      q += d * d;
    }
    const float rs = rsqrtf(block_sum(q, red) / D + eps);
    if (threadIdx.x == 0) {
      mean[row] = mu;
      rstd[row] = rs;
    }
    __nv_bfloat16* yr = y + row * D;
    for (int i = threadIdx.x; i < D; i += kThreads) {
      float v = (__bfloat162float(src[i]) - mu) * rs;
      if (w) v *= __bfloat162float(w[i]) + w_offset;
      if (b) v += __bfloat162float(b[i]);
      yr[i] = __float2bfloat16(v);
    }
  }
}

// s: the normalised input as stored (x + residual). dres: optional incoming gradient of the residual stream, added to dx.
__global__ void __launch_bounds__(kThreads)
    layernorm_bwd_kernel(const __nv_bfloat16* __restrict__ s, const __nv_bfloat16* __restrict__ dy,
                         const __nv_bfloat16* __restrict__ dres, const __nv_bfloat16* __restrict__ w,
                         const float* __restrict__ mean, const float* __restrict__ rstd, __nv_bfloat16* __restrict__ dx,
                         float* __restrict__ dw, float* __restrict__ db, long long T, int D, float w_offset) {
  extern __shared__ float acc[];          // [2][D]: weight and bias gradient partials of this CTA
  __shared__ float red[32];
  float* aw = acc;
  float* ab = acc + D;
  for (int i = threadIdx.x; i < D; i += kThreads) aw[i] = ab[i] = 0.f;
  for (long long row = blockIdx.x; row < T; row += gridDim.x) {
    const __nv_bfloat16* sr = s + row * D;
    const __nv_bfloat16* gr = dy + row * D;
    const float mu = mean[row], rs = rstd[row];
    float c1 = 0.f, c2 = 0.f;
    for (int i = threadIdx.x; i < D; i += kThreads) {
      const float xh = (__bfloat162float(sr[i]) - mu) * rs;
      const float g0 = __bfloat162float(gr[i]);
      const float g = w ? g0 * (__bfloat162float(w[i]) + w_offset) : g0;
      c1 += g;
      c2 += g * xh;
      aw[i] += g0 * xh;
      ab[i] += g0;
    }
    c1 = block_sum(c1, red) / D;
    c2 = block_sum(c2, red) / D;
    __nv_bfloat16* dxr = dx + row * D;
    const __nv_bfloat16* dr = dres ? dres + row * D : nullptr;
    for (int i = threadIdx.x; i < D; i += kThreads) {
      const float xh = (__bfloat162float(sr[i]) - mu) * rs;
      const float g0 = __bfloat162float(gr[i]);
      const float g = w ? g0 * (__bfloat162float(w[i]) + w_offset) : g0;
      float v = rs * (g - c1 - xh * c2);
      if (dr) v += __bfloat162float(dr[i]);
      dxr[i] = __float2bfloat16(v);
    }
  }
  __syncthreads();
  for (int i = threadIdx.x; i < D; i += kThreads) {
    if (dw) atomicAdd(&dw[i], aw[i]);
    if (db) atomicAdd(&db[i], ab[i]);
  }
}

int sm_count_ln() {
  static int n = 0;
  if (n == 0) {
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev);
    if (n <= 0) n = 148;
  }
  return n;
}

}  // namespace

extern "C" int axb_layernorm_fwd(const void* x, const void* res, const void* w, const void* b, void* y, void* res_out,
                                 float* mean, float* rstd, long long T, int D, float eps, float w_offset, void* stream) {
  if (T <= 0 || D <= 0) return 0;
  long long grid = T < (long long)sm_count_ln() * 8 ? T : (long long)sm_count_ln() * 8;
  layernorm_fwd_kernel<<<(unsigned)grid, kThreads, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
      static_cast<const __nv_bfloat16*>(x), static_cast<const __nv_bfloat16*>(res), static_cast<const __nv_bfloat16*>(w),
      static_cast<const __nv_bfloat16*>(b), static_cast<__nv_bfloat16*>(y), static_cast<__nv_bfloat16*>(res_out), mean,
      rstd, T, D, eps, w_offset);
  return (int)cudaGetLastError();
}

// dw / db (fp32 [D], zeroed by the caller) may be NULL when the norm has no such parameter.
extern "C" int axb_layernorm_bwd(const void* s, const void* dy, const void* dres, const void* w, const float* mean,
                                 const float* rstd, void* dx, float* dw, float* db, long long T, int D, float w_offset,
                                 void* stream) {
  if (T <= 0 || D <= 0) return 0;
  const size_t smem = 2ull * D * sizeof(float);
  if (smem > 200 * 1024) return -2;
  static size_t attr_set = 0;
  if (smem > 48 * 1024 && smem > attr_set) {
    cudaError_t e = cudaFuncSetAttribute(layernorm_bwd_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
    attr_set = smem;
  }
  long long grid = T < (long long)sm_count_ln() * 2 ? T : (long long)sm_count_ln() * 2;
  layernorm_bwd_kernel<<<(unsigned)grid, kThreads, smem, reinterpret_cast<cudaStream_t>(stream)>>>(
      static_cast<const __nv_bfloat16*>(s), static_cast<const __nv_bfloat16*>(dy), static_cast<const __nv_bfloat16*>(dres),
      static_cast<const __nv_bfloat16*>(w), mean, rstd, static_cast<__nv_bfloat16*>(dx), dw, db, T, D, w_offset);
  return (int)cudaGetLastError();
}
