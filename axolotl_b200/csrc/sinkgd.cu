// SinkGD update for sm_100a: alternating row / column normalisation of a gradient matrix
// (Sinkhorn-like sweeps) followed by an SGD step, without ever rewriting the matrix.
//
// After any number of sweeps the normalised gradient is diag(a) G diag(b), so only the two scale
// vectors change. A row half-sweep needs S_i = sum_j G_ij^2 b_j^2, a column half-sweep
// C_j = sum_i G_ij^2 a_i^2: one read of G each (from L2 for adapter-sized matrices), against the
// four full read+write passes per half-sweep of the elementwise formulation. The final kernel
// applies p <- p (1 - lr wd) - lr a_i G_ij b_j in one pass.
//
// Replaces the reference's Triton kernels (src/axolotl/utils/optimizers/sinkgd_triton.py:49-599).
#include "axb_common.cuh"

namespace {

#define ST(s) reinterpret_cast<cudaStream_t>(s)

__device__ __forceinline__ float warp_sum_f(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

// a_i <- a_i * target / (|a_i| * sqrt(S_i) + eps); one warp per row. b == nullptr means b = 1.
__global__ void __launch_bounds__(256)
    sink_row_kernel(const float* __restrict__ g, const float* __restrict__ b, float* __restrict__ a,
                    int m, int n, float target, float eps, int first) {
  const int row = blockIdx.x * 8 + (threadIdx.x >> 5);
  const int lane = threadIdx.x & 31;
  if (row >= m) return;
  const float* gr = g + (long long)row * n;
  float s = 0.f;
  if ((n & 3) == 0) {
    for (int j = lane * 4; j < n; j += 128) {
      const float4 v = *reinterpret_cast<const float4*>(gr + j);
      float4 w = make_float4(1.f, 1.f, 1.f, 1.f);
      if (b) w = *reinterpret_cast<const float4*>(b + j);
      s += v.x * v.x * w.x * w.x + v.y * v.y * w.y * w.y + v.z * v.z * w.z * w.z +
           v.w * v.w * w.w * w.w;
    }
  } else {
    for (int j = lane; j < n; j += 32) {
      const float w = b ? b[j] : 1.f;
      s += gr[j] * gr[j] * w * w;
    }
  }
  s = warp_sum_f(s);
  if (lane == 0) {
    const float prev = first ? 1.f : a[row];
    a[row] = prev * target / (fabsf(prev) * sqrtf(s) + eps);
  }
}

// b_j <- b_j * target / (|b_j| * sqrt(C_j) + eps); block = 32 columns x 8 row stripes.
__global__ void __launch_bounds__(256)
    sink_col_kernel(const float* __restrict__ g, const float* __restrict__ a, float* __restrict__ b,
                    int m, int n, float target, float eps, int first) {
  __shared__ float part[8][33];
  const int col = blockIdx.x * 32 + (threadIdx.x & 31);
  const int ry = threadIdx.x >> 5;
  float s = 0.f;
  if (col < n)
    for (int i = ry; i < m; i += 8) {
      const float v = g[(long long)i * n + col] * a[i];
      s += v * v;
    }
  part[ry][threadIdx.x & 31] = s;
  __syncthreads();
  if (ry == 0 && col < n) {
    float t = 0.f;
#pragma unroll
    for (int k = 0; k < 8; ++k) t += part[k][threadIdx.x];
    const float prev = first ? 1.f : b[col];
    b[col] = prev * target / (fabsf(prev) * sqrtf(t) + eps);
  }
}

template <typename T>
__global__ void sink_apply_kernel(T* __restrict__ p, const float* __restrict__ g,
                                  const float* __restrict__ a, const float* __restrict__ b, int m,
                                  int n, float lr, float decay) {
  const long long total = (long long)m * n;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total;
       i += (long long)gridDim.x * blockDim.x) {
    const int r = (int)(i / n), c = (int)(i % n);
    const float w = (float)p[i] * decay - lr * a[r] * g[i] * b[c];
    p[i] = (T)w;
  }
}

}  // namespace

// One SinkGD step on an [m, n] fp32 gradient. a [m] and b [n] are fp32 scratch vectors.
// p_dtype: 0 = fp32 parameter, 1 = bf16 parameter. p == nullptr only computes the scales.
extern "C" int axb_sinkgd_step(void* p, int p_dtype, const float* g, float* a, float* b, int m,
                               int n, int n_iters, float lr, float weight_decay, float eps,
                               void* stream) {
  if (m <= 0 || n <= 0 || n_iters <= 0) return -2;
  const float tr = sqrtf((float)n), tc = sqrtf((float)m);
  for (int it = 0; it < n_iters; ++it) {
    sink_row_kernel<<<(m + 7) / 8, 256, 0, ST(stream)>>>(g, it == 0 ? nullptr : b, a, m, n, tr, eps,
                                                         it == 0);
    sink_col_kernel<<<(n + 31) / 32, 256, 0, ST(stream)>>>(g, a, b, m, n, tc, eps, it == 0);
  }
  if (p) {
    const long long total = (long long)m * n;
    long long blocks = (total + 255) / 256;
    if (blocks > 148 * 16) blocks = 148 * 16;
    const float decay = 1.f - lr * weight_decay;
    if (p_dtype == 0)
      sink_apply_kernel<float><<<(unsigned)blocks, 256, 0, ST(stream)>>>((float*)p, g, a, b, m, n, lr, decay);
    else
      sink_apply_kernel<__nv_bfloat16><<<(unsigned)blocks, 256, 0, ST(stream)>>>((__nv_bfloat16*)p, g, a, b, m, n, lr, decay);
  }
  return (int)cudaGetLastError();
}
