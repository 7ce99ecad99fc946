// Feature-matching rewards of energy-based fine-tuning, one launch for a whole batch of prompt groups:
//   align[p, i] = 2 cos(g_pi, t_p)              div[p, i] = 2 / (n - 1) * sum_{j != i} <g_pi, g_pj>
// with g the embeddings of the n sampled completions of prompt p and t the embedding of its ground truth.
// `normalize` = 1 rates unit vectors (g / |g|), 0 takes the dot products as they are (whitened features).
// One block per prompt group: norms (one warp per row), the group's sum vector in shared memory, then one
// dot product per row against the sum and one against the ground truth: every embedding is read twice and no
// [n, n] similarity matrix or normalised copy is written. The reference's Triton kernels for these two
// quantities: src/axolotl/core/trainers/ebft/kernels.py:188-336.
#include "axb_common.cuh"

namespace {

constexpr int EB_T = 256;

__device__ __forceinline__ float warp_sum_f(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

__global__ void __launch_bounds__(EB_T)
    ebft_rewards_kernel(const float* __restrict__ gen, const float* __restrict__ gt, float* __restrict__ align,
                        float* __restrict__ div, int n, int D, int normalize) {
  extern __shared__ float sm[];
  float* s = sm;                // [D] sum of the (normalised) rows of the group
  float* inv = sm + D;          // [n] 1 / |g_i| (1 when not normalising); inv[n] = 1 / |t|
  float* sq = inv + n + 1;      // [n] |g_i|^2 in the units of the dot products
  const int p = blockIdx.x, warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nw = EB_T / 32;
  const float* g = gen + (long long)p * n * D;
  const float* t = gt + (long long)p * D;
  for (int i = warp; i <= n; i += nw) {
    const float* row = i < n ? g + (long long)i * D : t;
    float ss = 0.f;
    for (int d = lane; d < D; d += 32) ss += row[d] * row[d];
    ss = warp_sum_f(ss);
    if (lane == 0) {
      const float r = rsqrtf(fmaxf(ss, 1e-24f));
      inv[i] = (normalize || i == n) ? r : 1.f;
      if (i < n) sq[i] = normalize ? ss * r * r : ss;
      if (i == n) inv[n] = r;
    }
  }
  __syncthreads();
  for (int d = threadIdx.x; d < D; d += EB_T) {
    float acc = 0.f;
    for (int j = 0; j < n; ++j) acc += g[(long long)j * D + d] * inv[j];
    s[d] = acc;
  }
  __syncthreads();
  for (int i = warp; i < n; i += nw) {
    const float* row = g + (long long)i * D;
    float ds = 0.f, dt = 0.f, nn = 0.f;
    for (int d = lane; d < D; d += 32) {
      const float v = row[d];
      ds += v * s[d];
      dt += v * t[d];
      nn += v * v;
    }
    ds = warp_sum_f(ds);
    dt = warp_sum_f(dt);
    nn = warp_sum_f(nn);
    if (lane == 0) {
      const float cosv = dt * rsqrtf(fmaxf(nn, 1e-24f)) * inv[n];
      align[(long long)p * n + i] = 2.f * cosv;
      div[(long long)p * n + i] = n > 1 ? 2.f * (ds * inv[i] - sq[i]) / (float)(n - 1) : 0.f;
    }
  }
}

}  // namespace

// gen [P, n, D] fp32, gt [P, D] fp32 -> align [P * n], div [P * n] fp32. (D + 2 n + 1) floats of shared memory per block.
extern "C" int axb_ebft_rewards(const float* gen, const float* gt, float* align, float* div, int P, int n, int D,
                                int normalize, void* stream) {
  if (P <= 0 || n <= 0 || D <= 0) return 0;
  const size_t smem = sizeof(float) * ((size_t)D + 2 * (size_t)n + 1);
  if (smem > 200 * 1024) return -2;
  static bool attr = false;
  if (!attr) {
    cudaError_t e = cudaFuncSetAttribute(ebft_rewards_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
    if (e != cudaSuccess) return (int)e;
    attr = true;
  }
  ebft_rewards_kernel<<<P, EB_T, smem, reinterpret_cast<cudaStream_t>(stream)>>>(gen, gt, align, div, n, D, normalize);
  return (int)cudaGetLastError();
}
