// Two small bandwidth-bound operators for architectures outside the Llama mould (sm_100a build like the rest).
//
// xIELU (Apertus' MLP activation, two learnable scalars per layer):
//     y = alpha_p x^2 + beta x                              for x > 0
//     y = alpha_n (expm1(min(x, eps)) - x) + beta x          otherwise
//   forward: one pass, bf16 in / bf16 out, 8 elements per thread. backward: dx plus the two sums that carry the
//   gradients of alpha_p and alpha_n (sum dy x^2 over x > 0, sum dy (expm1(min(x, eps)) - x) over x <= 0), reduced per
//   warp, per block, then one atomic pair per block. The reference patches this activation in for Apertus
//   (src/axolotl/monkeypatch/models/apertus/activation.py; HF's XIELUActivation is the definition).
//
// Gated-softmax pooling (DeepSeek-V4 compressors and indexer):
//     out[m, d] = sum_w softmax_w(gate[m, :, d]) * kv[m, w, d]
//   one thread per (m, d) walks the W window rows twice (max, then sum); neighbouring threads read neighbouring d,
//   so every access is coalesced; fp32 throughout. backward recomputes the probabilities:
//     d_kv = p * d_out,   d_gate = p * d_out * (kv - out).
//   Reference: a Triton kernel pair, src/axolotl/integrations/kernels/libs/dsv4/gated_pool.py:27-104.
//
// Hyper-connection mixer (DeepSeek-V4: every layer keeps HC = 4 residual streams and mixes them twice). Per token, 24
// numbers `mixes` (a projection of the normalised streams) become
//     pre[j]  = sigmoid(mixes[j] s0 + base[j]) + eps                    weights that collapse the streams into the layer input
//     post[j] = post_mult sigmoid(mixes[4 + j] s1 + base[4 + j])        weights that spread the layer output over the streams
//     comb    = Sinkhorn(softmax_rows(mixes[8:] s2 + base[8:]) + eps)   a (nearly) doubly stochastic 4 x 4 stream mixer:
//               column-normalise, then (iters - 1) x [row-normalise, column-normalise], each as x / (sum + eps)
//   In eager form this is ~40 launches over [tokens, 4, 4]; here one thread holds a token's 16 numbers in registers.
//   backward: the thread reruns its forward keeping only the 4 sums of every normalisation (the input of a step is its
//   output times (sum + eps), so the chain is walked back without storing the matrices), applies
//   dx = (dy - sum(dy y)) / (sum + eps) per step, then the softmax and sigmoid derivatives; the gradients of the 3 scales
//   and 24 offsets are reduced per warp and added with one atomic per warp and value.
//   Reference: a Triton kernel pair, src/axolotl/integrations/kernels/libs/dsv4/mhc.py:29-350.
#include "axb_common.cuh"

namespace {

AXB_DEVICE float xielu_neg_core(float x, float eps) { return expm1f(fminf(x, eps)) - x; }

__global__ void xielu_fwd_kernel(const __nv_bfloat16* __restrict__ x, __nv_bfloat16* __restrict__ y, long long n,
                                 float ap, float an, float beta, float eps) {
  const long long i0 = ((long long)blockIdx.x * blockDim.x + threadIdx.x) * 8;
  if (i0 >= n) return;
  if (i0 + 8 <= n) {
    const uint4 in = *reinterpret_cast<const uint4*>(x + i0);
    const uint32_t w[4] = {in.x, in.y, in.z, in.w};
    uint32_t o[4];
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      const float2 v = unpack_bf16x2(w[k]);
      const float a = v.x > 0.f ? ap * v.x * v.x + beta * v.x : an * xielu_neg_core(v.x, eps) + beta * v.x;
      const float b = v.y > 0.f ? ap * v.y * v.y + beta * v.y : an * xielu_neg_core(v.y, eps) + beta * v.y;
      o[k] = pack_bf16x2(a, b);
    }
    *reinterpret_cast<uint4*>(y + i0) = make_uint4(o[0], o[1], o[2], o[3]);
  } else {
    for (long long i = i0; i < n; ++i) {
      const float v = __bfloat162float(x[i]);
      y[i] = __float2bfloat16(v > 0.f ? ap * v * v + beta * v : an * xielu_neg_core(v, eps) + beta * v);
    }
  }
}

__global__ void xielu_bwd_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ dy,
                                 __nv_bfloat16* __restrict__ dx, float* __restrict__ sums, long long n, float ap,
                                 float an, float beta, float eps) {
  __shared__ float red[2][32];
  float sp = 0.f, sn = 0.f;
  const long long stride = (long long)gridDim.x * blockDim.x;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride) {
    const float v = __bfloat162float(x[i]);
    const float g = __bfloat162float(dy[i]);
    float d;
    if (v > 0.f) {
      d = 2.f * ap * v + beta;
      sp += g * v * v;
    } else {
      d = an * ((v < eps ? __expf(v) : 0.f) - 1.f) + beta;
      sn += g * xielu_neg_core(v, eps);
    }
    dx[i] = __float2bfloat16(g * d);
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    sp += __shfl_xor_sync(0xffffffffu, sp, o);
    sn += __shfl_xor_sync(0xffffffffu, sn, o);
  }
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (lane == 0) {
    red[0][warp] = sp;
    red[1][warp] = sn;
  }
  __syncthreads();
  if (warp == 0) {
    const int nw = blockDim.x >> 5;
    sp = lane < nw ? red[0][lane] : 0.f;
    sn = lane < nw ? red[1][lane] : 0.f;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      sp += __shfl_xor_sync(0xffffffffu, sp, o);
      sn += __shfl_xor_sync(0xffffffffu, sn, o);
    }
    if (lane == 0) {
      atomicAdd(&sums[0], sp);
      atomicAdd(&sums[1], sn);
    }
  }
}

__global__ void gated_pool_fwd_kernel(const float* __restrict__ kv, const float* __restrict__ gate,
                                      float* __restrict__ out, long long M, int W, int D) {
  const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= M * D) return;
  const long long m = idx / D;
  const int d = (int)(idx - m * D);
  const float* g = gate + m * W * D + d;
  const float* v = kv + m * W * D + d;
  float mx = -INFINITY;
  for (int w = 0; w < W; ++w) mx = fmaxf(mx, g[(long long)w * D]);
  float den = 0.f, acc = 0.f;
  for (int w = 0; w < W; ++w) {
    const float e = __expf(g[(long long)w * D] - mx);
    den += e;
    acc += e * v[(long long)w * D];
  }
  out[idx] = acc / den;
}

__global__ void gated_pool_bwd_kernel(const float* __restrict__ kv, const float* __restrict__ gate,
                                      const float* __restrict__ out, const float* __restrict__ d_out,
                                      float* __restrict__ d_kv, float* __restrict__ d_gate, long long M, int W, int D) {
  const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= M * D) return;
  const long long m = idx / D;
  const int d = (int)(idx - m * D);
  const long long base = m * W * D + d;
  float mx = -INFINITY;
  for (int w = 0; w < W; ++w) mx = fmaxf(mx, gate[base + (long long)w * D]);
  float den = 0.f;
  for (int w = 0; w < W; ++w) den += __expf(gate[base + (long long)w * D] - mx);
  const float inv = 1.f / den, o = out[idx], go = d_out[idx];
  for (int w = 0; w < W; ++w) {
    const long long j = base + (long long)w * D;
    const float p = __expf(gate[j] - mx) * inv;
    d_kv[j] = p * go;
    d_gate[j] = p * go * (kv[j] - o);
  }
}

}  // namespace

namespace {

constexpr int MHC = 4;           // streams
constexpr int MHC_MAX_ITERS = 32;

AXB_DEVICE float sigmoidf_(float x) { return 1.f / (1.f + __expf(-x)); }

AXB_DEVICE float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

// one normalisation of c along rows (axis_col = false: every row sums to ~1) or columns; returns the 4 sums
AXB_DEVICE void mhc_normalise(float (&c)[MHC][MHC], bool cols, float eps, float (&sums)[MHC]) {
#pragma unroll
  for (int a = 0; a < MHC; ++a) {
    float t = 0.f;
#pragma unroll
    for (int b = 0; b < MHC; ++b) t += cols ? c[b][a] : c[a][b];
    sums[a] = t;
    const float inv = 1.f / (t + eps);
#pragma unroll
    for (int b = 0; b < MHC; ++b) {
      if (cols) c[b][a] *= inv; else c[a][b] *= inv;
    }
  }
}

AXB_DEVICE void mhc_softmax_rows(const float* __restrict__ mix, const float* __restrict__ base, float s2, float eps,
                                 float (&c)[MHC][MHC]) {
#pragma unroll
  for (int i = 0; i < MHC; ++i) {
    float mx = -INFINITY;
#pragma unroll
    for (int j = 0; j < MHC; ++j) {
      c[i][j] = mix[2 * MHC + i * MHC + j] * s2 + base[2 * MHC + i * MHC + j];
      mx = fmaxf(mx, c[i][j]);
    }
    float t = 0.f;
#pragma unroll
    for (int j = 0; j < MHC; ++j) { c[i][j] = __expf(c[i][j] - mx); t += c[i][j]; }
#pragma unroll
    for (int j = 0; j < MHC; ++j) c[i][j] = c[i][j] / t + eps;
  }
}

__global__ void mhc_mix_fwd_kernel(const float* __restrict__ mixes, const float* __restrict__ scale,
                                   const float* __restrict__ base, float* __restrict__ pre, float* __restrict__ post,
                                   float* __restrict__ comb, long long M, int iters, float eps, float post_mult) {
  const long long m = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (m >= M) return;
  const float* mix = mixes + m * (MHC * (2 + MHC));
  const float s0 = scale[0], s1 = scale[1], s2 = scale[2];
#pragma unroll
  for (int j = 0; j < MHC; ++j) {
    pre[m * MHC + j] = sigmoidf_(mix[j] * s0 + base[j]) + eps;
    post[m * MHC + j] = post_mult * sigmoidf_(mix[MHC + j] * s1 + base[MHC + j]);
  }
  float c[MHC][MHC], sums[MHC];
  mhc_softmax_rows(mix, base, s2, eps, c);
  mhc_normalise(c, true, eps, sums);
  for (int it = 1; it < iters; ++it) {
    mhc_normalise(c, false, eps, sums);
    mhc_normalise(c, true, eps, sums);
  }
#pragma unroll
  for (int i = 0; i < MHC; ++i)
#pragma unroll
    for (int j = 0; j < MHC; ++j) comb[m * MHC * MHC + i * MHC + j] = c[i][j];
}

// dx = (dy - sum(dy y)) / (sum + eps) along the normalised axis; y becomes the step's input x = y (sum + eps)
AXB_DEVICE void mhc_normalise_bwd(float (&y)[MHC][MHC], float (&g)[MHC][MHC], bool cols, float eps, const float* sums) {
#pragma unroll
  for (int a = 0; a < MHC; ++a) {
    float dot = 0.f;
#pragma unroll
    for (int b = 0; b < MHC; ++b) dot += cols ? g[b][a] * y[b][a] : g[a][b] * y[a][b];
    const float den = sums[a] + eps, inv = 1.f / den;
#pragma unroll
    for (int b = 0; b < MHC; ++b) {
      if (cols) { g[b][a] = (g[b][a] - dot) * inv; y[b][a] *= den; }
      else      { g[a][b] = (g[a][b] - dot) * inv; y[a][b] *= den; }
    }
  }
}

__global__ void mhc_mix_bwd_kernel(const float* __restrict__ mixes, const float* __restrict__ scale,
                                   const float* __restrict__ base, const float* __restrict__ d_pre,
                                   const float* __restrict__ d_post, const float* __restrict__ d_comb,
                                   float* __restrict__ d_mixes, float* __restrict__ d_scale, float* __restrict__ d_base,
                                   long long M, int iters, float eps, float post_mult) {
  const long long m = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  constexpr int N = MHC * (2 + MHC);
  float dm[N];            // d_mixes of this row before the scale factor, i.e. the gradient of (mix s + base) = d_base part
  float ds[3] = {0.f, 0.f, 0.f};
#pragma unroll
  for (int k = 0; k < N; ++k) dm[k] = 0.f;
  if (m < M) {
    const float* mix = mixes + m * N;
    const float s0 = scale[0], s1 = scale[1], s2 = scale[2];
#pragma unroll
    for (int j = 0; j < MHC; ++j) {
      const float a = sigmoidf_(mix[j] * s0 + base[j]);
      dm[j] = d_pre[m * MHC + j] * a * (1.f - a);
      const float b = sigmoidf_(mix[MHC + j] * s1 + base[MHC + j]);
      dm[MHC + j] = d_post[m * MHC + j] * post_mult * b * (1.f - b);
      ds[0] += dm[j] * mix[j];
      ds[1] += dm[MHC + j] * mix[MHC + j];
    }
    float c[MHC][MHC], g[MHC][MHC];
    float sums[2 * MHC_MAX_ITERS][MHC];
    mhc_softmax_rows(mix, base, s2, eps, c);
    int t = 0;
    mhc_normalise(c, true, eps, sums[t++]);
    for (int it = 1; it < iters; ++it) {
      mhc_normalise(c, false, eps, sums[t++]);
      mhc_normalise(c, true, eps, sums[t++]);
    }
#pragma unroll
    for (int i = 0; i < MHC; ++i)
#pragma unroll
      for (int j = 0; j < MHC; ++j) g[i][j] = d_comb[m * MHC * MHC + i * MHC + j];
    for (int it = iters - 1; it >= 1; --it) {
      mhc_normalise_bwd(c, g, true, eps, sums[--t]);
      mhc_normalise_bwd(c, g, false, eps, sums[--t]);
    }
    mhc_normalise_bwd(c, g, true, eps, sums[--t]);
    // c is now softmax + eps, g its gradient: d_logit = p (g - sum_j g p) per row
#pragma unroll
    for (int i = 0; i < MHC; ++i) {
      float dot = 0.f;
#pragma unroll
      for (int j = 0; j < MHC; ++j) dot += g[i][j] * (c[i][j] - eps);
#pragma unroll
      for (int j = 0; j < MHC; ++j) {
        const float dl = (c[i][j] - eps) * (g[i][j] - dot);
        dm[2 * MHC + i * MHC + j] = dl;
        ds[2] += dl * mix[2 * MHC + i * MHC + j];
      }
    }
#pragma unroll
    for (int k = 0; k < N; ++k) d_mixes[m * N + k] = dm[k] * (k < MHC ? s0 : (k < 2 * MHC ? s1 : s2));
  }
  // parameter gradients: per-warp sums, one atomic per warp and value (rows past M contribute zeros)
#pragma unroll
  for (int k = 0; k < N; ++k) {
    const float v = warp_sum(dm[k]);
    if ((threadIdx.x & 31) == 0 && v != 0.f) atomicAdd(d_base + k, v);
  }
#pragma unroll
  for (int k = 0; k < 3; ++k) {
    const float v = warp_sum(ds[k]);
    if ((threadIdx.x & 31) == 0 && v != 0.f) atomicAdd(d_scale + k, v);
  }
}

}  // namespace

extern "C" int axb_mhc_mix_fwd(const float* mixes, const float* scale, const float* base, float* pre, float* post,
                               float* comb, long long M, int hc, int iters, float eps, float post_mult, void* stream) {
  if (hc != MHC || iters < 1 || iters > MHC_MAX_ITERS) return -2;
  if (M <= 0) return 0;
  mhc_mix_fwd_kernel<<<(unsigned)((M + 127) / 128), 128, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
      mixes, scale, base, pre, post, comb, M, iters, eps, post_mult);
  return (int)cudaGetLastError();
}

// d_scale [3] and d_base [24] must be zeroed by the caller (they are accumulated with atomics).
extern "C" int axb_mhc_mix_bwd(const float* mixes, const float* scale, const float* base, const float* d_pre,
                               const float* d_post, const float* d_comb, float* d_mixes, float* d_scale, float* d_base,
                               long long M, int hc, int iters, float eps, float post_mult, void* stream) {
  if (hc != MHC || iters < 1 || iters > MHC_MAX_ITERS) return -2;
  if (M <= 0) return 0;
  mhc_mix_bwd_kernel<<<(unsigned)((M + 127) / 128), 128, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
      mixes, scale, base, d_pre, d_post, d_comb, d_mixes, d_scale, d_base, M, iters, eps, post_mult);
  return (int)cudaGetLastError();
}

extern "C" int axb_xielu_fwd(const void* x, void* y, long long n, float ap, float an, float beta, float eps,
                             void* stream) {
  if (n <= 0) return 0;
  const int threads = 256;
  const long long blocks = (n + threads * 8 - 1) / (threads * 8);
  xielu_fwd_kernel<<<(unsigned)blocks, threads, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
      static_cast<const __nv_bfloat16*>(x), static_cast<__nv_bfloat16*>(y), n, ap, an, beta, eps);
  return (int)cudaGetLastError();
}

// sums[0] += sum dy x^2 over x > 0, sums[1] += sum dy (expm1(min(x, eps)) - x) over x <= 0 (the caller zeroes them)
extern "C" int axb_xielu_bwd(const void* x, const void* dy, void* dx, float* sums, long long n, float ap, float an,
                             float beta, float eps, void* stream) {
  if (n <= 0) return 0;
  const int threads = 256;
  long long blocks = (n + threads * 8 - 1) / (threads * 8);
  if (blocks > 148 * 8) blocks = 148 * 8;
  xielu_bwd_kernel<<<(unsigned)blocks, threads, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
      static_cast<const __nv_bfloat16*>(x), static_cast<const __nv_bfloat16*>(dy), static_cast<__nv_bfloat16*>(dx),
      sums, n, ap, an, beta, eps);
  return (int)cudaGetLastError();
}

extern "C" int axb_gated_pool_fwd(const float* kv, const float* gate, float* out, long long M, int W, int D,
                                  void* stream) {
  if (M <= 0 || W <= 0 || D <= 0) return 0;
  const long long n = M * D;
  gated_pool_fwd_kernel<<<(unsigned)((n + 255) / 256), 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>(kv, gate, out, M, W, D);
  return (int)cudaGetLastError();
}

extern "C" int axb_gated_pool_bwd(const float* kv, const float* gate, const float* out, const float* d_out,
                                  float* d_kv, float* d_gate, long long M, int W, int D, void* stream) {
  if (M <= 0 || W <= 0 || D <= 0) return 0;
  const long long n = M * D;
  gated_pool_bwd_kernel<<<(unsigned)((n + 255) / 256), 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
      kv, gate, out, d_out, d_kv, d_gate, M, W, D);
  return (int)cudaGetLastError();
}
