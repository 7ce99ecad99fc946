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
