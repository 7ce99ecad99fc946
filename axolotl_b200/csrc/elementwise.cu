// Memory-bound fused ops for sm_100a: RMSNorm (+residual add) fwd/bwd, RoPE (+optional per-head
// q/k RMSNorm for Qwen3) fwd/bwd, SwiGLU / GeGLU fwd/bwd, embedding gather / scatter-add,
// in-place cross-entropy fwd+bwd over a logits chunk, fused multi-tensor AdamW with global-norm
// clipping. All kernels move 16-byte vectors and keep statistics in fp32.
//
// These replace the reference's Triton kernels (src/axolotl/kernels/swiglu.py, geglu.py,
// gemma4_fused_rope.py), the HF eager RMSNorm / rotary chains and torch's fused AdamW.
#include "axb_common.cuh"

namespace {

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}
template <int NT>
__device__ __forceinline__ float block_sum(float v, float* sh) {
  v = warp_sum(v);
  const int w = threadIdx.x >> 5, l = threadIdx.x & 31;
  __syncthreads();
  if (l == 0) sh[w] = v;
  __syncthreads();
  float r = (threadIdx.x < NT / 32) ? sh[threadIdx.x] : 0.f;
  if (w == 0) {
    r = warp_sum(r);
    if (l == 0) sh[0] = r;
  }
  __syncthreads();
  return sh[0];
}
template <int NT>
__device__ __forceinline__ float block_max(float v, float* sh) {
  v = warp_max(v);
  const int w = threadIdx.x >> 5, l = threadIdx.x & 31;
  __syncthreads();
  if (l == 0) sh[w] = v;
  __syncthreads();
  float r = (threadIdx.x < NT / 32) ? sh[threadIdx.x] : -INFINITY;
  if (w == 0) {
    r = warp_max(r);
    if (l == 0) sh[0] = r;
  }
  __syncthreads();
  return sh[0];
}

struct bf16x8 {
  uint4 u;
};
__device__ __forceinline__ void load8(const __nv_bfloat16* p, float (&f)[8]) {
  uint4 u = *reinterpret_cast<const uint4*>(p);
  float2 a = unpack_bf16x2(u.x), b = unpack_bf16x2(u.y), c = unpack_bf16x2(u.z),
         d = unpack_bf16x2(u.w);
  f[0] = a.x; f[1] = a.y; f[2] = b.x; f[3] = b.y; f[4] = c.x; f[5] = c.y; f[6] = d.x; f[7] = d.y;
}
__device__ __forceinline__ void store8(__nv_bfloat16* p, const float (&f)[8]) {
  uint4 u;
  u.x = pack_bf16x2(f[0], f[1]);
  u.y = pack_bf16x2(f[2], f[3]);
  u.z = pack_bf16x2(f[4], f[5]);
  u.w = pack_bf16x2(f[6], f[7]);
  *reinterpret_cast<uint4*>(p) = u;
}

// ---------------------------------------------------------------------------------- RMSNorm
// h = x (+ res);  res_out = h (optional);  y = h * rstd * (w + w_offset)
constexpr int NORM_T = 256;
__global__ void __launch_bounds__(NORM_T)
    rmsnorm_fwd_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ res,
                       const __nv_bfloat16* __restrict__ w, __nv_bfloat16* __restrict__ y,
                       __nv_bfloat16* __restrict__ res_out, float* __restrict__ rstd_out, int H,
                       float eps, float w_offset) {
  __shared__ float sh[32];
  const long long row = blockIdx.x;
  const __nv_bfloat16* xr = x + row * H;
  const __nv_bfloat16* rr = res ? res + row * H : nullptr;
  float ss = 0.f;
  // H <= 8 * NORM_T * 4 supported by keeping up to 4 vectors per thread in registers
  float cache[4][8];
  int nv = 0;
  for (int i = threadIdx.x * 8; i < H; i += NORM_T * 8, ++nv) {
    float f[8];
    load8(xr + i, f);
    if (rr) {
      float g[8];
      load8(rr + i, g);
#pragma unroll
      for (int j = 0; j < 8; ++j) f[j] += g[j];
    }
    if (res_out) {
      // round the residual stream to bf16 first so forward and backward see the same h (in
      // registers: a store followed by a load of the same address would wait for a trip to L2)
      uint4 u;
      u.x = pack_bf16x2(f[0], f[1]);
      u.y = pack_bf16x2(f[2], f[3]);
      u.z = pack_bf16x2(f[4], f[5]);
      u.w = pack_bf16x2(f[6], f[7]);
      *reinterpret_cast<uint4*>(res_out + row * H + i) = u;
      const float2 a = unpack_bf16x2(u.x), b = unpack_bf16x2(u.y), c = unpack_bf16x2(u.z), d = unpack_bf16x2(u.w);
      f[0] = a.x; f[1] = a.y; f[2] = b.x; f[3] = b.y; f[4] = c.x; f[5] = c.y; f[6] = d.x; f[7] = d.y;
    }
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      ss += f[j] * f[j];
      if (nv < 4) cache[nv][j] = f[j];
    }
  }
  ss = block_sum<NORM_T>(ss, sh);
  const float rstd = rsqrtf(ss / H + eps);
  if (threadIdx.x == 0 && rstd_out) rstd_out[row] = rstd;
  int k = 0;
  for (int i = threadIdx.x * 8; i < H; i += NORM_T * 8, ++k) {
    float f[8], wv[8];
    if (k < 4) {
#pragma unroll
      for (int j = 0; j < 8; ++j) f[j] = cache[k][j];
    } else {
      load8((res_out ? res_out + row * H : xr) + i, f);
    }
    load8(w + i, wv);
#pragma unroll
    for (int j = 0; j < 8; ++j) f[j] = f[j] * rstd * (wv[j] + w_offset);
    store8(y + row * H + i, f);
  }
}

// dx = rstd * (dy*w - xhat * mean(dy*w*xhat)) (+ dres). Each thread owns fixed columns, so the
// weight gradient is accumulated in registers over the rows of the block and flushed once.
__global__ void __launch_bounds__(NORM_T)
    rmsnorm_bwd_kernel(const __nv_bfloat16* __restrict__ dy, const __nv_bfloat16* __restrict__ h,
                       const __nv_bfloat16* __restrict__ w, const float* __restrict__ rstd_in,
                       const __nv_bfloat16* __restrict__ dres, __nv_bfloat16* __restrict__ dx,
                       float* __restrict__ dw, int H, int rows, float w_offset) {
  __shared__ float sh[32];
  float dw_acc[4][8];
#pragma unroll
  for (int a = 0; a < 4; ++a)
#pragma unroll
    for (int j = 0; j < 8; ++j) dw_acc[a][j] = 0.f;
  for (long long row = blockIdx.x; row < rows; row += gridDim.x) {
    const float rstd = rstd_in[row];
    float dot = 0.f;
    for (int i = threadIdx.x * 8; i < H; i += NORM_T * 8) {
      float a[8], b[8], c[8];
      load8(dy + row * H + i, a);
      load8(h + row * H + i, b);
      load8(w + i, c);
#pragma unroll
      for (int j = 0; j < 8; ++j) dot += a[j] * (c[j] + w_offset) * b[j] * rstd;
    }
    dot = block_sum<NORM_T>(dot, sh) / H;
    int k = 0;
    for (int i = threadIdx.x * 8; i < H; i += NORM_T * 8, ++k) {
      float a[8], b[8], c[8], o[8];
      load8(dy + row * H + i, a);
      load8(h + row * H + i, b);
      load8(w + i, c);
      if (dres) load8(dres + row * H + i, o);
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const float xhat = b[j] * rstd;
        const float g = rstd * (a[j] * (c[j] + w_offset) - xhat * dot);
        if (dw) {
          if (k < 4) dw_acc[k][j] += a[j] * xhat;
          else atomicAdd(dw + i + j, a[j] * xhat);
        }
        o[j] = dres ? o[j] + g : g;
      }
      store8(dx + row * H + i, o);
    }
  }
  if (dw) {
    int k = 0;
    for (int i = threadIdx.x * 8; i < H && k < 4; i += NORM_T * 8, ++k)
#pragma unroll
      for (int j = 0; j < 8; ++j) atomicAdd(dw + i + j, dw_acc[k][j]);
  }
}

// ---------------------------------------------------------------------------------- RoPE
// Rotates the q and k heads of a fused [T, (Hq + 2*Hk) * D] projection in place (rotate-half
// convention: out = x*cos + rotate_half(x)*sin, angles = pos * inv_freq[i], i < D/2).
// With norm weights given, a per-head RMSNorm over D is applied first (Qwen3 q_norm / k_norm),
// and the per-head rstd is saved for the backward pass. sign = -1 gives the inverse rotation.
__global__ void rope_qk_kernel(__nv_bfloat16* __restrict__ qkv, const int* __restrict__ pos,
                               const float* __restrict__ inv_freq, int T, int Hq, int Hk, int D,
                               long long row_stride, float sign, float attn_scale,
                               const __nv_bfloat16* __restrict__ qn_w,
                               const __nv_bfloat16* __restrict__ kn_w, float* __restrict__ rstd_out,
                               float eps) {
  // one warp per (token, head); lane handles pairs (i, i + D/2)
  const int warps_per_block = blockDim.x >> 5;
  const long long gw = (long long)blockIdx.x * warps_per_block + (threadIdx.x >> 5);
  const int lane = threadIdx.x & 31;
  const int nh = Hq + Hk;
  if (gw >= (long long)T * nh) return;
  const int t = (int)(gw / nh);
  const int hd = (int)(gw % nh);
  __nv_bfloat16* p = qkv + (long long)t * row_stride + (long long)hd * D;
  const float ps = (float)pos[t];
  const int half = D >> 1;
  const __nv_bfloat16* nw = (hd < Hq) ? qn_w : kn_w;
  float rstd = 1.f;
  if (nw) {
    float ss = 0.f;
    for (int i = lane; i < D; i += 32) {
      float v = __bfloat162float(p[i]);
      ss += v * v;
    }
    ss = warp_sum(ss);
    rstd = rsqrtf(ss / D + eps);
    if (lane == 0 && rstd_out) rstd_out[gw] = rstd;
  }
  for (int i = lane; i < half; i += 32) {
    float s, c;
    sincosf(ps * inv_freq[i], &s, &c);
    s *= sign * attn_scale;
    c *= attn_scale;
    float a = __bfloat162float(p[i]);
    float b = __bfloat162float(p[i + half]);
    if (nw) {
      a = __bfloat162float(__float2bfloat16(a * rstd * __bfloat162float(nw[i])));
      b = __bfloat162float(__float2bfloat16(b * rstd * __bfloat162float(nw[i + half])));
    }
    p[i] = __float2bfloat16(a * c - b * s);
    p[i + half] = __float2bfloat16(b * c + a * s);
  }
}

// Fast path without q/k norm: one warp per token. Each lane computes the sine / cosine of its two
// angles ONCE and reuses them for every q and k head of the token (the angles depend on the position
// only), and moves bf16 pairs (4-byte accesses, 128 B per warp instruction). sign = -1 is the
// inverse rotation, i.e. the backward pass.
// `rot` <= D: only the first `rot` dimensions of a head rotate (partial rotary embeddings: pairs (j, j + rot / 2));
// the rest of the head passes through untouched.
__global__ void rope_fast_kernel(__nv_bfloat16* __restrict__ qkv, const int* __restrict__ pos,
                                 const float* __restrict__ inv_freq, int T, int nh, int D,
                                 long long row_stride, float sign, float attn_scale, int rot) {
  const int warps_per_block = blockDim.x >> 5;
  const long long t = (long long)blockIdx.x * warps_per_block + (threadIdx.x >> 5);
  const int lane = threadIdx.x & 31;
  if (t >= T) return;
  const int half = rot >> 1;
  const float ps = (float)pos[t];
  __nv_bfloat16* row = qkv + t * row_stride;
  for (int j = 2 * lane; j < half; j += 64) {
    float s0, c0, s1, c1;
    sincosf(ps * inv_freq[j], &s0, &c0);
    sincosf(ps * inv_freq[j + 1], &s1, &c1);
    s0 *= sign * attn_scale;
    s1 *= sign * attn_scale;
    c0 *= attn_scale;
    c1 *= attn_scale;
#pragma unroll 4
    for (int hd = 0; hd < nh; ++hd) {
      uint32_t* pa = reinterpret_cast<uint32_t*>(row + (long long)hd * D + j);
      uint32_t* pb = reinterpret_cast<uint32_t*>(row + (long long)hd * D + half + j);
      const float2 a = unpack_bf16x2(*pa), b = unpack_bf16x2(*pb);
      *pa = pack_bf16x2(a.x * c0 - b.x * s0, a.y * c1 - b.y * s1);
      *pb = pack_bf16x2(b.x * c0 + a.x * s0, b.y * c1 + a.y * s1);
    }
  }
}

// Backward of (per-head RMSNorm ->) RoPE for the fused q/k gradient buffer, in place.
// x_pre holds the pre-norm projection (needed only when norm weights are given).
// NMAX: rotation pairs a lane keeps in registers (D <= 64 * NMAX).
template <int NMAX>
__global__ void rope_qk_bwd_kernel(__nv_bfloat16* __restrict__ dqkv,
                                   const __nv_bfloat16* __restrict__ x_pre,
                                   const int* __restrict__ pos, const float* __restrict__ inv_freq,
                                   int T, int Hq, int Hk, int D, long long row_stride,
                                   long long x_row_stride, float attn_scale,
                                   const __nv_bfloat16* __restrict__ qn_w,
                                   const __nv_bfloat16* __restrict__ kn_w,
                                   const float* __restrict__ rstd_in, float* __restrict__ dqn_w,
                                   float* __restrict__ dkn_w) {
  const int warps_per_block = blockDim.x >> 5;
  const long long gw = (long long)blockIdx.x * warps_per_block + (threadIdx.x >> 5);
  const int lane = threadIdx.x & 31;
  const int nh = Hq + Hk;
  if (gw >= (long long)T * nh) return;
  const int t = (int)(gw / nh);
  const int hd = (int)(gw % nh);
  __nv_bfloat16* g = dqkv + (long long)t * row_stride + (long long)hd * D;
  const float ps = (float)pos[t];
  const int half = D >> 1;
  const __nv_bfloat16* nw = (hd < Hq) ? qn_w : kn_w;
  float* dnw = (hd < Hq) ? dqn_w : dkn_w;
  // inverse rotation first
  float ga[NMAX], gb[NMAX];
  int n = 0;
  for (int i = lane; i < half; i += 32, ++n) {
    float s, c;
    sincosf(ps * inv_freq[i], &s, &c);
    s *= attn_scale;
    c *= attn_scale;
    const float a = __bfloat162float(g[i]);
    const float b = __bfloat162float(g[i + half]);
    ga[n] = a * c + b * s;
    gb[n] = b * c - a * s;
  }
  if (!nw) {
    n = 0;
    for (int i = lane; i < half; i += 32, ++n) {
      g[i] = __float2bfloat16(ga[n]);
      g[i + half] = __float2bfloat16(gb[n]);
    }
    return;
  }
  const __nv_bfloat16* x = x_pre + (long long)t * x_row_stride + (long long)hd * D;
  const float rstd = rstd_in[gw];
  float dot = 0.f;
  n = 0;
  for (int i = lane; i < half; i += 32, ++n) {
    const float xa = __bfloat162float(x[i]) * rstd, xb = __bfloat162float(x[i + half]) * rstd;
    const float wa = __bfloat162float(nw[i]), wb = __bfloat162float(nw[i + half]);
    dot += ga[n] * wa * xa + gb[n] * wb * xb;
    if (dnw) {
      atomicAdd(dnw + i, ga[n] * xa);
      atomicAdd(dnw + i + half, gb[n] * xb);
    }
  }
  dot = warp_sum(dot) / D;
  n = 0;
  for (int i = lane; i < half; i += 32, ++n) {
    const float xa = __bfloat162float(x[i]) * rstd, xb = __bfloat162float(x[i + half]) * rstd;
    const float wa = __bfloat162float(nw[i]), wb = __bfloat162float(nw[i + half]);
    g[i] = __float2bfloat16(rstd * (ga[n] * wa - xa * dot));
    g[i + half] = __float2bfloat16(rstd * (gb[n] * wb - xb * dot));
  }
}

// ---------------------------------------------------------------------------------- GLU
// Special-function-unit forms (ex2 / rcp / tanh approximations, a couple of ulp: far below the bf16
// rounding of the results); an IEEE division per element would make these kernels instruction-bound.
__device__ __forceinline__ float tanh_fast(float x) {
  float y;
  asm("tanh.approx.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
__device__ __forceinline__ float sigmoid_fast(float g) { return __fdividef(1.f, 1.f + __expf(-g)); }
// kind 0: silu, 1: gelu (tanh form), 2: g * sigmoid(1.702 g), whose GLU multiplies by (up + 1) (gpt-oss experts)
__device__ __forceinline__ float act_fwd(float g, int kind) {
  if (kind == 0) return g * sigmoid_fast(g);  // silu
  if (kind == 2) return g * sigmoid_fast(1.702f * g);
  const float k0 = 0.7978845608028654f, k1 = 0.044715f;  // gelu tanh
  const float t = tanh_fast(k0 * (g + k1 * g * g * g));
  return 0.5f * g * (1.f + t);
}
__device__ __forceinline__ float act_bwd(float g, int kind) {
  if (kind == 0) {
    const float s = sigmoid_fast(g);
    return s * (1.f + g * (1.f - s));
  }
  if (kind == 2) {
    const float s = sigmoid_fast(1.702f * g);
    return s * (1.f + 1.702f * g * (1.f - s));
  }
  const float k0 = 0.7978845608028654f, k1 = 0.044715f;
  const float t = tanh_fast(k0 * (g + k1 * g * g * g));
  return 0.5f * (1.f + t) + 0.5f * g * (1.f - t * t) * k0 * (1.f + 3.f * k1 * g * g);
}
// gu: [T, 2I] (gate | up);  h: [T, I] = act(gate) * up. With limit > 0 (clamped SwiGLU of the
// DeepSeek-V4 / gpt-oss experts): act(min(gate, limit)) * clamp(up, -limit, limit), and the
// gradients vanish where the clamp is active.
// `blocks_in_use` (optional, device): only the first *blocks_in_use * 128 rows are processed: the padded expert layout
// of a capacity-bounded plan uses a data-dependent prefix of its row buffer and nothing reads the rest.
__global__ void glu_fwd_kernel(const __nv_bfloat16* __restrict__ gu, __nv_bfloat16* __restrict__ h,
                               long long T, int I, int kind, float limit, const int* __restrict__ blocks_in_use) {
  if (blocks_in_use) T = min(T, (long long)(*blocks_in_use) * 128);
  const long long nvec = T * (I / 8);
  for (long long v = (long long)blockIdx.x * blockDim.x + threadIdx.x; v < nvec;
       v += (long long)gridDim.x * blockDim.x) {
    const long long t = v / (I / 8);
    const int c = (int)(v % (I / 8)) * 8;
    float g[8], u[8], o[8];
    load8(gu + t * 2 * I + c, g);
    load8(gu + t * 2 * I + I + c, u);
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const float gc = limit > 0.f ? fminf(g[j], limit) : g[j];
      const float uc = limit > 0.f ? fminf(fmaxf(u[j], -limit), limit) : u[j];
      o[j] = act_fwd(gc, kind) * (kind == 2 ? uc + 1.f : uc);
    }
    store8(h + t * I + c, o);
  }
}
// dgu[T,2I]: d_gate = dh * up * act'(gate), d_up = dh * act(gate). dgu may alias gu.
__global__ void glu_bwd_kernel(const __nv_bfloat16* __restrict__ dh,
                               const __nv_bfloat16* __restrict__ gu,
                               __nv_bfloat16* __restrict__ dgu, long long T, int I, int kind,
                               float limit, const int* __restrict__ blocks_in_use) {
  if (blocks_in_use) T = min(T, (long long)(*blocks_in_use) * 128);
  const long long nvec = T * (I / 8);
  for (long long v = (long long)blockIdx.x * blockDim.x + threadIdx.x; v < nvec;
       v += (long long)gridDim.x * blockDim.x) {
    const long long t = v / (I / 8);
    const int c = (int)(v % (I / 8)) * 8;
    float g[8], u[8], d[8], og[8], ou[8];
    load8(gu + t * 2 * I + c, g);
    load8(gu + t * 2 * I + I + c, u);
    load8(dh + t * I + c, d);
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const bool g_in = !(limit > 0.f) || g[j] <= limit;
      const bool u_in = !(limit > 0.f) || (u[j] >= -limit && u[j] <= limit);
      const float gc = g_in ? g[j] : limit;
      const float uc = u_in ? u[j] : (u[j] > 0.f ? limit : -limit);
      og[j] = g_in ? d[j] * (kind == 2 ? uc + 1.f : uc) * act_bwd(gc, kind) : 0.f;
      ou[j] = u_in ? d[j] * act_fwd(gc, kind) : 0.f;
    }
    store8(dgu + t * 2 * I + c, og);
    store8(dgu + t * 2 * I + I + c, ou);
  }
}

// ---------------------------------------------------------------------------------- DoRA weight norm
// norm[n] = sqrt(max(w2[n] + 2 s <W, BA>_n + s^2 |BA|_n^2, tiny)) with <W, BA>_n = sum_r WA[n,r] B[n,r] and
// |BA|_n^2 = sum_{q,r} B[n,q] G[q,r] B[n,r], G = A A^T [R, R] (fp32). One thread per output row, G in shared
// memory: the row-wise tail of the reference's fused DoRA-norm kernel (src/axolotl/kernels/dora.py:16-147)
// after the skinny tcgen05 GEMM W A^T.
__global__ void dora_norm_kernel(const float* __restrict__ WA, const float* __restrict__ B, const float* __restrict__ G,
                                 const float* __restrict__ w2, float* __restrict__ norm, long long N, int R, float s) {
  extern __shared__ float sG[];
  for (int i = threadIdx.x; i < R * R; i += blockDim.x) sG[i] = G[i];
  __syncthreads();
  const long long n = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (n >= N) return;
  const float* b = B + n * R;
  const float* wa = WA + n * R;
  float cross = 0.f, quad = 0.f;
  for (int r = 0; r < R; ++r) {
    const float br = b[r];
    cross += wa[r] * br;
    float acc = 0.f;
    for (int q = 0; q < R; ++q) acc += b[q] * sG[q * R + r];
    quad += acc * br;
  }
  norm[n] = sqrtf(fmaxf(w2[n] + 2.f * s * cross + s * s * quad, 1e-12f));
}

// ---------------------------------------------------------------------------------- embedding
__global__ void embedding_fwd_kernel(const __nv_bfloat16* __restrict__ table,
                                     const long long* __restrict__ ids,
                                     __nv_bfloat16* __restrict__ out, long long T, int H,
                                     long long vocab) {
  const long long nvec = T * (H / 8);
  for (long long v = (long long)blockIdx.x * blockDim.x + threadIdx.x; v < nvec;
       v += (long long)gridDim.x * blockDim.x) {
    const long long t = v / (H / 8);
    const int c = (int)(v % (H / 8)) * 8;
    long long id = ids[t];
    if (c == 0) (void)AXB_INDEX_OK(AXB_SITE_EMBED_ID, id, vocab);
    if (id < 0 || id >= vocab) id = 0;
    *reinterpret_cast<uint4*>(out + t * H + c) =
        *reinterpret_cast<const uint4*>(table + id * H + c);
  }
}
__global__ void embedding_bwd_kernel(const __nv_bfloat16* __restrict__ dout,
                                     const long long* __restrict__ ids, float* __restrict__ dtable,
                                     long long T, int H, long long vocab) {
  const long long n = T * H;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n;
       i += (long long)gridDim.x * blockDim.x) {
    const long long t = i / H;
    const int c = (int)(i % H);
    const long long id = ids[t];
    if (c == 0) (void)AXB_INDEX_OK(AXB_SITE_EMBED_GRAD_ID, id, vocab);
    if (id < 0 || id >= vocab) continue;
    atomicAdd(dtable + id * H + c, __bfloat162float(dout[i]));
  }
}

// ---------------------------------------------------------------------------------- cross entropy
// One block per row of a [R, V] bf16 logits chunk (optionally soft-capped). Computes
//   loss[r] = logsumexp(z) - z[label]   (0 when label == ignore_index)
// and overwrites the row with d loss_total / d z = (softmax(z) - onehot) * grad_scale, so the
// caller can feed the buffer straight into the dX / dW GEMMs. lse[r] is also returned.
constexpr int CE_T = 512;
// CAP: the logits are soft-capped first, z' = cap * tanh(z / cap) (Gemma 2 final_logit_softcapping); the
// gradient written back is with respect to the raw z.
template <bool CAP>
__global__ void __launch_bounds__(CE_T)
    ce_fwd_bwd_kernel(__nv_bfloat16* __restrict__ logits, const long long* __restrict__ labels,
                      float* __restrict__ loss, float* __restrict__ lse_out, int V,
                      long long ld, float grad_scale, long long ignore_index, int write_grad, float cap) {
  const float inv_cap = CAP ? 1.f / cap : 0.f;
  auto eff = [&](float v) -> float {
    if constexpr (CAP) return cap * tanhf(v * inv_cap);
    else return v;
  };
  __shared__ float sh[32];
  const long long r = blockIdx.x;
  __nv_bfloat16* z = logits + r * ld;
  const long long label = labels[r];
  if (threadIdx.x == 0 && label != ignore_index) (void)AXB_INDEX_OK(AXB_SITE_CE_LABEL, label, V);
  const bool ignored = (label == ignore_index) || label < 0 || label >= V;
  if (ignored && !lse_out) {
    if (threadIdx.x == 0) loss[r] = 0.f;
    if (write_grad) {
      const uint4 zero = make_uint4(0, 0, 0, 0);
      const int v8 = V & ~7;
      for (int i = threadIdx.x * 8; i < v8; i += CE_T * 8)
        *reinterpret_cast<uint4*>(z + i) = zero;
      for (int i = v8 + threadIdx.x; i < V; i += CE_T) z[i] = __float2bfloat16(0.f);
    }
    return;
  }
  const int v8 = V & ~7;
  float mx = -INFINITY;
  for (int i = threadIdx.x * 8; i < v8; i += CE_T * 8) {
    float f[8];
    load8(z + i, f);
#pragma unroll
    for (int j = 0; j < 8; ++j) mx = fmaxf(mx, f[j]);   // tanh is increasing: cap the maximum once below
  }
  for (int i = v8 + threadIdx.x; i < V; i += CE_T) mx = fmaxf(mx, __bfloat162float(z[i]));
  mx = eff(block_max<CE_T>(mx, sh));
  float se = 0.f;
  for (int i = threadIdx.x * 8; i < v8; i += CE_T * 8) {
    float f[8];
    load8(z + i, f);
#pragma unroll
    for (int j = 0; j < 8; ++j) se += __expf(eff(f[j]) - mx);
  }
  for (int i = v8 + threadIdx.x; i < V; i += CE_T) se += __expf(eff(__bfloat162float(z[i])) - mx);
  se = block_sum<CE_T>(se, sh);
  const float lse = mx + logf(se);
  if (threadIdx.x == 0) {
    if (lse_out) lse_out[r] = lse;
    loss[r] = ignored ? 0.f : lse - eff(__bfloat162float(z[label]));
  }
  if (!write_grad) return;
  __syncthreads();
  const float gs = ignored ? 0.f : grad_scale;
  for (int i = threadIdx.x * 8; i < v8; i += CE_T * 8) {
    float f[8];
    load8(z + i, f);
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const float ze = eff(f[j]);
      float pr = __expf(ze - lse);
      if (i + j == label) pr -= 1.f;
      if constexpr (CAP) pr *= 1.f - (ze * inv_cap) * (ze * inv_cap);   // d z' / d z = 1 - tanh^2
      f[j] = pr * gs;
    }
    store8(z + i, f);
  }
  for (int i = v8 + threadIdx.x; i < V; i += CE_T) {
    const float ze = eff(__bfloat162float(z[i]));
    float pr = __expf(ze - lse);
    if (i == label) pr -= 1.f;
    if constexpr (CAP) pr *= 1.f - (ze * inv_cap) * (ze * inv_cap);
    z[i] = __float2bfloat16(pr * gs);
  }
}

// ---------------------------------------------------------------------------------- gated RMSNorm
// y = (w + w_offset) * x * rstd(x) * silu(g): the output norm of gated linear-attention blocks
// (Qwen3.5 GatedDeltaNet). One block per row; x is kept in registers between the two passes.
__global__ void __launch_bounds__(NORM_T)
    rmsnorm_gated_fwd_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ g,
                             const __nv_bfloat16* __restrict__ w, __nv_bfloat16* __restrict__ y,
                             float* __restrict__ rstd_out, int H, float eps, float w_offset) {
  __shared__ float sh[32];
  const long long row = blockIdx.x;
  float ss = 0.f;
  for (int i = threadIdx.x * 8; i < H; i += NORM_T * 8) {
    float f[8];
    load8(x + row * H + i, f);
#pragma unroll
    for (int j = 0; j < 8; ++j) ss += f[j] * f[j];
  }
  ss = block_sum<NORM_T>(ss, sh);
  const float rstd = rsqrtf(ss / H + eps);
  if (threadIdx.x == 0) rstd_out[row] = rstd;
  for (int i = threadIdx.x * 8; i < H; i += NORM_T * 8) {
    float f[8], gv[8], wv[8];
    load8(x + row * H + i, f);
    load8(g + row * H + i, gv);
    load8(w + i, wv);
#pragma unroll
    for (int j = 0; j < 8; ++j)
      f[j] = f[j] * rstd * (wv[j] + w_offset) * (gv[j] * sigmoid_fast(gv[j]));
    store8(y + row * H + i, f);
  }
}
// With n = x*rstd*(w+off) and s = silu(g):  dg = dy*n*silu'(g);  dn = dy*s;
// dx = rstd * (dn*(w+off) - xhat * mean(dn*(w+off)*xhat));  dw += dn * xhat.
__global__ void __launch_bounds__(NORM_T)
    rmsnorm_gated_bwd_kernel(const __nv_bfloat16* __restrict__ dy, const __nv_bfloat16* __restrict__ x,
                             const __nv_bfloat16* __restrict__ g, const __nv_bfloat16* __restrict__ w,
                             const float* __restrict__ rstd_in, __nv_bfloat16* __restrict__ dx,
                             __nv_bfloat16* __restrict__ dg, float* __restrict__ dw, int H, int rows,
                             float w_offset) {
  __shared__ float sh[32];
  float dw_acc[4][8];
#pragma unroll
  for (int a = 0; a < 4; ++a)
#pragma unroll
    for (int j = 0; j < 8; ++j) dw_acc[a][j] = 0.f;
  for (long long row = blockIdx.x; row < rows; row += gridDim.x) {
    const float rstd = rstd_in[row];
    float dot = 0.f;
    for (int i = threadIdx.x * 8; i < H; i += NORM_T * 8) {
      float a[8], b[8], c[8], gv[8];
      load8(dy + row * H + i, a);
      load8(x + row * H + i, b);
      load8(w + i, c);
      load8(g + row * H + i, gv);
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const float s = gv[j] * sigmoid_fast(gv[j]);
        dot += a[j] * s * (c[j] + w_offset) * b[j] * rstd;
      }
    }
    dot = block_sum<NORM_T>(dot, sh) / H;
    int k = 0;
    for (int i = threadIdx.x * 8; i < H; i += NORM_T * 8, ++k) {
      float a[8], b[8], c[8], gv[8], ox[8], og[8];
      load8(dy + row * H + i, a);
      load8(x + row * H + i, b);
      load8(w + i, c);
      load8(g + row * H + i, gv);
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const float sg = sigmoid_fast(gv[j]);
        const float s = gv[j] * sg;
        const float xhat = b[j] * rstd;
        const float wj = c[j] + w_offset;
        const float dn = a[j] * s;
        ox[j] = rstd * (dn * wj - xhat * dot);
        og[j] = a[j] * xhat * wj * sg * (1.f + gv[j] * (1.f - sg));
        if (dw) {
          if (k < 4) dw_acc[k][j] += dn * xhat;
          else atomicAdd(dw + i + j, dn * xhat);
        }
      }
      store8(dx + row * H + i, ox);
      store8(dg + row * H + i, og);
    }
  }
  if (dw) {
    int k = 0;
    for (int i = threadIdx.x * 8; i < H && k < 4; i += NORM_T * 8, ++k)
#pragma unroll
      for (int j = 0; j < 8; ++j) atomicAdd(dw + i + j, dw_acc[k][j]);
  }
}

// ---------------------------------------------------------------------------------- entropy
// One block per row of a [R, V] bf16 logits chunk: a single online pass keeps the running maximum
// m, Z = sum exp(z - m) and S = sum (z - m) exp(z - m); entropy = log Z - S / Z. lse is returned
// as well. (The RL trainers log the policy entropy per token without a [R, V] fp32 softmax.)
__global__ void __launch_bounds__(CE_T)
    entropy_kernel(const __nv_bfloat16* __restrict__ logits, float* __restrict__ ent,
                   float* __restrict__ lse_out, int V, long long ld, float inv_temp) {
  __shared__ float sh[32];
  const long long r = blockIdx.x;
  const __nv_bfloat16* z = logits + r * ld;
  const int v8 = V & ~7;
  float m = -INFINITY, Z = 0.f, S = 0.f;
  auto push = [&](float v) {
    v *= inv_temp;
    if (v > m) {  // rescale the running sums to the new maximum
      const float c = __expf(m - v);
      S = (m == -INFINITY) ? 0.f : c * (S + (m - v) * Z);
      Z = (m == -INFINITY) ? 0.f : c * Z;
      m = v;
    }
    const float e = __expf(v - m);
    Z += e;
    S += (v - m) * e;
  };
  for (int i = threadIdx.x * 8; i < v8; i += CE_T * 8) {
    float f[8];
    load8(z + i, f);
#pragma unroll
    for (int j = 0; j < 8; ++j) push(f[j]);
  }
  for (int i = v8 + threadIdx.x; i < V; i += CE_T) push(__bfloat162float(z[i]));
  const float M = block_max<CE_T>(m, sh);
  const float c = (m == -INFINITY) ? 0.f : __expf(m - M);
  const float Zs = c * Z, Ss = c * (S + (m - M) * Z);
  const float Zt = block_sum<CE_T>(Zs, sh);
  const float St = block_sum<CE_T>((m == -INFINITY) ? 0.f : Ss, sh);
  if (threadIdx.x == 0) {
    ent[r] = logf(Zt) - St / Zt;
    if (lse_out) lse_out[r] = M + logf(Zt);  // of the scaled logits
  }
}

// ---------------------------------------------------------------------------------- optimizer
// sum of squares of a flat fp32 gradient buffer -> out[0] (atomic)
__global__ void sumsq_kernel(const float* __restrict__ g, long long n, float* __restrict__ out) {
  __shared__ float sh[32];
  float s = 0.f;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n;
       i += (long long)gridDim.x * blockDim.x)
    s += g[i] * g[i];
  s = block_sum<256>(s, sh);
  if (threadIdx.x == 0) atomicAdd(out, s);
}
// Fused AdamW over a flat fp32 master buffer. gnorm_sq (device scalar, optional) drives clipping:
// grads are scaled by min(1, max_norm / (sqrt(gnorm_sq) + 1e-6)) without a host round trip.
// bf16_copy (optional) receives the updated parameters for the bf16 compute path.
__global__ void adamw_kernel(float* __restrict__ p, const float* __restrict__ g,
                             float* __restrict__ m, float* __restrict__ v,
                             __nv_bfloat16* __restrict__ bf16_copy, long long n, float lr,
                             float beta1, float beta2, float eps, float wd, float bc1, float bc2,
                             const float* __restrict__ gnorm_sq, float max_norm,
                             float grad_scale) {
  float clip = grad_scale;
  if (gnorm_sq && max_norm > 0.f) {
    const float nrm = sqrtf(*gnorm_sq) * grad_scale;
    clip *= fminf(1.f, max_norm / (nrm + 1e-6f));
  }
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n;
       i += (long long)gridDim.x * blockDim.x) {
    const float gi = g[i] * clip;
    float pi = p[i];
    const float mi = beta1 * m[i] + (1.f - beta1) * gi;
    const float vi = beta2 * v[i] + (1.f - beta2) * gi * gi;
    m[i] = mi;
    v[i] = vi;
    pi *= (1.f - lr * wd);
    pi -= lr * (mi / bc1) / (sqrtf(vi / bc2) + eps);
    p[i] = pi;
    if (bf16_copy) bf16_copy[i] = __float2bfloat16(pi);
  }
}

// dst(bf16/fp32) = alpha * src (+ dst if accumulate)
__global__ void cast_bf16_to_f32_kernel(const __nv_bfloat16* __restrict__ s, float* __restrict__ d,
                                        long long n, float alpha, int accumulate) {
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n;
       i += (long long)gridDim.x * blockDim.x) {
    const float x = alpha * __bfloat162float(s[i]);
    d[i] = accumulate ? d[i] + x : x;
  }
}
__global__ void cast_f32_to_bf16_kernel(const float* __restrict__ s, __nv_bfloat16* __restrict__ d,
                                        long long n, float alpha) {
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n;
       i += (long long)gridDim.x * blockDim.x)
    d[i] = __float2bfloat16(alpha * s[i]);
}
// y[i] += x[i]  (bf16, 8-wide)
__global__ void add_bf16_kernel(__nv_bfloat16* __restrict__ y, const __nv_bfloat16* __restrict__ x,
                                long long n8) {
  for (long long v = (long long)blockIdx.x * blockDim.x + threadIdx.x; v < n8;
       v += (long long)gridDim.x * blockDim.x) {
    float a[8], b[8];
    load8(y + v * 8, a);
    load8(x + v * 8, b);
#pragma unroll
    for (int j = 0; j < 8; ++j) a[j] += b[j];
    store8(y + v * 8, a);
  }
}

inline int grid_for(long long work, int threads, int cap = 148 * 16) {
  long long g = (work + threads - 1) / threads;
  if (g > cap) g = cap;
  if (g < 1) g = 1;
  return (int)g;
}
}  // namespace

#define ST(s) reinterpret_cast<cudaStream_t>(s)

extern "C" int axb_rmsnorm_fwd(const void* x, const void* res, const void* w, void* y,
                               void* res_out, float* rstd, long long rows, int H, float eps,
                               float w_offset, void* stream) {
  if (H % 8) return -2;
  if (rows <= 0) return 0;
  rmsnorm_fwd_kernel<<<(unsigned)rows, NORM_T, 0, ST(stream)>>>(
      (const __nv_bfloat16*)x, (const __nv_bfloat16*)res, (const __nv_bfloat16*)w,
      (__nv_bfloat16*)y, (__nv_bfloat16*)res_out, rstd, H, eps, w_offset);
  return (int)cudaGetLastError();
}
extern "C" int axb_rmsnorm_bwd(const void* dy, const void* h, const void* w, const float* rstd,
                               const void* dres, void* dx, float* dw, long long rows, int H,
                               float w_offset, void* stream) {
  if (H % 8) return -2;
  if (rows <= 0) return 0;
  const int grid = rows < 148 * 8 ? (int)rows : 148 * 8;
  rmsnorm_bwd_kernel<<<grid, NORM_T, 0, ST(stream)>>>(
      (const __nv_bfloat16*)dy, (const __nv_bfloat16*)h, (const __nv_bfloat16*)w, rstd,
      (const __nv_bfloat16*)dres, (__nv_bfloat16*)dx, dw, H, (int)rows, w_offset);
  return (int)cudaGetLastError();
}
extern "C" int axb_rope_qk(void* qkv, const int* pos, const float* inv_freq, int T, int Hq, int Hk,
                           int D, long long row_stride, float sign, float attn_scale,
                           const void* qn_w, const void* kn_w, float* rstd_out, float eps,
                           void* stream) {
  if (T <= 0) return 0;
  if (!qn_w && !kn_w && (D % 4) == 0 && (row_stride % 2) == 0) {
    rope_fast_kernel<<<(unsigned)((T + 7) / 8), 256, 0, ST(stream)>>>((__nv_bfloat16*)qkv, pos, inv_freq, T, Hq + Hk, D,
                                                                     row_stride, sign, attn_scale, D);
    return (int)cudaGetLastError();
  }
  const long long warps = (long long)T * (Hq + Hk);
  const int wpb = 8;
  rope_qk_kernel<<<(unsigned)((warps + wpb - 1) / wpb), wpb * 32, 0, ST(stream)>>>(
      (__nv_bfloat16*)qkv, pos, inv_freq, T, Hq, Hk, D, row_stride, sign, attn_scale,
      (const __nv_bfloat16*)qn_w, (const __nv_bfloat16*)kn_w, rstd_out, eps);
  return (int)cudaGetLastError();
}
// Partial rotary embedding of the first `rot` dimensions of the q and k heads (sign = -1: the inverse rotation,
// i.e. the backward pass). rot % 4 == 0, rot <= D, row_stride % 2 == 0.
extern "C" int axb_rope_partial(void* qkv, const int* pos, const float* inv_freq, int T, int n_heads, int D, int rot,
                                long long row_stride, float sign, float attn_scale, void* stream) {
  if (T <= 0) return 0;
  if (rot <= 0 || rot > D || (rot & 3) || (row_stride & 1) || (D & 1)) return -2;
  rope_fast_kernel<<<(unsigned)((T + 7) / 8), 256, 0, ST(stream)>>>((__nv_bfloat16*)qkv, pos, inv_freq, T, n_heads, D,
                                                                   row_stride, sign, attn_scale, rot);
  return (int)cudaGetLastError();
}
extern "C" int axb_rope_qk_bwd(void* dqkv, const void* x_pre, const int* pos,
                               const float* inv_freq, int T, int Hq, int Hk, int D,
                               long long row_stride, long long x_row_stride, float attn_scale,
                               const void* qn_w, const void* kn_w, const float* rstd_in,
                               float* dqn_w, float* dkn_w, void* stream) {
  if (T <= 0) return 0;
  if (D > 512) return -2;
  if (!qn_w && !kn_w && (D % 4) == 0 && (row_stride % 2) == 0) {
    rope_fast_kernel<<<(unsigned)((T + 7) / 8), 256, 0, ST(stream)>>>((__nv_bfloat16*)dqkv, pos, inv_freq, T, Hq + Hk, D,
                                                                     row_stride, -1.f, attn_scale, D);
    return (int)cudaGetLastError();
  }
  const long long warps = (long long)T * (Hq + Hk);
  const int wpb = 8;
  if (D <= 256)
    rope_qk_bwd_kernel<4><<<(unsigned)((warps + wpb - 1) / wpb), wpb * 32, 0, ST(stream)>>>(
        (__nv_bfloat16*)dqkv, (const __nv_bfloat16*)x_pre, pos, inv_freq, T, Hq, Hk, D, row_stride,
        x_row_stride, attn_scale, (const __nv_bfloat16*)qn_w, (const __nv_bfloat16*)kn_w, rstd_in,
        dqn_w, dkn_w);
  else      // Gemma 4's global layers: 512-wide heads
    rope_qk_bwd_kernel<8><<<(unsigned)((warps + wpb - 1) / wpb), wpb * 32, 0, ST(stream)>>>(
        (__nv_bfloat16*)dqkv, (const __nv_bfloat16*)x_pre, pos, inv_freq, T, Hq, Hk, D, row_stride,
        x_row_stride, attn_scale, (const __nv_bfloat16*)qn_w, (const __nv_bfloat16*)kn_w, rstd_in,
        dqn_w, dkn_w);
  return (int)cudaGetLastError();
}
extern "C" int axb_rmsnorm_gated_fwd(const void* x, const void* g, const void* w, void* y,
                                     float* rstd, long long rows, int H, float eps,
                                     float w_offset, void* stream) {
  if (H % 8) return -2;
  if (rows <= 0) return 0;
  rmsnorm_gated_fwd_kernel<<<(unsigned)rows, NORM_T, 0, ST(stream)>>>(
      (const __nv_bfloat16*)x, (const __nv_bfloat16*)g, (const __nv_bfloat16*)w,
      (__nv_bfloat16*)y, rstd, H, eps, w_offset);
  return (int)cudaGetLastError();
}
extern "C" int axb_rmsnorm_gated_bwd(const void* dy, const void* x, const void* g, const void* w,
                                     const float* rstd, void* dx, void* dg, float* dw,
                                     long long rows, int H, float w_offset, void* stream) {
  if (H % 8) return -2;
  if (rows <= 0) return 0;
  const unsigned grid = (unsigned)(rows < 148 * 4 ? rows : 148 * 4);
  rmsnorm_gated_bwd_kernel<<<grid, NORM_T, 0, ST(stream)>>>(
      (const __nv_bfloat16*)dy, (const __nv_bfloat16*)x, (const __nv_bfloat16*)g,
      (const __nv_bfloat16*)w, rstd, (__nv_bfloat16*)dx, (__nv_bfloat16*)dg, dw, H, (int)rows,
      w_offset);
  return (int)cudaGetLastError();
}
extern "C" int axb_entropy(const void* logits, float* ent, float* lse, long long rows, int V,
                           long long ld, float inv_temp, void* stream) {
  if (rows <= 0) return 0;
  if (ld % 8) return -2;
  entropy_kernel<<<(unsigned)rows, CE_T, 0, ST(stream)>>>((const __nv_bfloat16*)logits, ent, lse, V,
                                                         ld, inv_temp);
  return (int)cudaGetLastError();
}
extern "C" int axb_dora_norm(const float* WA, const float* B, const float* G, const float* w2, float* norm, long long N,
                             int R, float s, void* stream) {
  if (N <= 0) return 0;
  if (R < 1 || R > 128) return -2;
  dora_norm_kernel<<<(unsigned)((N + 127) / 128), 128, R * R * sizeof(float), ST(stream)>>>(WA, B, G, w2, norm, N, R, s);
  return (int)cudaGetLastError();
}

extern "C" int axb_glu_fwd(const void* gu, void* h, long long T, int I, int kind, float limit,
                           void* stream) {
  if (I % 8) return -2;
  if (T <= 0) return 0;
  glu_fwd_kernel<<<grid_for(T * (I / 8), 256), 256, 0, ST(stream)>>>(
      (const __nv_bfloat16*)gu, (__nv_bfloat16*)h, T, I, kind, limit, nullptr);
  return (int)cudaGetLastError();
}
// the same over the first *blocks_in_use * 128 rows only (device-side count)
extern "C" int axb_glu_fwd_rows(const void* gu, void* h, long long T, int I, int kind, float limit,
                                const int* blocks_in_use, void* stream) {
  if (I % 8) return -2;
  if (T <= 0) return 0;
  glu_fwd_kernel<<<grid_for(T * (I / 8), 256), 256, 0, ST(stream)>>>(
      (const __nv_bfloat16*)gu, (__nv_bfloat16*)h, T, I, kind, limit, blocks_in_use);
  return (int)cudaGetLastError();
}
extern "C" int axb_glu_bwd_rows(const void* dh, const void* gu, void* dgu, long long T, int I, int kind,
                                float limit, const int* blocks_in_use, void* stream) {
  if (I % 8) return -2;
  if (T <= 0) return 0;
  glu_bwd_kernel<<<grid_for(T * (I / 8), 256), 256, 0, ST(stream)>>>(
      (const __nv_bfloat16*)dh, (const __nv_bfloat16*)gu, (__nv_bfloat16*)dgu, T, I, kind, limit, blocks_in_use);
  return (int)cudaGetLastError();
}
extern "C" int axb_glu_bwd(const void* dh, const void* gu, void* dgu, long long T, int I, int kind,
                           float limit, void* stream) {
  if (I % 8) return -2;
  if (T <= 0) return 0;
  glu_bwd_kernel<<<grid_for(T * (I / 8), 256), 256, 0, ST(stream)>>>(
      (const __nv_bfloat16*)dh, (const __nv_bfloat16*)gu, (__nv_bfloat16*)dgu, T, I, kind, limit, nullptr);
  return (int)cudaGetLastError();
}
extern "C" int axb_embedding_fwd(const void* table, const long long* ids, void* out, long long T,
                                 int H, long long vocab, void* stream) {
  if (H % 8) return -2;
  if (T <= 0) return 0;
  embedding_fwd_kernel<<<grid_for(T * (H / 8), 256), 256, 0, ST(stream)>>>(
      (const __nv_bfloat16*)table, ids, (__nv_bfloat16*)out, T, H, vocab);
  return (int)cudaGetLastError();
}
extern "C" int axb_embedding_bwd(const void* dout, const long long* ids, float* dtable,
                                 long long T, int H, long long vocab, void* stream) {
  if (T <= 0) return 0;
  embedding_bwd_kernel<<<grid_for(T * H, 256), 256, 0, ST(stream)>>>(
      (const __nv_bfloat16*)dout, ids, dtable, T, H, vocab);
  return (int)cudaGetLastError();
}
extern "C" int axb_ce_fwd_bwd(void* logits, const long long* labels, float* loss, float* lse,
                              long long rows, int V, long long ld, float grad_scale,
                              long long ignore_index, int write_grad, void* stream) {
  if (rows <= 0) return 0;
  if (ld % 8) return -2;
  ce_fwd_bwd_kernel<false><<<(unsigned)rows, CE_T, 0, ST(stream)>>>(
      (__nv_bfloat16*)logits, labels, loss, lse, V, ld, grad_scale, ignore_index, write_grad, 0.f);
  return (int)cudaGetLastError();
}
// the same with soft-capped logits, z' = softcap * tanh(z / softcap)
extern "C" int axb_ce_fwd_bwd_softcap(void* logits, const long long* labels, float* loss, float* lse,
                                      long long rows, int V, long long ld, float grad_scale,
                                      long long ignore_index, int write_grad, float softcap, void* stream) {
  if (rows <= 0) return 0;
  if (ld % 8 || !(softcap > 0.f)) return -2;
  ce_fwd_bwd_kernel<true><<<(unsigned)rows, CE_T, 0, ST(stream)>>>(
      (__nv_bfloat16*)logits, labels, loss, lse, V, ld, grad_scale, ignore_index, write_grad, softcap);
  return (int)cudaGetLastError();
}
extern "C" int axb_sumsq(const float* g, long long n, float* out, void* stream) {
  if (n <= 0) return 0;
  sumsq_kernel<<<grid_for(n, 256, 148 * 4), 256, 0, ST(stream)>>>(g, n, out);
  return (int)cudaGetLastError();
}
extern "C" int axb_adamw(float* p, const float* g, float* m, float* v, void* bf16_copy,
                         long long n, float lr, float beta1, float beta2, float eps, float wd,
                         float bc1, float bc2, const float* gnorm_sq, float max_norm,
                         float grad_scale, void* stream) {
  if (n <= 0) return 0;
  adamw_kernel<<<grid_for(n, 256), 256, 0, ST(stream)>>>(p, g, m, v, (__nv_bfloat16*)bf16_copy, n,
                                                         lr, beta1, beta2, eps, wd, bc1, bc2,
                                                         gnorm_sq, max_norm, grad_scale);
  return (int)cudaGetLastError();
}
extern "C" int axb_cast_bf16_to_f32(const void* s, float* d, long long n, float alpha,
                                    int accumulate, void* stream) {
  if (n <= 0) return 0;
  cast_bf16_to_f32_kernel<<<grid_for(n, 256), 256, 0, ST(stream)>>>((const __nv_bfloat16*)s, d, n,
                                                                    alpha, accumulate);
  return (int)cudaGetLastError();
}
extern "C" int axb_cast_f32_to_bf16(const float* s, void* d, long long n, float alpha,
                                    void* stream) {
  if (n <= 0) return 0;
  cast_f32_to_bf16_kernel<<<grid_for(n, 256), 256, 0, ST(stream)>>>(s, (__nv_bfloat16*)d, n,
                                                                    alpha);
  return (int)cudaGetLastError();
}
extern "C" int axb_add_bf16(void* y, const void* x, long long n, void* stream) {
  if (n % 8) return -2;
  if (n <= 0) return 0;
  add_bf16_kernel<<<grid_for(n / 8, 256), 256, 0, ST(stream)>>>((__nv_bfloat16*)y,
                                                                (const __nv_bfloat16*)x, n / 8);
  return (int)cudaGetLastError();
}
