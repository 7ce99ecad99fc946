// Single-query (decode) attention over a per-sequence KV cache for sm_100a.
//
// One CTA per (sequence, kv head) serves the whole GQA group of query heads: the cache rows of the
// head are read once for all of them. Positions are processed in chunks of 128: every thread scores
// one position (q . k over D, q broadcast from shared memory), the chunk goes through an online
// softmax, and the P.V product gives every thread one output dimension, so the V loads are
// coalesced. Memory-bound by construction: the cost is one pass over the live part of the cache.
//
// Generation in the reference goes through Hugging Face `generate` with its KV cache and SDPA /
// flash-attn decode kernels (src/axolotl/cli/inference.py, core/trainers/grpo rollouts).
#include "axb_common.cuh"

namespace {

constexpr int DEC_T = 128;
constexpr int MAX_G = 16;

template <int D>
__global__ void __launch_bounds__(DEC_T)
    decode_attn_kernel(const __nv_bfloat16* __restrict__ qkv, long long ld, int q_col0,
                       const __nv_bfloat16* __restrict__ kc, const __nv_bfloat16* __restrict__ vc,
                       const int* __restrict__ lens, __nv_bfloat16* __restrict__ out, long long out_ld,
                       int Hq, int Hk, long long max_len, float scale, int window) {
  constexpr int DPT = (D + DEC_T - 1) / DEC_T;  // output dims per thread
  __shared__ float sq[MAX_G][D];
  __shared__ float sp[MAX_G][DEC_T];
  __shared__ float s_red[MAX_G];
  const int b = blockIdx.y, kvh = blockIdx.x, tid = threadIdx.x;
  const int warp = tid >> 5, lane = tid & 31;
  const int G = Hq / Hk;
  const int n = lens[b];
  const int first = window > 0 ? max(0, n - window) : 0;   // sliding window: only the last `window` positions
  const long long row_elems = (long long)Hk * D;
  const __nv_bfloat16* kb = kc + (long long)b * max_len * row_elems + (long long)kvh * D;
  const __nv_bfloat16* vb = vc + (long long)b * max_len * row_elems + (long long)kvh * D;
  for (int i = tid; i < G * D; i += DEC_T) {
    const int g = i / D, d = i - g * D;
    sq[g][d] = __bfloat162float(qkv[(long long)b * ld + q_col0 + (long long)(kvh * G + g) * D + d]) * scale;
  }
  float acc[MAX_G][DPT];
  float m_run[MAX_G], l_run[MAX_G];
#pragma unroll
  for (int g = 0; g < MAX_G; ++g) {
    m_run[g] = -INFINITY;
    l_run[g] = 0.f;
#pragma unroll
    for (int j = 0; j < DPT; ++j) acc[g][j] = 0.f;
  }
  __syncthreads();
  for (int c0 = first; c0 < n; c0 += DEC_T) {
    const int pos = c0 + tid;
    const bool valid = pos < n;
    float s[MAX_G];
#pragma unroll
    for (int g = 0; g < MAX_G; ++g) s[g] = 0.f;
    if (valid) {
      const __nv_bfloat16* kr = kb + (long long)pos * row_elems;
#pragma unroll 4
      for (int i = 0; i < D; i += 8) {
        const uint4 u = *reinterpret_cast<const uint4*>(kr + i);
        const float2 a = unpack_bf16x2(u.x), bb = unpack_bf16x2(u.y), c = unpack_bf16x2(u.z), d = unpack_bf16x2(u.w);
        const float kv[8] = {a.x, a.y, bb.x, bb.y, c.x, c.y, d.x, d.y};
#pragma unroll
        for (int g = 0; g < MAX_G; ++g) {
          if (g < G) {
#pragma unroll
            for (int e = 0; e < 8; ++e) s[g] = fmaf(sq[g][i + e], kv[e], s[g]);
          }
        }
      }
    }
#pragma unroll
    for (int g = 0; g < MAX_G; ++g)
      if (g < G) sp[g][tid] = valid ? s[g] : -INFINITY;
    __syncthreads();
    // chunk maximum per query head: warp w reduces heads w, w+4, ...
    for (int g = warp; g < G; g += DEC_T / 32) {
      float mx = fmaxf(fmaxf(sp[g][lane], sp[g][lane + 32]), fmaxf(sp[g][lane + 64], sp[g][lane + 96]));
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
      if (lane == 0) s_red[g] = mx;
    }
    __syncthreads();
    float alpha[MAX_G];
#pragma unroll
    for (int g = 0; g < MAX_G; ++g) {
      if (g < G) {
        const float m_new = fmaxf(m_run[g], s_red[g]);   // finite: every chunk has a valid position
        alpha[g] = __expf(m_run[g] - m_new);
        m_run[g] = m_new;
        sp[g][tid] = valid ? __expf(s[g] - m_new) : 0.f;
      }
    }
    __syncthreads();
    for (int g = warp; g < G; g += DEC_T / 32) {
      float sm = sp[g][lane] + sp[g][lane + 32] + sp[g][lane + 64] + sp[g][lane + 96];
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) sm += __shfl_xor_sync(0xffffffffu, sm, o);
      if (lane == 0) s_red[g] = sm;
    }
    __syncthreads();
#pragma unroll
    for (int g = 0; g < MAX_G; ++g)
      if (g < G) l_run[g] = l_run[g] * alpha[g] + s_red[g];
    // P.V: thread owns output dims tid, tid + 128, ...
    const int cn = min(DEC_T, n - c0);
#pragma unroll
    for (int j = 0; j < DPT; ++j) {
      const int d = tid + j * DEC_T;
      if (d < D) {
#pragma unroll
        for (int g = 0; g < MAX_G; ++g)
          if (g < G) acc[g][j] *= alpha[g];
        const __nv_bfloat16* vr = vb + (long long)c0 * row_elems + d;
        // eight cache rows per step: their (strided) loads are issued together, then consumed;
        // probabilities of positions past the end of the sequence are zero already
        for (int p0 = 0; p0 < cn; p0 += 8) {
          float v[8];
#pragma unroll
          for (int k = 0; k < 8; ++k)
            v[k] = (p0 + k < cn) ? __bfloat162float(vr[(long long)(p0 + k) * row_elems]) : 0.f;
#pragma unroll
          for (int k = 0; k < 8; ++k) {
#pragma unroll
            for (int g = 0; g < MAX_G; ++g)
              if (g < G) acc[g][j] = fmaf(sp[g][p0 + k], v[k], acc[g][j]);
          }
        }
      }
    }
    __syncthreads();
  }
#pragma unroll
  for (int j = 0; j < DPT; ++j) {
    const int d = tid + j * DEC_T;
    if (d < D) {
#pragma unroll
      for (int g = 0; g < MAX_G; ++g)
        if (g < G)
          out[(long long)b * out_ld + (long long)(kvh * G + g) * D + d] =
              __float2bfloat16(n > 0 ? acc[g][j] / l_run[g] : 0.f);
    }
  }
}

}  // namespace

// qkv: [B, ld] fused projection of the new tokens (q block at column q_col0, already rotated);
// k_cache / v_cache: [B, max_len, Hk*D] (the new token's k / v already written at lens[b] - 1);
// lens[b]: live positions of sequence b including the new token; out: [B, out_ld >= Hq*D].
extern "C" int axb_decode_attn(const void* qkv, long long ld, int q_col0, const void* k_cache,
                               const void* v_cache, const int* lens, void* out, long long out_ld, int B,
                               int Hq, int Hk, int D, long long max_len, float scale, int window,
                               void* stream) {
  if (B <= 0) return 0;
  if (Hq % Hk || Hq / Hk > MAX_G || D % 8) return -2;
  dim3 grid(Hk, B);
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
#define LAUNCH(DD)                                                                                     \
  decode_attn_kernel<DD><<<grid, DEC_T, 0, st>>>((const __nv_bfloat16*)qkv, ld, q_col0,                \
                                                 (const __nv_bfloat16*)k_cache, (const __nv_bfloat16*)v_cache, \
                                                 lens, (__nv_bfloat16*)out, out_ld, Hq, Hk, max_len, scale, window)
  if (D == 64) LAUNCH(64);
  else if (D == 128) LAUNCH(128);
  else if (D == 256) LAUNCH(256);
  else return -2;
#undef LAUNCH
  return (int)cudaGetLastError();
}
