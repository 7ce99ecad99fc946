// Packed variable-length flash attention for sm_100a (forward + backward), GQA aware: causal
// inside each document, or bidirectional for documents whose tiles carry flag bit 0.
//
// Layout: tokens of all documents of a packed row are concatenated: q/k/v live in one fused
// projection buffer [T, (Hq + 2*Hk) * D] (bf16), documents are delimited by a host-built tile
// table (one entry per (document, 128-row tile)), so no [S,S] mask and no cross-document
// attention ever exists. Both kernels are warp-specialised:
//   warp 0: TMA producer, warp 1: tcgen05.mma issuer, warps 2-5: softmax / gradient math
// with S, P.V (forward) and S^T, dP^T, dK, dV, dQ^T (backward) accumulators living in TMEM.
//
// Replaces flash-attn varlen (FA2/FA4) that the reference reaches through HF's
// flash_attention_2 interface (src/axolotl/monkeypatch/attention/flash_attn_4.py:37-111) and its
// Triton varlen kernel (src/axolotl/monkeypatch/attention/flash_attn_d512.py:65-546).
#include "axb_common.cuh"
#include <type_traits>

namespace {

constexpr int kThreads = 192;
constexpr int HALF_BYTES = 128 * 128;  // 128 rows x 128 B (64 bf16) swizzled tile

struct AttnParams {
  const int4* tiles;  // (doc_start, doc_len, tile_start (doc relative), flags: bit 0 = bidirectional, bits 1.. = sliding window in tokens)
  int n_tiles;
  int Hq, Hk;
  int q_col0, k_col0, v_col0;  // element offsets of the q / k / v blocks inside a fused row
  __nv_bfloat16* out;          // [T, Hq*D]
  long long out_ld;
  float* lse2;  // [Hq, T]  log2-domain logsumexp of the scaled scores
  long long T;
  long long kv_rows;  // rows of the k / v buffer (the whole token stream under context parallelism)
  float sl2;  // softmax_scale * log2(e)
  int* status;
  // backward only
  const float* delta;  // [Hq, T]
  float* dq_acc;       // [T, Hq*D] fp32, accumulated with atomics
  __nv_bfloat16* dkv;  // fused gradient buffer, same layout as qkv (k and v blocks are written)
  long long dkv_ld;
  float scale;
  // context parallelism: the q / out / lse / dO / dq buffers hold only the rows
  // [q_row_off, q_row_off + q_rows) of the global token stream, K and V are global.
  int q_row_off, q_rows;
  // backward with context parallelism: dK / dV tiles are reduce-added (bf16x2 atomics over
  // NVLink) into the buffer of the rank that owns the kv rows: rank = row / cp_chunk.
  int dk_col0, dv_col0;  // column offsets of the dK / dV blocks in the gradient buffer
  int cp_world;
  long long cp_chunk;
  unsigned long long cp_dkv_ptrs[8];
  // backward: the q heads of one kv head may be split over `kv_split` CTAs (load balance for wide
  // GQA groups); their dK / dV partial tiles are then reduce-added into a pre-zeroed buffer
  int kv_split;
};

AXB_DEVICE float fast_exp2(float x) {
  float y;
  asm volatile("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

// byte offset of 8 consecutive bf16 (one 16-byte chunk) inside a [128 x 64] bf16 SW128 tile
AXB_DEVICE uint32_t sw128_chunk_off(int row, int chunk) {
  return (uint32_t)row * 128u + (uint32_t)((chunk ^ (row & 7)) << 4);
}

// =====================================================================================
// Forward
// =====================================================================================
template <int D>
struct FwdCfg {
  static constexpr int HALVES = D / 64;
  static constexpr int TILE_BYTES = HALVES * HALF_BYTES;  // Q / K / V tile of 128 rows
  static constexpr int P_BYTES = 2 * HALF_BYTES;          // P [128 x 128]
  static constexpr int KV_STAGES = 2;
  static constexpr int SMEM = TILE_BYTES * (1 + 2 * KV_STAGES) + P_BYTES + 1024 + 256;
  static constexpr int TMEM_COLS = 512;
  static constexpr int S_COL = 0;      // S buffers: 2 x 128 columns
  static constexpr int PV_COL = 256;   // PV buffers: 2 x D columns
};

template <int D>
__global__ void __launch_bounds__(kThreads, 1)
    flash_fwd_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_qkv,
                     const AttnParams p) {
  using C = FwdCfg<D>;
  const int tile_id = blockIdx.y;
  if (tile_id >= p.n_tiles) return;
  const int head = blockIdx.x;
  const int kv_head = head / (p.Hq / p.Hk);
  const int4 ti = p.tiles[tile_id];
  const int doc_start = ti.x, doc_len = ti.y, q0 = ti.z;
  if (!AXB_INDEX_OK(AXB_SITE_ATTN_TILE, (long long)doc_start + doc_len - 1, p.kv_rows) || !AXB_INDEX_OK(AXB_SITE_ATTN_TILE, q0, doc_len)) return;
  const bool bidir = ti.w & 1;  // every token of the document sees the whole document
  const int win = bidir ? 0 : (ti.w >> 1);  // sliding window: row q sees kv rows (q - win, q]; 0 = unlimited
  const int kv_end = bidir ? doc_len : min(q0 + 128, doc_len);
  const int jb0 = win > 0 ? max(0, q0 - win + 1) / 128 : 0;  // first kv block any row of the tile can see
  const int n_blocks = (kv_end + 127) / 128 - jb0;           // kv blocks visited: jb0 .. jb0 + n_blocks - 1

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~static_cast<uintptr_t>(1023));
  uint8_t* sQ = smem;
  uint8_t* sK = sQ + C::TILE_BYTES;
  uint8_t* sV = sK + C::KV_STAGES * C::TILE_BYTES;
  uint8_t* sP = sV + C::KV_STAGES * C::TILE_BYTES;
  uint64_t* bars = reinterpret_cast<uint64_t*>(sP + C::P_BYTES);
  uint64_t* q_full = bars + 0;
  uint64_t* k_full = bars + 1;    // [2]
  uint64_t* v_full = bars + 3;    // [2]
  uint64_t* kv_empty = bars + 5;  // [2]
  uint64_t* s_full = bars + 7;    // [2]
  uint64_t* s_empty = bars + 9;   // [2]
  uint64_t* p_full = bars + 11;
  uint64_t* p_empty = bars + 12;
  uint64_t* pv_full = bars + 13;   // [2]
  uint64_t* pv_empty = bars + 15;  // [2]
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 17);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (threadIdx.x == 0) {
    mbar_init(q_full, 1);
    for (int s = 0; s < 2; ++s) {
      mbar_init(&k_full[s], 1);
      mbar_init(&v_full[s], 1);
      mbar_init(&kv_empty[s], 1);
      mbar_init(&s_full[s], 1);
      mbar_init(&s_empty[s], 128);
      mbar_init(&pv_full[s], 1);
      mbar_init(&pv_empty[s], 128);
    }
    mbar_init(p_full, 128);
    mbar_init(p_empty, 1);
    mbar_fence_init();
    tma_prefetch_desc(&tm_qkv);
  }
  if (warp == 2) {
    tmem_alloc(tmem_slot, C::TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    if (lane == 0) {
      mbar_expect_tx(q_full, C::TILE_BYTES);
#pragma unroll
      for (int h = 0; h < C::HALVES; ++h)
        tma_load_2d(sQ + h * HALF_BYTES, &tm_q, q_full, p.q_col0 + head * D + h * 64,
                    doc_start + q0 - p.q_row_off);
      for (int j = 0; j < n_blocks; ++j) {
        const int st = j & 1;
        const uint32_t ph = (j >> 1) & 1;
        if (!mbar_wait(&kv_empty[st], ph ^ 1, p.status, AXB_TIMEOUT_EMPTY)) break;
        mbar_expect_tx(&k_full[st], C::TILE_BYTES);
#pragma unroll
        for (int h = 0; h < C::HALVES; ++h)
          tma_load_2d(sK + st * C::TILE_BYTES + h * HALF_BYTES, &tm_qkv, &k_full[st],
                      p.k_col0 + kv_head * D + h * 64, doc_start + (jb0 + j) * 128);
        mbar_expect_tx(&v_full[st], C::TILE_BYTES);
#pragma unroll
        for (int h = 0; h < C::HALVES; ++h)
          tma_load_2d(sV + st * C::TILE_BYTES + h * HALF_BYTES, &tm_qkv, &v_full[st],
                      p.v_col0 + kv_head * D + h * 64, doc_start + (jb0 + j) * 128);
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      constexpr uint32_t idesc_s = make_idesc_bf16(128, 128, 0, 0);  // Q (K-major) x K (K-major)
      constexpr uint32_t idesc_pv = make_idesc_bf16(128, D, 0, 1);   // P (K-major) x V (MN-major)
      const uint32_t q_addr = smem_u32(sQ);
      const uint32_t p_addr = smem_u32(sP);
      bool ok = mbar_wait(q_full, 0, p.status, AXB_TIMEOUT_FULL);
      auto issue_s = [&](int j) -> bool {
        const int st = j & 1;
        const uint32_t ph = (j >> 1) & 1;
        if (!mbar_wait(&k_full[st], ph, p.status, AXB_TIMEOUT_FULL)) return false;
        if (!mbar_wait(&s_empty[st], ph ^ 1, p.status, AXB_TIMEOUT_TMEM_EMPTY)) return false;
        tc_fence_after();
        const uint32_t k_addr = smem_u32(sK + st * C::TILE_BYTES);
#pragma unroll
        for (int kk = 0; kk < D / 16; ++kk) {
          const uint32_t off = (kk / 4) * HALF_BYTES + (kk % 4) * 32;
          umma_f16(tmem_base + C::S_COL + st * 128, make_smem_desc_sw128(q_addr + off, 16, 1024),
                   make_smem_desc_sw128(k_addr + off, 16, 1024), idesc_s, kk > 0);
        }
        umma_commit(&s_full[st]);
        return true;
      };
      if (ok) ok = issue_s(0);
      for (int j = 0; j < n_blocks && ok; ++j) {
        const int st = j & 1;
        const uint32_t ph = (j >> 1) & 1;
        if (j + 1 < n_blocks) {
          ok = issue_s(j + 1);
          if (!ok) break;
        }
        if (!mbar_wait(p_full, j & 1, p.status, AXB_TIMEOUT_GENERIC)) break;
        if (!mbar_wait(&v_full[st], ph, p.status, AXB_TIMEOUT_FULL)) break;
        if (!mbar_wait(&pv_empty[st], ph ^ 1, p.status, AXB_TIMEOUT_TMEM_EMPTY)) break;
        tc_fence_after();
        const uint32_t v_addr = smem_u32(sV + st * C::TILE_BYTES);
#pragma unroll
        for (int kk = 0; kk < 8; ++kk) {  // 128 kv rows / 16
          const uint32_t poff = (kk / 4) * HALF_BYTES + (kk % 4) * 32;
          umma_f16(tmem_base + C::PV_COL + st * D, make_smem_desc_sw128(p_addr + poff, 16, 1024),
                   make_smem_desc_sw128(v_addr + kk * 2048, HALF_BYTES, 1024), idesc_pv, kk > 0);
        }
        umma_commit(&pv_full[st]);
        umma_commit(&kv_empty[st]);
        umma_commit(p_empty);
      }
    }
  } else {
    // ---------------------------------------------------------------- softmax warps
    const int lg = warp & 3;
    const int r = lg * 32 + lane;  // row inside the tile
    const int q_idx = q0 + r;
    const uint32_t lane_off = uint32_t(lg * 32) << 16;
    float m = -INFINITY, l = 0.f, alpha_prev = 1.f;
    float o[D];
#pragma unroll
    for (int i = 0; i < D; ++i) o[i] = 0.f;
    bool ok = true;
    for (int j = 0; j < n_blocks && ok; ++j) {
      const int st = j & 1;
      const uint32_t ph = (j >> 1) & 1;
      if (!mbar_wait(&s_full[st], ph, p.status, AXB_TIMEOUT_TMEM_FULL)) {
        ok = false;
        break;
      }
      tc_fence_after();
      const uint32_t s_addr = tmem_base + lane_off + C::S_COL + st * 128;
      const int kv0 = (jb0 + j) * 128;
      const bool need_mask = (j == n_blocks - 1) || (win > 0 && kv0 < q0 + 128 - win);
      const int lim = (bidir ? doc_len - 1 : min(q_idx, doc_len - 1)) - kv0;  // columns <= lim are visible
      const int lo = win > 0 ? q_idx - win + 1 - kv0 : -(1 << 30);            // columns >= lo are visible
      float mx = -INFINITY;
      // two compiled variants of each pass: interior blocks carry no per-element compares
      auto max_pass = [&](auto masked) {
#pragma unroll 1
        for (int c = 0; c < 4; ++c) {
          uint32_t sr[32];
          tmem_ld_32x32(s_addr + c * 32, sr);
          tmem_ld_wait();
#pragma unroll
          for (int i = 0; i < 32; ++i) {
            float v = __uint_as_float(sr[i]);
            if constexpr (decltype(masked)::value) {
              if (c * 32 + i > lim || c * 32 + i < lo) v = -INFINITY;
            }
            mx = fmaxf(mx, v);
          }
        }
      };
      if (need_mask) max_pass(std::true_type{});
      else max_pass(std::false_type{});
      const float m_new = fmaxf(m, mx * p.sl2);
      const float m_use = (m_new == -INFINITY) ? 0.f : m_new;
      const float alpha = fast_exp2(m - m_use);
      if (!mbar_wait(p_empty, (j & 1) ^ 1, p.status, AXB_TIMEOUT_GENERIC)) {
        ok = false;
        break;
      }
      float rowsum = 0.f;
      auto p_pass = [&](auto masked) {
#pragma unroll 1
        for (int c = 0; c < 4; ++c) {
          uint32_t sr[32];
          tmem_ld_32x32(s_addr + c * 32, sr);
          tmem_ld_wait();
          uint32_t pk[16];
#pragma unroll
          for (int i = 0; i < 32; i += 2) {
            float v0 = __uint_as_float(sr[i]), v1 = __uint_as_float(sr[i + 1]);
            float p0 = fast_exp2(v0 * p.sl2 - m_use), p1 = fast_exp2(v1 * p.sl2 - m_use);
            if constexpr (decltype(masked)::value) {
              if (c * 32 + i > lim || c * 32 + i < lo) p0 = 0.f;
              if (c * 32 + i + 1 > lim || c * 32 + i + 1 < lo) p1 = 0.f;
            }
            rowsum += p0 + p1;
            pk[i >> 1] = pack_bf16x2(p0, p1);
          }
          // columns [c*32, c*32+32) -> half c/2, 16-byte chunks (c%2)*4 .. +3
          uint8_t* pbase = sP + (c >> 1) * HALF_BYTES;
#pragma unroll
          for (int q = 0; q < 4; ++q) {
            uint4 val = make_uint4(pk[q * 4], pk[q * 4 + 1], pk[q * 4 + 2], pk[q * 4 + 3]);
            *reinterpret_cast<uint4*>(pbase + sw128_chunk_off(r, (c & 1) * 4 + q)) = val;
          }
        }
      };
      if (need_mask) p_pass(std::true_type{});
      else p_pass(std::false_type{});
      tc_fence_before();
      mbar_arrive(&s_empty[st]);
      fence_proxy_async_smem();
      mbar_arrive(p_full);
      l = l * alpha + rowsum;
      m = m_new;
      if (j > 0) {
        const int pst = (j - 1) & 1;
        const uint32_t pph = ((j - 1) >> 1) & 1;
        if (!mbar_wait(&pv_full[pst], pph, p.status, AXB_TIMEOUT_TMEM_FULL)) {
          ok = false;
          break;
        }
        tc_fence_after();
        const uint32_t pv_addr = tmem_base + lane_off + C::PV_COL + pst * D;
#pragma unroll
        for (int c = 0; c < D / 32; ++c) {
          uint32_t vr[32];
          tmem_ld_32x32(pv_addr + c * 32, vr);
          tmem_ld_wait();
#pragma unroll
          for (int i = 0; i < 32; ++i)
            o[c * 32 + i] = o[c * 32 + i] * alpha_prev + __uint_as_float(vr[i]);
        }
        tc_fence_before();
        mbar_arrive(&pv_empty[pst]);
      }
      alpha_prev = alpha;
    }
    if (ok && n_blocks > 0) {
      const int pst = (n_blocks - 1) & 1;
      const uint32_t pph = ((n_blocks - 1) >> 1) & 1;
      if (mbar_wait(&pv_full[pst], pph, p.status, AXB_TIMEOUT_TMEM_FULL)) {
        tc_fence_after();
        const uint32_t pv_addr = tmem_base + lane_off + C::PV_COL + pst * D;
        const float inv_l = l > 0.f ? 1.f / l : 0.f;
        const long long lrow = (long long)doc_start + q_idx - p.q_row_off;  // row in the local buffers
        const bool row_ok = q_idx < doc_len && lrow >= 0 && lrow < p.q_rows;
        __nv_bfloat16* orow = p.out + lrow * p.out_ld + (long long)head * D;
#pragma unroll
        for (int c = 0; c < D / 32; ++c) {
          uint32_t vr[32];
          tmem_ld_32x32(pv_addr + c * 32, vr);
          tmem_ld_wait();
          if (row_ok) {
#pragma unroll
            for (int q = 0; q < 4; ++q) {
              float f[8];
#pragma unroll
              for (int i = 0; i < 8; ++i)
                f[i] = (o[c * 32 + q * 8 + i] * alpha_prev + __uint_as_float(vr[q * 8 + i])) *
                       inv_l;
              uint4 u;
              u.x = pack_bf16x2(f[0], f[1]);
              u.y = pack_bf16x2(f[2], f[3]);
              u.z = pack_bf16x2(f[4], f[5]);
              u.w = pack_bf16x2(f[6], f[7]);
              *reinterpret_cast<uint4*>(orow + c * 32 + q * 8) = u;
            }
          }
        }
        if (row_ok) p.lse2[(long long)head * p.q_rows + lrow] = m + log2f(l);
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 2) {
    tc_fence_after();
    tmem_dealloc(tmem_base, C::TMEM_COLS);
  }
}

// =====================================================================================
// Backward
// =====================================================================================
// delta[h][t] = sum_d dO[t,h,d] * O[t,h,d]
__global__ void attn_delta_kernel(const __nv_bfloat16* __restrict__ dout,
                                  const __nv_bfloat16* __restrict__ out, float* __restrict__ delta,
                                  long long T, int Hq, int D, long long ld_do, long long ld_o) {
  const long long gw = ((long long)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (gw >= T * Hq) return;
  const long long t = gw / Hq;
  const int h = (int)(gw % Hq);
  const __nv_bfloat16* a = dout + t * ld_do + (long long)h * D;
  const __nv_bfloat16* b = out + t * ld_o + (long long)h * D;
  float s = 0.f;
  for (int i = lane * 2; i < D; i += 64) {
    float2 x = unpack_bf16x2(*reinterpret_cast<const uint32_t*>(a + i));
    float2 y = unpack_bf16x2(*reinterpret_cast<const uint32_t*>(b + i));
    s += x.x * y.x + x.y * y.y;
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
  if (lane == 0) delta[(long long)h * T + t] = s;
}

// One CTA per (kv tile of 128 rows, kv head). Inner loop over the q heads of the GQA group and
// over 64-row q tiles at or below the diagonal. Every MMA has M = 128:
//   S^T  [kv, q]  = K . Q^T        dP^T [kv, q] = V . dO^T
//   dV   [kv, d] += P^T . dO       dK   [kv, d] += dS^T . Q
//   dQ^T [d,  q]  = K^T . dS^T     (drained with fp32 atomics into dq_acc)
// Two softmax warpgroups alternate iterations: S^T / dP^T (TMEM) and P^T / dS^T (shared memory)
// are double buffered, so the tensor core computes S^T, dP^T of iteration i+1 while warpgroup
// i % 2 turns S^T(i) into P^T, dS^T and drains dQ^T(i). dQ^T(i) reuses the TMEM columns of S^T(i),
// which is dead once P^T(i) is written; with D = 128 all 512 columns are in use:
//   [S^T0 | dP^T0 | S^T1 | dP^T1 | dV (D) | dK (D)]
constexpr int kBwdThreads = 320;  // TMA warp, MMA warp, 2 x 4 softmax warps
template <int D>
struct BwdCfg {
  static constexpr int HALVES = D / 64;
  static constexpr int KV_BYTES = HALVES * HALF_BYTES;  // K or V tile: 128 rows
  static constexpr int Q_HALF = 64 * 128;               // 64 rows x 128 B
  static constexpr int Q_BYTES = HALVES * Q_HALF;       // Q or dO tile: 64 rows
  static constexpr int PT_BYTES = HALF_BYTES;           // P^T / dS^T: [128 kv x 64 q]
  static constexpr int STAGES = 2;
  static constexpr int SMEM =
      2 * KV_BYTES + STAGES * 2 * Q_BYTES + 4 * PT_BYTES + 1024 /*lse+delta*/ + 1024 + 256;
  static constexpr int ST_COL = 0;     // S^T(b) at ST_COL + 128 b, 64 cols; dQ^T(b) aliases it
  static constexpr int DPT_COL = 64;   // dP^T(b) at DPT_COL + 128 b, 64 cols
  static constexpr int DV_COL = 256;   // D cols
  static constexpr int DK_COL = 256 + D;
  static constexpr int TMEM_COLS = 512;
};

template <int D>
__global__ void __launch_bounds__(kBwdThreads, 1)
    flash_bwd_kernel(const __grid_constant__ CUtensorMap tm_kv,   // box 64 x 128 over qkv
                     const __grid_constant__ CUtensorMap tm_q,    // box 64 x 64 over qkv
                     const __grid_constant__ CUtensorMap tm_do,   // box 64 x 64 over dO
                     const AttnParams p) {
  using C = BwdCfg<D>;
  const int tile_id = blockIdx.y;
  if (tile_id >= p.n_tiles) return;
  const int kv_head = blockIdx.x / p.kv_split;
  const int part = blockIdx.x - kv_head * p.kv_split;
  const int group_all = p.Hq / p.Hk;
  const int group = group_all / p.kv_split;             // q heads handled by this CTA
  const int head0 = kv_head * group_all + part * group;  // first of them
  const int4 ti = p.tiles[tile_id];
  const int doc_start = ti.x, doc_len = ti.y, kv0 = ti.z;
  if (!AXB_INDEX_OK(AXB_SITE_ATTN_TILE, (long long)doc_start + doc_len - 1, p.kv_rows) || !AXB_INDEX_OK(AXB_SITE_ATTN_TILE, kv0, doc_len)) return;
  const bool bidir = ti.w & 1;
  // 64-row q tiles at or below the diagonal (all of the document's when it is bidirectional)
  // that intersect this rank's q rows
  const int win = bidir ? 0 : (ti.w >> 1);  // sliding window (0 = unlimited): kv row c is seen by q rows [c, c + win)
  int q_first = bidir ? 0 : kv0 / 64;
  int q_last = (doc_len + 63) / 64;
  if (win > 0) q_last = min(q_last, (kv0 + 127 + win - 1) / 64 + 1);
  {
    const int lo = p.q_row_off - doc_start, hi = p.q_row_off + p.q_rows - doc_start;
    if (lo > 0) q_first = max(q_first, lo / 64);
    q_last = min(q_last, (hi + 63) / 64);
  }
  const int n_qt = q_last - q_first;  // q tiles per head
  const int n_iter = n_qt * group;
  if (n_iter <= 0) return;

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~static_cast<uintptr_t>(1023));
  uint8_t* sK = smem;
  uint8_t* sV = sK + C::KV_BYTES;
  uint8_t* sQ = sV + C::KV_BYTES;                    // [STAGES]
  uint8_t* sdO = sQ + C::STAGES * C::Q_BYTES;        // [STAGES]
  uint8_t* sPT = sdO + C::STAGES * C::Q_BYTES;       // [2]
  uint8_t* sdST = sPT + 2 * C::PT_BYTES;             // [2]
  float* s_lse = reinterpret_cast<float*>(sdST + 2 * C::PT_BYTES);  // [2][64]
  float* s_delta = s_lse + 128;                                     // [2][64]
  uint64_t* bars = reinterpret_cast<uint64_t*>(s_delta + 128);
  uint64_t* kv_full = bars + 0;
  uint64_t* q_full = bars + 1;    // [2]  (Q and dO of a stage)
  uint64_t* q_empty = bars + 3;   // [2]
  uint64_t* s_full = bars + 5;    // [2]  S^T(b) and dP^T(b) ready
  uint64_t* pt_full = bars + 7;   // [2]  P^T(b) / dS^T(b) written to smem
  uint64_t* dq_full = bars + 9;   // [2]  dQ^T(b) ready (and every MMA reading P^T(b)/dS^T(b) retired)
  uint64_t* st_free = bars + 11;  // [2]  dQ^T(b) drained: TMEM and smem buffers b reusable
  uint64_t* acc_full = bars + 13; // dK / dV final
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 14);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (threadIdx.x == 0) {
    mbar_init(kv_full, 1);
    for (int s = 0; s < 2; ++s) {
      mbar_init(&q_full[s], 1);
      mbar_init(&q_empty[s], 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(&s_full[b], 1);
      mbar_init(&pt_full[b], 128);
      mbar_init(&dq_full[b], 1);
      mbar_init(&st_free[b], 128);
    }
    mbar_init(acc_full, 1);
    mbar_fence_init();
  }
  if (warp == 2) {
    tmem_alloc(tmem_slot, C::TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    if (lane == 0) {
      mbar_expect_tx(kv_full, 2 * C::KV_BYTES);
#pragma unroll
      for (int h = 0; h < C::HALVES; ++h) {
        tma_load_2d(sK + h * HALF_BYTES, &tm_kv, kv_full, p.k_col0 + kv_head * D + h * 64,
                    doc_start + kv0);
        tma_load_2d(sV + h * HALF_BYTES, &tm_kv, kv_full, p.v_col0 + kv_head * D + h * 64,
                    doc_start + kv0);
      }
      for (int it = 0; it < n_iter; ++it) {
        const int st = it & 1;
        const uint32_t ph = (it >> 1) & 1;
        const int head = head0 + it / n_qt;
        const int qrow = doc_start + (q_first + it % n_qt) * 64 - p.q_row_off;
        if (!mbar_wait(&q_empty[st], ph ^ 1, p.status, AXB_TIMEOUT_EMPTY)) break;
        mbar_expect_tx(&q_full[st], 2 * C::Q_BYTES);
#pragma unroll
        for (int h = 0; h < C::HALVES; ++h) {
          tma_load_2d(sQ + st * C::Q_BYTES + h * C::Q_HALF, &tm_q, &q_full[st],
                      p.q_col0 + head * D + h * 64, qrow);
          tma_load_2d(sdO + st * C::Q_BYTES + h * C::Q_HALF, &tm_do, &q_full[st],
                      head * D + h * 64, qrow);
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      constexpr uint32_t idesc_st = make_idesc_bf16(128, 64, 0, 0);  // K/V (K-major) x Q/dO (K-major)
      constexpr uint32_t idesc_acc = make_idesc_bf16(128, D, 0, 1);  // P^T/dS^T x dO/Q (MN-major)
      constexpr uint32_t idesc_dq = make_idesc_bf16(128, 64, 1, 1);  // K^T (MN) x dS^T (MN)
      const uint32_t k_addr = smem_u32(sK), v_addr = smem_u32(sV);
      const uint32_t pt_addr = smem_u32(sPT), dst_addr = smem_u32(sdST);
      bool ok = mbar_wait(kv_full, 0, p.status, AXB_TIMEOUT_FULL);
      // S^T(i) = K . Q(i)^T and dP^T(i) = V . dO(i)^T into TMEM buffer i & 1
      auto issue_scores = [&](int i) -> bool {
        const int st = i & 1, b = i & 1;
        const uint32_t ph = (i >> 1) & 1;
        if (!mbar_wait(&q_full[st], ph, p.status, AXB_TIMEOUT_FULL)) return false;
        // buffer b was last used by iteration i - 2: its dQ^T must have been drained
        if (i >= 2 && !mbar_wait(&st_free[b], ((i - 2) >> 1) & 1, p.status, AXB_TIMEOUT_TMEM_EMPTY))
          return false;
        tc_fence_after();
        const uint32_t q_addr = smem_u32(sQ + st * C::Q_BYTES);
        const uint32_t do_addr = smem_u32(sdO + st * C::Q_BYTES);
#pragma unroll
        for (int kk = 0; kk < D / 16; ++kk) {  // reduce over d
          const uint32_t koff = (kk / 4) * HALF_BYTES + (kk % 4) * 32;
          const uint32_t qoff = (kk / 4) * C::Q_HALF + (kk % 4) * 32;
          umma_f16(tmem_base + C::ST_COL + 128 * b, make_smem_desc_sw128(k_addr + koff, 16, 1024),
                   make_smem_desc_sw128(q_addr + qoff, 16, 1024), idesc_st, kk > 0);
        }
#pragma unroll
        for (int kk = 0; kk < D / 16; ++kk) {
          const uint32_t koff = (kk / 4) * HALF_BYTES + (kk % 4) * 32;
          const uint32_t qoff = (kk / 4) * C::Q_HALF + (kk % 4) * 32;
          umma_f16(tmem_base + C::DPT_COL + 128 * b, make_smem_desc_sw128(v_addr + koff, 16, 1024),
                   make_smem_desc_sw128(do_addr + qoff, 16, 1024), idesc_st, kk > 0);
        }
        umma_commit(&s_full[b]);
        return true;
      };
      ok = ok && issue_scores(0);
      for (int it = 0; it < n_iter && ok; ++it) {
        const int st = it & 1, b = it & 1;
        const uint32_t ph = (it >> 1) & 1;
        if (it + 1 < n_iter && !issue_scores(it + 1)) break;   // keeps the tensor core busy during softmax(it)
        const uint32_t q_addr = smem_u32(sQ + st * C::Q_BYTES);
        const uint32_t do_addr = smem_u32(sdO + st * C::Q_BYTES);
        const uint32_t ptb = pt_addr + b * C::PT_BYTES, dstb = dst_addr + b * C::PT_BYTES;
        if (!mbar_wait(&pt_full[b], ph, p.status, AXB_TIMEOUT_GENERIC)) break;
        tc_fence_after();
        // reduce over the 64 q rows of this tile: 4 K-steps of 16
#pragma unroll
        for (int kk = 0; kk < 4; ++kk) {
          // dV += P^T . dO   (B = dO tile, MN-major: chunk stride = one 64x64 half)
          umma_f16(tmem_base + C::DV_COL, make_smem_desc_sw128(ptb + kk * 32, 16, 1024),
                   make_smem_desc_sw128(do_addr + kk * 2048, C::Q_HALF, 1024), idesc_acc,
                   (it > 0 || kk > 0));
        }
#pragma unroll
        for (int kk = 0; kk < 4; ++kk) {
          umma_f16(tmem_base + C::DK_COL, make_smem_desc_sw128(dstb + kk * 32, 16, 1024),
                   make_smem_desc_sw128(q_addr + kk * 2048, C::Q_HALF, 1024), idesc_acc,
                   (it > 0 || kk > 0));
        }
        umma_commit(&q_empty[st]);
        // dQ^T [d, q] = K^T . dS^T over the 128 kv rows (8 K-steps of 16), into the columns of S^T(b)
#pragma unroll
        for (int kk = 0; kk < 8; ++kk) {
          umma_f16(tmem_base + C::ST_COL + 128 * b,
                   make_smem_desc_sw128(k_addr + kk * 2048, HALF_BYTES, 1024),
                   make_smem_desc_sw128(dstb + kk * 2048, HALF_BYTES, 1024), idesc_dq, kk > 0);
        }
        umma_commit(&dq_full[b]);
      }
      umma_commit(acc_full);
    }
  } else {
    const int lg = warp & 3;
    const int grp = (warp - 2) >> 2;   // softmax warpgroup: handles iterations with it % 2 == grp
    const int r = lg * 32 + lane;      // kv row in tile (S^T, dP^T, dK, dV) or d row (dQ^T)
    const int st_tid = threadIdx.x - 64 - grp * 128;  // 0..127 inside the warpgroup
    const int kv_idx = kv0 + r;
    const uint32_t lane_off = uint32_t(lg * 32) << 16;
    const uint32_t st_col = C::ST_COL + 128 * grp, dpt_col = C::DPT_COL + 128 * grp;
    uint8_t* my_pt = sPT + grp * C::PT_BYTES;
    uint8_t* my_dst = sdST + grp * C::PT_BYTES;
    const float* lse = s_lse + grp * 64;
    const float* dlt = s_delta + grp * 64;
    bool ok = true;
    for (int it = grp; it < n_iter && ok; it += 2) {
      const uint32_t ph = (it >> 1) & 1;
      const int head = head0 + it / n_qt;
      const int qt0 = (q_first + it % n_qt) * 64;  // doc-relative first q row of the tile
      // stage lse / delta of the 64 q rows (one buffer per warpgroup; the previous iteration of
      // this group finished reading it before its threads got here: bar.sync below orders that)
      asm volatile("bar.sync %0, 128;" ::"r"(1 + grp) : "memory");
      {
        float* dst = (st_tid < 64 ? s_lse : s_delta) + grp * 64;
        const int i = st_tid & 63;
        const int q = qt0 + i;
        // rows outside the document or outside this rank's q window get lse = +inf -> P = 0
        // staged as -lse (so that P = exp2(S * sl2 + nlse)) and delta * scale
        float val = st_tid < 64 ? -INFINITY : 0.f;
        const long long lrow = (long long)doc_start + q - p.q_row_off;
        if (q < doc_len && lrow >= 0 && lrow < p.q_rows) {
          const long long off = (long long)head * p.q_rows + lrow;
          val = st_tid < 64 ? -p.lse2[off] : p.delta[off] * p.scale;
        }
        dst[i] = val;
      }
      asm volatile("bar.sync %0, 128;" ::"r"(1 + grp) : "memory");
      if (!mbar_wait(&s_full[grp], ph, p.status, AXB_TIMEOUT_TMEM_FULL)) {
        ok = false;
        break;
      }
      tc_fence_after();
      // Only tiles that touch the diagonal or the end of the document need per-element masks
      // (q rows outside the document already carry nlse = -inf, i.e. P = 0).
      const bool need_mask = (!bidir && qt0 < kv0 + 127) || (kv0 + 128 > doc_len) || (win > 0 && qt0 + 63 >= kv0 + win);
      const bool row_in_doc = kv_idx < doc_len;
      // q rows that see this thread's kv row: [q_lo, q_hi] (empty for kv rows beyond the document)
      const int q_lo = row_in_doc ? (bidir ? -(1 << 30) : kv_idx) : (1 << 30);
      const int q_hi = win > 0 ? kv_idx + win - 1 : (1 << 30);
#pragma unroll 1
      for (int c = 0; c < 2; ++c) {
        uint32_t sr[32], dr[32];
        tmem_ld_32x32(tmem_base + lane_off + st_col + c * 32, sr);
        tmem_ld_32x32(tmem_base + lane_off + dpt_col + c * 32, dr);
        tmem_ld_wait();
        uint32_t pk[16], dk[16];
#pragma unroll
        for (int i = 0; i < 32; i += 4) {
          const float4 nl = *reinterpret_cast<const float4*>(lse + c * 32 + i);
          const float4 ds = *reinterpret_cast<const float4*>(dlt + c * 32 + i);
          const float nlv[4] = {nl.x, nl.y, nl.z, nl.w};
          const float dsv[4] = {ds.x, ds.y, ds.z, ds.w};
          float pv[4], dv[4];
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            float pr = fast_exp2(fmaf(__uint_as_float(sr[i + e]), p.sl2, nlv[e]));
            if (need_mask) {
              const int q = qt0 + c * 32 + i + e;
              if (q < q_lo || q > q_hi) pr = 0.f;
            }
            pv[e] = pr;
            dv[e] = pr * fmaf(__uint_as_float(dr[i + e]), p.scale, -dsv[e]);
          }
          pk[i >> 1] = pack_bf16x2(pv[0], pv[1]);
          pk[(i >> 1) + 1] = pack_bf16x2(pv[2], pv[3]);
          dk[i >> 1] = pack_bf16x2(dv[0], dv[1]);
          dk[(i >> 1) + 1] = pack_bf16x2(dv[2], dv[3]);
        }
#pragma unroll
        for (int q = 0; q < 4; ++q) {
          const uint32_t off = sw128_chunk_off(r, c * 4 + q);
          *reinterpret_cast<uint4*>(my_pt + off) =
              make_uint4(pk[q * 4], pk[q * 4 + 1], pk[q * 4 + 2], pk[q * 4 + 3]);
          *reinterpret_cast<uint4*>(my_dst + off) =
              make_uint4(dk[q * 4], dk[q * 4 + 1], dk[q * 4 + 2], dk[q * 4 + 3]);
        }
      }
      tc_fence_before();
      fence_proxy_async_smem();
      mbar_arrive(&pt_full[grp]);
      // drain dQ^T: this thread owns d = r (only rows < D are meaningful)
      if (!mbar_wait(&dq_full[grp], ph, p.status, AXB_TIMEOUT_TMEM_FULL)) {
        ok = false;
        break;
      }
      tc_fence_after();
      {
        // valid q columns of this tile: inside the document and inside this rank's q window
        const long long row0 = (long long)doc_start + qt0 - p.q_row_off;   // local row of column 0
        int i_lo = row0 < 0 ? (int)(-row0) : 0;
        int i_hi = min(64, doc_len - qt0);
        if (row0 + i_hi > p.q_rows) i_hi = (int)(p.q_rows - row0);
        float* col = p.dq_acc + row0 * p.out_ld + (long long)head * D + r;
#pragma unroll 1
        for (int c = 0; c < 2; ++c) {
          uint32_t qr[32];
          tmem_ld_32x32(tmem_base + lane_off + st_col + c * 32, qr);
          tmem_ld_wait();
          if (r < D) {
            if (i_lo <= c * 32 && i_hi >= c * 32 + 32) {
#pragma unroll
              for (int i = 0; i < 32; ++i)
                atomicAdd(col + (long long)(c * 32 + i) * p.out_ld, __uint_as_float(qr[i]));
            } else {
#pragma unroll
              for (int i = 0; i < 32; ++i)
                if (c * 32 + i >= i_lo && c * 32 + i < i_hi)
                  atomicAdd(col + (long long)(c * 32 + i) * p.out_ld, __uint_as_float(qr[i]));
            }
          }
        }
      }
      tc_fence_before();
      mbar_arrive(&st_free[grp]);
    }
    // final dK / dV (warpgroup 0)
    if (grp == 0 && ok && mbar_wait(acc_full, 0, p.status, AXB_TIMEOUT_TMEM_FULL)) {
      tc_fence_after();
      const bool row_ok = kv_idx < doc_len && n_iter > 0;
      const long long grow = (long long)doc_start + kv_idx;  // global kv row
      __nv_bfloat16* base = p.dkv;
      long long brow = grow;
      if (p.cp_world > 1) {
        const long long owner = min(grow / p.cp_chunk, (long long)p.cp_world - 1);
        base = reinterpret_cast<__nv_bfloat16*>(p.cp_dkv_ptrs[owner]);
        brow = grow - owner * p.cp_chunk;
      }
      __nv_bfloat16* krow = base + brow * p.dkv_ld + p.dk_col0 + (long long)kv_head * D;
      __nv_bfloat16* vrow = base + brow * p.dkv_ld + p.dv_col0 + (long long)kv_head * D;
#pragma unroll 1
      for (int c = 0; c < D / 32; ++c) {
        uint32_t a[32], b[32];
        tmem_ld_32x32(tmem_base + lane_off + C::DK_COL + c * 32, a);
        tmem_ld_32x32(tmem_base + lane_off + C::DV_COL + c * 32, b);
        tmem_ld_wait();
        if (row_ok) {
#pragma unroll
          for (int q = 0; q < 4; ++q) {
            uint4 u, w;
            u.x = pack_bf16x2(__uint_as_float(a[q * 8 + 0]), __uint_as_float(a[q * 8 + 1]));
            u.y = pack_bf16x2(__uint_as_float(a[q * 8 + 2]), __uint_as_float(a[q * 8 + 3]));
            u.z = pack_bf16x2(__uint_as_float(a[q * 8 + 4]), __uint_as_float(a[q * 8 + 5]));
            u.w = pack_bf16x2(__uint_as_float(a[q * 8 + 6]), __uint_as_float(a[q * 8 + 7]));
            w.x = pack_bf16x2(__uint_as_float(b[q * 8 + 0]), __uint_as_float(b[q * 8 + 1]));
            w.y = pack_bf16x2(__uint_as_float(b[q * 8 + 2]), __uint_as_float(b[q * 8 + 3]));
            w.z = pack_bf16x2(__uint_as_float(b[q * 8 + 4]), __uint_as_float(b[q * 8 + 5]));
            w.w = pack_bf16x2(__uint_as_float(b[q * 8 + 6]), __uint_as_float(b[q * 8 + 7]));
            if (p.cp_world > 1 || p.kv_split > 1) {
              asm volatile("red.relaxed.sys.global.add.noftz.v4.bf16x2 [%0], {%1, %2, %3, %4};" ::"l"(
                               krow + c * 32 + q * 8),
                           "r"(u.x), "r"(u.y), "r"(u.z), "r"(u.w)
                           : "memory");
              asm volatile("red.relaxed.sys.global.add.noftz.v4.bf16x2 [%0], {%1, %2, %3, %4};" ::"l"(
                               vrow + c * 32 + q * 8),
                           "r"(w.x), "r"(w.y), "r"(w.z), "r"(w.w)
                           : "memory");
            } else {
              *reinterpret_cast<uint4*>(krow + c * 32 + q * 8) = u;
              *reinterpret_cast<uint4*>(vrow + c * 32 + q * 8) = w;
            }
          }
        }
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 2) {
    tc_fence_after();
    tmem_dealloc(tmem_base, C::TMEM_COLS);
  }
}

// dq (bf16, q block of the fused gradient buffer) = dq_acc (fp32)
__global__ void dq_convert_kernel(const float* __restrict__ acc, __nv_bfloat16* __restrict__ dqkv,
                                  long long T, int width, long long acc_ld, long long ld,
                                  int q_col0) {
  const long long n = T * (width / 4);
  for (long long v = (long long)blockIdx.x * blockDim.x + threadIdx.x; v < n;
       v += (long long)gridDim.x * blockDim.x) {
    const long long t = v / (width / 4);
    const int c = (int)(v % (width / 4)) * 4;
    const float4 f = *reinterpret_cast<const float4*>(acc + t * acc_ld + c);
    uint2 u;
    u.x = pack_bf16x2(f.x, f.y);
    u.y = pack_bf16x2(f.z, f.w);
    *reinterpret_cast<uint2*>(dqkv + t * ld + q_col0 + c) = u;
  }
}

template <int D>
int launch_fwd(const CUtensorMap& tq, const CUtensorMap& tm, const AttnParams& p, cudaStream_t st) {
  using C = FwdCfg<D>;
  auto kern = flash_fwd_kernel<D>;
  static bool attr = false;
  if (!attr) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, C::SMEM);
    if (e != cudaSuccess) return (int)e;
    attr = true;
  }
  dim3 grid(p.Hq, p.n_tiles);
  kern<<<grid, kThreads, C::SMEM, st>>>(tq, tm, p);
  return (int)cudaGetLastError();
}
template <int D>
int launch_bwd(const CUtensorMap& tkv, const CUtensorMap& tq, const CUtensorMap& tdo,
               const AttnParams& p, cudaStream_t st) {
  using C = BwdCfg<D>;
  auto kern = flash_bwd_kernel<D>;
  static bool attr = false;
  if (!attr) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, C::SMEM);
    if (e != cudaSuccess) return (int)e;
    attr = true;
  }
  dim3 grid(p.Hk * p.kv_split, p.n_tiles);
  kern<<<grid, kBwdThreads, C::SMEM, st>>>(tkv, tq, tdo, p);
  return (int)cudaGetLastError();
}
}  // namespace

namespace {

struct AttnGeom {
  const void* q_buf;   // rows [q_row_off, q_row_off + q_rows) of the token stream; q heads at q_col0
  long long q_ld;
  long long q_rows;
  int q_row_off;
  const void* kv_buf;  // all kv_rows rows; k heads at k_col0, v heads at v_col0
  long long kv_ld;
  long long kv_rows;
};

int flash_fwd_impl(const AttnGeom& g, int Hq, int Hk, int D, int q_col0, int k_col0, int v_col0,
                   const void* tiles, int n_tiles, void* out, long long out_ld, float* lse2,
                   float softmax_scale, int* status, void* stream) {
  if (g.q_rows <= 0 || n_tiles <= 0) return 0;
  if (D != 64 && D != 128) return -2;
  if ((g.q_ld & 7) || (g.kv_ld & 7) || (out_ld & 7) || (q_col0 & 7) || (k_col0 & 7) || (v_col0 & 7)) return -3;
  CUtensorMap tq, tkv;
  if (axb_make_tmap_2d(&tq, g.q_buf, g.q_rows, g.q_ld, g.q_ld, 128, 64)) return -4;
  if (axb_make_tmap_2d(&tkv, g.kv_buf, g.kv_rows, g.kv_ld, g.kv_ld, 128, 64)) return -4;
  AttnParams p = {};
  p.tiles = reinterpret_cast<const int4*>(tiles);
  p.n_tiles = n_tiles;
  p.Hq = Hq;
  p.Hk = Hk;
  p.q_col0 = q_col0;
  p.k_col0 = k_col0;
  p.v_col0 = v_col0;
  p.out = reinterpret_cast<__nv_bfloat16*>(out);
  p.out_ld = out_ld;
  p.lse2 = lse2;
  p.T = g.q_rows;
  p.kv_rows = g.kv_rows;
  p.q_row_off = g.q_row_off;
  p.q_rows = (int)g.q_rows;
  p.sl2 = softmax_scale * 1.4426950408889634f;
  p.scale = softmax_scale;
  p.status = status;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  return D == 128 ? launch_fwd<128>(tq, tkv, p, st) : launch_fwd<64>(tq, tkv, p, st);
}

int flash_bwd_impl(const AttnGeom& g, const void* dout, const void* out, long long o_ld, const float* lse2,
                   int Hq, int Hk, int D, int q_col0, int k_col0, int v_col0, const void* tiles, int n_tiles,
                   void* dqkv, long long dqkv_ld, int dq_col0, int dk_col0, int dv_col0, float* dq_acc,
                   float* delta, float softmax_scale, int cp_world, long long cp_chunk,
                   const unsigned long long* cp_dkv_ptrs, int* status, void* stream) {
  if (g.q_rows <= 0 || n_tiles <= 0) return 0;
  if (D != 64 && D != 128) return -2;
  if ((g.q_ld & 7) || (g.kv_ld & 7) || (o_ld & 7) || (dqkv_ld & 7) || cp_world > 8) return -3;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  const long long T = g.q_rows;
  CUtensorMap tkv, tq, tdo;
  if (axb_make_tmap_2d(&tkv, g.kv_buf, g.kv_rows, g.kv_ld, g.kv_ld, 128, 64)) return -4;
  if (axb_make_tmap_2d(&tq, g.q_buf, T, g.q_ld, g.q_ld, 64, 64)) return -4;
  if (axb_make_tmap_2d(&tdo, dout, T, (long long)Hq * D, o_ld, 64, 64)) return -4;
  cudaError_t e = cudaMemsetAsync(dq_acc, 0, sizeof(float) * T * Hq * D, st);
  if (e != cudaSuccess) return (int)e;
  {
    const long long warps = T * Hq;
    const int tpb = 256;
    attn_delta_kernel<<<(unsigned)((warps * 32 + tpb - 1) / tpb), tpb, 0, st>>>(
        (const __nv_bfloat16*)dout, (const __nv_bfloat16*)out, delta, T, Hq, D, o_ld, o_ld);
  }
  AttnParams p = {};
  p.tiles = reinterpret_cast<const int4*>(tiles);
  p.n_tiles = n_tiles;
  p.Hq = Hq;
  p.Hk = Hk;
  p.q_col0 = q_col0;
  p.k_col0 = k_col0;
  p.v_col0 = v_col0;
  p.out_ld = (long long)Hq * D;  // leading dimension of dq_acc
  p.lse2 = const_cast<float*>(lse2);
  p.T = T;
  p.kv_rows = g.kv_rows;
  p.q_row_off = g.q_row_off;
  p.q_rows = (int)T;
  p.sl2 = softmax_scale * 1.4426950408889634f;
  p.scale = softmax_scale;
  p.status = status;
  p.delta = delta;
  p.dq_acc = dq_acc;
  p.dkv = reinterpret_cast<__nv_bfloat16*>(dqkv);
  p.dkv_ld = dqkv_ld;
  p.dk_col0 = dk_col0;
  p.dv_col0 = dv_col0;
  p.cp_world = cp_world > 1 ? cp_world : 1;
  p.cp_chunk = cp_chunk;
  // Wide GQA groups: one CTA per (kv tile, kv head) loops over group * q-tiles iterations, and the
  // longest such CTA bounds the launch. Two CTAs per kv head halve it; their dK / dV partials meet
  // in the (zeroed) gradient buffer through bf16x2 reduce-adds.
  p.kv_split = (cp_world <= 1 && Hq / Hk >= 8 && (Hq / Hk) % 2 == 0 && dv_col0 == dk_col0 + Hk * D) ? 2 : 1;
  if (p.kv_split > 1) {
    e = cudaMemset2DAsync(reinterpret_cast<__nv_bfloat16*>(dqkv) + dk_col0, (size_t)dqkv_ld * 2, 0,
                          (size_t)2 * Hk * D * 2, (size_t)g.kv_rows, st);
    if (e != cudaSuccess) return (int)e;
  }
  for (int i = 0; i < 8; ++i) p.cp_dkv_ptrs[i] = (cp_world > 1 && i < cp_world) ? cp_dkv_ptrs[i] : 0ull;
  int rc = D == 128 ? launch_bwd<128>(tkv, tq, tdo, p, st) : launch_bwd<64>(tkv, tq, tdo, p, st);
  if (rc) return rc;
  const long long n = T * (long long)(Hq * D / 4);
  int grid = (int)((n + 255) / 256 > 148 * 16 ? 148 * 16 : (n + 255) / 256);
  dq_convert_kernel<<<grid, 256, 0, st>>>(dq_acc, (__nv_bfloat16*)dqkv, T, Hq * D, (long long)Hq * D, dqkv_ld,
                                          dq_col0);
  return (int)cudaGetLastError();
}

}  // namespace

// qkv: fused projection [T, ld] bf16 with q heads at column q_col0, k heads at k_col0, v at
// v_col0 (head-major, D per head). tiles: device int4 array built by axb_build_attn_tiles
// (tile rows = 128). out: [T, out_ld] bf16, lse2: [Hq, T] fp32.
extern "C" int axb_flash_varlen_fwd(const void* qkv, long long ld, long long T, int Hq, int Hk,
                                    int D, int q_col0, int k_col0, int v_col0, const void* tiles,
                                    int n_tiles, void* out, long long out_ld, float* lse2,
                                    float softmax_scale, int* status, void* stream) {
  AttnGeom g = {qkv, ld, T, 0, qkv, ld, T};
  return flash_fwd_impl(g, Hq, Hk, D, q_col0, k_col0, v_col0, tiles, n_tiles, out, out_ld, lse2,
                        softmax_scale, status, stream);
}

// Backward. dout/out: [T, o_ld] bf16; dqkv: fused gradient buffer with the layout of qkv (all
// three blocks are written); dq_acc: fp32 [T, Hq*D] scratch (zeroed here); delta: fp32 [Hq, T]
// scratch. tiles must have been built with 128-row tiles.
extern "C" int axb_flash_varlen_bwd(const void* qkv, long long ld, const void* dout,
                                    const void* out, long long o_ld, const float* lse2,
                                    long long T, int Hq, int Hk, int D, int q_col0, int k_col0,
                                    int v_col0, const void* tiles, int n_tiles, void* dqkv,
                                    long long dqkv_ld, float* dq_acc, float* delta,
                                    float softmax_scale, int* status, void* stream) {
  AttnGeom g = {qkv, ld, T, 0, qkv, ld, T};
  return flash_bwd_impl(g, dout, out, o_ld, lse2, Hq, Hk, D, q_col0, k_col0, v_col0, tiles, n_tiles, dqkv,
                        dqkv_ld, q_col0, k_col0, v_col0, dq_acc, delta, softmax_scale, 1, 0, nullptr, status,
                        stream);
}

// Context-parallel forward: q rows [q_row_off, q_row_off + q_rows) come from the local fused
// projection `q_buf`; K and V of the WHOLE token stream come from `kv_buf` ([kv_rows, kv_ld], k
// heads at column 0, v heads at Hk*D), which the ranks filled by storing their rows into every
// peer's buffer. tiles: (doc_start, doc_len, tile_start) in GLOBAL rows, only tiles that
// intersect the local q rows. out [q_rows, out_ld], lse2 [Hq, q_rows].
extern "C" int axb_flash_varlen_fwd_cp(const void* q_buf, long long q_ld, long long q_rows, int q_row_off,
                                       const void* kv_buf, long long kv_ld, long long kv_rows, int Hq,
                                       int Hk, int D, const void* tiles, int n_tiles, void* out,
                                       long long out_ld, float* lse2, float softmax_scale, int* status,
                                       void* stream) {
  AttnGeom g = {q_buf, q_ld, q_rows, q_row_off, kv_buf, kv_ld, kv_rows};
  return flash_fwd_impl(g, Hq, Hk, D, 0, 0, Hk * D, tiles, n_tiles, out, out_ld, lse2, softmax_scale, status,
                        stream);
}

// Context-parallel backward: dQ of the local rows goes to the q block of `dqkv` ([q_rows, dqkv_ld],
// fused layout); the dK / dV tiles this rank computes for ANY kv row are reduce-added over NVLink
// into the k / v blocks of the owner's gradient buffer cp_dkv_ptrs[row / cp_chunk] (HOST array of
// peer-mapped addresses, same fused layout, zeroed by the caller before any rank starts).
extern "C" int axb_flash_varlen_bwd_cp(const void* q_buf, long long q_ld, long long q_rows, int q_row_off,
                                       const void* kv_buf, long long kv_ld, long long kv_rows,
                                       const void* dout, const void* out, long long o_ld, const float* lse2,
                                       int Hq, int Hk, int D, const void* tiles, int n_tiles, void* dqkv,
                                       long long dqkv_ld, float* dq_acc, float* delta, float softmax_scale,
                                       int cp_world, long long cp_chunk,
                                       const unsigned long long* cp_dkv_ptrs, int* status, void* stream) {
  AttnGeom g = {q_buf, q_ld, q_rows, q_row_off, kv_buf, kv_ld, kv_rows};
  return flash_bwd_impl(g, dout, out, o_ld, lse2, Hq, Hk, D, 0, 0, Hk * D, tiles, n_tiles, dqkv, dqkv_ld, 0,
                        Hq * D, (Hq + Hk) * D, dq_acc, delta, softmax_scale, cp_world, cp_chunk, cp_dkv_ptrs,
                        status, stream);
}

// ---------------------------------------------------------------------------------------------
// Allocation-free variant of the backward pass (declared and documented in axb_noalloc.h): the
// dQ accumulator and the delta vector live in a fixed device array inside this library instead
// of caller-provided scratch, for callers that cannot allocate device memory.
#include <cstdio>

#include "axb_noalloc.h"

static __device__ __align__(256) float
    g_noalloc_scratch[AXB_NOALLOC_MAX_DQ_FLOATS + AXB_NOALLOC_MAX_DELTA_FLOATS];

namespace {
constexpr int kMaxDevices = 64;
float* g_noalloc_ptr[kMaxDevices] = {nullptr};

void set_err(char* err, int err_len, const char* msg) {
  if (err && err_len > 0) std::snprintf(err, (size_t)err_len, "%s", msg);
}
}  // namespace

extern "C" int axb_flash_varlen_bwd_noalloc(const void* qkv, long long ld, const void* dout,
                                            const void* out, long long o_ld, const float* lse2,
                                            long long T, int Hq, int Hk, int D, int q_col0,
                                            int k_col0, int v_col0, const void* tiles, int n_tiles,
                                            void* dqkv, long long dqkv_ld, float softmax_scale,
                                            int* status, void* stream, char* err, int err_len) {
  if (T < 0 || Hq <= 0 || D <= 0) {
    set_err(err, err_len, "axb_flash_varlen_bwd_noalloc: T must be >= 0 and Hq, D must be positive");
    return AXB_NOALLOC_BAD_SIZE;
  }
  if (T == 0 || n_tiles <= 0) return 0;  // an empty batch: nothing to compute, nothing launched
  const long long dq_floats = T * (long long)Hq * D;
  const long long delta_floats = T * (long long)Hq;
  if (dq_floats > AXB_NOALLOC_MAX_DQ_FLOATS || delta_floats > AXB_NOALLOC_MAX_DELTA_FLOATS) {
    char msg[256];
    std::snprintf(msg, sizeof(msg),
                  "axb_flash_varlen_bwd_noalloc: T*Hq*D = %lld (max %d) or T*Hq = %lld (max %d) "
                  "exceeds the built-in scratch array; use axb_flash_varlen_bwd with your own scratch",
                  dq_floats, AXB_NOALLOC_MAX_DQ_FLOATS, delta_floats, AXB_NOALLOC_MAX_DELTA_FLOATS);
    set_err(err, err_len, msg);
    return AXB_NOALLOC_TOO_LARGE;
  }
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) {
    set_err(err, err_len, "axb_flash_varlen_bwd_noalloc: no current CUDA device");
    return AXB_NOALLOC_SETUP_FAILED;
  }
  if (g_noalloc_ptr[dev] == nullptr) {
    // one-time set-up per device: in host code the array's name is only a stand-in, the kernels
    // need its device address
    float* p = nullptr;
    cudaError_t e = cudaGetSymbolAddress(reinterpret_cast<void**>(&p), g_noalloc_scratch);
    if (e != cudaSuccess || p == nullptr) {
      set_err(err, err_len, cudaGetErrorString(e));
      return AXB_NOALLOC_SETUP_FAILED;
    }
    g_noalloc_ptr[dev] = p;
  }
  float* dq_acc = g_noalloc_ptr[dev];
  float* delta = g_noalloc_ptr[dev] + AXB_NOALLOC_MAX_DQ_FLOATS;
  // the callee clears dq_acc (it must start at zero) and overwrites delta completely
  const int rc = axb_flash_varlen_bwd(qkv, ld, dout, out, o_ld, lse2, T, Hq, Hk, D, q_col0, k_col0,
                                      v_col0, tiles, n_tiles, dqkv, dqkv_ld, dq_acc, delta,
                                      softmax_scale, status, stream);
  if (rc != 0) set_err(err, err_len, "axb_flash_varlen_bwd_noalloc: kernel launch failed");
  return rc;
}
