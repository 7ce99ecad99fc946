// Packed variable-length flash attention for WIDE heads on sm_100a: q/k head width 192 or 256, v head width
// 128 or 256 (Gemma 1/2/3 with head_dim 256; multi-head latent attention with 192-wide q/k and 128-wide v),
// optional tanh soft-capping of the scores (Gemma 2), causal or bidirectional documents, sliding windows.
//
// The 128-wide kernels of flash_varlen.cu keep a whole head in shared memory and TMEM with double buffers;
// at 256 that does not fit (Q + K + V tiles of 128 rows are 192 KB, dK + dV accumulators are all 512 TMEM
// columns). Here every CTA produces one 128-column PART of the outputs and contracts S = Q.K^T (and
// dP = dO.V^T) over the full width:
//   forward   grid (q head, q tile, v part):   S over Dqk, O[:, part] = P . V[:, part]
//   backward  grid (kv head, kv tile, part):   S^T, dP^T over the full widths; dV[:, part], dK[:, part] and
//                                              dQ^T[part, :] for this part only
// so the score GEMMs are computed once per part (1.4x the minimum FLOPs at 256/256) and nothing else grows.
// Stages are single-buffered (shared memory is full); the pipeline still overlaps the K load and the next S
// with the softmax of the current block. Same tile table, same packed fused-projection layout
// [T, Hq*Dqk | Hk*Dqk | Hk*Dv] and the same bounded waits as flash_varlen.cu.
//
// Takes the place of the reference's flash-attn / SDPA paths for these head sizes
// (src/axolotl/monkeypatch/attention/flash_attn_4.py:37-111; Gemma attention soft-capping reaches the
// reference through HF's eager/flash paths selected in src/axolotl/loaders/model.py:560-640).
#include "axb_common.cuh"
#include <type_traits>

namespace {

constexpr int HALF_BYTES = 128 * 128;  // 128 rows x 128 B (64 bf16), swizzled
constexpr int QH_BYTES = 64 * 128;     // 64 rows x 128 B

struct WideParams {
  const int4* tiles;  // (doc_start, doc_len, tile_start, flags: bit 0 bidirectional, bits 1.. sliding window)
  int n_tiles;
  int Hq, Hk;
  int q_col0, k_col0, v_col0;
  __nv_bfloat16* out;  // [T, Hq * Dv]
  long long out_ld;
  float* lse2;         // [Hq, T], log2 domain
  long long T;
  float sl2;           // softmax_scale * log2(e)
  float scale;
  float cap_in;        // soft cap: u = s * cap_in (= scale / cap); effective score (log2 domain) = tanh(u) * cap_out2
  float cap_out2;      // cap * log2(e)
  int* status;
  // backward
  const float* delta;  // [Hq, T]
  float* dq_acc;       // [T, Hq * Dqk] fp32 (atomics)
  long long dq_ld;
  __nv_bfloat16* dkv;  // gradient buffer, same layout as qkv
  long long dkv_ld;
  int dk_col0, dv_col0;
};

AXB_DEVICE float fast_exp2(float x) {
  float y;
  asm volatile("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
AXB_DEVICE uint32_t sw128_chunk_off(int row, int chunk) {
  return (uint32_t)row * 128u + (uint32_t)((chunk ^ (row & 7)) << 4);
}

// =====================================================================================================
// Forward: 192 threads = TMA warp, MMA warp, 4 softmax warps. One CTA per (q head, 128-row q tile, v part).
// =====================================================================================================
template <int DQK>
struct WFwd {
  static constexpr int QK_BYTES = (DQK / 64) * HALF_BYTES;
  static constexpr int V_BYTES = 2 * HALF_BYTES;   // 128 kv rows x 128 v columns of this part
  static constexpr int P_BYTES = 2 * HALF_BYTES;
  static constexpr int SMEM = 2 * QK_BYTES + V_BYTES + P_BYTES + 1024 + 256;
};

template <int DQK, int DV, bool SOFTCAP>
__global__ void __launch_bounds__(192, 1)
    flash_wide_fwd_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_kv,
                          const WideParams p) {
  using C = WFwd<DQK>;
  const int tile_id = blockIdx.y;
  if (tile_id >= p.n_tiles) return;
  const int head = blockIdx.x, part = blockIdx.z;
  const int kv_head = head / (p.Hq / p.Hk);
  const int4 ti = p.tiles[tile_id];
  const int doc_start = ti.x, doc_len = ti.y, q0 = ti.z;
  if (!AXB_INDEX_OK(AXB_SITE_ATTN_TILE, (long long)doc_start + doc_len - 1, p.T) || !AXB_INDEX_OK(AXB_SITE_ATTN_TILE, q0, doc_len)) return;
  const bool bidir = ti.w & 1;
  const int win = bidir ? 0 : (ti.w >> 1);
  const int kv_end = bidir ? doc_len : min(q0 + 128, doc_len);
  const int jb0 = win > 0 ? max(0, q0 - win + 1) / 128 : 0;
  const int n_blocks = (kv_end + 127) / 128 - jb0;

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
  uint8_t* sQ = smem;
  uint8_t* sK = sQ + C::QK_BYTES;
  uint8_t* sV = sK + C::QK_BYTES;
  uint8_t* sP = sV + C::V_BYTES;
  uint64_t* bars = reinterpret_cast<uint64_t*>(sP + C::P_BYTES);
  uint64_t* q_full = bars + 0;
  uint64_t* k_full = bars + 1;
  uint64_t* v_full = bars + 2;
  uint64_t* k_empty = bars + 3;
  uint64_t* v_empty = bars + 4;
  uint64_t* s_full = bars + 5;    // [2]
  uint64_t* s_empty = bars + 7;   // [2]
  uint64_t* p_full = bars + 9;
  uint64_t* p_empty = bars + 10;
  uint64_t* pv_full = bars + 11;  // [2]
  uint64_t* pv_empty = bars + 13; // [2]
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 15);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (threadIdx.x == 0) {
    mbar_init(q_full, 1);
    mbar_init(k_full, 1);
    mbar_init(v_full, 1);
    mbar_init(k_empty, 1);
    mbar_init(v_empty, 1);
    for (int s = 0; s < 2; ++s) {
      mbar_init(&s_full[s], 1);
      mbar_init(&s_empty[s], 128);
      mbar_init(&pv_full[s], 1);
      mbar_init(&pv_empty[s], 128);
    }
    mbar_init(p_full, 128);
    mbar_init(p_empty, 1);
    mbar_fence_init();
    tma_prefetch_desc(&tm_kv);
  }
  if (warp == 2) {
    tmem_alloc(tmem_slot, 512);   // S: 2 x 128 columns at 0; P.V: 2 x 128 columns at 256
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    if (lane == 0) {
      mbar_expect_tx(q_full, C::QK_BYTES);
#pragma unroll
      for (int h = 0; h < DQK / 64; ++h)
        tma_load_2d(sQ + h * HALF_BYTES, &tm_q, q_full, p.q_col0 + head * DQK + h * 64, doc_start + q0);
      for (int j = 0; j < n_blocks; ++j) {
        const uint32_t ph = j & 1;
        if (!mbar_wait(k_empty, ph ^ 1, p.status, AXB_TIMEOUT_EMPTY)) break;
        mbar_expect_tx(k_full, C::QK_BYTES);
#pragma unroll
        for (int h = 0; h < DQK / 64; ++h)
          tma_load_2d(sK + h * HALF_BYTES, &tm_kv, k_full, p.k_col0 + kv_head * DQK + h * 64, doc_start + (jb0 + j) * 128);
        if (!mbar_wait(v_empty, ph ^ 1, p.status, AXB_TIMEOUT_EMPTY)) break;
        mbar_expect_tx(v_full, C::V_BYTES);
#pragma unroll
        for (int h = 0; h < 2; ++h)
          tma_load_2d(sV + h * HALF_BYTES, &tm_kv, v_full, p.v_col0 + kv_head * DV + part * 128 + h * 64,
                      doc_start + (jb0 + j) * 128);
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      constexpr uint32_t idesc_s = make_idesc_bf16(128, 128, 0, 0);
      constexpr uint32_t idesc_pv = make_idesc_bf16(128, 128, 0, 1);
      const uint32_t q_addr = smem_u32(sQ), k_addr = smem_u32(sK), v_addr = smem_u32(sV), p_addr = smem_u32(sP);
      bool ok = mbar_wait(q_full, 0, p.status, AXB_TIMEOUT_FULL);
      auto issue_s = [&](int j) -> bool {
        const int b = j & 1;
        if (!mbar_wait(k_full, j & 1, p.status, AXB_TIMEOUT_FULL)) return false;
        if (!mbar_wait(&s_empty[b], ((j >> 1) & 1) ^ 1, p.status, AXB_TIMEOUT_TMEM_EMPTY)) return false;
        tc_fence_after();
#pragma unroll
        for (int kk = 0; kk < DQK / 16; ++kk) {
          const uint32_t off = (kk / 4) * HALF_BYTES + (kk % 4) * 32;
          umma_f16(tmem_base + b * 128, make_smem_desc_sw128(q_addr + off, 16, 1024),
                   make_smem_desc_sw128(k_addr + off, 16, 1024), idesc_s, kk > 0);
        }
        umma_commit(&s_full[b]);
        umma_commit(k_empty);
        return true;
      };
      if (ok) ok = issue_s(0);
      for (int j = 0; j < n_blocks && ok; ++j) {
        const int b = j & 1;
        if (j + 1 < n_blocks) {
          ok = issue_s(j + 1);
          if (!ok) break;
        }
        if (!mbar_wait(p_full, j & 1, p.status, AXB_TIMEOUT_GENERIC)) break;
        if (!mbar_wait(v_full, j & 1, p.status, AXB_TIMEOUT_FULL)) break;
        if (!mbar_wait(&pv_empty[b], ((j >> 1) & 1) ^ 1, p.status, AXB_TIMEOUT_TMEM_EMPTY)) break;
        tc_fence_after();
#pragma unroll
        for (int kk = 0; kk < 8; ++kk) {
          const uint32_t poff = (kk / 4) * HALF_BYTES + (kk % 4) * 32;
          umma_f16(tmem_base + 256 + b * 128, make_smem_desc_sw128(p_addr + poff, 16, 1024),
                   make_smem_desc_sw128(v_addr + kk * 2048, HALF_BYTES, 1024), idesc_pv, kk > 0);
        }
        umma_commit(&pv_full[b]);
        umma_commit(v_empty);
        umma_commit(p_empty);
      }
    }
  } else {
    const int lg = warp & 3;
    const int r = lg * 32 + lane;
    const int q_idx = q0 + r;
    const uint32_t lane_off = uint32_t(lg * 32) << 16;
    // effective score in the log2 domain
    auto eff = [&](float v) -> float {
      if constexpr (SOFTCAP) return tanhf(v * p.cap_in) * p.cap_out2;
      else return v * p.sl2;
    };
    float m = -INFINITY, l = 0.f, alpha_prev = 1.f;
    float o[128];
#pragma unroll
    for (int i = 0; i < 128; ++i) o[i] = 0.f;
    bool ok = true;
    for (int j = 0; j < n_blocks && ok; ++j) {
      const int b = j & 1;
      const uint32_t ph = (j >> 1) & 1;
      if (!mbar_wait(&s_full[b], ph, p.status, AXB_TIMEOUT_TMEM_FULL)) {
        ok = false;
        break;
      }
      tc_fence_after();
      const uint32_t s_addr = tmem_base + lane_off + b * 128;
      const int kv0 = (jb0 + j) * 128;
      const int lim = (bidir ? doc_len - 1 : min(q_idx, doc_len - 1)) - kv0;
      const int lo = win > 0 ? q_idx - win + 1 - kv0 : -(1 << 30);
      float mx = -INFINITY;
#pragma unroll 1
      for (int c = 0; c < 4; ++c) {
        uint32_t sr[32];
        tmem_ld_32x32(s_addr + c * 32, sr);
        tmem_ld_wait();
#pragma unroll
        for (int i = 0; i < 32; ++i) {
          float v = __uint_as_float(sr[i]);
          if (c * 32 + i > lim || c * 32 + i < lo) v = -INFINITY;
          mx = fmaxf(mx, v);
        }
      }
      const float m_new = fmaxf(m, mx == -INFINITY ? -INFINITY : eff(mx));   // eff is increasing
      const float m_use = (m_new == -INFINITY) ? 0.f : m_new;
      const float alpha = fast_exp2(m - m_use);
      if (!mbar_wait(p_empty, (j & 1) ^ 1, p.status, AXB_TIMEOUT_GENERIC)) {
        ok = false;
        break;
      }
      float rowsum = 0.f;
#pragma unroll 1
      for (int c = 0; c < 4; ++c) {
        uint32_t sr[32];
        tmem_ld_32x32(s_addr + c * 32, sr);
        tmem_ld_wait();
        uint32_t pk[16];
#pragma unroll
        for (int i = 0; i < 32; i += 2) {
          float p0 = fast_exp2(eff(__uint_as_float(sr[i])) - m_use), p1 = fast_exp2(eff(__uint_as_float(sr[i + 1])) - m_use);
          if (c * 32 + i > lim || c * 32 + i < lo) p0 = 0.f;
          if (c * 32 + i + 1 > lim || c * 32 + i + 1 < lo) p1 = 0.f;
          rowsum += p0 + p1;
          pk[i >> 1] = pack_bf16x2(p0, p1);
        }
        uint8_t* pbase = sP + (c >> 1) * HALF_BYTES;
#pragma unroll
        for (int q = 0; q < 4; ++q)
          *reinterpret_cast<uint4*>(pbase + sw128_chunk_off(r, (c & 1) * 4 + q)) =
              make_uint4(pk[q * 4], pk[q * 4 + 1], pk[q * 4 + 2], pk[q * 4 + 3]);
      }
      tc_fence_before();
      mbar_arrive(&s_empty[b]);
      fence_proxy_async_smem();
      mbar_arrive(p_full);
      l = l * alpha + rowsum;
      m = m_new;
      if (j > 0) {
        const int pb = (j - 1) & 1;
        if (!mbar_wait(&pv_full[pb], ((j - 1) >> 1) & 1, p.status, AXB_TIMEOUT_TMEM_FULL)) {
          ok = false;
          break;
        }
        tc_fence_after();
        const uint32_t pv_addr = tmem_base + lane_off + 256 + pb * 128;
#pragma unroll
        for (int c = 0; c < 4; ++c) {
          uint32_t vr[32];
          tmem_ld_32x32(pv_addr + c * 32, vr);
          tmem_ld_wait();
#pragma unroll
          for (int i = 0; i < 32; ++i) o[c * 32 + i] = o[c * 32 + i] * alpha_prev + __uint_as_float(vr[i]);
        }
        tc_fence_before();
        mbar_arrive(&pv_empty[pb]);
      }
      alpha_prev = alpha;
    }
    if (ok && n_blocks > 0) {
      const int pb = (n_blocks - 1) & 1;
      if (mbar_wait(&pv_full[pb], ((n_blocks - 1) >> 1) & 1, p.status, AXB_TIMEOUT_TMEM_FULL)) {
        tc_fence_after();
        const uint32_t pv_addr = tmem_base + lane_off + 256 + pb * 128;
        const float inv_l = l > 0.f ? 1.f / l : 0.f;
        const long long row = (long long)doc_start + q_idx;
        const bool row_ok = q_idx < doc_len && row < p.T;
        __nv_bfloat16* orow = p.out + row * p.out_ld + (long long)head * DV + part * 128;
#pragma unroll
        for (int c = 0; c < 4; ++c) {
          uint32_t vr[32];
          tmem_ld_32x32(pv_addr + c * 32, vr);
          tmem_ld_wait();
          if (row_ok) {
#pragma unroll
            for (int q = 0; q < 4; ++q) {
              float f[8];
#pragma unroll
              for (int i = 0; i < 8; ++i) f[i] = (o[c * 32 + q * 8 + i] * alpha_prev + __uint_as_float(vr[q * 8 + i])) * inv_l;
              uint4 u;
              u.x = pack_bf16x2(f[0], f[1]);
              u.y = pack_bf16x2(f[2], f[3]);
              u.z = pack_bf16x2(f[4], f[5]);
              u.w = pack_bf16x2(f[6], f[7]);
              *reinterpret_cast<uint4*>(orow + c * 32 + q * 8) = u;
            }
          }
        }
        if (row_ok && part == 0) p.lse2[(long long)head * p.T + row] = m + log2f(l);
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 2) {
    tc_fence_after();
    tmem_dealloc(tmem_base, 512);
  }
}

// =====================================================================================================
// Backward: 192 threads = TMA warp, MMA warp, one softmax warpgroup. One CTA per (kv head, 128-row kv tile,
// part); loops over the q heads of the GQA group and the 64-row q tiles that see the kv tile. Per iteration
//   S^T [kv, q] = K . Q^T (over Dqk)      dP^T [kv, q] = V . dO^T (over Dv)
//   dV[:, part] += P^T . dO[:, part]      dK[:, part] += dS^T . Q[:, part]
//   dQ^T[part, q] = K[:, part]^T . dS^T   (fp32 atomics into dq_acc; reuses the TMEM columns of S^T)
// A 192-wide q/k head has the parts [0, 128) and [64, 192): the second stores only its upper 64 columns.
// =====================================================================================================
template <int DQK, int DV>
struct WBwd {
  static constexpr int K_BYTES = (DQK / 64) * HALF_BYTES;
  static constexpr int V_BYTES = (DV / 64) * HALF_BYTES;
  static constexpr int Q_BYTES = (DQK / 64) * QH_BYTES;
  static constexpr int DO_BYTES = (DV / 64) * QH_BYTES;
  static constexpr int PT_BYTES = HALF_BYTES;   // [128 kv x 64 q]
  static constexpr int SMEM = K_BYTES + V_BYTES + Q_BYTES + DO_BYTES + 2 * PT_BYTES + 512 + 128 + 1024;
  static constexpr int ST_COL = 0, DPT_COL = 64, DV_COL = 128, DK_COL = 256;
};

template <int DQK, int DV, bool SOFTCAP>
__global__ void __launch_bounds__(192, 1)
    flash_wide_bwd_kernel(const __grid_constant__ CUtensorMap tm_kv, const __grid_constant__ CUtensorMap tm_q,
                          const __grid_constant__ CUtensorMap tm_do, const WideParams p) {
  using C = WBwd<DQK, DV>;
  const int tile_id = blockIdx.y;
  if (tile_id >= p.n_tiles) return;
  const int kv_head = blockIdx.x, part = blockIdx.z;
  const int group = p.Hq / p.Hk, head0 = kv_head * group;
  const int4 ti = p.tiles[tile_id];
  const int doc_start = ti.x, doc_len = ti.y, kv0 = ti.z;
  if (!AXB_INDEX_OK(AXB_SITE_ATTN_TILE, (long long)doc_start + doc_len - 1, p.T) || !AXB_INDEX_OK(AXB_SITE_ATTN_TILE, kv0, doc_len)) return;
  const bool bidir = ti.w & 1;
  const int win = bidir ? 0 : (ti.w >> 1);
  const int q_first = bidir ? 0 : kv0 / 64;
  int q_last = (doc_len + 63) / 64;
  if (win > 0) q_last = min(q_last, (kv0 + 127 + win - 1) / 64 + 1);
  const int n_qt = q_last - q_first;
  const int n_iter = n_qt * group;
  if (n_iter <= 0) return;
  // column parts of this CTA
  const bool has_k = part * 128 < DQK, has_v = part * 128 < DV;
  const int kpart = has_k ? min(part * 128, DQK - 128) : 0;   // first q/k column of the 128-wide window
  const int k_lo = has_k ? part * 128 - kpart : 128;          // columns of the window below k_lo belong to another part
  const int vpart = has_v ? part * 128 : 0;

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
  uint8_t* sK = smem;
  uint8_t* sV = sK + C::K_BYTES;
  uint8_t* sQ = sV + C::V_BYTES;
  uint8_t* sdO = sQ + C::Q_BYTES;
  uint8_t* sPT = sdO + C::DO_BYTES;
  uint8_t* sdST = sPT + C::PT_BYTES;
  float* s_lse = reinterpret_cast<float*>(sdST + C::PT_BYTES);   // [64]
  float* s_delta = s_lse + 64;                                   // [64]
  uint64_t* bars = reinterpret_cast<uint64_t*>(s_delta + 64);
  uint64_t* kv_full = bars + 0;
  uint64_t* q_full = bars + 1;
  uint64_t* q_empty = bars + 2;
  uint64_t* s_full = bars + 3;
  uint64_t* pt_full = bars + 4;
  uint64_t* dq_full = bars + 5;
  uint64_t* st_free = bars + 6;
  uint64_t* acc_full = bars + 7;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 8);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (threadIdx.x == 0) {
    mbar_init(kv_full, 1);
    mbar_init(q_full, 1);
    mbar_init(q_empty, 1);
    mbar_init(s_full, 1);
    mbar_init(pt_full, 128);
    mbar_init(dq_full, 1);
    mbar_init(st_free, 128);
    mbar_init(acc_full, 1);
    mbar_fence_init();
  }
  if (warp == 2) {
    tmem_alloc(tmem_slot, 512);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    if (lane == 0) {
      mbar_expect_tx(kv_full, C::K_BYTES + C::V_BYTES);
#pragma unroll
      for (int h = 0; h < DQK / 64; ++h)
        tma_load_2d(sK + h * HALF_BYTES, &tm_kv, kv_full, p.k_col0 + kv_head * DQK + h * 64, doc_start + kv0);
#pragma unroll
      for (int h = 0; h < DV / 64; ++h)
        tma_load_2d(sV + h * HALF_BYTES, &tm_kv, kv_full, p.v_col0 + kv_head * DV + h * 64, doc_start + kv0);
      for (int it = 0; it < n_iter; ++it) {
        const int head = head0 + it / n_qt;
        const int qrow = doc_start + (q_first + it % n_qt) * 64;
        if (!mbar_wait(q_empty, (it & 1) ^ 1, p.status, AXB_TIMEOUT_EMPTY)) break;
        mbar_expect_tx(q_full, C::Q_BYTES + C::DO_BYTES);
#pragma unroll
        for (int h = 0; h < DQK / 64; ++h)
          tma_load_2d(sQ + h * QH_BYTES, &tm_q, q_full, p.q_col0 + head * DQK + h * 64, qrow);
#pragma unroll
        for (int h = 0; h < DV / 64; ++h)
          tma_load_2d(sdO + h * QH_BYTES, &tm_do, q_full, head * DV + h * 64, qrow);
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      constexpr uint32_t idesc_st = make_idesc_bf16(128, 64, 0, 0);
      constexpr uint32_t idesc_acc = make_idesc_bf16(128, 128, 0, 1);
      constexpr uint32_t idesc_dq = make_idesc_bf16(128, 64, 1, 1);
      const uint32_t k_addr = smem_u32(sK), v_addr = smem_u32(sV), q_addr = smem_u32(sQ), do_addr = smem_u32(sdO);
      const uint32_t pt_addr = smem_u32(sPT), dst_addr = smem_u32(sdST);
      bool ok = mbar_wait(kv_full, 0, p.status, AXB_TIMEOUT_FULL);
      for (int it = 0; it < n_iter && ok; ++it) {
        const uint32_t ph = it & 1;
        if (!mbar_wait(q_full, ph, p.status, AXB_TIMEOUT_FULL)) break;
        // the S^T columns carried dQ^T of the previous iteration: it must have been drained
        if (it > 0 && !mbar_wait(st_free, (it - 1) & 1, p.status, AXB_TIMEOUT_TMEM_EMPTY)) break;
        tc_fence_after();
#pragma unroll
        for (int kk = 0; kk < DQK / 16; ++kk) {
          const uint32_t koff = (kk / 4) * HALF_BYTES + (kk % 4) * 32, qoff = (kk / 4) * QH_BYTES + (kk % 4) * 32;
          umma_f16(tmem_base + C::ST_COL, make_smem_desc_sw128(k_addr + koff, 16, 1024),
                   make_smem_desc_sw128(q_addr + qoff, 16, 1024), idesc_st, kk > 0);
        }
#pragma unroll
        for (int kk = 0; kk < DV / 16; ++kk) {
          const uint32_t koff = (kk / 4) * HALF_BYTES + (kk % 4) * 32, qoff = (kk / 4) * QH_BYTES + (kk % 4) * 32;
          umma_f16(tmem_base + C::DPT_COL, make_smem_desc_sw128(v_addr + koff, 16, 1024),
                   make_smem_desc_sw128(do_addr + qoff, 16, 1024), idesc_st, kk > 0);
        }
        umma_commit(s_full);
        if (!mbar_wait(pt_full, ph, p.status, AXB_TIMEOUT_GENERIC)) break;
        tc_fence_after();
        if (has_v) {
#pragma unroll
          for (int kk = 0; kk < 4; ++kk)
            umma_f16(tmem_base + C::DV_COL, make_smem_desc_sw128(pt_addr + kk * 32, 16, 1024),
                     make_smem_desc_sw128(do_addr + (vpart / 64) * QH_BYTES + kk * 2048, QH_BYTES, 1024), idesc_acc,
                     (it > 0 || kk > 0));
        }
        if (has_k) {
#pragma unroll
          for (int kk = 0; kk < 4; ++kk)
            umma_f16(tmem_base + C::DK_COL, make_smem_desc_sw128(dst_addr + kk * 32, 16, 1024),
                     make_smem_desc_sw128(q_addr + (kpart / 64) * QH_BYTES + kk * 2048, QH_BYTES, 1024), idesc_acc,
                     (it > 0 || kk > 0));
#pragma unroll
          for (int kk = 0; kk < 8; ++kk)
            umma_f16(tmem_base + C::ST_COL, make_smem_desc_sw128(k_addr + (kpart / 64) * HALF_BYTES + kk * 2048, HALF_BYTES, 1024),
                     make_smem_desc_sw128(dst_addr + kk * 2048, HALF_BYTES, 1024), idesc_dq, kk > 0);
        }
        umma_commit(q_empty);   // Q, dO, P^T, dS^T of this iteration are consumed
        umma_commit(dq_full);
      }
      umma_commit(acc_full);
    }
  } else {
    const int lg = warp & 3;
    const int r = lg * 32 + lane;   // kv row of the tile (S^T, dP^T, dK, dV) or column of the part (dQ^T)
    const int tid = threadIdx.x - 64;
    const int kv_idx = kv0 + r;
    const uint32_t lane_off = uint32_t(lg * 32) << 16;
    bool ok = true;
    for (int it = 0; it < n_iter && ok; ++it) {
      const uint32_t ph = it & 1;
      const int head = head0 + it / n_qt;
      const int qt0 = (q_first + it % n_qt) * 64;
      asm volatile("bar.sync 1, 128;" ::: "memory");   // everyone finished reading the previous lse / delta
      {
        const int i = tid & 63;
        const int q = qt0 + i;
        float val = tid < 64 ? -INFINITY : 0.f;
        const long long row = (long long)doc_start + q;
        if (q < doc_len && row < p.T) {
          const long long off = (long long)head * p.T + row;
          val = tid < 64 ? -p.lse2[off] : p.delta[off] * p.scale;
        }
        (tid < 64 ? s_lse : s_delta)[i] = val;
      }
      asm volatile("bar.sync 1, 128;" ::: "memory");
      if (!mbar_wait(s_full, ph, p.status, AXB_TIMEOUT_TMEM_FULL)) {
        ok = false;
        break;
      }
      tc_fence_after();
      const bool row_in_doc = kv_idx < doc_len;
      const int q_lo = row_in_doc ? (bidir ? -(1 << 30) : kv_idx) : (1 << 30);
      const int q_hi = win > 0 ? kv_idx + win - 1 : (1 << 30);
#pragma unroll 1
      for (int c = 0; c < 2; ++c) {
        uint32_t sr[32], dr[32];
        tmem_ld_32x32(tmem_base + lane_off + C::ST_COL + c * 32, sr);
        tmem_ld_32x32(tmem_base + lane_off + C::DPT_COL + c * 32, dr);
        tmem_ld_wait();
        uint32_t pk[16], dk[16];
#pragma unroll
        for (int i = 0; i < 32; i += 2) {
          float pv[2], dv[2];
#pragma unroll
          for (int e = 0; e < 2; ++e) {
            const float s = __uint_as_float(sr[i + e]);
            const float nl = s_lse[c * 32 + i + e], dl = s_delta[c * 32 + i + e];
            float pr, g = 1.f;
            if constexpr (SOFTCAP) {
              const float t = tanhf(s * p.cap_in);
              pr = fast_exp2(fmaf(t, p.cap_out2, nl));
              g = 1.f - t * t;
            } else {
              pr = fast_exp2(fmaf(s, p.sl2, nl));
            }
            const int q = qt0 + c * 32 + i + e;
            if (q < q_lo || q > q_hi) pr = 0.f;
            pv[e] = pr;
            dv[e] = pr * fmaf(__uint_as_float(dr[i + e]), p.scale, -dl) * g;
          }
          pk[i >> 1] = pack_bf16x2(pv[0], pv[1]);
          dk[i >> 1] = pack_bf16x2(dv[0], dv[1]);
        }
#pragma unroll
        for (int q = 0; q < 4; ++q) {
          const uint32_t off = sw128_chunk_off(r, c * 4 + q);
          *reinterpret_cast<uint4*>(sPT + off) = make_uint4(pk[q * 4], pk[q * 4 + 1], pk[q * 4 + 2], pk[q * 4 + 3]);
          *reinterpret_cast<uint4*>(sdST + off) = make_uint4(dk[q * 4], dk[q * 4 + 1], dk[q * 4 + 2], dk[q * 4 + 3]);
        }
      }
      tc_fence_before();
      fence_proxy_async_smem();
      mbar_arrive(pt_full);
      if (!mbar_wait(dq_full, ph, p.status, AXB_TIMEOUT_TMEM_FULL)) {
        ok = false;
        break;
      }
      tc_fence_after();
      if (has_k) {
        const long long row0 = (long long)doc_start + qt0;
        int i_hi = min(64, doc_len - qt0);
        if (row0 + i_hi > p.T) i_hi = (int)(p.T - row0);
        float* col = p.dq_acc + row0 * p.dq_ld + (long long)head * DQK + kpart + r;
#pragma unroll 1
        for (int c = 0; c < 2; ++c) {
          uint32_t qr[32];
          tmem_ld_32x32(tmem_base + lane_off + C::ST_COL + c * 32, qr);
          tmem_ld_wait();
          if (r >= k_lo) {
#pragma unroll
            for (int i = 0; i < 32; ++i)
              if (c * 32 + i < i_hi) atomicAdd(col + (long long)(c * 32 + i) * p.dq_ld, __uint_as_float(qr[i]));
          }
        }
      }
      tc_fence_before();
      mbar_arrive(st_free);
    }
    if (ok && mbar_wait(acc_full, 0, p.status, AXB_TIMEOUT_TMEM_FULL)) {
      tc_fence_after();
      const bool row_ok = kv_idx < doc_len;
      const long long grow = (long long)doc_start + kv_idx;
      __nv_bfloat16* krow = p.dkv + grow * p.dkv_ld + p.dk_col0 + (long long)kv_head * DQK + kpart;
      __nv_bfloat16* vrow = p.dkv + grow * p.dkv_ld + p.dv_col0 + (long long)kv_head * DV + vpart;
#pragma unroll 1
      for (int c = 0; c < 4; ++c) {
        uint32_t a[32], b[32];
        tmem_ld_32x32(tmem_base + lane_off + C::DK_COL + c * 32, a);
        tmem_ld_32x32(tmem_base + lane_off + C::DV_COL + c * 32, b);
        tmem_ld_wait();
        if (row_ok) {
#pragma unroll
          for (int q = 0; q < 4; ++q) {
            if (has_k && c * 32 + q * 8 >= k_lo) {
              uint4 u;
              u.x = pack_bf16x2(__uint_as_float(a[q * 8 + 0]), __uint_as_float(a[q * 8 + 1]));
              u.y = pack_bf16x2(__uint_as_float(a[q * 8 + 2]), __uint_as_float(a[q * 8 + 3]));
              u.z = pack_bf16x2(__uint_as_float(a[q * 8 + 4]), __uint_as_float(a[q * 8 + 5]));
              u.w = pack_bf16x2(__uint_as_float(a[q * 8 + 6]), __uint_as_float(a[q * 8 + 7]));
              *reinterpret_cast<uint4*>(krow + c * 32 + q * 8) = u;
            }
            if (has_v) {
              uint4 w;
              w.x = pack_bf16x2(__uint_as_float(b[q * 8 + 0]), __uint_as_float(b[q * 8 + 1]));
              w.y = pack_bf16x2(__uint_as_float(b[q * 8 + 2]), __uint_as_float(b[q * 8 + 3]));
              w.z = pack_bf16x2(__uint_as_float(b[q * 8 + 4]), __uint_as_float(b[q * 8 + 5]));
              w.w = pack_bf16x2(__uint_as_float(b[q * 8 + 6]), __uint_as_float(b[q * 8 + 7]));
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
    tmem_dealloc(tmem_base, 512);
  }
}

__global__ void wide_delta_kernel(const __nv_bfloat16* __restrict__ dout, const __nv_bfloat16* __restrict__ out,
                                  float* __restrict__ delta, long long T, int Hq, int D, long long ld) {
  const long long gw = ((long long)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (gw >= T * Hq) return;
  const long long t = gw / Hq;
  const int h = (int)(gw % Hq);
  const __nv_bfloat16* a = dout + t * ld + (long long)h * D;
  const __nv_bfloat16* b = out + t * ld + (long long)h * D;
  float s = 0.f;
  for (int i = lane * 2; i < D; i += 64) {
    const float2 x = unpack_bf16x2(*reinterpret_cast<const uint32_t*>(a + i));
    const float2 y = unpack_bf16x2(*reinterpret_cast<const uint32_t*>(b + i));
    s += x.x * y.x + x.y * y.y;
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
  if (lane == 0) delta[(long long)h * T + t] = s;
}

__global__ void wide_dq_convert_kernel(const float* __restrict__ acc, __nv_bfloat16* __restrict__ dqkv, long long T,
                                       int width, long long ld, int q_col0) {
  const long long n = T * (width / 4);
  for (long long v = (long long)blockIdx.x * blockDim.x + threadIdx.x; v < n; v += (long long)gridDim.x * blockDim.x) {
    const long long t = v / (width / 4);
    const int c = (int)(v % (width / 4)) * 4;
    const float4 f = *reinterpret_cast<const float4*>(acc + t * width + c);
    uint2 u;
    u.x = pack_bf16x2(f.x, f.y);
    u.y = pack_bf16x2(f.z, f.w);
    *reinterpret_cast<uint2*>(dqkv + t * ld + q_col0 + c) = u;
  }
}

template <int DQK, int DV, bool SC>
int launch_wide_fwd(const CUtensorMap& tq, const CUtensorMap& tkv, const WideParams& p, cudaStream_t st) {
  auto kern = flash_wide_fwd_kernel<DQK, DV, SC>;
  static bool attr = false;
  if (!attr) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, WFwd<DQK>::SMEM);
    if (e != cudaSuccess) return (int)e;
    attr = true;
  }
  dim3 grid(p.Hq, p.n_tiles, DV / 128);
  kern<<<grid, 192, WFwd<DQK>::SMEM, st>>>(tq, tkv, p);
  return (int)cudaGetLastError();
}
template <int DQK, int DV, bool SC>
int launch_wide_bwd(const CUtensorMap& tkv, const CUtensorMap& tq, const CUtensorMap& tdo, const WideParams& p,
                    cudaStream_t st) {
  using C = WBwd<DQK, DV>;
  auto kern = flash_wide_bwd_kernel<DQK, DV, SC>;
  static bool attr = false;
  if (!attr) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, C::SMEM);
    if (e != cudaSuccess) return (int)e;
    attr = true;
  }
  constexpr int pk = (DQK + 127) / 128, pv = (DV + 127) / 128;
  constexpr int parts = pk > pv ? pk : pv;
  dim3 grid(p.Hk, p.n_tiles, parts);
  kern<<<grid, 192, C::SMEM, st>>>(tkv, tq, tdo, p);
  return (int)cudaGetLastError();
}

void fill_common(WideParams& p, const void* tiles, int n_tiles, int Hq, int Hk, int q_col0, int k_col0, int v_col0,
                 long long T, float scale, float softcap, int* status) {
  p.tiles = reinterpret_cast<const int4*>(tiles);
  p.n_tiles = n_tiles;
  p.Hq = Hq;
  p.Hk = Hk;
  p.q_col0 = q_col0;
  p.k_col0 = k_col0;
  p.v_col0 = v_col0;
  p.T = T;
  p.scale = scale;
  p.sl2 = scale * 1.4426950408889634f;
  p.cap_in = softcap > 0.f ? scale / softcap : 0.f;
  p.cap_out2 = softcap * 1.4426950408889634f;
  p.status = status;
}

}  // namespace

// qkv [T, Hq*Dqk | Hk*Dqk | Hk*Dv] bf16 (column offsets given), out [T, Hq*Dv], lse2 [Hq, T] fp32.
// (Dqk, Dv) in {(256, 256), (192, 128)}; softcap 0 = none.
extern "C" int axb_flash_wide_fwd(const void* qkv, long long ld, long long T, int Hq, int Hk, int Dqk, int Dv,
                                  int q_col0, int k_col0, int v_col0, const void* tiles, int n_tiles, void* out,
                                  long long out_ld, float* lse2, float softmax_scale, float softcap, int* status,
                                  void* stream) {
  if (T <= 0 || n_tiles <= 0) return 0;
  if (!((Dqk == 256 && Dv == 256) || (Dqk == 192 && Dv == 128))) return -2;
  if ((ld & 7) || (out_ld & 7) || (q_col0 & 7) || (k_col0 & 7) || (v_col0 & 7) || Hk <= 0 || Hq % Hk) return -3;
  CUtensorMap tq;
  if (axb_make_tmap_2d(&tq, qkv, T, ld, ld, 128, 64)) return -4;
  WideParams p = {};
  fill_common(p, tiles, n_tiles, Hq, Hk, q_col0, k_col0, v_col0, T, softmax_scale, softcap, status);
  p.out = reinterpret_cast<__nv_bfloat16*>(out);
  p.out_ld = out_ld;
  p.lse2 = lse2;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  const bool sc = softcap > 0.f;
  if (Dqk == 256) return sc ? launch_wide_fwd<256, 256, true>(tq, tq, p, st) : launch_wide_fwd<256, 256, false>(tq, tq, p, st);
  return sc ? launch_wide_fwd<192, 128, true>(tq, tq, p, st) : launch_wide_fwd<192, 128, false>(tq, tq, p, st);
}

// dout / out [T, Hq*Dv] (ld o_ld); dqkv same layout as qkv; dq_acc fp32 [T, Hq*Dqk] and delta fp32 [Hq, T] scratch.
extern "C" int axb_flash_wide_bwd(const void* qkv, long long ld, const void* dout, const void* out, long long o_ld,
                                  const float* lse2, long long T, int Hq, int Hk, int Dqk, int Dv, int q_col0,
                                  int k_col0, int v_col0, const void* tiles, int n_tiles, void* dqkv,
                                  long long dqkv_ld, float* dq_acc, float* delta, float softmax_scale, float softcap,
                                  int* status, void* stream) {
  if (T <= 0 || n_tiles <= 0) return 0;
  if (!((Dqk == 256 && Dv == 256) || (Dqk == 192 && Dv == 128))) return -2;
  if ((ld & 7) || (o_ld & 7) || (dqkv_ld & 7) || (q_col0 & 7) || (k_col0 & 7) || (v_col0 & 7) || Hk <= 0 || Hq % Hk) return -3;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  CUtensorMap tkv, tq, tdo;
  if (axb_make_tmap_2d(&tkv, qkv, T, ld, ld, 128, 64)) return -4;
  if (axb_make_tmap_2d(&tq, qkv, T, ld, ld, 64, 64)) return -4;
  if (axb_make_tmap_2d(&tdo, dout, T, (long long)Hq * Dv, o_ld, 64, 64)) return -4;
  cudaError_t e = cudaMemsetAsync(dq_acc, 0, sizeof(float) * T * Hq * Dqk, st);
  if (e != cudaSuccess) return (int)e;
  {
    const long long warps = T * Hq;
    wide_delta_kernel<<<(unsigned)((warps * 32 + 255) / 256), 256, 0, st>>>(
        (const __nv_bfloat16*)dout, (const __nv_bfloat16*)out, delta, T, Hq, Dv, o_ld);
  }
  WideParams p = {};
  fill_common(p, tiles, n_tiles, Hq, Hk, q_col0, k_col0, v_col0, T, softmax_scale, softcap, status);
  p.lse2 = const_cast<float*>(lse2);
  p.delta = delta;
  p.dq_acc = dq_acc;
  p.dq_ld = (long long)Hq * Dqk;
  p.dkv = reinterpret_cast<__nv_bfloat16*>(dqkv);
  p.dkv_ld = dqkv_ld;
  p.dk_col0 = k_col0;
  p.dv_col0 = v_col0;
  const bool sc = softcap > 0.f;
  int rc;
  if (Dqk == 256) rc = sc ? launch_wide_bwd<256, 256, true>(tkv, tq, tdo, p, st) : launch_wide_bwd<256, 256, false>(tkv, tq, tdo, p, st);
  else rc = sc ? launch_wide_bwd<192, 128, true>(tkv, tq, tdo, p, st) : launch_wide_bwd<192, 128, false>(tkv, tq, tdo, p, st);
  if (rc) return rc;
  const long long n = T * (long long)(Hq * Dqk / 4);
  const int grid = (int)((n + 255) / 256 > 148 * 16 ? 148 * 16 : (n + 255) / 256);
  wide_dq_convert_kernel<<<grid, 256, 0, st>>>(dq_acc, (__nv_bfloat16*)dqkv, T, Hq * Dqk, dqkv_ld, q_col0);
  return (int)cudaGetLastError();
}
