// Grouped bf16 GEMMs for mixture-of-experts layers on sm_100a: one persistent tcgen05 kernel runs
// the GEMMs of ALL experts of a layer in a single launch.
//
// Token rows are sorted by expert and every expert's segment is padded (with zero rows) to a
// multiple of 128 rows, so a 128-row M tile never straddles two experts. The layout lives in
// device memory (built without any host synchronisation):
//   blk_expert[b]  expert of 128-row block b          n_blocks[0]  blocks in use
//   seg_start[e]   first row of expert e's segment    seg_rows[e]  padded rows of that segment
//
// Three modes share the TMA -> smem ring -> tcgen05.mma -> TMEM -> epilogue pipeline:
//   FWD   C[rows, N]   = alpha * (A[rows, K] . W[e]^T + A2[rows, K2] . W2[e]^T)  W: [E, N, K]
//   DX    C[rows, N]   = alpha * (A[rows, K] . W[e]   + A2[rows, K2] . W2[e])    W: [E, K, N]
//   GRAM  C[e][Mg, Ng] = alpha * sum over the rows of segment e of A[row, :]^T B[row, :]
// FWD is the expert projection with the LoRA update as K-extension, DX its input gradient, GRAM
// the per-expert weight / adapter gradients. They replace the reference's Triton scatter2scatter
// and groupXtY kernels (src/axolotl/integrations/kernels/libs/scattermoe_lora/kernels/ops.py:17-683,
// lora_ops.py:251-2370), which loop over experts inside a tile scheduler driven by sorted indices.
#include "axb_common.cuh"

namespace {

constexpr int BM = 128;
constexpr int BK = 64;
constexpr int kThreads = 192;
constexpr int kSmemBudget = 220 * 1024;

enum Mode { FWD = 0, DX = 1, GRAM = 2 };

struct GParams {
  int N, K, K2;       // FWD / DX: output columns, contraction, K-extension. GRAM: N = Ng
  int Mg;             // GRAM: rows of every output matrix
  int E;
  void* C;
  long long ldc;
  long long c_batch;  // GRAM: elements between consecutive output matrices
  float alpha;
  int out_mode;       // 0 bf16 store, 1 fp32 store, 2 fp32 accumulate (C += result)
  const int* blk_expert;
  const int* n_blocks;
  const int* seg_start;
  const int* seg_rows;
  int* status;
};

template <int BN>
struct Cfg {
  static constexpr int A_BYTES = BM * BK * 2;
  static constexpr int B_BYTES = BN * BK * 2;
  static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
  static constexpr int STAGES =
      (kSmemBudget - 1024) / STAGE_BYTES > 8 ? 8 : (kSmemBudget - 1024) / STAGE_BYTES;
  static constexpr int TMEM_COLS = 2 * BN < 32 ? 32 : 2 * BN;
  static constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + 1024 + 256;
};

struct Tile {
  int m0, n0, k0, nk_main, nk_ext, zb, m_lim;
  long long c_off;
};

// Every role decodes the same tile sequence; a tile with no K blocks (empty expert in GRAM mode)
// is handled by the epilogue alone and uses no accumulator.
template <int BN, int MODE>
__device__ __forceinline__ bool decode(const GParams& p, int tile, int n_blocks, Tile& t) {
  const int num_n = (p.N + BN - 1) / BN;
  if (MODE == GRAM) {
    const int num_m = (p.Mg + BM - 1) / BM;
    const int per_e = num_m * num_n;
    if (tile >= p.E * per_e) return false;
    const int e = tile / per_e;
    const int r = tile - e * per_e;
    t.m0 = (r / num_n) * BM;
    t.n0 = (r % num_n) * BN;
    t.k0 = p.seg_start[e];
    t.nk_main = p.seg_rows[e] / BK;
    t.nk_ext = 0;
    t.zb = 0;
    t.m_lim = p.Mg;
    t.c_off = (long long)e * p.c_batch;
  } else {
    if (tile >= n_blocks * num_n) return false;
    const int blk = tile / num_n;
    t.m0 = blk * BM;
    t.n0 = (tile - blk * num_n) * BN;
    t.k0 = 0;
    t.nk_main = (p.K + BK - 1) / BK;
    t.nk_ext = (p.K2 + BK - 1) / BK;
    t.zb = p.blk_expert[blk];
    if (!AXB_INDEX_OK(AXB_SITE_GROUPED_EXPERT, t.zb, p.E)) return false;   // checked build: stop this CTA's tile loop
    t.m_lim = t.m0 + BM;
    t.c_off = 0;
  }
  return true;
}

template <int BN, int MODE>
__global__ void __launch_bounds__(kThreads, 1)
    grouped_gemm_kernel(const __grid_constant__ CUtensorMap tmA,
                        const __grid_constant__ CUtensorMap tmB,
                        const __grid_constant__ CUtensorMap tmA2,
                        const __grid_constant__ CUtensorMap tmB2, const GParams p) {
  using C = Cfg<BN>;
  constexpr bool A_MN = MODE == GRAM;
  constexpr bool B_MN = MODE != FWD;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~static_cast<uintptr_t>(1023));
  uint8_t* sA = smem;
  uint8_t* sB = smem + C::STAGES * C::A_BYTES;
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + C::STAGES * C::STAGE_BYTES);
  uint64_t* full_bar = bars;
  uint64_t* empty_bar = bars + C::STAGES;
  uint64_t* tfull_bar = bars + 2 * C::STAGES;
  uint64_t* tempty_bar = bars + 2 * C::STAGES + 2;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * C::STAGES + 4);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int n_blocks = MODE == GRAM ? 0 : *p.n_blocks;

  if (threadIdx.x == 0) {
    for (int s = 0; s < C::STAGES; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 1);
    }
    for (int s = 0; s < 2; ++s) {
      mbar_init(&tfull_bar[s], 1);
      mbar_init(&tempty_bar[s], 4);
    }
    mbar_fence_init();
    tma_prefetch_desc(&tmA);
    tma_prefetch_desc(&tmB);
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
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      Tile t;
      for (int tile = blockIdx.x; ok && decode<BN, MODE>(p, tile, n_blocks, t); tile += gridDim.x) {
        const int nk = t.nk_main + t.nk_ext;
        for (int kb = 0; kb < nk; ++kb) {
          if (!mbar_wait(&empty_bar[stage], phase ^ 1, p.status, AXB_TIMEOUT_EMPTY)) {
            ok = false;
            break;
          }
          mbar_expect_tx(&full_bar[stage], C::STAGE_BYTES);
          const bool ext = kb >= t.nk_main;
          const CUtensorMap* ma = ext ? &tmA2 : &tmA;
          const CUtensorMap* mb = ext ? &tmB2 : &tmB;
          const int k = ext ? (kb - t.nk_main) * BK : t.k0 + kb * BK;
          uint8_t* a_dst = sA + stage * C::A_BYTES;
          uint8_t* b_dst = sB + stage * C::B_BYTES;
          if (!A_MN) {
            tma_load_2d(a_dst, ma, &full_bar[stage], k, t.m0);
          } else {
#pragma unroll
            for (int c = 0; c < BM / 64; ++c)
              tma_load_2d(a_dst + c * 8192, ma, &full_bar[stage], t.m0 + c * 64, k);
          }
          if (!B_MN) {
            tma_load_3d(b_dst, mb, &full_bar[stage], k, t.n0, t.zb);
          } else {
#pragma unroll
            for (int c = 0; c < BN / 64; ++c)
              tma_load_3d(b_dst + c * 8192, mb, &full_bar[stage], t.n0 + c * 64, k, t.zb);
          }
          if (++stage == C::STAGES) {
            stage = 0;
            phase ^= 1;
          }
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      constexpr uint32_t idesc = make_idesc_bf16(BM, BN, A_MN ? 1 : 0, B_MN ? 1 : 0);
      int stage = 0;
      uint32_t phase = 0;
      int it = 0;
      bool ok = true;
      Tile t;
      for (int tile = blockIdx.x; ok && decode<BN, MODE>(p, tile, n_blocks, t); tile += gridDim.x) {
        const int nk = t.nk_main + t.nk_ext;
        if (nk == 0) continue;
        const int acc = it & 1;
        const uint32_t acc_phase = (it >> 1) & 1;
        ++it;
        if (!mbar_wait(&tempty_bar[acc], acc_phase ^ 1, p.status, AXB_TIMEOUT_TMEM_EMPTY)) break;
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + acc * BN;
        for (int kb = 0; kb < nk; ++kb) {
          if (!mbar_wait(&full_bar[stage], phase, p.status, AXB_TIMEOUT_FULL)) {
            ok = false;
            break;
          }
          tc_fence_after();
          const uint32_t a_addr = smem_u32(sA + stage * C::A_BYTES);
          const uint32_t b_addr = smem_u32(sB + stage * C::B_BYTES);
#pragma unroll
          for (int kk = 0; kk < BK / 16; ++kk) {
            const uint64_t da = A_MN ? make_smem_desc_sw128(a_addr + kk * 2048, 8192, 1024)
                                     : make_smem_desc_sw128(a_addr + kk * 32, 16, 1024);
            const uint64_t db = B_MN ? make_smem_desc_sw128(b_addr + kk * 2048, 8192, 1024)
                                     : make_smem_desc_sw128(b_addr + kk * 32, 16, 1024);
            umma_f16(d_tmem, da, db, idesc, (kb > 0 || kk > 0) ? 1u : 0u);
          }
          umma_commit(&empty_bar[stage]);
          if (++stage == C::STAGES) {
            stage = 0;
            phase ^= 1;
          }
        }
        if (!ok) break;
        umma_commit(&tfull_bar[acc]);
      }
    }
  } else {
    const int lane_group = warp & 3;
    int it = 0;
    bool ok = true;
    Tile t;
    for (int tile = blockIdx.x; ok && decode<BN, MODE>(p, tile, n_blocks, t); tile += gridDim.x) {
      const int nk = t.nk_main + t.nk_ext;
      int acc = 0;
      if (nk > 0) {
        acc = it & 1;
        const uint32_t acc_phase = (it >> 1) & 1;
        ++it;
        if (!mbar_wait(&tfull_bar[acc], acc_phase, p.status, AXB_TIMEOUT_TMEM_FULL)) break;
        tc_fence_after();
      } else if (p.out_mode == 2) {
        continue;  // nothing to add
      }
      const long long row = (long long)t.m0 + lane_group * 32 + lane;
      const bool row_ok = row < t.m_lim;
      const uint32_t t_addr = tmem_base + (uint32_t(lane_group * 32) << 16) + acc * BN;
#pragma unroll 1
      for (int c = 0; c < BN / 32; ++c) {
        uint32_t r[32];
        if (nk > 0) {
          tmem_ld_32x32(t_addr + c * 32, r);
          tmem_ld_wait();
        } else {
#pragma unroll
          for (int j = 0; j < 32; ++j) r[j] = 0u;
        }
        const int col0 = t.n0 + c * 32;
        if (!row_ok || col0 >= p.N) continue;
        float v[32];
#pragma unroll
        for (int j = 0; j < 32; ++j) v[j] = __uint_as_float(r[j]) * p.alpha;
        const bool full_chunk = col0 + 32 <= p.N;
        const long long off = t.c_off + row * p.ldc + col0;
        if (p.out_mode == 0) {
          __nv_bfloat16* crow = reinterpret_cast<__nv_bfloat16*>(p.C) + off;
          if (full_chunk && (p.ldc & 7) == 0) {
#pragma unroll
            for (int q = 0; q < 4; ++q) {
              uint4 o;
              o.x = pack_bf16x2(v[q * 8 + 0], v[q * 8 + 1]);
              o.y = pack_bf16x2(v[q * 8 + 2], v[q * 8 + 3]);
              o.z = pack_bf16x2(v[q * 8 + 4], v[q * 8 + 5]);
              o.w = pack_bf16x2(v[q * 8 + 6], v[q * 8 + 7]);
              *reinterpret_cast<uint4*>(crow + q * 8) = o;
            }
          } else {
            for (int j = 0; j < 32 && col0 + j < p.N; ++j) crow[j] = __float2bfloat16(v[j]);
          }
        } else {
          float* crow = reinterpret_cast<float*>(p.C) + off;
          const bool add = p.out_mode == 2;
          if (full_chunk && (p.ldc & 3) == 0 && (t.c_off & 3) == 0) {
#pragma unroll
            for (int q = 0; q < 8; ++q) {
              float4 o = make_float4(v[q * 4], v[q * 4 + 1], v[q * 4 + 2], v[q * 4 + 3]);
              if (add) {
                const float4 in = *reinterpret_cast<const float4*>(crow + q * 4);
                o.x += in.x;
                o.y += in.y;
                o.z += in.z;
                o.w += in.w;
              }
              *reinterpret_cast<float4*>(crow + q * 4) = o;
            }
          } else {
            for (int j = 0; j < 32 && col0 + j < p.N; ++j) crow[j] = v[j] + (add ? crow[j] : 0.f);
          }
        }
      }
      if (nk > 0) {
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(&tempty_bar[acc]);
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

int g_sms = 0;
int sm_count() {
  if (g_sms == 0) {
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&g_sms, cudaDevAttrMultiProcessorCount, dev);
    if (g_sms <= 0) g_sms = 148;
  }
  return g_sms;
}

template <int BN, int MODE>
int launch(const CUtensorMap& tA, const CUtensorMap& tB, const CUtensorMap& tA2,
           const CUtensorMap& tB2, const GParams& p, int max_tiles, cudaStream_t stream) {
  using C = Cfg<BN>;
  auto kern = grouped_gemm_kernel<BN, MODE>;
  static bool attr_set = false;
  if (!attr_set) {
    cudaError_t e =
        cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, C::SMEM_BYTES);
    if (e != cudaSuccess) return (int)e;
    attr_set = true;
  }
  int grid = sm_count();
  if (max_tiles < grid) grid = max_tiles;
  if (grid < 1) return 0;
  kern<<<grid, kThreads, C::SMEM_BYTES, stream>>>(tA, tB, tA2, tB2, p);
  return (int)cudaGetLastError();
}

template <int MODE>
int launch_bn(int bn, const CUtensorMap& tA, const CUtensorMap& tB, const CUtensorMap& tA2,
              const CUtensorMap& tB2, const GParams& p, int max_tiles, cudaStream_t stream) {
  switch (bn) {
    case 64:
      return launch<64, MODE>(tA, tB, tA2, tB2, p, max_tiles, stream);
    case 128:
      return launch<128, MODE>(tA, tB, tA2, tB2, p, max_tiles, stream);
    case 256:
      return launch<256, MODE>(tA, tB, tA2, tB2, p, max_tiles, stream);
    default:
      return -5;
  }
}

}  // namespace

// Expert projections over padded, expert-sorted rows.
//   trans_w = 0: C[rows, N] = alpha * (A . W[e]^T + A2 . W2[e]^T),  W [E, N, K],  W2 [E, N, K2]
//   trans_w = 1: C[rows, N] = alpha * (A . W[e]   + A2 . W2[e]),    W [E, K, N],  W2 [E, K2, N]
// A [max_rows, K] (lda), A2 [max_rows, K2] (lda2) or NULL; max_rows = 128 * max_blocks.
// All leading dimensions in elements and multiples of 8. out_mode 0 bf16 / 1 fp32 / 2 fp32 +=.
extern "C" int axb_grouped_gemm(const void* A, long long lda, const void* W, const void* A2,
                                long long lda2, const void* W2, void* C, long long ldc, int E,
                                int N, int K, int K2, int trans_w, float alpha, int out_mode,
                                int bn, const int* blk_expert, const int* n_blocks,
                                int max_blocks, int* status, void* stream) {
  if (max_blocks <= 0 || N <= 0 || K <= 0) return 0;
  if ((lda & 7) || (K & 7) || (N & 7) || (K2 > 0 && ((lda2 & 7) || (K2 & 7)))) return -2;
  const unsigned long long rows = (unsigned long long)max_blocks * BM;
  CUtensorMap tA, tB, tA2, tB2;
  int rc = axb_make_tmap_2d(&tA, A, rows, K, lda, BM, 64);
  if (!trans_w)
    rc |= axb_make_tmap_3d(&tB, W, E, N, K, K, (unsigned long long)N * K, bn, 64);
  else
    rc |= axb_make_tmap_3d(&tB, W, E, K, N, N, (unsigned long long)N * K, 64, 64);
  if (K2 > 0) {
    rc |= axb_make_tmap_2d(&tA2, A2, rows, K2, lda2, BM, 64);
    if (!trans_w)
      rc |= axb_make_tmap_3d(&tB2, W2, E, N, K2, K2, (unsigned long long)N * K2, bn, 64);
    else
      rc |= axb_make_tmap_3d(&tB2, W2, E, K2, N, N, (unsigned long long)N * K2, 64, 64);
  } else {
    tA2 = tA;
    tB2 = tB;
  }
  if (rc) return -4;
  GParams p = {};
  p.N = N;
  p.K = K;
  p.K2 = K2 > 0 ? K2 : 0;
  p.E = E;
  p.C = C;
  p.ldc = ldc;
  p.alpha = alpha;
  p.out_mode = out_mode;
  p.blk_expert = blk_expert;
  p.n_blocks = n_blocks;
  p.status = status;
  const int max_tiles = max_blocks * ((N + bn - 1) / bn);
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  return trans_w ? launch_bn<DX>(bn, tA, tB, tA2, tB2, p, max_tiles, st)
                 : launch_bn<FWD>(bn, tA, tB, tA2, tB2, p, max_tiles, st);
}

// Per-expert Gram products: C[e] [Mg, Ng] = alpha * A[seg_e, :Mg]^T . B[seg_e, :Ng] over the rows of
// expert e's padded segment (pad rows must be zero). A [rows, Mg] (lda), B [rows, Ng] (ldb),
// C [E, Mg, Ng] with row stride ldc and matrix stride c_batch (elements).
extern "C" int axb_grouped_gram(const void* A, long long lda, const void* B, long long ldb, void* C,
                                long long ldc, long long c_batch, int E, int Mg, int Ng,
                                long long rows, float alpha, int out_mode, int bn,
                                const int* seg_start, const int* seg_rows, int* status,
                                void* stream) {
  if (E <= 0 || Mg <= 0 || Ng <= 0 || rows <= 0) return 0;
  if ((lda & 7) || (ldb & 7) || out_mode == 0) return -2;
  CUtensorMap tA, tB;
  int rc = axb_make_tmap_2d(&tA, A, rows, Mg, lda, 64, 64);
  rc |= axb_make_tmap_3d(&tB, B, 1, rows, Ng, ldb, (unsigned long long)rows * ldb, 64, 64);
  if (rc) return -4;
  GParams p = {};
  p.N = Ng;
  p.Mg = Mg;
  p.E = E;
  p.C = C;
  p.ldc = ldc;
  p.c_batch = c_batch;
  p.alpha = alpha;
  p.out_mode = out_mode;
  p.seg_start = seg_start;
  p.seg_rows = seg_rows;
  p.status = status;
  const int max_tiles = E * ((Mg + BM - 1) / BM) * ((Ng + bn - 1) / bn);
  return launch_bn<GRAM>(bn, tA, tB, tA, tB, p, max_tiles, reinterpret_cast<cudaStream_t>(stream));
}
