// Grouped expert GEMM with NVFP4 weights decoded inside the kernel (W4A16): the bf16 weight stack of a
// mixture-of-experts projection never exists in global memory.
//
//   FWD  C[rows, N] = alpha * (A[rows, K] . W[e]^T + A2[rows, K2] . W2[e]^T)     W[e] logical [N, K]
//   DX   C[rows, K] = alpha * (A[rows, N] . W[e]   + A2[rows, K2] . W2[e])       (input gradient)
//
// W is stored as packed E2M1 nibbles [E, N, K/2] (low nibble = even k), E4M3 block scales [E, N, K/16] and
// one fp32 scale per expert; W2 / A2 (the LoRA K-extension) are bf16. Rows are expert-sorted and padded to
// 128-row blocks (blk_expert[b] = expert of block b), exactly as in grouped_gemm.cu.
//
// Per k block the TMA producer brings the bf16 A tile and the PACKED weight tile (4 KB instead of 16 KB)
// into shared memory; four converter warps expand the nibbles through a register lookup table, multiply
// by the block scale and write the bf16 tile in the 128-byte-swizzled layout tcgen05.mma reads; the MMA
// warp accumulates in TMEM; four epilogue warps store the result. The decoded values are bit-identical to
// nvfp4_dequant_kernel's, so the product equals dequantise-then-GEMM exactly, at a quarter of the weight
// traffic and without the bf16 scratch. This is the role the Marlin W4A16 grouped kernel and the
// dequantise-into-a-chunk path play in the reference
// (src/axolotl/integrations/kernels/libs/scattermoe_lora/marlin_w4a16/_csrc/libtorch_stable/moe/marlin_moe_wna16/marlin_template.h:251,
//  src/axolotl/integrations/kernels/libs/scattermoe_lora/grouped_train.py:446-596).
#include "axb_common.cuh"

namespace {

constexpr int BM = 128;
constexpr int BN = 128;
constexpr int BK = 64;
constexpr int W4_THREADS = 320;   // TMA, MMA, 4 epilogue warps, 4 converter warps
constexpr int W4_STAGES = 5;
constexpr int A_BYTES = BM * BK * 2;
constexpr int B_BYTES = BN * BK * 2;
constexpr int RAW_BYTES = 4096;   // FWD: 128 rows x 32 bytes; DX: 64 rows x 64 bytes
constexpr int W4_SMEM = W4_STAGES * (A_BYTES + B_BYTES + RAW_BYTES) + 1024 + 256;

constexpr unsigned long long kE2M1Lo = 0x3fc03f803f000000ull;  // bf16 bits of 1.5, 1.0, 0.5, 0.0
constexpr unsigned long long kE2M1Hi = 0x40c0408040404000ull;  // 6.0, 4.0, 3.0, 2.0

AXB_DEVICE float e2m1_to_float(uint32_t code) {
  const unsigned long long tbl = (code & 4) ? kE2M1Hi : kE2M1Lo;
  const uint32_t bits = (uint32_t)(tbl >> ((code & 3) * 16)) & 0xFFFFu;
  return __uint_as_float((bits | ((code & 8) << 12)) << 16);
}
AXB_DEVICE float e4m3_to_float(uint32_t v) {
  const uint32_t sign = (v >> 7) & 1, exp = (v >> 3) & 0xF, man = v & 7;
  float f;
  if (exp == 0) f = ldexpf((float)man, -9);
  else if (exp == 15 && man == 7) f = __int_as_float(0x7fc00000);
  else f = __uint_as_float(((exp + 120u) << 23) | (man << 20));
  return sign ? -f : f;
}
// 8 packed codes (one 32-bit word, low nibble first) times one scale -> 8 bf16 in a 16-byte chunk
AXB_DEVICE uint4 decode8(uint32_t w, float s) {
  uint4 o;
  o.x = pack_bf16x2(e2m1_to_float(w & 0xF) * s, e2m1_to_float((w >> 4) & 0xF) * s);
  o.y = pack_bf16x2(e2m1_to_float((w >> 8) & 0xF) * s, e2m1_to_float((w >> 12) & 0xF) * s);
  o.z = pack_bf16x2(e2m1_to_float((w >> 16) & 0xF) * s, e2m1_to_float((w >> 20) & 0xF) * s);
  o.w = pack_bf16x2(e2m1_to_float((w >> 24) & 0xF) * s, e2m1_to_float(w >> 28) * s);
  return o;
}

struct W4Params {
  int N, K, K2;   // FWD: N output columns, K contraction. DX: N = output columns (the weight's K), K = contraction (the weight's N)
  int Wn, Wk;     // logical weight shape [Wn, Wk] per expert
  void* C;
  long long ldc;
  float alpha;
  int out_mode;   // 0 bf16, 1 fp32
  const uint8_t* scale;   // [E, Wn, Wk / 16] e4m3 bytes
  const float* pts;       // [E]
  const int* blk_expert;
  const int* n_blocks;
  int* status;
};

// tensor map over the packed weight bytes [E, Wn, Wk/2], box [1, box_rows, box_bytes], no swizzle
int make_tmap_u8_3d(CUtensorMap* out, const void* base, uint64_t batch, uint64_t rows, uint64_t row_bytes,
                    uint32_t box_rows, uint32_t box_bytes) {
  AxbEncodeTiledFn fn = axb_get_encode_fn();
  if (!fn) return -1;
  cuuint64_t dims[3] = {row_bytes, rows, batch};
  cuuint64_t strides[2] = {row_bytes, rows * row_bytes};
  cuuint32_t box[3] = {box_bytes, box_rows, 1};
  cuuint32_t estr[3] = {1, 1, 1};
  CUresult r = CUDA_SUCCESS;
  for (int attempt = 0; attempt < 2; ++attempt) {
    r = fn(out, CU_TENSOR_MAP_DATA_TYPE_UINT8, 3, const_cast<void*>(base), dims, strides, box, estr,
           CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
           CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_ERROR_INVALID_CONTEXT) break;
    cudaFree(nullptr);
  }
  return r == CUDA_SUCCESS ? 0 : (int)r;
}

template <bool DX>
__global__ void __launch_bounds__(W4_THREADS, 1)
    grouped_w4a16_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmQ,
                         const __grid_constant__ CUtensorMap tmA2, const __grid_constant__ CUtensorMap tmB2,
                         const W4Params p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
  uint8_t* sA = smem;
  uint8_t* sB = smem + W4_STAGES * A_BYTES;
  uint8_t* sRaw = sB + W4_STAGES * B_BYTES;
  uint64_t* bars = reinterpret_cast<uint64_t*>(sRaw + W4_STAGES * RAW_BYTES);
  uint64_t* raw_full = bars;                    // TMA landed: A tile + packed weights (or the bf16 LoRA tile)
  uint64_t* full_bar = bars + W4_STAGES;        // converters done: the bf16 B tile is in place (4 arrivals)
  uint64_t* empty_bar = bars + 2 * W4_STAGES;   // MMAs retired
  uint64_t* tfull_bar = bars + 3 * W4_STAGES;
  uint64_t* tempty_bar = bars + 3 * W4_STAGES + 2;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 3 * W4_STAGES + 4);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int n_blocks = *p.n_blocks;
  const int num_n = (p.N + BN - 1) / BN;
  const int nk_main = (p.K + BK - 1) / BK, nk_ext = (p.K2 + BK - 1) / BK;
  const int nk = nk_main + nk_ext;
  const int total = n_blocks * num_n;

  if (threadIdx.x == 0) {
    for (int s = 0; s < W4_STAGES; ++s) {
      mbar_init(&raw_full[s], 1);
      mbar_init(&full_bar[s], 4);
      mbar_init(&empty_bar[s], 1);
    }
    for (int s = 0; s < 2; ++s) {
      mbar_init(&tfull_bar[s], 1);
      mbar_init(&tempty_bar[s], 4);
    }
    mbar_fence_init();
    tma_prefetch_desc(&tmA);
    tma_prefetch_desc(&tmQ);
  }
  if (warp == 2) {
    tmem_alloc(tmem_slot, 2 * BN);
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
      for (int tile = blockIdx.x; tile < total && ok; tile += gridDim.x) {
        const int blk = tile / num_n, n0 = (tile - blk * num_n) * BN, e = p.blk_expert[blk];
        for (int kb = 0; kb < nk; ++kb) {
          if (!mbar_wait(&empty_bar[stage], phase ^ 1, p.status, AXB_TIMEOUT_EMPTY)) {
            ok = false;
            break;
          }
          const bool ext = kb >= nk_main;
          uint8_t* a_dst = sA + stage * A_BYTES;
          if (!ext) {
            mbar_expect_tx(&raw_full[stage], A_BYTES + RAW_BYTES);
            tma_load_2d(a_dst, &tmA, &raw_full[stage], kb * BK, blk * BM);
            if (!DX) tma_load_3d(sRaw + stage * RAW_BYTES, &tmQ, &raw_full[stage], kb * (BK / 2), n0, e);       // [128 n, 32 B of k]
            else tma_load_3d(sRaw + stage * RAW_BYTES, &tmQ, &raw_full[stage], n0 / 2, kb * BK, e);             // [64 n, 64 B of k]
          } else {
            mbar_expect_tx(&raw_full[stage], A_BYTES + B_BYTES);
            const int k = (kb - nk_main) * BK;
            uint8_t* b_dst = sB + stage * B_BYTES;
            tma_load_2d(a_dst, &tmA2, &raw_full[stage], k, blk * BM);
            if (!DX) {
              tma_load_3d(b_dst, &tmB2, &raw_full[stage], k, n0, e);
            } else {
              tma_load_3d(b_dst, &tmB2, &raw_full[stage], n0, k, e);
              tma_load_3d(b_dst + 8192, &tmB2, &raw_full[stage], n0 + 64, k, e);
            }
          }
          if (++stage == W4_STAGES) {
            stage = 0;
            phase ^= 1;
          }
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      constexpr uint32_t idesc = make_idesc_bf16(BM, BN, 0, DX ? 1 : 0);
      int stage = 0, it = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < total && ok; tile += gridDim.x, ++it) {
        const int acc = it & 1;
        if (!mbar_wait(&tempty_bar[acc], ((it >> 1) & 1) ^ 1, p.status, AXB_TIMEOUT_TMEM_EMPTY)) break;
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + acc * BN;
        for (int kb = 0; kb < nk; ++kb) {
          // raw_full: the TMA writes (A tile, LoRA B tile) observed by this thread itself; full_bar: the decoded tile
          if (!mbar_wait(&raw_full[stage], phase, p.status, AXB_TIMEOUT_FULL) ||
              !mbar_wait(&full_bar[stage], phase, p.status, AXB_TIMEOUT_FULL)) {
            ok = false;
            break;
          }
          tc_fence_after();
          const uint32_t a_addr = smem_u32(sA + stage * A_BYTES), b_addr = smem_u32(sB + stage * B_BYTES);
#pragma unroll
          for (int kk = 0; kk < BK / 16; ++kk) {
            const uint64_t da = make_smem_desc_sw128(a_addr + kk * 32, 16, 1024);
            const uint64_t db = DX ? make_smem_desc_sw128(b_addr + kk * 2048, 8192, 1024)
                                   : make_smem_desc_sw128(b_addr + kk * 32, 16, 1024);
            umma_f16(d_tmem, da, db, idesc, (kb > 0 || kk > 0) ? 1u : 0u);
          }
          umma_commit(&empty_bar[stage]);
          if (++stage == W4_STAGES) {
            stage = 0;
            phase ^= 1;
          }
        }
        if (!ok) break;
        umma_commit(&tfull_bar[acc]);
      }
    }
  } else if (warp >= 6) {
    // ------------------------------------------------------------ converters: packed tile -> bf16 B tile
    const int ct = threadIdx.x - 192;   // 0..127
    int stage = 0;
    uint32_t phase = 0;
    bool ok = true;
    for (int tile = blockIdx.x; tile < total && ok; tile += gridDim.x) {
      const int blk = tile / num_n, n0 = (tile - blk * num_n) * BN, e = p.blk_expert[blk];
      const float g = p.pts[e];
      const long long sc_row_bytes = p.Wk / 16;
      // FWD: thread = weight row n0 + ct, the 64 k values of the block (4 scale bytes).
      // DX : thread = contraction row (weight row) kb * 64 + ct % 64, half ct / 64 of the 128 output columns
      //      (64 k values starting at n0 + 64 * half, 4 scale bytes).
      for (int kb = 0; kb < nk; ++kb) {
        if (!mbar_wait(&raw_full[stage], phase, p.status, AXB_TIMEOUT_FULL)) {
          ok = false;
          break;
        }
        if (kb < nk_main) {
          const uint8_t* raw = sRaw + stage * RAW_BYTES;
          uint8_t* bt = sB + stage * B_BYTES;
          uint32_t sc4 = 0;
          uint4 w0, w1;
          uint8_t* dst_row;
          int sw;
          if (!DX) {
            const int n = n0 + ct;
            if (n < p.Wn) sc4 = *reinterpret_cast<const uint32_t*>(p.scale + ((long long)e * p.Wn + n) * sc_row_bytes + kb * 4);
            w0 = *reinterpret_cast<const uint4*>(raw + ct * 32);
            w1 = *reinterpret_cast<const uint4*>(raw + ct * 32 + 16);
            dst_row = bt + ct * 128;       // K-major tile: row = n, 128 bytes = 64 k values
            sw = ct & 7;
          } else {
            const int r = ct & 63, half = ct >> 6;
            const int wn = kb * BK + r, k0 = n0 + half * 64;
            if (wn < p.Wn && k0 < p.Wk)
              sc4 = *reinterpret_cast<const uint32_t*>(p.scale + ((long long)e * p.Wn + wn) * sc_row_bytes + k0 / 16);
            w0 = *reinterpret_cast<const uint4*>(raw + r * 64 + half * 32);
            w1 = *reinterpret_cast<const uint4*>(raw + r * 64 + half * 32 + 16);
            dst_row = bt + half * 8192 + r * 128;   // MN-major tile: chunk of 64 columns, row = contraction index
            sw = r & 7;
          }
          const float s0 = e4m3_to_float(sc4 & 0xFF) * g, s1 = e4m3_to_float((sc4 >> 8) & 0xFF) * g;
          const float s2 = e4m3_to_float((sc4 >> 16) & 0xFF) * g, s3 = e4m3_to_float(sc4 >> 24) * g;
          *reinterpret_cast<uint4*>(dst_row + ((0 ^ sw) << 4)) = decode8(w0.x, s0);
          *reinterpret_cast<uint4*>(dst_row + ((1 ^ sw) << 4)) = decode8(w0.y, s0);
          *reinterpret_cast<uint4*>(dst_row + ((2 ^ sw) << 4)) = decode8(w0.z, s1);
          *reinterpret_cast<uint4*>(dst_row + ((3 ^ sw) << 4)) = decode8(w0.w, s1);
          *reinterpret_cast<uint4*>(dst_row + ((4 ^ sw) << 4)) = decode8(w1.x, s2);
          *reinterpret_cast<uint4*>(dst_row + ((5 ^ sw) << 4)) = decode8(w1.y, s2);
          *reinterpret_cast<uint4*>(dst_row + ((6 ^ sw) << 4)) = decode8(w1.z, s3);
          *reinterpret_cast<uint4*>(dst_row + ((7 ^ sw) << 4)) = decode8(w1.w, s3);
          fence_proxy_async_smem();
        }
        __syncwarp();
        if (lane == 0) mbar_arrive(&full_bar[stage]);
        if (++stage == W4_STAGES) {
          stage = 0;
          phase ^= 1;
        }
      }
    }
  } else {
    // ------------------------------------------------------------ epilogue warps 2..5
    const int lane_group = warp & 3;
    int it = 0;
    for (int tile = blockIdx.x; tile < total; tile += gridDim.x, ++it) {
      const int blk = tile / num_n, n0 = (tile - blk * num_n) * BN;
      const int acc = it & 1;
      if (!mbar_wait(&tfull_bar[acc], (it >> 1) & 1, p.status, AXB_TIMEOUT_TMEM_FULL)) break;
      tc_fence_after();
      const long long row = (long long)blk * BM + lane_group * 32 + lane;
      const uint32_t t_addr = tmem_base + (uint32_t(lane_group * 32) << 16) + acc * BN;
#pragma unroll 1
      for (int c = 0; c < BN / 32; ++c) {
        uint32_t r[32];
        tmem_ld_32x32(t_addr + c * 32, r);
        tmem_ld_wait();
        const int col0 = n0 + c * 32;
        if (col0 >= p.N) continue;
        const bool full_chunk = col0 + 32 <= p.N;
        if (p.out_mode == 0) {
          __nv_bfloat16* crow = reinterpret_cast<__nv_bfloat16*>(p.C) + row * p.ldc + col0;
          if (full_chunk && (p.ldc & 7) == 0) {
#pragma unroll
            for (int q = 0; q < 4; ++q) {
              uint4 o;
              o.x = pack_bf16x2(__uint_as_float(r[q * 8 + 0]) * p.alpha, __uint_as_float(r[q * 8 + 1]) * p.alpha);
              o.y = pack_bf16x2(__uint_as_float(r[q * 8 + 2]) * p.alpha, __uint_as_float(r[q * 8 + 3]) * p.alpha);
              o.z = pack_bf16x2(__uint_as_float(r[q * 8 + 4]) * p.alpha, __uint_as_float(r[q * 8 + 5]) * p.alpha);
              o.w = pack_bf16x2(__uint_as_float(r[q * 8 + 6]) * p.alpha, __uint_as_float(r[q * 8 + 7]) * p.alpha);
              *reinterpret_cast<uint4*>(crow + q * 8) = o;
            }
          } else {
            for (int j = 0; j < 32 && col0 + j < p.N; ++j) crow[j] = __float2bfloat16(__uint_as_float(r[j]) * p.alpha);
          }
        } else {
          float* crow = reinterpret_cast<float*>(p.C) + row * p.ldc + col0;
          for (int j = 0; j < 32 && col0 + j < p.N; ++j) crow[j] = __uint_as_float(r[j]) * p.alpha;
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&tempty_bar[acc]);
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 2) {
    tc_fence_after();
    tmem_dealloc(tmem_base, 2 * BN);
  }
}

}  // namespace

// A [max_blocks * 128, Ka] bf16 (lda); qdata [E, Wn, Wk/2] uint8, scale [E, Wn, Wk/16] e4m3 bytes, pts [E] fp32.
//   trans_w = 0 (forward):        Ka = Wk, C [rows, Wn];  A2 [rows, K2], W2 [E, Wn, K2] (bf16, optional)
//   trans_w = 1 (input gradient): Ka = Wn, C [rows, Wk];  A2 [rows, K2], W2 [E, K2, Wk] (bf16, optional)
// Wk must be a multiple of 64, Wn a multiple of 8; out_mode 0 bf16 / 1 fp32.
extern "C" int axb_grouped_gemm_w4a16(const void* A, long long lda, const void* qdata, const void* scale, const float* pts,
                                      const void* A2, long long lda2, const void* W2, void* C, long long ldc, int E,
                                      int Wn, int Wk, int K2, int trans_w, float alpha, int out_mode,
                                      const int* blk_expert, const int* n_blocks, int max_blocks, int* status,
                                      void* stream) {
  if (max_blocks <= 0 || Wn <= 0 || Wk <= 0) return 0;
  if ((lda & 7) || (Wk & 63) || (Wn & 7) || (K2 > 0 && ((lda2 & 7) || (K2 & 7))) || out_mode < 0 || out_mode > 1) return -2;
  const unsigned long long rows = (unsigned long long)max_blocks * BM;
  const int Ka = trans_w ? Wn : Wk, N = trans_w ? Wk : Wn;
  CUtensorMap tA, tQ, tA2, tB2;
  int rc = axb_make_tmap_2d(&tA, A, rows, Ka, lda, BM, 64);
  rc |= trans_w ? make_tmap_u8_3d(&tQ, qdata, E, Wn, Wk / 2, 64, 64) : make_tmap_u8_3d(&tQ, qdata, E, Wn, Wk / 2, 128, 32);
  if (K2 > 0) {
    rc |= axb_make_tmap_2d(&tA2, A2, rows, K2, lda2, BM, 64);
    rc |= trans_w ? axb_make_tmap_3d(&tB2, W2, E, K2, Wk, Wk, (unsigned long long)Wk * K2, 64, 64)
                  : axb_make_tmap_3d(&tB2, W2, E, Wn, K2, K2, (unsigned long long)Wn * K2, BN, 64);
  } else {
    tA2 = tA;
    tB2 = tA;
  }
  if (rc) return -4;
  W4Params p = {};
  p.N = N; p.K = Ka; p.K2 = K2 > 0 ? K2 : 0; p.Wn = Wn; p.Wk = Wk;
  p.C = C; p.ldc = ldc; p.alpha = alpha; p.out_mode = out_mode;
  p.scale = reinterpret_cast<const uint8_t*>(scale); p.pts = pts;
  p.blk_expert = blk_expert; p.n_blocks = n_blocks; p.status = status;
  int dev = 0, sms = 148;
  cudaGetDevice(&dev);
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  const int max_tiles = max_blocks * ((N + BN - 1) / BN);
  int grid = sms < max_tiles ? sms : max_tiles;
  if (grid < 1) return 0;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  if (trans_w) {
    static bool set = false;
    if (!set) {
      cudaError_t e = cudaFuncSetAttribute(grouped_w4a16_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, W4_SMEM);
      if (e != cudaSuccess) return (int)e;
      set = true;
    }
    grouped_w4a16_kernel<true><<<grid, W4_THREADS, W4_SMEM, st>>>(tA, tQ, tA2, tB2, p);
  } else {
    static bool set = false;
    if (!set) {
      cudaError_t e = cudaFuncSetAttribute(grouped_w4a16_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, W4_SMEM);
      if (e != cudaSuccess) return (int)e;
      set = true;
    }
    grouped_w4a16_kernel<false><<<grid, W4_THREADS, W4_SMEM, st>>>(tA, tQ, tA2, tB2, p);
  }
  return (int)cudaGetLastError();
}
