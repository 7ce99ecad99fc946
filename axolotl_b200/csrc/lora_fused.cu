// One pass over dY for the adapter side of a LoRA projection's backward pass.
//
//   t32[T, R]  += dY[T, N] . B[N, R]            (the low-rank activation gradient, before scaling)
//   dB32[N, R] += dY[T, N]^T . xa[T, R]         (gradient of B; only the columns of the diagonal block a
//                                                row belongs to are written: B is block diagonal when
//                                                several projections share one fused weight)
//
// Both products consume the same dY tile, which is brought into shared memory once (TMA, 128-byte
// swizzle) and fed to tcgen05.mma twice: as the K-major A operand of the first product and, read the
// other way round (MN-major), as the A operand of the second. The reference computes the two with
// separate cuBLAS calls per projection (src/axolotl/kernels/lora.py:283-705: `dY @ B.t()`, `dY.t() @ (X A^T)`),
// i.e. two or more full reads of dY.
//
// A CTA owns 512 token rows (4 sub-tiles of 128) and a contiguous range of 128-column blocks of dY:
//   warp 0 (one lane): TMA producer   - xa sub-tiles once, then per column block the B tile and 4 dY tiles
//   warp 1 (one lane): MMA issuer     - t accumulators (4 x R columns of TMEM) live for the whole CTA,
//                                       dB accumulators are double buffered per column block
//   warps 2-5        : epilogue       - fp32 reductions into t32 / dB32 (several CTAs share every row)
#include "axb_common.cuh"

namespace {

constexpr int LF_THREADS = 192;
constexpr int LF_ROWS = 512;                 // token rows per CTA
constexpr int LF_SUB = 4;                    // 128-row sub-tiles
constexpr int LF_DY_STAGES = 3;
constexpr int LF_DY_BYTES = 128 * 128 * 2;   // two 64-column halves of 128 rows x 128 bytes
constexpr int LF_SMALL_BYTES = 128 * 64 * 2; // [128 rows, 64 columns] tile of xa / B (columns >= R are zero)
constexpr int LF_SMEM = LF_DY_STAGES * LF_DY_BYTES + LF_SUB * LF_SMALL_BYTES + 2 * LF_SMALL_BYTES + 1024 + 256;

struct LoraBwdParams {
  int T, N, R, Rpad;
  int n_blocks;        // ceil(N / 128)
  int n_splits;        // CTAs along N
  float* t32;          // [T, R]
  float* dB32;         // [N, ldb32]
  long long ldb32;
  int n_lora_blocks;
  int blk_row0[8], blk_rows[8], blk_r0[8], blk_r[8];
  int* status;
};

__global__ void __launch_bounds__(LF_THREADS, 1)
    lora_bwd_dy_kernel(const __grid_constant__ CUtensorMap tmDY, const __grid_constant__ CUtensorMap tmB,
                       const __grid_constant__ CUtensorMap tmXA, const LoraBwdParams p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
  uint8_t* sDY = smem;
  uint8_t* sXA = smem + LF_DY_STAGES * LF_DY_BYTES;
  uint8_t* sB = sXA + LF_SUB * LF_SMALL_BYTES;
  uint64_t* bars = reinterpret_cast<uint64_t*>(sB + 2 * LF_SMALL_BYTES);
  uint64_t* dy_full = bars;                     // [3]
  uint64_t* dy_empty = bars + 3;                // [3]
  uint64_t* b_full = bars + 6;                  // [2]
  uint64_t* b_empty = bars + 8;                 // [2]
  uint64_t* db_full = bars + 10;                // [2]
  uint64_t* db_empty = bars + 12;               // [2]
  uint64_t* xa_full = bars + 14;
  uint64_t* t_done = bars + 15;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 16);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int t_chunk = blockIdx.x / p.n_splits, split = blockIdx.x % p.n_splits;
  const int row0 = t_chunk * LF_ROWS;
  const int nb0 = (int)((long long)p.n_blocks * split / p.n_splits);
  const int nb1 = (int)((long long)p.n_blocks * (split + 1) / p.n_splits);
  const int n_sub = min(LF_SUB, (p.T - row0 + 127) / 128);

  if (threadIdx.x == 0) {
    for (int s = 0; s < 3; ++s) {
      mbar_init(&dy_full[s], 1);
      mbar_init(&dy_empty[s], 1);
    }
    for (int s = 0; s < 2; ++s) {
      mbar_init(&b_full[s], 1);
      mbar_init(&b_empty[s], 1);
      mbar_init(&db_full[s], 1);
      mbar_init(&db_empty[s], 4);
    }
    mbar_init(xa_full, 1);
    mbar_init(t_done, 1);
    mbar_fence_init();
    tma_prefetch_desc(&tmDY);
  }
  if (warp == 2) {
    tmem_alloc(tmem_slot, 512);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  // TMEM columns: t accumulators [sub * 64, +Rpad), dB accumulators [256 + buf * 64, +Rpad)
  if (nb1 > nb0 && n_sub > 0) {
    if (warp == 0) {
      if (lane == 0) {
        mbar_expect_tx(xa_full, n_sub * LF_SMALL_BYTES);
        for (int s = 0; s < n_sub; ++s) {
          tma_load_2d(sXA + s * LF_SMALL_BYTES, &tmXA, xa_full, 0, row0 + s * 128);
          tma_load_2d(sXA + s * LF_SMALL_BYTES + 8192, &tmXA, xa_full, 0, row0 + s * 128 + 64);
        }
        int stage = 0;
        uint32_t phase = 0;
        bool ok = true;
        for (int nb = nb0, i = 0; nb < nb1 && ok; ++nb, ++i) {
          const int bb = i & 1;
          if (!mbar_wait(&b_empty[bb], ((i >> 1) & 1) ^ 1, p.status, AXB_TIMEOUT_EMPTY)) break;
          mbar_expect_tx(&b_full[bb], LF_SMALL_BYTES);
          tma_load_2d(sB + bb * LF_SMALL_BYTES, &tmB, &b_full[bb], 0, nb * 128);
          tma_load_2d(sB + bb * LF_SMALL_BYTES + 8192, &tmB, &b_full[bb], 0, nb * 128 + 64);
          for (int s = 0; s < n_sub; ++s) {
            if (!mbar_wait(&dy_empty[stage], phase ^ 1, p.status, AXB_TIMEOUT_EMPTY)) {
              ok = false;
              break;
            }
            mbar_expect_tx(&dy_full[stage], LF_DY_BYTES);
            uint8_t* dst = sDY + stage * LF_DY_BYTES;
            tma_load_2d(dst, &tmDY, &dy_full[stage], nb * 128, row0 + s * 128);
            tma_load_2d(dst + 16384, &tmDY, &dy_full[stage], nb * 128 + 64, row0 + s * 128);
            if (++stage == LF_DY_STAGES) {
              stage = 0;
              phase ^= 1;
            }
          }
        }
      }
    } else if (warp == 1) {
      if (lane == 0) {
        const uint32_t idesc1 = make_idesc_bf16(128, p.Rpad, 0, 1);   // A = dY tile K-major, B = B tile MN-major
        const uint32_t idesc2 = make_idesc_bf16(128, p.Rpad, 1, 1);   // A = dY tile read MN-major, B = xa MN-major
        bool ok = mbar_wait(xa_full, 0, p.status, AXB_TIMEOUT_FULL);
        int stage = 0;
        uint32_t phase = 0;
        for (int nb = nb0, i = 0; nb < nb1 && ok; ++nb, ++i) {
          const int bb = i & 1;
          const uint32_t use = (i >> 1) & 1;
          if (!mbar_wait(&b_full[bb], use, p.status, AXB_TIMEOUT_FULL) ||
              !mbar_wait(&db_empty[bb], use ^ 1, p.status, AXB_TIMEOUT_TMEM_EMPTY)) {
            ok = false;
            break;
          }
          tc_fence_after();
          const uint32_t b_addr = smem_u32(sB + bb * LF_SMALL_BYTES);
          const uint32_t d_db = tmem_base + 256 + bb * 64;
          for (int s = 0; s < n_sub; ++s) {
            if (!mbar_wait(&dy_full[stage], phase, p.status, AXB_TIMEOUT_FULL)) {
              ok = false;
              break;
            }
            tc_fence_after();
            const uint32_t a_addr = smem_u32(sDY + stage * LF_DY_BYTES);
            const uint32_t xa_addr = smem_u32(sXA + s * LF_SMALL_BYTES);
            const uint32_t d_t = tmem_base + s * 64;
            // t[s] += dY(128 x 128) . B(128 x R): k runs over the 128 columns of the tile (two 64-column halves)
#pragma unroll
            for (int kk = 0; kk < 8; ++kk) {
              const uint64_t da = make_smem_desc_sw128(a_addr + (kk >> 2) * 16384 + (kk & 3) * 32, 16, 1024);
              const uint64_t db = make_smem_desc_sw128(b_addr + kk * 2048, 8192, 1024);
              umma_f16(d_t, da, db, idesc1, (i > 0 || kk > 0) ? 1u : 0u);
            }
            // dB[nb] += dY^T(128 cols x 128 rows) . xa(128 rows x R): k runs over the 128 token rows
#pragma unroll
            for (int kk = 0; kk < 8; ++kk) {
              const uint64_t da = make_smem_desc_sw128(a_addr + kk * 2048, 16384, 1024);
              const uint64_t db = make_smem_desc_sw128(xa_addr + kk * 2048, 8192, 1024);
              umma_f16(d_db, da, db, idesc2, (s > 0 || kk > 0) ? 1u : 0u);
            }
            umma_commit(&dy_empty[stage]);
            if (++stage == LF_DY_STAGES) {
              stage = 0;
              phase ^= 1;
            }
          }
          if (!ok) break;
          umma_commit(&db_full[bb]);
          umma_commit(&b_empty[bb]);
        }
        if (ok) umma_commit(t_done);
      }
    } else {
      const int lg = warp & 3;   // TMEM lanes [32 lg, 32 lg + 32)
      bool ok = true;
      for (int nb = nb0, i = 0; nb < nb1 && ok; ++nb, ++i) {
        const int bb = i & 1;
        if (!mbar_wait(&db_full[bb], (i >> 1) & 1, p.status, AXB_TIMEOUT_TMEM_FULL)) {
          ok = false;
          break;
        }
        tc_fence_after();
        const int n = nb * 128 + lg * 32 + lane;   // this thread's column of dY = row of dB
        int r0 = 0, r = 0;
        for (int b = 0; b < p.n_lora_blocks; ++b)
          if (n >= p.blk_row0[b] && n < p.blk_row0[b] + p.blk_rows[b]) {
            r0 = p.blk_r0[b];
            r = p.blk_r[b];
          }
        const uint32_t t_addr = tmem_base + (uint32_t(lg * 32) << 16) + 256 + bb * 64;
        for (int c = 0; c < p.Rpad; c += 16) {
          uint32_t v[16];
          tmem_ld_32x16(t_addr + c, v);
          tmem_ld_wait();
          if (n < p.N && c < r0 + r && c + 16 > r0) {
            float* dst = p.dB32 + (long long)n * p.ldb32 + c;
#pragma unroll
            for (int j = 0; j < 16; ++j)
              if (c + j >= r0 && c + j < r0 + r) atomicAdd(dst + j, __uint_as_float(v[j]));
          }
        }
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(&db_empty[bb]);
      }
      if (ok && mbar_wait(t_done, 0, p.status, AXB_TIMEOUT_TMEM_FULL)) {
        tc_fence_after();
        for (int s = 0; s < n_sub; ++s) {
          const int t = row0 + s * 128 + lg * 32 + lane;
          const uint32_t t_addr = tmem_base + (uint32_t(lg * 32) << 16) + s * 64;
          for (int c = 0; c < p.Rpad; c += 16) {
            uint32_t v[16];
            tmem_ld_32x16(t_addr + c, v);
            tmem_ld_wait();
            if (t < p.T) {
              float* dst = p.t32 + (long long)t * p.R + c;
#pragma unroll
              for (int j = 0; j < 16; ++j)
                if (c + j < p.R) atomicAdd(dst + j, __uint_as_float(v[j]));
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

}  // namespace

// dY [T, N] (ld_dy), B [N, R] (ld_b), xa [T, R] (ld_xa): bf16 row-major, R <= 64, all leading dimensions
// multiples of 8. t32 [T, R] and dB32 [N, ldb32] are fp32 and are ACCUMULATED into (zero t32 first).
// blocks: n_blocks x (row0, rows, r0, r) diagonal blocks of B (HOST array of 4 * n_blocks ints).
extern "C" int axb_lora_bwd_dy(const void* dy, long long ld_dy, const void* B, long long ld_b, const void* xa,
                               long long ld_xa, float* t32, float* dB32, long long ldb32, int T, int N, int R,
                               const int* blocks, int n_lora_blocks, int* status, void* stream) {
  if (T <= 0 || N <= 0 || R <= 0) return 0;
  if (R > 64 || n_lora_blocks < 1 || n_lora_blocks > 8) return -3;
  if ((ld_dy & 7) || (ld_b & 7) || (ld_xa & 7)) return -2;
  CUtensorMap tDY, tB, tXA;
  int rc = 0;
  rc |= axb_make_tmap_2d(&tDY, dy, T, N, ld_dy, 128, 64);
  rc |= axb_make_tmap_2d(&tB, B, N, R, ld_b, 64, 64);
  rc |= axb_make_tmap_2d(&tXA, xa, T, R, ld_xa, 64, 64);
  if (rc) return -4;
  LoraBwdParams p = {};
  p.T = T; p.N = N; p.R = R; p.Rpad = (R + 15) & ~15;
  p.n_blocks = (N + 127) / 128;
  const int t_chunks = (T + LF_ROWS - 1) / LF_ROWS;
  int dev = 0, sms = 148;
  cudaGetDevice(&dev);
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  int splits = sms / t_chunks;
  if (splits < 1) splits = 1;
  if (splits > p.n_blocks) splits = p.n_blocks;
  p.n_splits = splits;
  p.t32 = t32; p.dB32 = dB32; p.ldb32 = ldb32;
  p.n_lora_blocks = n_lora_blocks;
  for (int b = 0; b < n_lora_blocks; ++b) {
    p.blk_row0[b] = blocks[4 * b]; p.blk_rows[b] = blocks[4 * b + 1];
    p.blk_r0[b] = blocks[4 * b + 2]; p.blk_r[b] = blocks[4 * b + 3];
  }
  p.status = status;
  static bool attr_set = false;
  if (!attr_set) {
    cudaError_t e = cudaFuncSetAttribute(lora_bwd_dy_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, LF_SMEM);
    if (e != cudaSuccess) return (int)e;
    attr_set = true;
  }
  lora_bwd_dy_kernel<<<t_chunks * splits, LF_THREADS, LF_SMEM, reinterpret_cast<cudaStream_t>(stream)>>>(tDY, tB, tXA, p);
  return (int)cudaGetLastError();
}
