// Lightning-indexer scores for sparse attention (GLM-5 / DeepSeek-V3.2 style dynamic sparse attention)
// on sm_100a:
//
//   out[s, t] = sum over heads h of  w[s, h] * relu(q[s, h, :] . k[t, :])      for t <= s + causal_off
//             = -inf                                                          otherwise
//
// q [Lq, H, 128] bf16, k [Lk, 128] bf16 (one key vector per position, shared by all heads), w [Lq, H] fp32
// (the caller folds the softmax scale and H^-1/2 into w: relu commutes with a positive scale).
//
// The contraction is one GEMM [Lk, 128] x [128, Lq*H] on the tensor cores with the KEYS on the accumulator rows and
// (query position, head) on its columns, so the [Lq, H, Lk] score tensor is never written and the head sum needs no
// exchange between threads: an epilogue thread owns one key, reads the H accumulator columns of a query position,
// applies relu * w and adds them up in registers, and the 32 lanes of a warp store 32 consecutive keys of the output
// row. One CTA owns a block of 128 / H query positions, keeps its Q tile resident in shared memory and streams the
// key tiles of the causal range through a TMA ring; accumulators are double-buffered in TMEM so the epilogue of tile
// i overlaps the MMAs of tile i+1. Eight epilogue warps: two per TMEM lane quadrant, each taking half of the columns
// (for H = 128 a position spans all columns and one warp per quadrant does the work).
//
// The reference computes the same scores with a Triton kernel that loops over heads inside a program
// (src/axolotl/integrations/kernels/libs/glm_dsa/indexer.py:38-176, .../dsv4/indexer.py:38-138).
#include "axb_common.cuh"

#include <cmath>

namespace {

constexpr int BM = 128;        // (query position, head) rows of the resident Q tile = accumulator columns
constexpr int BN = 128;        // keys per tile = accumulator rows
constexpr int DI = 128;        // index head width
constexpr int STAGES = 4;
constexpr int kEpiWarps = 8;
constexpr int kThreads = 64 + 32 * kEpiWarps;  // TMA warp, MMA warp, epilogue warps
constexpr int A_BYTES = BM * DI * 2;
constexpr int B_BYTES = BN * DI * 2;
constexpr int PART_BYTES = kEpiWarps * BM * 4;   // every epilogue warp's own copy of the tile's head weights
constexpr int SMEM_BYTES = A_BYTES + STAGES * B_BYTES + PART_BYTES + 256 + 1024;
constexpr int TMEM_COLS = 2 * BN;

struct IParams {
  const float* w;   // [Lq * H]
  float* out;       // [Lq, ldo]
  long long ldo;
  int Lq, Lk, H;
  int causal_off;   // key t is visible to query s when t <= s + causal_off
  int* status;
};

AXB_DEVICE int last_k_tile(const IParams& p, int qt, int P) {
  long long last_pos = (long long)qt * P + P - 1;
  if (last_pos > p.Lq - 1) last_pos = p.Lq - 1;
  long long last_key = last_pos + p.causal_off;
  if (last_key > p.Lk - 1) last_key = p.Lk - 1;
  return last_key < 0 ? -1 : (int)(last_key / BN);
}

__global__ void __launch_bounds__(kThreads, 1)
    indexer_scores_kernel(const __grid_constant__ CUtensorMap tmQ,
                          const __grid_constant__ CUtensorMap tmK, const IParams p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~static_cast<uintptr_t>(1023));
  uint8_t* sA = smem;
  uint8_t* sB = smem + A_BYTES;
  float* w_s = reinterpret_cast<float*>(smem + A_BYTES + STAGES * B_BYTES);    // [kEpiWarps][BM]
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + A_BYTES + STAGES * B_BYTES + PART_BYTES);
  uint64_t* full_bar = bars;                 // key tile landed
  uint64_t* empty_bar = bars + STAGES;       // key tile consumed
  uint64_t* a_full = bars + 2 * STAGES;      // Q tile landed
  uint64_t* a_empty = bars + 2 * STAGES + 1; // all MMAs that read the Q tile are done
  uint64_t* tfull_bar = bars + 2 * STAGES + 2;
  uint64_t* tempty_bar = bars + 2 * STAGES + 4;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * STAGES + 6);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int P = BM / p.H;                                  // query positions per tile
  const int num_q = (p.Lq + P - 1) / P;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 1);
    }
    mbar_init(a_full, 1);
    mbar_init(a_empty, 1);
    for (int s = 0; s < 2; ++s) {
      mbar_init(&tfull_bar[s], 1);
      mbar_init(&tempty_bar[s], kEpiWarps);
    }
    mbar_fence_init();
    tma_prefetch_desc(&tmQ);
    tma_prefetch_desc(&tmK);
  }
  if (warp == 2) {
    tmem_alloc(tmem_slot, TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0, a_phase = 0;
      bool ok = true;
      for (int qt = blockIdx.x; ok && qt < num_q; qt += gridDim.x) {
        const int kt_last = last_k_tile(p, qt, P);
        if (kt_last < 0) continue;
        if (!mbar_wait(a_empty, a_phase ^ 1, p.status, AXB_TIMEOUT_EMPTY)) break;
        a_phase ^= 1;
        mbar_expect_tx(a_full, A_BYTES);
        tma_load_2d(sA, &tmQ, a_full, 0, qt * BM);
        tma_load_2d(sA + A_BYTES / 2, &tmQ, a_full, 64, qt * BM);
        for (int kt = 0; kt <= kt_last; ++kt) {
          if (!mbar_wait(&empty_bar[stage], phase ^ 1, p.status, AXB_TIMEOUT_EMPTY)) {
            ok = false;
            break;
          }
          mbar_expect_tx(&full_bar[stage], B_BYTES);
          uint8_t* b_dst = sB + stage * B_BYTES;
          tma_load_2d(b_dst, &tmK, &full_bar[stage], 0, kt * BN);
          tma_load_2d(b_dst + B_BYTES / 2, &tmK, &full_bar[stage], 64, kt * BN);
          if (++stage == STAGES) {
            stage = 0;
            phase ^= 1;
          }
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      constexpr uint32_t idesc = make_idesc_bf16(BN, BM, 0, 0);
      int stage = 0;
      uint32_t phase = 0, a_phase = 0;
      int it = 0;
      bool ok = true;
      const uint32_t a_addr = smem_u32(sA);
      for (int qt = blockIdx.x; ok && qt < num_q; qt += gridDim.x) {
        const int kt_last = last_k_tile(p, qt, P);
        if (kt_last < 0) continue;
        if (!mbar_wait(a_full, a_phase, p.status, AXB_TIMEOUT_FULL)) break;
        a_phase ^= 1;
        for (int kt = 0; kt <= kt_last; ++kt) {
          const int acc = it & 1;
          const uint32_t acc_phase = (it >> 1) & 1;
          ++it;
          if (!mbar_wait(&tempty_bar[acc], acc_phase ^ 1, p.status, AXB_TIMEOUT_TMEM_EMPTY) ||
              !mbar_wait(&full_bar[stage], phase, p.status, AXB_TIMEOUT_FULL)) {
            ok = false;
            break;
          }
          tc_fence_after();
          const uint32_t d_tmem = tmem_base + acc * BM;
          const uint32_t b_addr = smem_u32(sB + stage * B_BYTES);
#pragma unroll
          for (int kb = 0; kb < DI / 64; ++kb) {
#pragma unroll
            for (int kk = 0; kk < 4; ++kk) {
              // keys are the M operand (accumulator rows), the resident Q tile the N operand
              const uint64_t dq = make_smem_desc_sw128(a_addr + kb * (A_BYTES / 2) + kk * 32, 16, 1024);
              const uint64_t dk = make_smem_desc_sw128(b_addr + kb * (B_BYTES / 2) + kk * 32, 16, 1024);
              umma_f16(d_tmem, dk, dq, idesc, (kb > 0 || kk > 0) ? 1u : 0u);
            }
          }
          umma_commit(&empty_bar[stage]);
          umma_commit(&tfull_bar[acc]);
          if (++stage == STAGES) {
            stage = 0;
            phase ^= 1;
          }
        }
        if (ok) umma_commit(a_empty);
      }
    }
  } else {
    const int ew = warp - 2;
    const int lane_group = warp & 3;             // TMEM lane quadrant this warp may read: keys lane_group*32 ..
    const int half = ew >> 2;                    // which half of the accumulator columns
    // H <= 64: the two warps of a quadrant split the columns (a position never straddles the halves);
    // H = 128: one position spans all columns, the first warp of the quadrant takes them all
    const int c_lo = p.H == 128 ? 0 : half * 2;
    const int c_hi = p.H == 128 ? (half == 0 ? 4 : 0) : half * 2 + 2;
    const long long n_rows = (long long)p.Lq * p.H;
    const float neg_inf = -INFINITY;
    float* my_w = w_s + ew * BM;
    int it = 0;
    bool ok = true;
    for (int qt = blockIdx.x; ok && qt < num_q; qt += gridDim.x) {
      const int kt_last = last_k_tile(p, qt, P);
      if (kt_last < 0) continue;
      __syncwarp();
#pragma unroll
      for (int i = 0; i < BM / 32; ++i) {
        const long long row = (long long)qt * BM + i * 32 + lane;
        my_w[i * 32 + lane] = row < n_rows ? p.w[row] : 0.f;
      }
      __syncwarp();
      for (int kt = 0; kt <= kt_last; ++kt) {
        const int acc = it & 1;
        const uint32_t acc_phase = (it >> 1) & 1;
        ++it;
        if (!mbar_wait(&tfull_bar[acc], acc_phase, p.status, AXB_TIMEOUT_TMEM_FULL)) {
          ok = false;
          break;
        }
        tc_fence_after();
        const uint32_t t_addr = tmem_base + (uint32_t(lane_group * 32) << 16) + acc * BM;
        const int key = kt * BN + lane_group * 32 + lane;
        float s = 0.f;
#pragma unroll 1
        for (int c = c_lo; c < c_hi; ++c) {
          uint32_t r[32];
          tmem_ld_32x32(t_addr + c * 32, r);
          tmem_ld_wait();
          const float4* wv = reinterpret_cast<const float4*>(my_w + c * 32);
          float s0 = 0.f, s1 = 0.f, s2 = 0.f, s3 = 0.f;
#pragma unroll
          for (int j = 0; j < 8; ++j) {
            const float4 w4 = wv[j];                                   // the same address in every lane: a broadcast
            s0 = fmaf(fmaxf(__uint_as_float(r[4 * j + 0]), 0.f), w4.x, s0);
            s1 = fmaf(fmaxf(__uint_as_float(r[4 * j + 1]), 0.f), w4.y, s1);
            s2 = fmaf(fmaxf(__uint_as_float(r[4 * j + 2]), 0.f), w4.z, s2);
            s3 = fmaf(fmaxf(__uint_as_float(r[4 * j + 3]), 0.f), w4.w, s3);
          }
          s += (s0 + s1) + (s2 + s3);
          if (((c + 1) * 32) % p.H == 0) {                              // last head of a query position
            const long long pos = (long long)qt * P + ((c + 1) * 32) / p.H - 1;
            if (pos < p.Lq && key < p.Lk) p.out[pos * p.ldo + key] = key <= pos + p.causal_off ? s : neg_inf;
            s = 0.f;
          }
        }
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
    tmem_dealloc(tmem_base, TMEM_COLS);
  }
}

}  // namespace

// out[s, t] for t in [0, Lk) of every key tile that holds a visible key of the CTA's query block; entries to the
// right of those tiles are NOT written (the caller pre-fills `out` with -inf). q rows are [Lq * H, 128] with leading
// dimension ldq (elements, multiple of 8), k rows [Lk, 128] with ldk. H in {32, 64, 128}.
extern "C" int axb_indexer_scores(const void* q, long long ldq, const void* k, long long ldk,
                                  const float* w, float* out, long long ldo, int Lq, int Lk, int H,
                                  int Di, int causal_off, int* status, void* stream) {
  if (Lq <= 0 || Lk <= 0) return 0;
  if (Di != DI || (H != 32 && H != 64 && H != 128) || (ldq & 7) || (ldk & 7)) return -2;
  CUtensorMap tQ, tK;
  int rc = axb_make_tmap_2d(&tQ, q, (unsigned long long)Lq * H, DI, ldq, BM, 64);
  rc |= axb_make_tmap_2d(&tK, k, Lk, DI, ldk, BN, 64);
  if (rc) return -4;
  IParams p = {};
  p.w = w;
  p.out = out;
  p.ldo = ldo;
  p.Lq = Lq;
  p.Lk = Lk;
  p.H = H;
  p.causal_off = causal_off;
  p.status = status;
  static bool attr_set = false;
  if (!attr_set) {
    cudaError_t e = cudaFuncSetAttribute(indexer_scores_kernel,
                                         cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES);
    if (e != cudaSuccess) return (int)e;
    attr_set = true;
  }
  int sms = 0, dev = 0;
  cudaGetDevice(&dev);
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  if (sms <= 0) sms = 148;
  const int P = BM / H;
  const int num_q = (Lq + P - 1) / P;
  const int grid = num_q < sms ? num_q : sms;
  indexer_scores_kernel<<<grid, kThreads, SMEM_BYTES, reinterpret_cast<cudaStream_t>(stream)>>>(tQ, tK, p);
  return (int)cudaGetLastError();
}
