// bf16 GEMM core for sm_100a: TMA -> shared-memory ring -> tcgen05.mma (accumulators in TMEM,
// double buffered) -> tcgen05.ld epilogue. Persistent, warp-specialised:
//   warp 0   : TMA producer (one lane)
//   warp 1   : MMA issuer   (one lane)
//   warps 2-5: epilogue (each warp owns the 32 TMEM lanes its warp-id % 4 selects)
//
// Logical problem: C[M,N] = alpha * (A[M,K] . B[N,K]^T  +  A2[M,K2] . B2[N,K2]^T) + beta * Cin
// Either operand may be stored "MN-major" (the transposed matrix, [K,M] / [K,N] row-major), which
// lets one kernel serve X.W^T (forward), dY.W (input gradient) and dY^T.X (weight gradient).
// The second operand pair is the K-extension used to fuse the LoRA low-rank update: the product
// (X.A^T) . B^T is simply one more K block accumulated into the same TMEM tile.
//
// Replaces the cuBLAS calls behind the reference's LoRA kernels (src/axolotl/kernels/lora.py:226-280).
#include "axb_common.cuh"

namespace {

constexpr int BM = 128;
constexpr int BK = 64;  // 64 bf16 = 128 bytes = one swizzle row
constexpr int kThreads = 192;
constexpr int kSmemBudget = 220 * 1024;

struct GemmParams {
  int M, N, K, K2;
  void* C;
  const void* Cin;
  long long ldc, ldcin;
  float alpha, beta;
  int out_mode;  // 0: bf16 store, 1: fp32 store, 2: fp32 atomic add (split-K)
  int splits;
  int* status;
  // fused all-gather (GATHER kernels only): the B operand is row-sharded over `g_world` GPUs.
  // Every CTA's gather warp copies 8 KB chunks of the peers' shards into the local staging
  // buffer the B tensor map points at and counts finished chunks per 256-row block in g_ready.
  const unsigned long long* g_peer_bases;  // [g_world] base address of each rank's shard arena
  unsigned long long g_shard_offset;       // byte offset of this weight's shard inside the arena
  unsigned long long g_shard_bytes;        // bytes per rank ( = rows/world * row_bytes )
  unsigned long long g_total_bytes;        // rows * row_bytes
  unsigned char* g_dst;                    // local staging buffer [rows, row_bytes]
  unsigned int* g_ready;                   // [rows/256] finished-chunk counters (zeroed by host)
  unsigned int g_chunks_per_block;         // 256 * row_bytes / 8192
  int g_world;
};

constexpr int GATHER_CHUNK = 8192;
constexpr int GATHER_SLOTS = 4;

template <int BN>
struct Cfg {
  static constexpr int A_BYTES = BM * BK * 2;
  static constexpr int B_BYTES = BN * BK * 2;
  static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
  static constexpr int STAGES = (kSmemBudget - 1024) / STAGE_BYTES > 8
                                    ? 8
                                    : (kSmemBudget - 1024) / STAGE_BYTES;
  static constexpr int TMEM_COLS = 2 * BN < 32 ? 32 : 2 * BN;
  static constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + 1024 /*align slack*/ + 256 /*barriers*/;
  // gather variant: one stage less is never needed; the bounce slots live after the barriers
  static constexpr int GATHER_STAGES =
      (kSmemBudget - 1024 - GATHER_SLOTS * GATHER_CHUNK) / STAGE_BYTES > 8
          ? 8
          : (kSmemBudget - 1024 - GATHER_SLOTS * GATHER_CHUNK) / STAGE_BYTES;
};

__device__ __forceinline__ void decode_tile(int tile, int num_m, int num_n, int splits, int& m_blk,
                                            int& n_blk, int& split, bool n_major = false) {
  split = tile % splits;
  tile /= splits;
  if (n_major) {  // weights are consumed block by block in the order the gather warps fetch them
    n_blk = tile / num_m;
    m_blk = tile - n_blk * num_m;
    return;
  }
  constexpr int GROUP_M = 8;
  const int per_group = GROUP_M * num_n;
  const int group = tile / per_group;
  const int first_m = group * GROUP_M;
  const int gsz = min(num_m - first_m, GROUP_M);
  const int in_group = tile - group * per_group;
  m_blk = first_m + in_group % gsz;
  n_blk = in_group / gsz;
}

// bounded poll of a chunk counter written by other CTAs' gather warps
__device__ __forceinline__ bool wait_block_ready(const unsigned int* ctr, unsigned int target,
                                                 int* status) {
  unsigned int v;
  asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(ctr) : "memory");
  if (v >= target) return true;
  const uint64_t t0 = global_timer_ns();
  uint32_t spins = 0;
  while (true) {
    asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(ctr) : "memory");
    if (v >= target) return true;
    if ((++spins & 0xFF) == 0 && global_timer_ns() - t0 > AXB_WAIT_BUDGET_NS) {
      if (status) atomicCAS(status, 0, AXB_TIMEOUT_PEER_FLAG);
      return false;
    }
    __nanosleep(64);
  }
}

template <int BN, bool A_MN, bool B_MN, bool GATHER>
__global__ void __launch_bounds__(GATHER ? kThreads + 32 : kThreads, 1)
    gemm_bf16_tcgen05_kernel(const __grid_constant__ CUtensorMap tmA,
                             const __grid_constant__ CUtensorMap tmB,
                             const __grid_constant__ CUtensorMap tmA2,
                             const __grid_constant__ CUtensorMap tmB2, const GemmParams p) {
  using C = Cfg<BN>;
  constexpr int STAGES = GATHER ? C::GATHER_STAGES : C::STAGES;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~static_cast<uintptr_t>(1023));
  uint8_t* sA = smem;
  uint8_t* sB = smem + STAGES * C::A_BYTES;
  uint8_t* sBounce = smem + STAGES * C::STAGE_BYTES;  // GATHER only: 4 x 8 KB
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + STAGES * C::STAGE_BYTES +
                                               (GATHER ? GATHER_SLOTS * GATHER_CHUNK : 0));
  uint64_t* full_bar = bars;
  uint64_t* empty_bar = bars + STAGES;
  uint64_t* tfull_bar = bars + 2 * STAGES;
  uint64_t* tempty_bar = bars + 2 * STAGES + 2;
  uint64_t* bounce_bar = bars + 2 * STAGES + 4;  // [GATHER_SLOTS]
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * STAGES + 4 + GATHER_SLOTS);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;

  const int num_m = (p.M + BM - 1) / BM;
  const int num_n = (p.N + BN - 1) / BN;
  const int nk_main = (p.K + BK - 1) / BK;
  const int nk_ext = (p.K2 + BK - 1) / BK;
  const int nk_total = nk_main + nk_ext;
  const int total_tiles = num_m * num_n * p.splits;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 1);
    }
    if (GATHER)
      for (int s = 0; s < GATHER_SLOTS; ++s) mbar_init(&bounce_bar[s], 1);
    for (int s = 0; s < 2; ++s) {
      mbar_init(&tfull_bar[s], 1);
      mbar_init(&tempty_bar[s], 4);  // one arrival per epilogue warp
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
    // ------------------------------------------------------------ TMA producer
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      unsigned long long seen[2] = {0ull, 0ull};  // 256-row blocks already seen complete
      for (int tile = blockIdx.x; tile < total_tiles && ok; tile += gridDim.x) {
        int m_blk, n_blk, split;
        decode_tile(tile, num_m, num_n, p.splits, m_blk, n_blk, split, GATHER && !B_MN);
        const int kb0 = (int)((long long)nk_total * split / p.splits);
        const int kb1 = (int)((long long)nk_total * (split + 1) / p.splits);
        for (int kb = kb0; kb < kb1; ++kb) {
          if (!mbar_wait(&empty_bar[stage], phase ^ 1, p.status, AXB_TIMEOUT_EMPTY)) {
            ok = false;
            break;
          }
          const bool ext = kb >= nk_main;
          if (GATHER && !ext) {
            // rows of the (row-sharded) B operand this k block / tile reads, in 256-row blocks
            const int blk_lo = B_MN ? (kb * BK) >> 8 : (n_blk * BN) >> 8;
            const int blk_hi = B_MN ? (kb * BK + BK - 1) >> 8 : (n_blk * BN + BN - 1) >> 8;
            const int last_blk = (int)(p.g_total_bytes / ((unsigned long long)p.g_chunks_per_block * GATHER_CHUNK)) - 1;
            for (int b = blk_lo; b <= min(blk_hi, last_blk) && ok; ++b) {
              const bool known = b < 128 && ((seen[b >> 6] >> (b & 63)) & 1ull);
              if (!known) {
                if (!wait_block_ready(p.g_ready + b, p.g_chunks_per_block, p.status)) ok = false;
                else if (b < 128) seen[b >> 6] |= 1ull << (b & 63);
              }
            }
            if (!ok) break;
            asm volatile("fence.proxy.async;" ::: "memory");
          }
          mbar_expect_tx(&full_bar[stage], C::STAGE_BYTES);
          const CUtensorMap* ma = ext ? &tmA2 : &tmA;
          const CUtensorMap* mb = ext ? &tmB2 : &tmB;
          const int k0 = (ext ? kb - nk_main : kb) * BK;
          uint8_t* a_dst = sA + stage * C::A_BYTES;
          uint8_t* b_dst = sB + stage * C::B_BYTES;
          if (!A_MN) {
            tma_load_2d(a_dst, ma, &full_bar[stage], k0, m_blk * BM);
          } else {
#pragma unroll
            for (int c = 0; c < BM / 64; ++c)
              tma_load_2d(a_dst + c * 8192, ma, &full_bar[stage], m_blk * BM + c * 64, k0);
          }
          if (!B_MN) {
            tma_load_2d(b_dst, mb, &full_bar[stage], k0, n_blk * BN);
          } else {
#pragma unroll
            for (int c = 0; c < BN / 64; ++c)
              tma_load_2d(b_dst + c * 8192, mb, &full_bar[stage], n_blk * BN + c * 64, k0);
          }
          if (++stage == STAGES) {
            stage = 0;
            phase ^= 1;
          }
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------ MMA issuer
    if (lane == 0) {
      constexpr uint32_t idesc = make_idesc_bf16(BM, BN, A_MN ? 1 : 0, B_MN ? 1 : 0);
      int stage = 0;
      uint32_t phase = 0;
      int it = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < total_tiles && ok; tile += gridDim.x, ++it) {
        int m_blk, n_blk, split;
        decode_tile(tile, num_m, num_n, p.splits, m_blk, n_blk, split, GATHER && !B_MN);
        const int kb0 = (int)((long long)nk_total * split / p.splits);
        const int kb1 = (int)((long long)nk_total * (split + 1) / p.splits);
        const int acc = it & 1;
        const uint32_t acc_phase = (it >> 1) & 1;
        if (!mbar_wait(&tempty_bar[acc], acc_phase ^ 1, p.status, AXB_TIMEOUT_TMEM_EMPTY)) {
          ok = false;
          break;
        }
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + acc * BN;
        for (int kb = kb0; kb < kb1; ++kb) {
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
            umma_f16(d_tmem, da, db, idesc, (kb > kb0 || kk > 0) ? 1u : 0u);
          }
          umma_commit(&empty_bar[stage]);  // releases the smem stage when these MMAs retire
          if (++stage == STAGES) {
            stage = 0;
            phase ^= 1;
          }
        }
        if (!ok) break;
        umma_commit(&tfull_bar[acc]);
      }
    }
  } else if (GATHER && warp == 6) {
    // ------------------------------------------------------------ gather warp (all-gather of B)
    if (lane == 0) {
      const unsigned long long n_chunks = p.g_total_bytes / GATHER_CHUNK;
      const unsigned long long block_bytes = (unsigned long long)p.g_chunks_per_block * GATHER_CHUNK;
      auto src_of = [&](unsigned long long c) -> const unsigned char* {
        const unsigned long long byte = c * GATHER_CHUNK;
        const unsigned long long owner = byte / p.g_shard_bytes;
        return reinterpret_cast<const unsigned char*>(p.g_peer_bases[owner]) + p.g_shard_offset +
               (byte - owner * p.g_shard_bytes);
      };
      auto issue_load = [&](unsigned long long c, int slot) {
        mbar_expect_tx(&bounce_bar[slot], GATHER_CHUNK);
        bulk_load(sBounce + slot * GATHER_CHUNK, src_of(c), GATHER_CHUNK, &bounce_bar[slot]);
      };
      auto signal_done = [&](unsigned long long c) {
        asm volatile("fence.proxy.async;" ::: "memory");
        unsigned int* ctr = p.g_ready + (c * GATHER_CHUNK) / block_bytes;
        asm volatile("red.release.gpu.global.add.u32 [%0], 1;" ::"l"(ctr) : "memory");
      };
      // prologue: up to GATHER_SLOTS loads in flight
      unsigned long long c_issue = blockIdx.x;
      int n_issued = 0;
      for (; n_issued < GATHER_SLOTS && c_issue < n_chunks; ++n_issued, c_issue += gridDim.x)
        issue_load(c_issue, n_issued);
      unsigned long long prev = ~0ull;
      int i = 0;
      bool ok = true;
      for (unsigned long long c = blockIdx.x; c < n_chunks && ok; c += gridDim.x, ++i) {
        const int slot = i % GATHER_SLOTS;
        const uint32_t ph = (i / GATHER_SLOTS) & 1;
        if (!mbar_wait(&bounce_bar[slot], ph, p.status, AXB_TIMEOUT_PEER_FLAG)) {
          ok = false;
          break;
        }
        // smem -> local staging buffer
        asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], %2;" ::"l"(
                         p.g_dst + c * GATHER_CHUNK),
                     "r"(smem_u32(sBounce + slot * GATHER_CHUNK)), "r"(GATHER_CHUNK)
                     : "memory");
        asm volatile("cp.async.bulk.commit_group;" ::: "memory");
        if (prev != ~0ull) {  // everything but the newest store is globally complete
          asm volatile("cp.async.bulk.wait_group 1;" ::: "memory");
          signal_done(prev);
        }
        prev = c;
        if (c_issue < n_chunks) {  // refill this slot once the store has read it
          asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");
          issue_load(c_issue, slot);
          c_issue += gridDim.x;
        }
      }
      asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");
      if (ok && prev != ~0ull) signal_done(prev);
    }
  } else {
    // ------------------------------------------------------------ epilogue warps
    const int lane_group = warp & 3;  // TMEM lanes [32*lane_group, 32*lane_group+32)
    int it = 0;
    bool ok = true;
    for (int tile = blockIdx.x; tile < total_tiles && ok; tile += gridDim.x, ++it) {
      int m_blk, n_blk, split;
      decode_tile(tile, num_m, num_n, p.splits, m_blk, n_blk, split, GATHER && !B_MN);
      const int kb0 = (int)((long long)nk_total * split / p.splits);
      const int kb1 = (int)((long long)nk_total * (split + 1) / p.splits);
      const int acc = it & 1;
      const uint32_t acc_phase = (it >> 1) & 1;
      if (!mbar_wait(&tfull_bar[acc], acc_phase, p.status, AXB_TIMEOUT_TMEM_FULL)) {
        ok = false;
        break;
      }
      tc_fence_after();
      const long long row = (long long)m_blk * BM + lane_group * 32 + lane;
      const bool row_ok = row < p.M && kb1 > kb0;
      const uint32_t t_addr = tmem_base + (uint32_t(lane_group * 32) << 16) + acc * BN;
#pragma unroll 1
      for (int c = 0; c < BN / 32; ++c) {
        uint32_t r[32];
        tmem_ld_32x32(t_addr + c * 32, r);
        tmem_ld_wait();
        const int col0 = n_blk * BN + c * 32;
        if (!row_ok || col0 >= p.N) continue;
        float v[32];
#pragma unroll
        for (int j = 0; j < 32; ++j) v[j] = __uint_as_float(r[j]) * p.alpha;
        const bool full_chunk = col0 + 32 <= p.N;
        if (p.out_mode == 0) {
          __nv_bfloat16* crow = reinterpret_cast<__nv_bfloat16*>(p.C) + row * p.ldc + col0;
          const __nv_bfloat16* irow =
              p.Cin ? reinterpret_cast<const __nv_bfloat16*>(p.Cin) + row * p.ldcin + col0 : nullptr;
          if (full_chunk && (p.ldc & 7) == 0 && (!irow || (p.ldcin & 7) == 0)) {
#pragma unroll
            for (int q = 0; q < 4; ++q) {
              if (irow) {
                uint4 in = *reinterpret_cast<const uint4*>(irow + q * 8);
                const uint32_t w[4] = {in.x, in.y, in.z, in.w};
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                  float2 f = unpack_bf16x2(w[e]);
                  v[q * 8 + 2 * e] += p.beta * f.x;
                  v[q * 8 + 2 * e + 1] += p.beta * f.y;
                }
              }
              uint4 o;
              o.x = pack_bf16x2(v[q * 8 + 0], v[q * 8 + 1]);
              o.y = pack_bf16x2(v[q * 8 + 2], v[q * 8 + 3]);
              o.z = pack_bf16x2(v[q * 8 + 4], v[q * 8 + 5]);
              o.w = pack_bf16x2(v[q * 8 + 6], v[q * 8 + 7]);
              *reinterpret_cast<uint4*>(crow + q * 8) = o;
            }
          } else {
            for (int j = 0; j < 32 && col0 + j < p.N; ++j) {
              float x = v[j];
              if (irow) x += p.beta * __bfloat162float(irow[j]);
              crow[j] = __float2bfloat16(x);
            }
          }
        } else if (p.out_mode == 1) {
          float* crow = reinterpret_cast<float*>(p.C) + row * p.ldc + col0;
          const float* irow =
              p.Cin ? reinterpret_cast<const float*>(p.Cin) + row * p.ldcin + col0 : nullptr;
          if (full_chunk && (p.ldc & 3) == 0 && (!irow || (p.ldcin & 3) == 0)) {
#pragma unroll
            for (int q = 0; q < 8; ++q) {
              float4 o = make_float4(v[q * 4], v[q * 4 + 1], v[q * 4 + 2], v[q * 4 + 3]);
              if (irow) {
                float4 in = *reinterpret_cast<const float4*>(irow + q * 4);
                o.x += p.beta * in.x;
                o.y += p.beta * in.y;
                o.z += p.beta * in.z;
                o.w += p.beta * in.w;
              }
              *reinterpret_cast<float4*>(crow + q * 4) = o;
            }
          } else {
            for (int j = 0; j < 32 && col0 + j < p.N; ++j)
              crow[j] = v[j] + (irow ? p.beta * irow[j] : 0.f);
          }
        } else {
          float* crow = reinterpret_cast<float*>(p.C) + row * p.ldc + col0;
          for (int j = 0; j < 32 && col0 + j < p.N; ++j) atomicAdd(crow + j, v[j]);
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
    tmem_dealloc(tmem_base, C::TMEM_COLS);
  }
}

template <int BN, bool A_MN, bool B_MN, bool GATHER>
int launch_gemm(const CUtensorMap& tA, const CUtensorMap& tB, const CUtensorMap& tA2,
                const CUtensorMap& tB2, const GemmParams& p, int sm_count, cudaStream_t stream) {
  using C = Cfg<BN>;
  constexpr int smem_bytes =
      GATHER ? C::GATHER_STAGES * C::STAGE_BYTES + GATHER_SLOTS * GATHER_CHUNK + 1024 + 256
             : C::SMEM_BYTES;
  auto kern = gemm_bf16_tcgen05_kernel<BN, A_MN, B_MN, GATHER>;
  static bool attr_set = false;
  if (!attr_set) {
    cudaError_t e =
        cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem_bytes);
    if (e != cudaSuccess) return (int)e;
    attr_set = true;
  }
  const int num_m = (p.M + BM - 1) / BM;
  const int num_n = (p.N + BN - 1) / BN;
  const int tiles = num_m * num_n * p.splits;
  // gather kernels always launch one CTA per SM: every CTA carries a share of the all-gather
  const int grid = GATHER ? sm_count : (tiles < sm_count ? tiles : sm_count);
  kern<<<grid, GATHER ? kThreads + 32 : kThreads, smem_bytes, stream>>>(tA, tB, tA2, tB2, p);
  return (int)cudaGetLastError();
}

template <int BN>
int dispatch_major(int a_mn, int b_mn, const CUtensorMap& tA, const CUtensorMap& tB,
                   const CUtensorMap& tA2, const CUtensorMap& tB2, const GemmParams& p,
                   int sm_count, cudaStream_t stream) {
  if (!a_mn && !b_mn)
    return launch_gemm<BN, false, false, false>(tA, tB, tA2, tB2, p, sm_count, stream);
  if (!a_mn && b_mn)
    return launch_gemm<BN, false, true, false>(tA, tB, tA2, tB2, p, sm_count, stream);
  if (a_mn && !b_mn)
    return launch_gemm<BN, true, false, false>(tA, tB, tA2, tB2, p, sm_count, stream);
  return launch_gemm<BN, true, true, false>(tA, tB, tA2, tB2, p, sm_count, stream);
}

int g_sm_count = 0;


struct GatherArgs {
  const unsigned long long* peer_bases = nullptr;
  unsigned long long shard_offset = 0, shard_bytes = 0;
  void* staging = nullptr;
  unsigned int* ready = nullptr;
  int world = 0;
};

static int gemm_entry(const void* A, long long lda, int a_mn, const void* B, long long ldb, int b_mn,
                      void* C, long long ldc, const void* Cin, long long ldcin, int M, int N, int K,
                      const void* A2, long long lda2, const void* B2, long long ldb2, int K2,
                      float alpha, float beta, int out_mode, int splits, int bn, int* status,
                      void* stream, const GatherArgs* ga) {
  if (M <= 0 || N <= 0 || (K <= 0 && K2 <= 0)) return 0;
  if ((lda & 7) || (ldb & 7) || (K2 > 0 && ((lda2 & 7) || (ldb2 & 7)))) return -2;
  if (splits < 1) splits = 1;
  if (splits > 1 && out_mode != 2) return -3;
  if (g_sm_count == 0) {
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&g_sm_count, cudaDevAttrMultiProcessorCount, dev);
    if (g_sm_count <= 0) g_sm_count = 148;
  }
  CUtensorMap tA, tB, tA2, tB2;
  int rc = 0;
  // K-major operand [R, K]: box [BM|BN rows, 64 cols]; MN-major operand [K, R]: box [64, 64].
  rc |= a_mn ? axb_make_tmap_2d(&tA, A, K, M, lda, 64, 64)
             : axb_make_tmap_2d(&tA, A, M, K, lda, BM, 64);
  rc |= b_mn ? axb_make_tmap_2d(&tB, B, K, N, ldb, 64, 64)
             : axb_make_tmap_2d(&tB, B, N, K, ldb, bn, 64);
  if (K2 > 0) {
    rc |= a_mn ? axb_make_tmap_2d(&tA2, A2, K2, M, lda2, 64, 64)
               : axb_make_tmap_2d(&tA2, A2, M, K2, lda2, BM, 64);
    rc |= b_mn ? axb_make_tmap_2d(&tB2, B2, K2, N, ldb2, 64, 64)
               : axb_make_tmap_2d(&tB2, B2, N, K2, ldb2, bn, 64);
  } else {
    tA2 = tA;
    tB2 = tB;
  }
  if (rc) return -4;
  GemmParams p = {};
  p.M = M;
  p.N = N;
  p.K = K;
  p.K2 = K2 > 0 ? K2 : 0;
  p.C = C;
  p.Cin = Cin;
  p.ldc = ldc;
  p.ldcin = ldcin;
  p.alpha = alpha;
  p.beta = beta;
  p.out_mode = out_mode;
  p.splits = splits;
  p.status = status;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  if (ga != nullptr) {
    // B is the staging buffer: [N, K] (b_mn = 0) or [K, N] (b_mn = 1), contiguous rows
    const unsigned long long rows = b_mn ? (unsigned long long)K : (unsigned long long)N;
    const unsigned long long row_bytes = 2ull * (b_mn ? (unsigned long long)N : (unsigned long long)K);
    if (a_mn || splits != 1 || (bn != 128 && bn != 256)) return -6;
    if (rows % 256 || (256 * row_bytes) % GATHER_CHUNK || ga->shard_bytes % GATHER_CHUNK ||
        (unsigned long long)ldb * 2 != row_bytes || ga->shard_bytes * ga->world != rows * row_bytes)
      return -7;
    p.g_peer_bases = ga->peer_bases;
    p.g_shard_offset = ga->shard_offset;
    p.g_shard_bytes = ga->shard_bytes;
    p.g_total_bytes = rows * row_bytes;
    p.g_dst = reinterpret_cast<unsigned char*>(ga->staging);
    p.g_ready = ga->ready;
    p.g_chunks_per_block = (unsigned int)(256 * row_bytes / GATHER_CHUNK);
    p.g_world = ga->world;
    cudaError_t e = cudaMemsetAsync(ga->ready, 0, sizeof(unsigned int) * (rows / 256), st);
    if (e != cudaSuccess) return (int)e;
    if (bn == 256)
      return b_mn ? launch_gemm<256, false, true, true>(tA, tB, tA2, tB2, p, g_sm_count, st)
                  : launch_gemm<256, false, false, true>(tA, tB, tA2, tB2, p, g_sm_count, st);
    return b_mn ? launch_gemm<128, false, true, true>(tA, tB, tA2, tB2, p, g_sm_count, st)
                : launch_gemm<128, false, false, true>(tA, tB, tA2, tB2, p, g_sm_count, st);
  }
  switch (bn) {
    case 64:
      return dispatch_major<64>(a_mn, b_mn, tA, tB, tA2, tB2, p, g_sm_count, st);
    case 128:
      return dispatch_major<128>(a_mn, b_mn, tA, tB, tA2, tB2, p, g_sm_count, st);
    case 256:
      return dispatch_major<256>(a_mn, b_mn, tA, tB, tA2, tB2, p, g_sm_count, st);
    default:
      return -5;
  }
}

}  // namespace

// C[M,N] = alpha * (A.B^T + A2.B2^T) + beta * Cin
//   a_mn = 0: A is [M,K] row-major (lda);  a_mn = 1: A is stored transposed, [K,M] row-major.
//   b_mn = 0: B is [N,K] row-major (ldb);  b_mn = 1: B is stored transposed, [K,N] row-major.
//   A2/B2 (optional, K2 > 0) use the same storage convention as A/B.
//   out_mode 0: bf16 C, 1: fp32 C, 2: fp32 atomic accumulate into C (required when splits > 1).
//   bn: tile width 64 / 128 / 256. Leading dimensions must be multiples of 8 elements.
// Returns 0 or a CUDA / driver error code; asynchronous device-side wait timeouts land in *status.
extern "C" int axb_gemm_bf16(const void* A, long long lda, int a_mn, const void* B, long long ldb,
                             int b_mn, void* C, long long ldc, const void* Cin, long long ldcin,
                             int M, int N, int K, const void* A2, long long lda2, const void* B2,
                             long long ldb2, int K2, float alpha, float beta, int out_mode,
                             int splits, int bn, int* status, void* stream) {
  return gemm_entry(A, lda, a_mn, B, ldb, b_mn, C, ldc, Cin, ldcin, M, N, K, A2, lda2, B2, ldb2, K2,
                    alpha, beta, out_mode, splits, bn, status, stream, nullptr);
}

// Same contraction with the all-gather of a row-sharded B fused in: rank r owns rows
// [r*rows/world, (r+1)*rows/world) of the stored B matrix at `peer_bases[r] + shard_offset`
// (peer_bases: DEVICE array of `world` arena addresses, peer-mapped). `staging` is a local
// buffer of the full B size that the kernel fills block by block while the MMA warps consume
// it; `ready` is a zero-able counter array with one entry per 256 stored rows.
extern "C" int axb_gemm_bf16_allgather(const void* A, long long lda, void* staging, int b_mn,
                                       void* C, long long ldc, const void* Cin, long long ldcin,
                                       int M, int N, int K, const void* A2, long long lda2,
                                       const void* B2, long long ldb2, int K2, float alpha,
                                       float beta, int out_mode, int bn,
                                       const unsigned long long* peer_bases,
                                       unsigned long long shard_offset,
                                       unsigned long long shard_bytes, int world,
                                       unsigned int* ready, int* status, void* stream) {
  GatherArgs ga;
  ga.peer_bases = peer_bases;
  ga.shard_offset = shard_offset;
  ga.shard_bytes = shard_bytes;
  ga.staging = staging;
  ga.ready = ready;
  ga.world = world;
  const long long ldb = b_mn ? N : K;
  return gemm_entry(A, lda, 0, staging, ldb, b_mn, C, ldc, Cin, ldcin, M, N, K, A2, lda2, B2, ldb2,
                    K2, alpha, beta, out_mode, 1, bn, status, stream, &ga);
}
